"""Parity of fused attention (Op::Sdpa on the tcgen05 kernel) and of the decomposed form with the CPU
oracle. Tolerance: rel 2e-2 against the f64 interpreter run, as stated for bf16 attention."""
import numpy as np
import pytest

from kurumi_b200 import api, configs
from tests import util
from tests.util import Pair

pytestmark = pytest.mark.gpu


def bf16(rng, shape, scale=1.0):
    return api.f32_to_bf16((rng.standard_normal(shape) * scale).astype(np.float32))


@pytest.mark.parametrize("shape,causal", [((2, 3, 256, 128), True), ((1, 2, 384, 64), True), ((2, 200, 128), True), ((1, 1, 128, 128), False),
                                          ((3, 130, 64), False), ((1, 4, 1, 128), True), ((1, 2, 640, 128), True), ((2, 1100, 64), True), ((1, 2, 1000, 128), False)])
def test_fused_attention_matches_oracle(oracle_lib, cuda_lib, cpu, cpu64, gpu, shape, causal):
    rng = np.random.default_rng(40)
    p = Pair(oracle_lib, cuda_lib)
    q, k, v = (p.feed(shape, api.BF16, bf16(rng, shape)) for _ in range(3))
    out = p.sdpa_fused(q, k, v, causal)
    assert api.compile_check(cuda_lib, p.gc, [out]) == ["attention_tc"]
    o, c, dts = p.run(cpu, gpu, [out])
    w, _, _ = p.run(cpu64, gpu, [out])
    got = util.to_f64(c[0], dts[0])
    util.assert_band(w[0], got, 2e-2, 2.0 ** -8, f"fused attention {shape} vs f64 run")
    # the native-dtype oracle rounds raw scores, scaled scores and probabilities to bf16 on the way: it is itself further
    # from the f64 run than the kernel is, so this is a cross-check with a wide band (the stated band is the one above)
    util.assert_band(util.to_f64(o[0], dts[0]), got, 6e-2, 2.0 ** -6, f"fused attention {shape} vs bf16 oracle")
    if causal:   # query 0 attends to key 0 only (kurumi_core/tests/ops.rs:258-270)
        vv = util.to_f64(p.feeds[v][0], api.BF16)
        assert np.array_equal(got[..., 0, :], vv[..., 0, :])


def test_decomposed_attention_and_auto_selection(oracle_lib, cuda_lib, cpu, cpu64, gpu):
    rng = np.random.default_rng(41)
    for tag, mk in ((api.F32, lambda s: rng.standard_normal(s).astype(np.float32)), (api.BF16, lambda s: bf16(rng, s))):
        p = Pair(oracle_lib, cuda_lib)
        shape = (2, 2, 48, 16)
        q, k, v = (p.feed(shape, tag, mk(shape)) for _ in range(3))
        nodes = [p.sdpa(q, k, v, True), p.sdpa_decomposed(q, k, v, False), p.sdpa_fused(q, k, v, True)]   # dh = 16: the fused primitive runs decomposed on device
        o, c, dts = p.run(cpu, gpu, nodes)
        w, _, _ = p.run(cpu64, gpu, nodes)
        for a, b, z, dt in zip(o, c, w, dts):
            if tag == api.F32:
                util.assert_close(z, util.to_f64(b, dt), 1e-4, 1e-4 * np.abs(z).max(), "decomposed attention f32")
            else:   # scores and probabilities are rounded to bf16 between the kernels, exactly the interpreter's steps: the
                # native oracle is the reference here (one bf16 step); those roundings put the interpreter itself, and so this
                # path, further from the f64 run than the fused kernel is
                util.assert_band(util.to_f64(a, dt), util.to_f64(b, dt), 2.0 ** -6, 2.0 ** -7, "decomposed attention bf16 vs bf16 oracle")
                util.assert_band(z, util.to_f64(b, dt), 6e-2, 2.0 ** -6, "decomposed attention bf16 vs f64 run")


def test_attention_config_graph_uses_the_fused_primitive(cuda_lib):
    g = api.Graph(cuda_lib)
    root, _ = configs.causal_attention(g)     # [8, 32, 4096, 128]: score buffer over 1 GiB -> Op::Sdpa
    assert "Sdpa" in g.dump(root)
    assert api.compile_check(cuda_lib, g, [root]) == ["attention_tc"]


def test_the_decomposition_runs_the_same_fused_kernel(oracle_lib, cuda_lib, cpu64, gpu):
    """Graph::sdpa records dot -> scale -> causal bias -> softmax -> dot below its 1 GiB score-buffer threshold and the
    fused primitive above it (kurumi_core/src/graph/ops/nn/attention.rs:78-113): the backend finds the decomposition again,
    so the same call runs the same kernel at every size. A decomposition whose scores are also wanted stays decomposed."""
    rng = np.random.default_rng(44)
    small, big = api.Graph(cuda_lib), api.Graph(cuda_lib)
    for g, shape in ((small, [2, 2, 512, 128]), (big, [8, 32, 4096, 128])):
        q, k, v = (g.input(shape, api.BF16) for _ in range(3))
        root = g.sdpa(q, k, v, True)
        assert ("Sdpa" in g.dump(root)) == (g is big)
        assert api.compile_check(cuda_lib, g, [root]) == ["attention_tc"]
    for shape, causal in (((2, 2, 512, 128), True), ((1, 3, 300, 64), False)):
        p = Pair(oracle_lib, cuda_lib)
        q, k, v = (p.feed(shape, api.BF16, bf16(rng, shape)) for _ in range(3))
        out = p.sdpa_decomposed(q, k, v, causal)
        assert api.compile_check(cuda_lib, p.gc, [out]) == ["attention_tc"]
        w, c, dts = p.run(cpu64, gpu, [out])
        util.assert_band(w[0], util.to_f64(c[0], dts[0]), 2e-2, 2.0 ** -8, f"decomposition on the fused kernel {shape}")
    # the probabilities are an output too: nothing may be skipped
    p = Pair(oracle_lib, cuda_lib)
    shape = (1, 2, 256, 128)
    q, k, v = (p.feed(shape, api.BF16, bf16(rng, shape)) for _ in range(3))
    out = p.sdpa_decomposed(q, k, v, True)
    probs = p.go.node_src(out)[0] if hasattr(p.go, "node_src") else None
    fams = api.compile_check(cuda_lib, p.gc, [out, p.mul(out, out)])
    assert fams[0] == "attention_tc"
