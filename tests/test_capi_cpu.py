"""C-ABI boundary without a GPU: the product library loads, exports every declared symbol, survives
null handles and bad ids (kurumi/src/capi/tests.rs:236-276), refuses to create anything but a CUDA
backend, and every kernel it would launch for the benchmark graphs compiles for sm_100a."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from kurumi_b200 import api, configs

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = []
    for h in ("kurumi.h", "kurumi_cuda.h"):
        text = open(os.path.join(ROOT, "include", h)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names += re.findall(r"\b(ku_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_every_declared_symbol_is_exported(cuda_lib):
    names = declared_symbols()
    assert len(names) > 120
    missing = [n for n in names if not cuda_lib.has(n)]
    assert not missing, missing


def test_oracle_exports_the_same_builder_abi(oracle_lib):
    text = re.sub(r"/\*.*?\*/", "", open(os.path.join(ROOT, "include", "kurumi.h")).read(), flags=re.S)
    for n in sorted(set(re.findall(r"\b(ku_[a-z0-9_]+)\s*\(", text))):
        assert oracle_lib.has(n), n


def test_null_handles_and_bad_ids_do_not_crash(cuda_lib):
    L = cuda_lib.lib
    assert cuda_lib.node_fn("ku_add")(None, C.c_uint32(0), C.c_uint32(1)) == api.KU_ERR
    assert "null graph" in cuda_lib.last_error()
    g = api.Graph(cuda_lib)
    with pytest.raises(api.Error):
        g.add(7, 9)                       # ids that do not exist
    with pytest.raises(api.Error):
        g.input([2], 99)                  # bad dtype tag
    assert L.ku_eval(None, C.c_uint32(0), None) is None
    assert L.ku_eval_many(None, None, C.c_size_t(0), None, None, None) == -1
    assert L.ku_tensor_rank(None) == 0 and L.ku_tensor_nbytes(None) == 0
    L.ku_tensor_free(None); L.ku_graph_free(None); L.ku_feeds_free(None); L.ku_backend_free(None)
    L.ku_feeds_set(None, C.c_uint32(0), None)
    assert L.ku_node_rank(g.h, C.c_uint32(1234)) == C.c_size_t(-1).value
    assert L.ku_node_dtype(g.h, C.c_uint32(1234)) == api.KU_ERR
    assert L.ku_tensor_new(C.c_uint32(99), None, C.c_size_t(0), None, C.c_size_t(0)) is None
    t = api.Tensor.from_numpy(cuda_lib, np.arange(6, dtype=np.int32).reshape(2, 3))
    assert t.shape == (2, 3) and t.dtype == api.I32 and t.numpy().tolist() == [[0, 1, 2], [3, 4, 5]]
    out = (C.c_float * 6)()
    assert L.ku_tensor_data_f32(t.h, out, C.c_size_t(6)) == -1 and "not F32" in cuda_lib.last_error()


def test_only_the_cuda_backend_exists_in_the_product_library(cuda_lib):
    for kind in (api.KU_CPU, api.KU_METAL, 7):
        with pytest.raises(api.Error):
            api.Backend(cuda_lib, kind)
    assert "only KU_CUDA" in cuda_lib.last_error() or "unknown kind" in cuda_lib.last_error()


def test_builders_record_the_reference_decompositions(cuda_lib, oracle_lib):
    """Same builder calls give the same graph in both libraries (they share the IR sources)."""
    dumps = []
    for lib in (cuda_lib, oracle_lib):
        g = api.Graph(lib)
        x = g.input([4, 8], api.BF16)
        y = g.gelu(g.add(g.matmul(x, g.input([8, 8], api.BF16)), g.broadcast_to(g.input([8], api.BF16), [4, 8])))
        dumps.append(g.dump(y))
        assert g.node_count(y) == len(dumps[-1].splitlines())
    assert dumps[0] == dumps[1] and dumps[0].count("Exp2") == 1 and dumps[0].count("DotGeneral") == 1


@pytest.mark.parametrize("name", ["c1", "c2", "c3", "c4", "c5", "c5_plain"])
def test_generated_kernels_compile_for_sm100a(cuda_lib, name):
    """NVRTC cross-compiles every kernel of the five benchmark graphs (reduced sizes) without a GPU."""
    g = api.Graph(cuda_lib)
    root = {"c1": lambda: configs.fused_reduce(g, 256, 512)[0],
            "c2": lambda: configs.transposed_softmax(g, 1024)[0],
            "c3": lambda: configs.gemm_bias_gelu(g, 256, 512, 384)[0],
            "c4": lambda: configs.causal_attention(g, 1, 2, 256, 128, fused=True)[0],
            "c5": lambda: configs.fp8_weight_gemm(g, 256, 384, 512, amp=True)[0],
            "c5_plain": lambda: configs.fp8_weight_gemm(g, 256, 384, 512, amp=False)[0]}[name]()
    fams = api.compile_check(cuda_lib, g, [root])
    assert fams, fams


def test_input_generators_compile(cuda_lib):
    g = api.Graph(cuda_lib)
    _, gens = configs.fp8_weight_gemm(g, 128, 256, 128)
    h = api.Graph(cuda_lib)
    roots = [gen(h) for gen in gens.values()]
    assert api.compile_check(cuda_lib, h, roots)


def test_plan_compile_and_replay(oracle_lib, cpu):
    """ku_plan_compile / ku_plan_run (kurumi/src/capi/eval.rs:152-182): a plan replays with fresh feeds and equals
    ku_eval_with; off the f32 fused path the reference returns NULL with a message, and so does the CPU oracle."""
    import numpy as np
    from kurumi_b200 import api
    g = api.Graph(oracle_lib)
    x, y = g.input([4, 6], api.F32), g.input([4, 6], api.F32)
    root = g.sum(g.relu(g.add(g.mul(x, y), g.mul(g.scalar(x, 0.5), x))), 1)
    plan = api.Plan(g, root)
    rng = np.random.default_rng(2)
    for _ in range(2):
        xv, yv = rng.standard_normal((4, 6)).astype(np.float32), rng.standard_normal((4, 6)).astype(np.float32)
        f = api.Feeds(oracle_lib).set(x, xv).set(y, yv)
        assert np.array_equal(plan.run(f).numpy(), cpu.eval_with(g, root, f).numpy())
    with pytest.raises(api.Error, match="not on the f32 fused plan path"):
        api.Plan(g, g.softmax(x, 1))
    other = api.Graph(oracle_lib)
    other.input([4, 6], api.F32)
    with pytest.raises(api.Error, match="another graph"):
        plan.run(api.Feeds(oracle_lib), other)
    with pytest.raises(api.Error):
        api.Plan(g, 10 ** 6)
