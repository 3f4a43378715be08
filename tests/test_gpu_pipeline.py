"""ku_eval_with on host tensors streams a large row-separable evaluation through the device in chunks (upload, kernels
and download overlapped, kurumi_b200/csrc/cuda/pipeline.cc): the result equals the evaluation done in one piece on
device-resident inputs, bit for bit, for each of the five benchmark graphs; graphs that do not separate, and small
ones, take the one-piece path."""
import numpy as np
import pytest

from kurumi_b200 import api, configs

pytestmark = pytest.mark.gpu

CASES = [
    (configs.fused_reduce, dict(rows=2048, cols=2048)),
    (configs.transposed_softmax, dict(n=2048)),
    (configs.gemm_bias_gelu, dict(m=4096, n=1024, kdim=1024)),
    (configs.causal_attention, dict(batch=8, heads=4, seq=1024, dh=128, fused=True)),
    (configs.fp8_weight_gemm, dict(m=4096, kdim=1024, n=2048, amp=True)),
    # what one of eight ranks evaluates of each full-size configuration: the chunks of a shard are the smallest pieces
    # the kernels meet (128 softmax lines, 64 rows of a reduction, 128 rows of a contraction, 4 heads)
    (configs.fused_reduce, dict(rows=512, cols=4096)),
    (configs.transposed_softmax, dict(n=8192, lines=1024)),
    (configs.gemm_bias_gelu, dict(m=1024, n=8192, kdim=8192)),
    (configs.causal_attention, dict(batch=1, heads=32, seq=4096, dh=128)),
    (configs.fp8_weight_gemm, dict(m=2048, kdim=8192, n=28672, amp=True)),
    # and one of four ranks
    (configs.fused_reduce, dict(rows=1024, cols=4096)),
    (configs.transposed_softmax, dict(n=8192, lines=2048)),
    (configs.gemm_bias_gelu, dict(m=2048, n=8192, kdim=8192)),
    (configs.causal_attention, dict(batch=2, heads=32, seq=4096, dh=128)),
    (configs.fp8_weight_gemm, dict(m=4096, kdim=8192, n=28672, amp=True)),
]


@pytest.mark.parametrize("make,kwargs", CASES)
def test_chunked_host_evaluation_equals_one_piece(cuda_lib, gpu, make, kwargs):
    g = api.Graph(cuda_lib)
    root, gens = make(g, **kwargs)
    dev, host = {}, api.Feeds(cuda_lib)
    for node, mk in gens.items():
        h = api.Graph(cuda_lib)
        dev[node] = gpu.eval_device(h, [mk(h)])[0]
        host.set(node, dev[node].numpy(), dev[node].dtype)
    one_piece = gpu.eval_device(g, [root], None, dev)[0].numpy()
    before = gpu.stats()
    chunked = gpu.eval_with(g, root, host)
    after = gpu.stats()
    got = chunked.numpy()

    def same(a, b):
        if make is configs.transposed_softmax:   # a chunk of lines may run another softmax kernel (another summation order): the f32 band applies
            return a.shape == b.shape and np.allclose(a, b, rtol=1e-5, atol=1e-12)
        if a.shape == b.shape and a.tobytes() == b.tobytes():
            return True
        # a chunk of few rows may take the one-SM form of the contraction kernel instead of the SM-pair form: the same
        # products, accumulated in f32 in another grouping, so results may differ by one rounding step of bf16
        if chunked.dtype != api.BF16 or a.shape != b.shape:
            return False
        fa, fb = api.bf16_to_f32(a).astype(np.float64), api.bf16_to_f32(b).astype(np.float64)
        return bool((np.abs(fa - fb) <= 2.0 ** -7 * np.maximum(np.abs(fa), np.abs(fb)) + 1e-30).all())
    assert same(got, one_piece)
    # it really ran in chunks: several launches of the same program, and exactly the input / output bytes crossed the bus
    if make is configs.causal_attention and kwargs["batch"] == 1:
        assert after["launches"] - before["launches"] == 1      # attention separates over the batch axis only: one piece
    else:
        assert after["launches"] - before["launches"] >= 2
    assert after["h2d_bytes"] - before["h2d_bytes"] == sum(d.nbytes for d in dev.values())
    assert after["d2h_bytes"] - before["d2h_bytes"] == one_piece.nbytes
    # a second call replays the cached pipeline
    again = gpu.eval_with(g, root, host).numpy()
    assert again.tobytes() == got.tobytes()
    gpu.release_graph(g)
    assert gpu.eval_with(g, root, host).numpy().tobytes() == got.tobytes()


def test_graphs_that_do_not_separate_run_in_one_piece(cuda_lib, gpu):
    rng = np.random.default_rng(3)
    g = api.Graph(cuda_lib)
    x = g.input([4096, 2048], api.F32)
    root = g.softmax(x, 0)                       # normalises along the rows
    xv = rng.standard_normal((4096, 2048)).astype(np.float32)
    before = gpu.stats()["launches"]
    got = gpu.eval_with(g, root, api.Feeds(cuda_lib).set(x, xv)).numpy()
    assert gpu.stats()["launches"] - before <= 2
    e = np.exp(xv.astype(np.float64) - xv.max(axis=0))
    assert np.abs(got - e / e.sum(axis=0)).max() < 1e-6


def test_missing_and_misshapen_feeds_fail_before_anything_is_queued(cuda_lib, gpu):
    g = api.Graph(cuda_lib)
    root, gens = configs.fused_reduce(g, rows=2048, cols=2048)
    x, y = list(gens)
    ok = np.zeros((2048, 2048), np.float32)
    gpu.eval_with(g, root, api.Feeds(cuda_lib).set(x, ok).set(y, ok))
    with pytest.raises(api.Error, match="missing feed"):
        gpu.eval_with(g, root, api.Feeds(cuda_lib).set(x, ok))
    with pytest.raises(api.Error, match="has shape"):
        gpu.eval_with(g, root, api.Feeds(cuda_lib).set(x, ok).set(y, np.zeros((2048, 1024), np.float32)))
    assert np.array_equal(gpu.eval_with(g, root, api.Feeds(cuda_lib).set(x, ok).set(y, ok)).numpy(), np.zeros(2048, np.float32))


def test_plan_compile_and_replay_on_the_device(cuda_lib, gpu):
    """ku_plan_compile builds the device program ahead of the first run; ku_plan_run replays it with fresh feeds and
    equals ku_eval_with. A graph off the reference's f32 fused path (a softmax) compiles here too."""
    rng = np.random.default_rng(8)
    g = api.Graph(cuda_lib)
    root, gens = configs.fused_reduce(g, rows=96, cols=512)
    x, y = list(gens)
    plan = api.Plan(g, root)
    for _ in range(2):
        xv, yv = rng.uniform(-1, 1, (96, 512)).astype(np.float32), rng.uniform(-1, 1, (96, 512)).astype(np.float32)
        f = api.Feeds(cuda_lib).set(x, xv).set(y, yv)
        assert np.array_equal(plan.run(f).numpy(), gpu.eval_with(g, root, f).numpy())
    sm = g.softmax(g.mul(x, y), 1)
    p2 = api.Plan(g, sm)
    xv = rng.standard_normal((96, 512)).astype(np.float32)
    out = p2.run(api.Feeds(cuda_lib).set(x, xv).set(y, xv)).numpy()
    assert np.abs(out.sum(axis=1) - 1).max() < 1e-5
    with pytest.raises(api.Error, match="missing feed"):
        plan.run(api.Feeds(cuda_lib).set(x, xv))
