"""Parity of the tensor-core contraction (tcgen05 / TMEM, TMA-fed) with the CPU oracle, through the
C ABI. Tolerance: rel 2e-2 against the f64 interpreter run (stated for bf16 / fp8 GEMM), and one
narrow-format rounding step against the native-dtype oracle, whose f32 accumulation order differs."""
import numpy as np
import pytest

from kurumi_b200 import api, configs
from tests import util
from tests.util import Pair

pytestmark = pytest.mark.gpu


def bf16(rng, shape, scale=1.0):
    return api.f32_to_bf16((rng.standard_normal(shape) * scale).astype(np.float32))


def check(p, cpu, cpu64, gpu, nodes, what, families=None):
    o, c, dts = p.run(cpu, gpu, nodes)
    w, _, _ = p.run(cpu64, gpu, nodes)
    for i, (x, y, z, dt) in enumerate(zip(o, c, w, dts)):
        scale = np.abs(z).max() + 1e-30
        util.assert_close(z, util.to_f64(y, dt), 2e-2, 2e-3 * scale, f"{what} node {i} vs f64 run")
        ulp = {api.BF16: 2.0 ** -7, api.F16: 2.0 ** -10}.get(dt, 2.0 ** -7)
        util.assert_close(util.to_f64(x, dt), util.to_f64(y, dt), 2 * ulp, 2e-3 * scale, f"{what} node {i} vs native oracle")


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (256, 512, 384), (200, 328, 264), (8, 16, 8), (1000, 72, 1032), (130, 1000, 40)])
def test_bf16_gemm_all_layouts(oracle_lib, cuda_lib, cpu, cpu64, gpu, m, n, k):
    rng = np.random.default_rng(20)
    p = Pair(oracle_lib, cuda_lib)
    a, b = p.feed((m, k), api.BF16, bf16(rng, (m, k), 0.5)), p.feed((k, n), api.BF16, bf16(rng, (k, n), 0.5))
    at, bt = p.feed((k, m), api.BF16, bf16(rng, (k, m), 0.5)), p.feed((n, k), api.BF16, bf16(rng, (n, k), 0.5))
    nodes = [p.matmul(a, b), p.dot_general(a, bt, [1], [1]), p.dot_general(at, b, [0], [0]), p.dot_general(at, bt, [0], [1])]
    before = gpu.stats()["launches"]
    check(p, cpu, cpu64, gpu, nodes, f"bf16 {m}x{n}x{k}")
    assert gpu.stats()["launches"] > before


def test_tensor_core_kernel_is_the_one_that_runs(cuda_lib):
    g = api.Graph(cuda_lib)
    root, _ = configs.gemm_bias_gelu(g, 256, 512, 384)
    assert api.compile_check(cuda_lib, g, [root]) == ["gemm_tc"]          # contraction + bias + gelu in one kernel
    g = api.Graph(cuda_lib)
    root, _ = configs.fp8_weight_gemm(g, 256, 384, 512, amp=True)
    assert api.compile_check(cuda_lib, g, [root]) == ["pointwise", "gemm_tc_f8"]   # quantise X, then fp8 x fp8 contraction + scale + silu


def test_gemm_bias_gelu_config(oracle_lib, cuda_lib, cpu, cpu64, gpu):
    """Configuration 3 at a reduced size, inputs from the seeded generators."""
    rng = np.random.default_rng(21)
    m, n, k = 384, 512, 640
    p = Pair(oracle_lib, cuda_lib)
    a = p.feed((m, k), api.BF16, bf16(rng, (m, k), 1 / np.sqrt(k)))
    b = p.feed((k, n), api.BF16, bf16(rng, (k, n), 1.0))
    bias = p.feed((n,), api.BF16, api.f32_to_bf16(rng.uniform(-0.1, 0.1, n).astype(np.float32)))
    out = p.gelu(p.add(p.matmul(a, b), p.broadcast_to(bias, [m, n])))
    check(p, cpu, cpu64, gpu, [out], "gemm+bias+gelu")
    # epilogue variants: relu, silu on f32-cast result with a per-column scale, a residual that is a full matrix
    res = p.feed((m, n), api.BF16, bf16(rng, (m, n)))
    sc = p.feed((n,), api.F32, rng.uniform(0.5, 2, n).astype(np.float32))
    acc = p.matmul(a, b)
    nodes = [p.relu(p.add(acc, res)), p.cast(p.silu(p.mul(p.cast(acc, api.F32), p.broadcast_to(sc, [m, n]))), api.BF16)]
    check(p, cpu, cpu64, gpu, nodes, "epilogues")


def test_f16_and_batched(oracle_lib, cuda_lib, cpu, cpu64, gpu):
    rng = np.random.default_rng(22)
    p = Pair(oracle_lib, cuda_lib)
    a = p.feed((3, 136, 72), api.F16, (rng.standard_normal((3, 136, 72)) * 0.5).astype(np.float16))
    b = p.feed((3, 72, 264), api.F16, (rng.standard_normal((3, 72, 264)) * 0.5).astype(np.float16))
    q = p.feed((2, 4, 64, 32), api.BF16, bf16(rng, (2, 4, 64, 32), 0.5))
    nodes = [p.dot_general(a, b, [2], [1], [0], [0]), p.dot_general(a, a, [2], [2], [0], [0]),
             p.dot_general(q, q, [3], [3], [0, 1], [0, 1])]       # q @ q^T per (batch, head)
    check(p, cpu, cpu64, gpu, nodes, "batched")


def test_fp8_weight_gemm_config(oracle_lib, cuda_lib, cpu, cpu64, gpu):
    """Configuration 5 at a reduced size: plain (bf16 MMA on dequantised weights) and with the fp8
    mixed-precision pass (fp8 x fp8 MMA). Both are compared with the oracle on the same graph."""
    rng = np.random.default_rng(23)
    m, k, n = 256, 512, 384
    wf = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
    scales = (np.abs(wf).max(axis=0) / 448).astype(np.float32)
    import torch
    wq = torch.from_numpy(wf / scales).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    for amp in (False, True):
        p = Pair(oracle_lib, cuda_lib)
        x = p.feed((m, k), api.BF16, bf16(rng, (m, k)))
        w = p.feed((k, n), api.F8E4M3, wq)
        s = p.feed((n,), api.F32, scales)
        acc = p.matmul(x, p.cast(w, api.BF16))
        out = p.cast(p.silu(p.mul(p.cast(acc, api.F32), p.broadcast_to(s, [m, n]))), api.BF16)
        if amp:
            out = p.amp_to(out, api.F8E4M3)
        check(p, cpu, cpu64, gpu, [out], f"fp8 weights amp={amp}")


def test_gemm_linearity_at_benchmark_width(cuda_lib, gpu):
    """Size-independent property at K = N = 8192: A @ (B1 + B2) == A @ B1 + A @ B2 up to bf16 rounding,
    and identity weights reproduce the input exactly."""
    rng = np.random.default_rng(24)
    m, k = 256, 8192
    g = api.Graph(cuda_lib)
    a = g.input([m, k], api.BF16)
    eye = g.cast(g.eq(g.iota([k, k], 0, api.I32), g.iota([k, k], 1, api.I32)), api.BF16)
    out = g.matmul(a, eye)
    av = bf16(rng, (m, k))
    got = gpu.eval_with(g, out, api.Feeds(cuda_lib).set(a, av, api.BF16)).numpy()
    assert np.array_equal(got, av)
