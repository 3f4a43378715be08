"""Op::QuantMatmul on the device against the oracle: the streaming kernel for a few activation rows
(reads the packed weight directly) and the lowering onto the pointwise + contraction kernels for many rows."""
import numpy as np
import pytest

from kurumi_b200 import api
from tests import util

pytestmark = pytest.mark.gpu


def build(lib, m, n, k, bits, group, sym, act_dtype, seed):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((n, k)) * 0.5).astype(np.float32)
    act = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    packed, scales, mins = api.quantize(lib, w, bits, group, sym)
    g = api.Graph(lib)
    a = g.input([m, k], act_dtype)
    qw, sc = g.input(list(packed.shape), api.U8), g.input(list(scales.shape), api.F16)
    mn = None if sym else g.input(list(mins.shape), api.F16)
    out = g.quant_matmul(a, qw, sc, mn, bits, group)
    f = api.Feeds(lib)
    if act_dtype == api.F32:
        f.set(a, act)
    elif act_dtype == api.BF16:
        f.set(a, api.f32_to_bf16(act), api.BF16)
    else:
        f.set(a, act.astype(np.float16).view(np.uint16), api.F16)
    f.set(qw, packed).set(sc, scales.view(np.uint16), api.F16)
    if mn is not None:
        f.set(mn, mins.view(np.uint16), api.F16)
    return g, out, f


@pytest.mark.parametrize("bits,group", [(2, 32), (2, 128), (4, 32), (4, 128), (8, 64)])
@pytest.mark.parametrize("sym", [True, False])
@pytest.mark.parametrize("m", [1, 3, 8])
def test_few_rows_stream_the_packed_weight(oracle_lib, cuda_lib, cpu64, gpu, bits, group, sym, m):
    n, k = 96, 1024
    go, ro, fo = build(oracle_lib, m, n, k, bits, group, sym, api.F32, 5)
    gc, rc, fc = build(cuda_lib, m, n, k, bits, group, sym, api.F32, 5)
    assert api.compile_check(cuda_lib, gc, [rc]) == ["quant_gemv"]
    got = gpu.eval_with(gc, rc, fc).numpy()
    want = cpu64.eval_with(go, ro, fo).numpy()
    util.assert_close(want, got, 1e-5, 1e-5 * np.abs(want).max(), f"gemv bits={bits} sym={sym} m={m}")


@pytest.mark.parametrize("act_dtype", [api.BF16, api.F16])
def test_few_rows_low_precision_activation(oracle_lib, cuda_lib, cpu, cpu64, gpu, act_dtype):
    go, ro, fo = build(oracle_lib, 4, 256, 2048, 4, 128, False, act_dtype, 9)
    gc, rc, fc = build(cuda_lib, 4, 256, 2048, 4, 128, False, act_dtype, 9)
    got = util.to_f64(gpu.eval_with(gc, rc, fc).numpy(), act_dtype)
    native = util.to_f64(cpu.eval_with(go, ro, fo).numpy(), act_dtype)
    wide = cpu64.eval_with(go, ro, fo).numpy()
    step = 2.0 ** -7 if act_dtype == api.BF16 else 2.0 ** -10
    util.assert_close(wide, got, step, step * np.abs(wide).max(), "gemv low precision vs f64 run")
    assert (got != native).mean() < 0.05      # one rounding at the end on both sides: different summation order flips few results


@pytest.mark.parametrize("act_dtype,m,tol", [(api.F32, 40, 1e-5), (api.BF16, 192, 2.0 ** -6)])
def test_many_rows_lowering(oracle_lib, cuda_lib, cpu64, gpu, act_dtype, m, tol):
    go, ro, fo = build(oracle_lib, m, 320, 512, 4, 64, True, act_dtype, 3)
    gc, rc, fc = build(cuda_lib, m, 320, 512, 4, 64, True, act_dtype, 3)
    fams = api.compile_check(cuda_lib, gc, [rc])
    assert "quant_gemv" not in fams and any(f.startswith("gemm") for f in fams)
    got = util.to_f64(gpu.eval_with(gc, rc, fc).numpy(), act_dtype)
    want = cpu64.eval_with(go, ro, fo).numpy()
    util.assert_close(want, got, tol, tol * np.abs(want).max(), f"quant matmul m={m}")


@pytest.mark.parametrize("bits,group", [(4, 128), (4, 256), (2, 256)])
@pytest.mark.parametrize("sym", [True, False])
@pytest.mark.parametrize("act_dtype,m", [(api.BF16, 1), (api.F16, 3), (api.BF16, 8)])
def test_few_rows_16_bit_activations_on_the_tensor_cores(oracle_lib, cuda_lib, cpu, cpu64, gpu, bits, group, sym, act_dtype, m):
    """2- and 4-bit weights against 16-bit activations run their products on mma.sync with the raw field values as one
    operand (kernels/quant_gemv_mma.cuh): the sums are exact up to f32 accumulation, scale and minimum applied in f32, one
    rounding at the end - as close to the interpreter as the scalar kernel is. Ragged N, several K chunks."""
    n, k = 200, 4096 + 1024
    go, ro, fo = build(oracle_lib, m, n, k, bits, group, sym, act_dtype, 17)
    gc, rc, fc = build(cuda_lib, m, n, k, bits, group, sym, act_dtype, 17)
    assert api.compile_check(cuda_lib, gc, [rc]) == ["quant_gemv"]
    got = util.to_f64(gpu.eval_with(gc, rc, fc).numpy(), act_dtype)
    native = util.to_f64(cpu.eval_with(go, ro, fo).numpy(), act_dtype)
    wide = cpu64.eval_with(go, ro, fo).numpy()
    step = 2.0 ** -7 if act_dtype == api.BF16 else 2.0 ** -10
    util.assert_close(wide, got, step, step * np.abs(wide).max(), f"mma gemv bits={bits} group={group} sym={sym} m={m} vs f64 run")
    assert (got != native).mean() < 0.05, (got != native).mean()   # one rounding at the end on both sides


def test_more_rows_than_one_wave_of_ctas_covers(oracle_lib, cuda_lib, cpu64, gpu):
    """With more 16-row tiles than one wave of CTAs holds, the CTAs of the mma kernel loop over blocks of rows and stage the
    activations once; the ragged last block is cut at N."""
    m, n, k, bits, group = 2, 148 * 4 * 128 + 1000 + 7, 512, 4, 128
    go, ro, fo = build(oracle_lib, m, n, k, bits, group, False, api.F16, 23)
    gc, rc, fc = build(cuda_lib, m, n, k, bits, group, False, api.F16, 23)
    assert api.compile_check(cuda_lib, gc, [rc]) == ["quant_gemv"]
    got = util.to_f64(gpu.eval_with(gc, rc, fc).numpy(), api.F16)
    wide = cpu64.eval_with(go, ro, fo).numpy()
    util.assert_close(wide, got, 2.0 ** -10, 2.0 ** -10 * np.abs(wide).max(), "mma gemv over several blocks per CTA")
