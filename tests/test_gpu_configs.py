"""The five benchmark configurations end to end through the C ABI: at reduced sizes against the CPU
oracle on identical seeded inputs, and at the baseline's full sizes through row samples and
size-independent properties."""
import numpy as np
import pytest

from kurumi_b200 import api, configs
from tests import util

pytestmark = pytest.mark.gpu


def oracle_inputs(oracle_lib, cpu, gens):
    """Evaluate the seeded generator graphs on the oracle: {node: (array, dtype)}."""
    out = {}
    for node, mk in gens.items():
        h = api.Graph(oracle_lib)
        t = cpu.eval(h, mk(h))
        out[node] = (t.numpy(), t.dtype)
    return out


def run_config(make, kwargs, oracle_lib, cuda_lib, cpu, cpu64, gpu):
    go, gc = api.Graph(oracle_lib), api.Graph(cuda_lib)
    ro, gens = make(go, **kwargs)
    rc, gens_c = make(gc, **kwargs)
    assert ro == rc
    vals = oracle_inputs(oracle_lib, cpu, gens)
    fo, fc = api.Feeds(oracle_lib), api.Feeds(cuda_lib)
    for n, (v, dt) in vals.items():
        fo.set(n, v, dt); fc.set(n, v, dt)
    got = gpu.eval_with(gc, rc, fc)
    native = cpu.eval_with(go, ro, fo)
    wide = cpu64.eval_with(go, ro, fo).numpy()
    # the device's own generators reproduce the seeded inputs (threefry is integer work: the uniform draws are bit-equal)
    for n, mk in gens_c.items():
        h = api.Graph(cuda_lib)
        dv = gpu.eval(h, mk(h)).numpy()
        ref = util.to_f64(vals[n][0], vals[n][1])
        dev = util.to_f64(dv, vals[n][1])
        # the float steps after the draws (log, cos, the quantising divide) may differ in the last place, which
        # a narrow output type turns into at most one of ITS steps, and only at a rounding boundary
        step = {api.F32: 0.0, api.F8E4M3: 2.0 ** -3}.get(vals[n][1], 2.0 ** -7)
        assert (np.abs(dev - ref) <= 1e-5 * np.abs(ref) + 1e-6 + step * np.abs(ref)).all()
        if step:
            assert (dev != ref).mean() <= 2e-3
    return util.to_f64(got.numpy(), got.dtype), util.to_f64(native.numpy(), native.dtype), wide, got.dtype


def test_c1_fused_reduce(oracle_lib, cuda_lib, cpu, cpu64, gpu):
    got, native, wide, _ = run_config(configs.fused_reduce, dict(rows=96, cols=2048), oracle_lib, cuda_lib, cpu, cpu64, gpu)
    util.assert_close(wide, got, 1e-5, 0, "c1 vs f64 run")           # all terms are >= 0: a plain relative bound
    util.assert_close(native, got, 2048 * 2.0 ** -24, 0, "c1 vs f32 oracle")


def test_c2_transposed_softmax(oracle_lib, cuda_lib, cpu, cpu64, gpu):
    for n in (512, 2048):
        got, native, wide, _ = run_config(configs.transposed_softmax, dict(n=n), oracle_lib, cuda_lib, cpu, cpu64, gpu)
        util.assert_close(wide, got, 1e-5, 1e-12, f"c2 n={n} vs f64 run")
        util.assert_close(native, got, max(1e-5, n * 2.0 ** -24), 1e-9, f"c2 n={n} vs f32 oracle")


def test_c3_gemm_bias_gelu(oracle_lib, cuda_lib, cpu, cpu64, gpu):
    got, native, wide, _ = run_config(configs.gemm_bias_gelu, dict(m=256, n=384, kdim=512), oracle_lib, cuda_lib, cpu, cpu64, gpu)
    util.assert_close(wide, got, 2e-2, 2e-2 * np.abs(wide).max(), "c3 vs f64 run")
    util.assert_close(native, got, 2.0 ** -6, 2e-2 * np.abs(wide).max(), "c3 vs bf16 oracle")


def test_c4_causal_attention(oracle_lib, cuda_lib, cpu, cpu64, gpu):
    got, native, wide, _ = run_config(configs.causal_attention, dict(batch=1, heads=2, seq=256, dh=128, fused=True), oracle_lib, cuda_lib, cpu, cpu64, gpu)
    util.assert_close(wide, got, 2e-2, 2e-2 * np.abs(wide).max(), "c4 vs f64 run")
    util.assert_close(native, got, 2e-2, 2e-2 * np.abs(wide).max(), "c4 vs bf16 oracle")


@pytest.mark.parametrize("amp", [False, True])
def test_c5_fp8_weight_gemm(oracle_lib, cuda_lib, cpu, cpu64, gpu, amp):
    got, native, wide, _ = run_config(configs.fp8_weight_gemm, dict(m=128, kdim=512, n=384, amp=amp), oracle_lib, cuda_lib, cpu, cpu64, gpu)
    util.assert_close(wide, got, 2e-2, 2e-2 * np.abs(wide).max(), f"c5 amp={amp} vs f64 run")
    util.assert_close(native, got, 2.0 ** -6, 2e-2 * np.abs(wide).max(), f"c5 amp={amp} vs bf16 oracle")


# ---- full sizes -------------------------------------------------------------------------------------
def device_inputs(cuda_lib, gpu, gens):
    out = {}
    for node, mk in gens.items():
        h = api.Graph(cuda_lib)
        out[node] = gpu.eval_device(h, [mk(h)])[0]
    return out


def rows_of(cuda_lib, gpu, dev, lo, hi):
    """Rows [lo, hi) of a device tensor, brought to the host."""
    g = api.Graph(cuda_lib)
    x = g.input(list(dev.shape), dev.dtype)
    ranges = [(lo, hi)] + [(0, d) for d in dev.shape[1:]]
    return gpu.eval_device(g, [g.slice(x, ranges)], None, {x: dev})[0].numpy()


def test_c1_full_size_against_the_oracle(oracle_lib, cuda_lib, cpu, gpu):
    g = api.Graph(cuda_lib)
    root, gens = configs.fused_reduce(g)
    dev = device_inputs(cuda_lib, gpu, gens)
    got = gpu.eval_device(g, [root], None, dev)[0].numpy()
    go = api.Graph(oracle_lib)
    ro, gens_o = configs.fused_reduce(go)
    f = api.Feeds(oracle_lib)
    for (n, d) in dev.items():
        f.set(n, d.numpy())
    want = cpu.eval_with(go, ro, f).numpy()
    assert got.shape == (4096,)
    util.assert_close(want, got, 1e-5, 0, "c1 full size")   # the stated bound for f32 reductions


def test_c2_full_size_lines_against_the_oracle(oracle_lib, cuda_lib, cpu64, gpu):
    n = 8192
    g = api.Graph(cuda_lib)
    root, gens = configs.transposed_softmax(g, n)
    dev = device_inputs(cuda_lib, gpu, gens)
    out = gpu.eval_device(g, [root], None, dev)[0]
    (Ln, bn) = list(gens)
    L, bias = dev[Ln].numpy(), dev[bn].numpy()
    got = out.numpy()
    assert np.abs(got.sum(axis=1) - 1).max() < 1e-4 and (got >= 0).all()
    lines = [0, 1, 31, 32, 4095, 8191]                     # softmax lines are columns of L
    x = (L[:, lines].astype(np.float64) + bias[:, None].astype(np.float64)).T
    e = np.exp(x - x.max(axis=1, keepdims=True))
    util.assert_close(e / e.sum(axis=1, keepdims=True), got[lines], 1e-5, 1e-12, "c2 full-size lines vs f64")


def test_c3_full_size_row_sample(oracle_lib, cuda_lib, cpu, gpu):
    g = api.Graph(cuda_lib)
    root, gens = configs.gemm_bias_gelu(g)
    dev = device_inputs(cuda_lib, gpu, gens)
    out = gpu.eval_device(g, [root], None, dev)[0]
    (An, Bn, bn) = list(gens)
    rows = (4000, 4008)
    go = api.Graph(oracle_lib)
    ro, gens_o = configs.gemm_bias_gelu(go, m=rows[1] - rows[0])
    (Ao, Bo, bo) = list(gens_o)
    f = api.Feeds(oracle_lib).set(Ao, rows_of(cuda_lib, gpu, dev[An], *rows), api.BF16).set(Bo, dev[Bn].numpy(), api.BF16).set(bo, dev[bn].numpy(), api.BF16)
    want = util.to_f64(cpu.eval_with(go, ro, f).numpy(), api.BF16)
    got = util.to_f64(rows_of(cuda_lib, gpu, out, *rows), api.BF16)
    util.assert_close(want, got, 2e-2, 2e-2 * np.abs(want).max(), "c3 full-size rows")


def test_c4_full_size_properties(cuda_lib, gpu):
    g = api.Graph(cuda_lib)
    root, gens = configs.causal_attention(g)
    dev = device_inputs(cuda_lib, gpu, gens)
    (qn, kn, vn) = list(gens)
    out = gpu.eval_device(g, [root], None, dev)[0]
    o = util.to_f64(out.numpy(), api.BF16)
    v = util.to_f64(dev[vn].numpy(), api.BF16)
    assert np.isfinite(o).all()
    assert np.array_equal(o[:, :, 0, :], v[:, :, 0, :])          # query 0 sees key 0 only
    # each output row is a convex combination of value rows 0..i: bounded by their running extremes
    hi, lo = np.maximum.accumulate(v, axis=2), np.minimum.accumulate(v, axis=2)
    assert (o <= hi + 2e-2 * np.abs(hi) + 1e-2).all() and (o >= lo - 2e-2 * np.abs(lo) - 1e-2).all()
    # linearity in V: doubling V doubles the output exactly (a power of two commutes with every rounding)
    g2 = api.Graph(cuda_lib)
    q2, k2, v2 = (g2.input([8, 32, 4096, 128], api.BF16) for _ in range(3))
    root2 = g2.sdpa(q2, k2, g2.mul(v2, g2.scalar(v2, 2.0)), True)
    o2 = util.to_f64(gpu.eval_device(g2, [root2], None, {q2: dev[qn], k2: dev[kn], v2: dev[vn]})[0].numpy(), api.BF16)
    assert np.array_equal(o2, 2 * o)


def test_c5_full_size_row_sample(oracle_lib, cuda_lib, cpu, gpu):
    g = api.Graph(cuda_lib)
    root, gens = configs.fp8_weight_gemm(g, amp=True)
    dev = device_inputs(cuda_lib, gpu, gens)
    out = gpu.eval_device(g, [root], None, dev)[0]
    (Xn, Wn, sn) = list(gens)
    rows = (9000, 9004)
    go = api.Graph(oracle_lib)
    ro, gens_o = configs.fp8_weight_gemm(go, m=rows[1] - rows[0], amp=True)
    (Xo, Wo, so) = list(gens_o)
    f = api.Feeds(oracle_lib).set(Xo, rows_of(cuda_lib, gpu, dev[Xn], *rows), api.BF16).set(Wo, dev[Wn].numpy(), api.F8E4M3).set(so, dev[sn].numpy())
    want = util.to_f64(cpu.eval_with(go, ro, f).numpy(), api.BF16)
    got = util.to_f64(rows_of(cuda_lib, gpu, out, *rows), api.BF16)
    util.assert_close(want, got, 2e-2, 2e-2 * np.abs(want).max(), "c5 full-size rows")
    w = dev[Wn].numpy()
    assert ((w & 0x7F) != 0x7F).all()                            # no NaN codes in the quantised weights
    assert (util.to_f64(w, api.F8E4M3).__abs__().max(axis=0) == 448).all()   # every channel uses the full e4m3 range
