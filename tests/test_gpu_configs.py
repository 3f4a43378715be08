"""The five benchmark configurations end to end through the C ABI: at reduced sizes against the CPU
oracle on identical seeded inputs, and at the baseline's full sizes through row samples and
size-independent properties."""
import os

import numpy as np
import pytest

from kurumi_b200 import api, configs
from tests import util

pytestmark = pytest.mark.gpu

# Band for bf16 / fp8 contractions and attention against the f64 interpreter run: relative 2e-2, and near zero one bf16
# step (2^-8) of the row's largest magnitude (an output element is the rounded sum of products far larger than itself).
STEP_BF16 = 2.0 ** -8


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
    util.assert_band(wide, got, 2e-2, STEP_BF16, "c3 reduced size vs f64 run")
    util.assert_band(native, got, 2e-2, 2 * STEP_BF16, "c3 reduced size vs bf16 oracle")


def test_c4_causal_attention(oracle_lib, cuda_lib, cpu, cpu64, gpu):
    got, native, wide, _ = run_config(configs.causal_attention, dict(batch=1, heads=2, seq=256, dh=128, fused=True), oracle_lib, cuda_lib, cpu, cpu64, gpu)
    util.assert_band(wide, got, 2e-2, STEP_BF16, "c4 reduced size vs f64 run")
    util.assert_band(native, got, 6e-2, 4 * STEP_BF16, "c4 reduced size vs bf16 oracle")   # a cross-check: the bf16 interpreter rounds its scores and is itself further from the f64 run


@pytest.mark.parametrize("amp", [False, True])
def test_c5_fp8_weight_gemm(oracle_lib, cuda_lib, cpu, cpu64, gpu, amp):
    got, native, wide, _ = run_config(configs.fp8_weight_gemm, dict(m=128, kdim=512, n=384, amp=amp), oracle_lib, cuda_lib, cpu, cpu64, gpu)
    util.assert_band(wide, got, 2e-2, STEP_BF16, f"c5 reduced size amp={amp} vs f64 run")
    util.assert_band(native, got, 2e-2, 2 * STEP_BF16, f"c5 reduced size amp={amp} vs bf16 oracle")


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


def f64_run_in_threads(oracle_lib, jobs):
    """Evaluate independent oracle graphs under the f64 interpreter run on host threads (the C calls release the GIL;
    every job has its own graph, feeds and backend handle). jobs: callables taking a backend, returning an array."""
    from concurrent.futures import ThreadPoolExecutor
    with ThreadPoolExecutor(max_workers=min(len(jobs), max(1, (os.cpu_count() or 2) - 1))) as ex:
        return list(ex.map(lambda job: job(api.Backend(oracle_lib, 64)), jobs))


def spread_rows(m, rng, per_block=2, block=256):
    """Random rows hitting every 256-row block (one SM-pair tile) and both 128-row halves of it (one CTA each)."""
    rows = []
    for b0 in range(0, m, block):
        for half in range(per_block):
            lo = b0 + half * (block // per_block)
            rows.append(int(rng.integers(lo, min(lo + block // per_block, m))))
    return np.array(sorted(rows))


def test_c3_full_size_random_rows_against_the_f64_run(oracle_lib, cuda_lib, gpu):
    """All 8192 columns of 64 random rows of the full-size result (two rows in every 256-row tile, one per CTA of the
    SM pair) against the f64 interpreter run of the same graph on those rows of A."""
    g = api.Graph(cuda_lib)
    root, gens = configs.gemm_bias_gelu(g)
    dev = device_inputs(cuda_lib, gpu, gens)
    out = gpu.eval_device(g, [root], None, dev)[0]
    (An, Bn, bn) = list(gens)
    rows = spread_rows(8192, np.random.default_rng(3))
    assert len(rows) == 64
    A, B, bias, got_all = dev[An].numpy(), dev[Bn].numpy(), dev[bn].numpy(), out.numpy()

    def job(chunk):
        def run(cpu64):
            go = api.Graph(oracle_lib)
            ro, gens_o = configs.gemm_bias_gelu(go, m=len(chunk))
            (Ao, Bo, bo) = list(gens_o)
            f = api.Feeds(oracle_lib).set(Ao, np.ascontiguousarray(A[chunk]), api.BF16).set(Bo, B, api.BF16).set(bo, bias, api.BF16)
            return cpu64.eval_with(go, ro, f).numpy()
        return run
    want = np.concatenate(f64_run_in_threads(oracle_lib, [job(c) for c in np.array_split(rows, 8)]), 0)
    util.assert_band(want, util.to_f64(got_all[rows], api.BF16), 2e-2, STEP_BF16, "c3 full size, 64 random rows vs f64 run")


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


def test_c4_full_size_heads_against_the_f64_run(oracle_lib, cuda_lib, gpu):
    """Four random (batch, head) pairs of the full-size result, every query row over all 32 key blocks, against the f64
    interpreter run of the same attention on that head's Q, K, V."""
    g = api.Graph(cuda_lib)
    root, gens = configs.causal_attention(g)
    dev = device_inputs(cuda_lib, gpu, gens)
    (qn, kn, vn) = list(gens)
    out = gpu.eval_device(g, [root], None, dev)[0]
    rng = np.random.default_rng(4)
    heads = [(int(rng.integers(8)), int(rng.integers(32))) for _ in range(4)]
    heads[0] = (7, 31)                                   # the last head in memory

    def head_of(t, b, h):
        gs = api.Graph(cuda_lib)
        x = gs.input(list(t.shape), t.dtype)
        return gpu.eval_device(gs, [gs.slice(x, [(b, b + 1), (h, h + 1), (0, 4096), (0, 128)])], None, {x: t})[0].numpy()

    def job(b, h):
        q, k, v = (head_of(dev[n], b, h) for n in (qn, kn, vn))

        def run(cpu64):
            go = api.Graph(oracle_lib)
            qo, ko, vo = (go.input([1, 1, 4096, 128], api.BF16) for _ in range(3))
            ro = go.sdpa_fused(qo, ko, vo, True)
            f = api.Feeds(oracle_lib).set(qo, q, api.BF16).set(ko, k, api.BF16).set(vo, v, api.BF16)
            return cpu64.eval_with(go, ro, f).numpy()
        return run
    wants = f64_run_in_threads(oracle_lib, [job(b, h) for b, h in heads])
    for (b, h), want in zip(heads, wants):
        got = util.to_f64(head_of(out, b, h), api.BF16)
        util.assert_band(want, got, 2e-2, STEP_BF16, f"c4 full size, head ({b}, {h}) vs f64 run")


def test_c5_full_size_random_rows_against_the_f64_run(oracle_lib, cuda_lib, gpu):
    """All 28672 columns of 64 random rows of the full-size result (one row in every 256-row tile, alternating between
    the two CTAs of the SM pair) against the f64 interpreter run of the same graph on those rows of X."""
    g = api.Graph(cuda_lib)
    root, gens = configs.fp8_weight_gemm(g, amp=True)
    dev = device_inputs(cuda_lib, gpu, gens)
    out = gpu.eval_device(g, [root], None, dev)[0]
    (Xn, Wn, sn) = list(gens)
    rng = np.random.default_rng(5)
    rows = np.array([b0 + (i % 2) * 128 + int(rng.integers(128)) for i, b0 in enumerate(range(0, 16384, 256))])
    assert len(rows) == 64
    X, w, sc = dev[Xn].numpy(), dev[Wn].numpy(), dev[sn].numpy()
    got = np.stack([rows_of(cuda_lib, gpu, out, int(r) // 256 * 256, int(r) // 256 * 256 + 256)[int(r) % 256] for r in rows])

    def job(chunk):
        def run(cpu64):
            go = api.Graph(oracle_lib)
            ro, gens_o = configs.fp8_weight_gemm(go, m=len(chunk), amp=True)
            (Xo, Wo, so) = list(gens_o)
            f = api.Feeds(oracle_lib).set(Xo, np.ascontiguousarray(X[chunk]), api.BF16).set(Wo, w, api.F8E4M3).set(so, sc)
            return cpu64.eval_with(go, ro, f).numpy()
        return run
    want = np.concatenate(f64_run_in_threads(oracle_lib, [job(c) for c in np.array_split(rows, 4)]), 0)   # each job widens W to f64 once (1.9 GB)
    util.assert_band(want, util.to_f64(got, api.BF16), 2e-2, STEP_BF16, "c5 full size, 64 random rows vs f64 run")
    assert ((w & 0x7F) != 0x7F).all()                            # no NaN codes in the quantised weights
    assert (util.to_f64(w, api.F8E4M3).__abs__().max(axis=0) == 448).all()   # every channel uses the full e4m3 range


def test_quantised_decode_step_full_size_channels_against_the_f64_run(oracle_lib, cuda_lib, cpu64, gpu):
    """The decode-step workload of the bench (one bf16 activation row against [28672, 8192] 4-bit weights): 2048 output
    channels, eight in every 112-row stretch so that every CTA of the kernel's one wave is sampled, against the f64
    interpreter run on those rows of the packed weight, scales and minima."""
    g = api.Graph(cuda_lib)
    root, gens = configs.quant_gemv(g)
    assert api.compile_check(cuda_lib, g, [root]) == ["quant_gemv"]
    dev = device_inputs(cuda_lib, gpu, gens)
    out = gpu.eval_device(g, [root], None, dev)[0].numpy()
    (an, qn, sn, mn) = list(gens)
    rng = np.random.default_rng(8)
    rows = np.sort(np.concatenate([b0 + rng.choice(112, 8, replace=False) for b0 in range(0, 28672, 112)]))
    assert len(rows) == 2048
    act, qw, sc, mins = (dev[n].numpy() for n in (an, qn, sn, mn))
    assert len(np.unique(qw[rows])) == 256                                  # every byte value: every field value in both positions
    go = api.Graph(oracle_lib)
    ro, gens_o = configs.quant_gemv(go, n=len(rows))
    (ao, qo, so, mo) = list(gens_o)
    f = api.Feeds(oracle_lib).set(ao, act, api.BF16).set(qo, np.ascontiguousarray(qw[rows]), api.U8)
    f.set(so, np.ascontiguousarray(sc[rows]), api.F16).set(mo, np.ascontiguousarray(mins[rows]), api.F16)
    want = cpu64.eval_with(go, ro, f).numpy()
    util.assert_band(want, util.to_f64(out[:, rows], api.BF16), 2.0 ** -7, STEP_BF16, "quantised decode step, 2048 channels vs f64 run")
