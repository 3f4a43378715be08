"""Parity of the CUDA backend with the CPU oracle, op by op, through the C ABI (ku_eval_many).
Bool / integer / movement / indexing results must be bit-exact; f32 pointwise within 2 ulp per
primitive; f32 reductions within rel 1e-5; low-precision pointwise bit-exact except where a
transcendental differs by its ulp budget."""
import numpy as np
import pytest

from kurumi_b200 import api
from tests import util
from tests.util import Pair

pytestmark = pytest.mark.gpu

INT_TYPES = [(api.U8, np.uint8), (api.U16, np.uint16), (api.U32, np.uint32), (api.U64, np.uint64), (api.I8, np.int8),
             (api.I16, np.int16), (api.I32, np.int32), (api.I64, np.int64)]


def rng_f32(rng, shape, scale=1.0):
    return (rng.standard_normal(shape) * scale).astype(np.float32)


def test_f32_pointwise_primitives_within_2ulp(oracle_lib, cuda_lib, cpu, gpu):
    rng = np.random.default_rng(0)
    p = Pair(oracle_lib, cuda_lib)
    shape = (37, 129)   # ragged: not a multiple of any vector width
    a = p.feed(shape, api.F32, rng_f32(rng, shape, 3.0))
    b = p.feed(shape, api.F32, rng_f32(rng, shape, 3.0))
    pos = p.feed(shape, api.F32, np.abs(rng_f32(rng, shape, 50.0)) + np.float32(1e-3))
    special = np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 1e-40, -1e-40, 3.4e38, 1.0, -1.0], np.float32)
    sp = p.feed((10,), api.F32, special)
    sp2 = p.feed((10,), api.F32, special[::-1].copy())
    nodes = {"add": p.add(a, b), "mul": p.mul(a, b), "max": p.max(a, b), "neg": p.neg(a), "recip": p.recip(a), "sqrt": p.sqrt(pos),
             "exp2": p.exp2(a), "log2": p.log2(pos), "sin": p.sin(a), "floor": p.floor(a),
             "sp_add": p.add(sp, sp2), "sp_mul": p.mul(sp, sp2), "sp_max": p.max(sp, sp2), "sp_recip": p.recip(sp), "sp_sqrt": p.sqrt(sp),
             "sp_floor": p.floor(sp), "sp_relu": p.relu(sp)}
    o, c, _ = p.run(cpu, gpu, list(nodes.values()))
    for name, x, y in zip(nodes, o, c):
        assert np.array_equal(np.isnan(x), np.isnan(y)), name
        if name in ("add", "mul", "max", "neg", "recip", "sqrt", "floor") or name.startswith("sp_"):
            util.assert_ulp(x, y, 0, name)     # IEEE-exact operations
        else:
            util.assert_ulp(x, y, 2, name)     # exp2 / log2 / sin: library ulp budget


def test_no_fma_contraction(oracle_lib, cuda_lib, cpu, gpu):
    """x*y + 0.5*x must round after each primitive (the reference never fuses a*b+c)."""
    rng = np.random.default_rng(1)
    p = Pair(oracle_lib, cuda_lib)
    x = rng.uniform(-1, 1, (64, 256)).astype(np.float32)
    y = (np.float32(-0.5) + rng.uniform(-1e-4, 1e-4, (64, 256)).astype(np.float32))   # near-cancelling products
    xn, yn = p.feed(x.shape, api.F32, x), p.feed(x.shape, api.F32, y)
    out = p.add(p.mul(xn, yn), p.mul(p.scalar(xn, 0.5), xn))
    o, c, _ = p.run(cpu, gpu, [out])
    util.assert_exact(o[0], c[0], "x*y + 0.5*x")


def test_activations_f32_and_f64(oracle_lib, cuda_lib, cpu, gpu):
    rng = np.random.default_rng(2)
    p = Pair(oracle_lib, cuda_lib)
    x = p.feed((33, 65), api.F32, rng_f32(rng, (33, 65), 2.0))
    xd = p.feed((9, 17), api.F64, rng.standard_normal((9, 17)))
    nodes = [p.relu(x), p.sigmoid(x), p.silu(x), p.gelu(x), p.tanh(x), p.exp(x), p.cos(x), p.gelu(xd), p.ln(p.abs(xd))]
    o, c, _ = p.run(cpu, gpu, nodes)
    for i, (a, b) in enumerate(zip(o, c)):
        if a.dtype == np.float32:
            util.assert_close(a, b, 2e-6, 2e-7, f"act {i}")   # chains of <= 2-ulp primitives
        else:
            util.assert_close(a, b, 1e-14, 1e-15, f"act64 {i}")


@pytest.mark.parametrize("tag,np_t", INT_TYPES)
def test_integer_ops_bit_exact(oracle_lib, cuda_lib, cpu, gpu, tag, np_t):
    rng = np.random.default_rng(3)
    info = np.iinfo(np_t)
    p = Pair(oracle_lib, cuda_lib)
    n = 1031
    a = rng.integers(info.min, info.max, n, dtype=np_t, endpoint=True)
    b = rng.integers(info.min, info.max, n, dtype=np_t, endpoint=True)
    b[:50] = 0
    a[50:60] = info.min
    b[50:60] = np_t(-1) if info.min < 0 else np_t(1)
    sh = rng.integers(0, 80, n).astype(np_t)
    an, bn, sn = p.feed((n,), tag, a), p.feed((n,), tag, b), p.feed((n,), tag, sh)
    nodes = [p.add(an, bn), p.mul(an, bn), p.max(an, bn), p.idiv(an, bn), p.and_(an, bn), p.or_(an, bn), p.xor(an, bn), p.shl(an, sn),
             p.shr(an, sn), p.lt(an, bn), p.eq(an, bn), p.where(p.lt(an, bn), an, bn), p.min(an, bn)]
    if info.min < 0:
        nodes += [p.neg(an), p.abs(an)]
    nodes += [p.sum(p.reshape(an, [n, 1]), 0), p.sum(an, 0), p.prod(p.reshape(p.slice(an, [(0, 1024)]), [32, 32]), 1), p.reduce_max(an, 0)]
    nodes += [p.cast(an, t) for t in (api.F32, api.F64, api.I32, api.U8, api.I64, api.BOOL, api.BF16, api.F16)]
    o, c, _ = p.run(cpu, gpu, nodes)
    for i, (x, y) in enumerate(zip(o, c)):
        util.assert_exact(x, y, f"{api.DTYPES[tag]} node {i}")


def test_bool_ops_and_casts_bit_exact(oracle_lib, cuda_lib, cpu, gpu):
    rng = np.random.default_rng(4)
    p = Pair(oracle_lib, cuda_lib)
    a = p.feed((257,), api.BOOL, rng.integers(0, 2, 257).astype(np.uint8))
    b = p.feed((257,), api.BOOL, rng.integers(0, 2, 257).astype(np.uint8))
    f = np.concatenate([rng_f32(rng, 240, 1e5), np.array([np.nan, np.inf, -np.inf, 0, -0.0, 1e20, -1e20, 255.5, 256, -1, 127.9, -128.9, 2 ** 31, -2 ** 31, 2 ** 63, 1.8e19, 65535.5], np.float32)])
    fn = p.feed((257,), api.F32, f)
    fd = p.feed((257,), api.F64, f.astype(np.float64) * 1.0000001)
    nodes = [p.and_(a, b), p.or_(a, b), p.xor(a, b), p.logical_not(a), p.lt(a, b), p.eq(a, b), p.cast(a, api.F32), p.cast(a, api.I8)]
    for t in (api.BOOL, api.U8, api.U16, api.U32, api.U64, api.I8, api.I16, api.I32, api.I64):
        nodes += [p.cast(fn, t), p.cast(fd, t)]
    nodes += [p.cast(fd, api.F32), p.cast(fd, api.BF16), p.cast(fd, api.F16), p.cast(fn, api.BF16), p.cast(fn, api.F16), p.cast(fn, api.F8E4M3), p.cast(fn, api.F8E5M2),
              p.cast(fd, api.F8E4M3), p.ge(fn, p.scalar(fn, 0.0)), p.ne(fn, fn), p.le(fn, p.neg(fn))]
    o, c, dts = p.run(cpu, gpu, nodes)
    for i, (x, y, dt) in enumerate(zip(o, c, dts)):
        if dt in (api.F32, api.F64, api.F16):
            assert np.array_equal(x, y, equal_nan=True), i
        elif dt in (api.BF16, api.F8E4M3, api.F8E5M2):   # NaN payloads may differ; compare values
            assert np.array_equal(util.to_f64(x, dt), util.to_f64(y, dt), equal_nan=True), (i, api.DTYPES[dt])
        else:
            util.assert_exact(x, y, f"node {i} {api.DTYPES[dt]}")


def test_bitcast_iota_random_bit_exact(oracle_lib, cuda_lib, cpu, gpu):
    rng = np.random.default_rng(5)
    p = Pair(oracle_lib, cuda_lib)
    f = p.feed((64,), api.F32, rng_f32(rng, 64))
    h = p.feed((64,), api.BF16, rng.integers(0, 2 ** 16, 64).astype(np.uint16))
    d = p.feed((16,), api.F64, rng.standard_normal(16))
    seed = p.feed((1,), api.I64, np.array([-12345], np.int64))
    nodes = [p.bitcast(f, api.U32), p.bitcast(p.bitcast(f, api.I32), api.F32), p.bitcast(h, api.U16), p.bitcast(h, api.F16), p.bitcast(d, api.I64),
             p.iota([5, 7, 3], 1, api.I32), p.iota([300], 0, api.U8), p.iota([4, 6], 1, api.F32), p.iota([2, 3], 0, api.BF16),
             p.transpose(p.iota([5, 7], 0, api.I64), 0, 1),
             p.rand_uniform([1000], 42), p.rand_uniform([3, 5, 7], 2 ** 64 - 1), p.rand_uniform_keyed([64], seed),
             p.slice(p.rand_uniform([100], 7), [(10, 60)]), p.permute(p.rand_uniform([6, 8], 9), [1, 0])]
    o, c, dts = p.run(cpu, gpu, nodes)
    for i, (x, y) in enumerate(zip(o, c)):
        assert np.array_equal(x.view(np.uint8), y.view(np.uint8)), f"node {i}"
    # the decompositions on top of the uniform draw: same primitives, library ulp budget
    q = Pair(oracle_lib, cuda_lib)
    o, c, _ = q.run(cpu, gpu, [q.randn([4096], 11), q.rand_range([4096], 12, -0.1, 0.1)])
    util.assert_close(o[0], c[0], 1e-5, 1e-6, "randn")
    util.assert_exact(o[1], c[1], "rand_range")


def test_movement_bit_exact(oracle_lib, cuda_lib, cpu, gpu):
    rng = np.random.default_rng(6)
    p = Pair(oracle_lib, cuda_lib)
    x = p.feed((4, 6, 10), api.F32, rng_f32(rng, (4, 6, 10)))
    xi = p.feed((12, 10), api.I16, rng.integers(-1000, 1000, (12, 10)).astype(np.int16))
    xb = p.feed((3, 8), api.BF16, rng.integers(0, 2 ** 15, (3, 8)).astype(np.uint16))
    nodes = [p.permute(x, [2, 0, 1]), p.reshape(p.permute(x, [1, 0, 2]), [6, 40]), p.reshape(x, [24, 10]), p.reshape(p.permute(x, [2, 1, 0]), [240]),
             p.expand(p.reshape(p.slice(x, [(0, 4), (0, 1), (0, 10)]), [4, 1, 10]), [4, 5, 10]),
             p.slice_step(x, [(1, 4, 2), (0, 6, 3), (2, 9, 2)]), p.flip(x, [0, 2]), p.pad(x, [(1, 0), (0, 2), (3, 1)]),
             p.pad(p.permute(x, [1, 0, 2]), [(0, 1), (2, 0), (0, 0)]), p.slice(p.pad(xi, [(2, 2), (1, 1)]), [(1, 15), (0, 11)]),
             p.flip(p.pad(xi, [(0, 3), (0, 0)]), [0]), p.transpose(xi, 0, 1), p.broadcast_to(p.slice(xi, [(0, 1), (0, 10)]), [7, 1, 10]),
             p.permute(xb, [1, 0]), p.pad(xb, [(1, 1), (0, 3)]), p.reshape(p.flip(xb, [1]), [4, 6]),
             p.add(p.pad(p.relu(p.slice(x, [(0, 4), (0, 6), (0, 5)])), [(0, 0), (0, 0), (0, 5)]), x),   # pad of an expression
             p.reshape(p.expand(p.reshape(p.sum(x, 2), [4, 6, 1]), [4, 6, 10]), [24, 10])]
    o, c, _ = p.run(cpu, gpu, nodes)
    for i, (a, b) in enumerate(zip(o, c)):
        util.assert_exact(a, b, f"movement {i}")


def test_transposed_operands_go_through_shared_memory_tiles(oracle_lib, cuda_lib, cpu, gpu):
    """A leaf that is contiguous along another dim than the output's innermost one (a transpose, a permuted batch) is
    read along its own rows into shared-memory tiles and read back transposed; every other operand is read in place.
    Bit for bit the interpreter's values: ragged tile edges in both dims, leading batch dims, 1-, 2-, 4- and 8-byte
    types (a copy of 16-bit floats keeps NaN payloads), a second transposed leaf, a row-major one, a broadcast one, a
    padded (guarded) one, and a transposed slice that starts inside its buffer."""
    rng = np.random.default_rng(16)
    p = Pair(oracle_lib, cuda_lib)
    x = p.feed((300, 500), api.F32, rng_f32(rng, (300, 500)))
    y = p.feed((500, 300), api.F32, rng_f32(rng, (500, 300)))
    bias = p.feed((300,), api.F32, rng_f32(rng, (300,)))
    xb = p.feed((4, 70, 90), api.BF16, rng.integers(0, 2 ** 16, (4, 70, 90)).astype(np.uint16))       # every bit pattern, NaNs included
    xi = p.feed((64, 3, 128), api.I64, rng.integers(-2 ** 62, 2 ** 62, (64, 3, 128)).astype(np.int64))
    x8 = p.feed((100, 200), api.U8, rng.integers(0, 256, (100, 200)).astype(np.uint8))
    xt = p.permute(x, [1, 0])
    nodes = [p.add(xt, y),                                                     # transposed + row-major
             p.mul(p.add(xt, p.broadcast_to(bias, [500, 300])), xt),          # the same transposed leaf twice + a broadcast
             p.permute(xb, [0, 2, 1]),                                         # pure copy, 2-byte, batch dim
             p.mul(p.permute(xi, [2, 1, 0]), p.permute(xi, [2, 1, 0])),       # 8-byte, three dims reversed
             p.permute(x8, [1, 0]),                                            # 1-byte
             p.add(p.permute(p.slice(x, [(7, 300), (33, 500)]), [1, 0]), p.slice(y, [(33, 500), (7, 300)])),   # offsets inside the buffers
             p.add(p.pad(p.slice(xt, [(0, 499), (0, 300)]), [(1, 0), (0, 0)]), y),                            # a guarded transposed leaf stays on direct reads
             p.add(xt, p.pad(p.slice(y, [(0, 500), (0, 299)]), [(0, 0), (0, 1)])),                            # a guarded row-major leaf beside a staged one
             p.cast(xt, api.BF16)]
    assert api.compile_check(cuda_lib, p.gc, [nodes[0]]) == ["pointwise_tiled"]
    assert api.compile_check(cuda_lib, p.gc, [nodes[2]]) == ["pointwise_tiled"]
    o, c, _ = p.run(cpu, gpu, nodes)
    for i, (a, b) in enumerate(zip(o, c)):
        util.assert_exact(a, b, f"transposed operand {i}")


def test_empty_and_rank0(oracle_lib, cuda_lib, cpu, gpu):
    p = Pair(oracle_lib, cuda_lib)
    e = p.feed((0, 5), api.F32, np.zeros((0, 5), np.float32))
    s = p.feed((), api.F32, np.array(3.0, np.float32))
    one = p.feed((1, 1), api.I32, np.array([[7]], np.int32))
    nodes = [p.add(e, e), p.sum(e, 0), p.sum(e, 1), p.reduce_max(e, 0), p.add(s, s), p.sqrt(s), p.sum(p.reshape(s, [1]), 0), p.sum(one, 0),
             p.expand(one, [3, 4]), p.matmul(p.reshape(e, [5, 0]), e)]
    o, c, _ = p.run(cpu, gpu, nodes)
    for i, (a, b) in enumerate(zip(o, c)):
        util.assert_exact(a, b, f"edge {i}")


# (12000 rows: more than eight residencies of CTAs, so the row kernel's CTAs loop over rows instead of taking one each)
@pytest.mark.parametrize("shape,axis", [((64, 4096), 1), ((7, 1000), 1), ((300, 33), 0), ((5, 64, 9), 1), ((3, 129), 1), ((1, 100000), 1), ((2049,), 0), ((12000, 256), 1)])
def test_f32_reductions(oracle_lib, cuda_lib, cpu, cpu64, gpu, shape, axis):
    rng = np.random.default_rng(7)
    p = Pair(oracle_lib, cuda_lib)
    x = p.feed(shape, api.F32, rng.uniform(-1, 1, shape).astype(np.float32))
    y = p.feed(shape, api.F32, rng.uniform(-1, 1, shape).astype(np.float32))
    fused = p.relu(p.add(p.mul(x, y), p.mul(p.scalar(x, 0.5), x)))
    nodes = [p.sum(fused, axis), p.sum(x, axis), p.reduce_max(x, axis), p.reduce_min(y, axis), p.mean(x, axis),
             p.prod(p.add(p.mul(x, p.scalar(x, 0.01)), p.scalar(x, 1.0)), axis)]
    o, c, _ = p.run(cpu, gpu, nodes)
    o64, _, _ = p.run(cpu64, gpu, nodes)
    n = shape[axis]
    eps = 2.0 ** -24
    for i, (a, b, w) in enumerate(zip(o, c, o64)):
        if i in (2, 3):
            util.assert_exact(a, b, f"max/min {i}")       # order-independent
            continue
        # against the f64 interpreter run: rel 1e-5, with an absolute floor for sums that cancel
        # (1e-6 of the line's L1 mass, which for |x| <= 1 is at most n)
        floor = 1e-6 * n if i in (0, 1, 4) else 0.0
        # (a product of n factors accumulates ~sqrt(n) roundings in any order)
        rel = 1e-5 if i != 5 else max(1e-5, 4 * np.sqrt(n) * eps)
        util.assert_close(w, b, rel, floor, f"reduce {i} vs f64 run")
        # against the f32 oracle: its strict left fold carries its own rounding, bounded by n * eps
        # of the L1 mass; the device's tree order must not be further from the f64 run than that
        util.assert_close(a, b, n * eps, n * eps * n if i in (0, 1, 4) else 0.0, f"reduce {i} vs f32 oracle")


def test_low_precision_pointwise_and_reduce(oracle_lib, cuda_lib, cpu, gpu):
    rng = np.random.default_rng(8)
    p = Pair(oracle_lib, cuda_lib)
    shape = (48, 256)
    xb = p.feed(shape, api.BF16, api.f32_to_bf16(rng_f32(rng, shape)))
    yb = p.feed(shape, api.BF16, api.f32_to_bf16(rng_f32(rng, shape)))
    xh = p.feed(shape, api.F16, rng_f32(rng, shape).astype(np.float16))
    x8 = p.feed(shape, api.F8E4M3, rng.integers(0, 256, shape).astype(np.uint8))
    exact = [p.add(xb, yb), p.mul(xb, yb), p.max(xb, yb), p.neg(xb), p.recip(xb), p.sqrt(p.abs(xb)), p.relu(xb), p.add(xh, xh), p.mul(xh, xh),
             p.cast(xb, api.F32), p.cast(x8, api.BF16), p.cast(x8, api.F32), p.cast(p.cast(x8, api.F32), api.F8E4M3), p.add(p.mul(xb, yb), p.mul(p.scalar(xb, 0.5), xb)),
             p.lt(xb, yb), p.where(p.lt(xb, yb), xb, yb), p.sum(xb, 1), p.reduce_max(xb, 1), p.sum(xh, 0), p.reduce_max(x8, 1)]
    o, c, dts = p.run(cpu, gpu, exact)
    for i, (a, b, dt) in enumerate(zip(o, c, dts)):
        va, vb = util.to_f64(a, dt), util.to_f64(b, dt)
        if i in (16, 18):   # f32-accumulated sums rounded once: within one unit of the narrow format
            util.assert_close(va, vb, 2.0 ** -7 if dt == api.BF16 else 2.0 ** -10, 1e-3, f"low sum {i}")
        else:
            assert np.array_equal(va, vb, equal_nan=True), f"low-precision node {i} ({api.DTYPES[dt]})"
    chains = [p.gelu(xb), p.silu(xb), p.sigmoid(xh), p.exp(xb), p.tanh(xb)]
    o, c, dts = p.run(cpu, gpu, chains)
    for i, (a, b, dt) in enumerate(zip(o, c, dts)):
        va, vb = util.to_f64(a, dt), util.to_f64(b, dt)
        # a transcendental that differs in its last f32 bits can flip one narrow-format rounding
        assert (np.abs(va - vb) <= np.abs(va) * 2.0 ** -6 + 1e-6).all(), i
        assert (va != vb).mean() < 0.02, f"chain {i}: {(va != vb).mean():.4f} of elements differ"


@pytest.mark.parametrize("shape,axis", [((16, 8192), 1), ((33, 1000), 1), ((8, 77), 1), ((40, 50), 0), ((3, 20, 7), 1), ((2, 20000), 1), ((12000, 256), 1)])
def test_softmax_and_rmsnorm(oracle_lib, cuda_lib, cpu, cpu64, gpu, shape, axis):
    rng = np.random.default_rng(9)
    p = Pair(oracle_lib, cuda_lib)
    x = p.feed(shape, api.F32, rng_f32(rng, shape, 2.0))
    xb = p.feed(shape, api.BF16, api.f32_to_bf16(rng_f32(rng, shape, 2.0)))
    nodes = [p.softmax(x, axis), p.softmax(p.add(x, x), axis), p.rmsnorm(x, axis, 1e-5), p.softmax(xb, axis), p.rmsnorm(xb, axis, 1e-6)]
    o, c, dts = p.run(cpu, gpu, nodes)
    w, _, _ = p.run(cpu64, gpu, nodes)
    n = shape[axis]
    for i, (a, b, dt) in enumerate(zip(o, c, dts)):
        if dt == api.F32:
            # rel 1e-5 against the f64 interpreter run; the f32 oracle's serial line sum carries up to
            # n * 2^-24 of relative rounding of its own, which every element of that line inherits
            util.assert_close(w[i], b, 1e-5, 1e-12, f"line op {i} vs f64 run")
            util.assert_close(a, b, max(1e-5, n * 2.0 ** -24), 1e-9, f"line op {i} vs f32 oracle")
        else:
            util.assert_close(util.to_f64(a, dt), util.to_f64(b, dt), 2.0 ** -7, 1e-9, f"bf16 line op {i}")
    s = c[0].sum(axis=axis)
    assert np.abs(s - 1).max() < 1e-4


def test_softmax_through_transpose_and_bias(oracle_lib, cuda_lib, cpu, cpu64, gpu):
    rng = np.random.default_rng(10)
    for n, m in ((256, 384), (130, 70), (1024, 1024)):
        p = Pair(oracle_lib, cuda_lib)
        L = p.feed((n, m), api.F32, rng_f32(rng, (n, m), 2.0))
        bias = p.feed((n,), api.F32, rng.uniform(-1, 1, n).astype(np.float32))
        out = p.softmax(p.add(p.permute(L, [1, 0]), p.broadcast_to(bias, [m, n])), 1)
        o, c, _ = p.run(cpu, gpu, [out])
        w, _, _ = p.run(cpu64, gpu, [out])
        util.assert_close(w[0], c[0], 1e-5, 1e-12, f"transposed softmax {n}x{m} vs f64 run")
        util.assert_close(o[0], c[0], max(1e-5, n * 2.0 ** -24), 1e-9, f"transposed softmax {n}x{m} vs f32 oracle")
        assert c[0].shape == (m, n)


@pytest.mark.parametrize("family,env", [("softmax_groups_tma", {}), ("softmax_panels_tma", {"KURUMI_SMT_NO_GROUPS": "1"})])
def test_large_transposed_softmax_ragged_and_special_lines(oracle_lib, cuda_lib, cpu64, gpu, monkeypatch, family, env):
    """Each of the two large-problem kernels on a shape that divides into nothing (2100 positions, 2052 lines),
    with lines that are all -inf, hold a NaN, hold +inf, or a single finite entry."""
    for k, v in env.items():
        monkeypatch.setenv(k, v)
    rng = np.random.default_rng(21)
    n, m = 2100, 2052                       # positions (rows of L), lines (columns of L)
    Lv = rng_f32(rng, (n, m), 2.0)
    Lv[:, 5] = -np.inf                      # nothing finite: the line is NaN
    Lv[:, 6] = -np.inf; Lv[1234, 6] = 0.5   # one finite entry: a one-hot line
    Lv[17, 7] = np.nan                      # NaN poisons its line
    Lv[99, 2051] = np.inf                   # +inf: inf - inf in the exponent
    Lv[:, 2050] = 60.0; Lv[3, 2050] = 88.0  # large but finite
    bv = rng.uniform(-1, 1, n).astype(np.float32)
    p = Pair(oracle_lib, cuda_lib)
    L = p.feed((n, m), api.F32, Lv)
    bias = p.feed((n,), api.F32, bv)
    out = p.softmax(p.add(p.permute(L, [1, 0]), p.broadcast_to(bias, [m, n])), 1)
    assert api.compile_check(cuda_lib, p.gc, [out]) == [family]
    w, c, _ = p.run(cpu64, gpu, [out])
    want, got = w[0], c[0]
    assert got.shape == (m, n)
    nan_lines = [5, 7, 2051]
    for i in nan_lines:
        assert np.isnan(want[i]).all() and np.isnan(got[i]).all(), i
    keep = np.setdiff1d(np.arange(m), nan_lines)
    util.assert_close(want[keep], got[keep], 1e-5, 1e-12, f"{family} ragged")
    assert abs(got[6, 1234] - 1.0) < 1e-6 and np.count_nonzero(got[6]) == 1


@pytest.mark.parametrize("n,m", [(8192, 128), (4096, 288)])
def test_transposed_softmax_with_a_short_last_panel(oracle_lib, cuda_lib, cpu64, gpu, n, m):
    """The panel kernel cuts the lines into panels of 256: a line count that is a multiple of 32 but not of 256 leaves the
    last panel with fewer than its eight strips (a row shard of the softmax configuration on eight GPUs, streamed in
    eight chunks, is 128 lines). Strips past the last line write nothing: the result is right and the inputs, which lie
    next to the result in device memory, are untouched."""
    rng = np.random.default_rng(22)
    Lv, bv = rng_f32(rng, (n, m), 2.0), rng.uniform(-1, 1, n).astype(np.float32)
    g = api.Graph(cuda_lib)
    L, bias = g.input([n, m], api.F32), g.input([n], api.F32)
    out = g.softmax(g.add(g.permute(L, [1, 0]), g.broadcast_to(bias, [m, n])), 1)
    assert api.compile_check(cuda_lib, g, [out]) == ["softmax_panels_tma"]
    dL, db = gpu.upload(Lv), gpu.upload(bv)
    tail = gpu.upload(np.full((m, n), 7.0, np.float32))            # allocations around the result's
    got = gpu.eval_device(g, [out], None, {L: dL, bias: db})[0]
    tail2 = gpu.upload(np.full((m, n), 9.0, np.float32))
    for _ in range(2):
        got.free()
        got = gpu.eval_device(g, [out], None, {L: dL, bias: db})[0]
    x = Lv.T.astype(np.float64) + bv.astype(np.float64)[None, :]
    e = np.exp(x - x.max(axis=1, keepdims=True))
    util.assert_close(e / e.sum(axis=1, keepdims=True), got.numpy(), 1e-5, 1e-12, f"panels, {m} lines of {n}")
    assert np.array_equal(dL.numpy(), Lv) and np.array_equal(db.numpy(), bv)
    assert (tail.numpy() == 7.0).all() and (tail2.numpy() == 9.0).all()


def test_softmax_special_values(oracle_lib, cuda_lib, cpu, gpu):
    p = Pair(oracle_lib, cuda_lib)
    v = np.zeros((4, 256), np.float32)
    v[0, :] = -np.inf; v[0, 3] = 0.0          # a single finite entry
    v[1, :] = 80.0; v[1, 7] = 88.0            # large but finite
    v[2, 5] = np.nan                          # NaN poisons the line (max drops it, exp does not)
    v[3, :] = np.linspace(-100, 0, 256)
    x = p.feed(v.shape, api.F32, v)
    o, c, _ = p.run(cpu, gpu, [p.softmax(x, 1)])
    util.assert_close(o[0], c[0], 1e-5, 1e-30, "softmax specials")


@pytest.mark.parametrize("tag", [api.F32, api.F64, api.I32, api.I8, api.U16, api.BF16, api.F16])
def test_dot_general_layouts(oracle_lib, cuda_lib, cpu, cpu64, gpu, tag):
    rng = np.random.default_rng(11)

    def vals(shape):
        if tag in (api.I32, api.I8, api.U16):
            np_t = {api.I32: np.int32, api.I8: np.int8, api.U16: np.uint16}[tag]
            return rng.integers(0 if tag == api.U16 else -9, 9, shape).astype(np_t)
        f = rng_f32(rng, shape, 0.5)
        return {api.F32: f, api.F64: f.astype(np.float64), api.BF16: api.f32_to_bf16(f), api.F16: f.astype(np.float16)}[tag]
    p = Pair(oracle_lib, cuda_lib)
    a, b = p.feed((37, 50), tag, vals((37, 50))), p.feed((50, 29), tag, vals((50, 29)))
    bt = p.feed((29, 50), tag, vals((29, 50)))
    a3, b3 = p.feed((3, 20, 16), tag, vals((3, 20, 16))), p.feed((3, 16, 24), tag, vals((3, 16, 24)))
    a4, b4 = p.feed((2, 5, 3, 4), tag, vals((2, 5, 3, 4))), p.feed((4, 2, 3, 6), tag, vals((4, 2, 3, 6)))
    nodes = [p.matmul(a, b), p.dot_general(a, bt, [1], [1]), p.dot_general(p.permute(a, [1, 0]), b, [0], [0]),
             p.dot_general(a3, b3, [2], [1], [0], [0]), p.dot_general(a3, a3, [2], [2], [0], [0]),
             p.dot_general(a4, b4, [3, 2], [0, 2], [0], [1]),     # two contract axes, batch in different positions
             p.matmul(p.slice(a, [(1, 33), (2, 50)]), p.slice(b, [(2, 50), (0, 29)])),
             p.relu(p.add(p.matmul(a, b), p.broadcast_to(p.slice(b, [(0, 1), (0, 29)]), [37, 29])))]   # epilogue fusion
    o, c, dts = p.run(cpu, gpu, nodes)
    w, _, _ = p.run(cpu64, gpu, nodes)
    for i, (x, y, z, dt) in enumerate(zip(o, c, w, dts)):
        if tag in (api.I32, api.I8, api.U16):
            util.assert_exact(x, y, f"int dot {i}")
        elif tag == api.F64:
            util.assert_close(x, y, 1e-12, 1e-13, f"f64 dot {i}")
        elif tag == api.F32:
            util.assert_close(x, y, 1e-5, 1e-5, f"f32 dot {i}")
        else:   # rel 2e-2 against the f64 interpreter run; and within one narrow ulp of the native oracle
            util.assert_close(z, util.to_f64(y, dt), 2e-2, 2e-2, f"low dot {i} vs f64")
            util.assert_close(util.to_f64(x, dt), util.to_f64(y, dt), 2.0 ** -6, 1e-2, f"low dot {i} vs native")


def test_eval_many_shares_subgraphs_and_missing_feed_is_an_error(oracle_lib, cuda_lib, cpu, gpu):
    rng = np.random.default_rng(12)
    p = Pair(oracle_lib, cuda_lib)
    x = p.feed((16, 32), api.F32, rng_f32(rng, (16, 32)))
    trunk = p.gelu(p.matmul(x, p.permute(x, [1, 0])))
    nodes = [trunk, p.sum(trunk, 1), p.softmax(trunk, 1), trunk]
    o, c, _ = p.run(cpu, gpu, nodes)
    for a, b in zip(o, c):
        util.assert_close(a, b, 2e-5, 1e-5, "eval_many")
    assert np.array_equal(c[0], c[3])
    g = api.Graph(cuda_lib)
    y = g.relu(g.input([4], api.F32))
    with pytest.raises(api.Error, match="missing feed"):
        gpu.eval(g, y)
    f = api.Feeds(cuda_lib).set(0, np.zeros((5,), np.float32))
    with pytest.raises(api.Error, match="shape"):
        gpu.eval_with(g, y, f)
    # the context is still usable after an error
    assert gpu.eval_with(g, y, api.Feeds(cuda_lib).set(0, np.array([-1, 2, -3, 4], np.float32))).numpy().tolist() == [0, 2, 0, 4]


def test_random_graph_fuzz(oracle_lib, cuda_lib, cpu, gpu):
    """Differential fuzz in the shape of kurumi_core/src/realize/fuzz.rs:37-112 and
    kurumi_metal/src/tests/fuzz.rs:86-180: random unary/binary/reduce/movement graphs, f32 within a
    band, integer graphs exact."""
    rng = np.random.default_rng(13)
    for seed in range(24):
        is_int = seed % 3 == 2
        p = Pair(oracle_lib, cuda_lib)
        shape = [int(rng.integers(1, 6)), int(rng.integers(1, 40))]
        mk = (lambda s: rng.integers(-50, 50, s).astype(np.int32)) if is_int else (lambda s: rng_f32(rng, s))
        tag = api.I32 if is_int else api.F32
        vals = [p.feed(tuple(shape), tag, mk(shape)) for _ in range(3)]
        for _ in range(int(rng.integers(3, 12))):
            a = vals[int(rng.integers(len(vals)))]
            sh = list(p.go.shape(a))
            same = [v for v in vals if list(p.go.shape(v)) == sh]
            b = same[int(rng.integers(len(same)))]
            op = int(rng.integers(0, 10))
            if op == 0: r = p.add(a, b)
            elif op == 1: r = p.mul(a, b)
            elif op == 2: r = p.max(a, b)
            elif op == 3: r = p.neg(a) if is_int else [p.neg, p.sqrt, p.sin, p.abs, p.relu][int(rng.integers(5))](a)
            elif op == 4 and len(sh) == 2: r = p.permute(a, [1, 0])
            elif op == 5 and len(sh) >= 1: r = [p.sum, p.reduce_max][int(rng.integers(2))](a, int(rng.integers(len(sh))))
            elif op == 6 and len(sh) == 2: r = p.reshape(a, [sh[0] * sh[1]])
            elif op == 7 and len(sh) >= 1 and sh[-1] > 2: r = p.slice(a, [(0, d) for d in sh[:-1]] + [(1, sh[-1] - 1)])
            elif op == 8 and len(sh) >= 1: r = p.pad(a, [(0, 1)] * (len(sh) - 1) + [(2, 1)])
            elif op == 9 and len(sh) >= 1: r = p.flip(a, [len(sh) - 1])
            else: r = p.where(p.lt(a, b), a, b)
            vals.append(r)
        o, c, _ = p.run(cpu, gpu, vals[-3:])
        for a, b in zip(o, c):
            if is_int:
                util.assert_exact(a, b, f"fuzz seed {seed}")
            else:
                util.assert_close(a, b, 2e-5, 2e-5, f"fuzz seed {seed}")
