"""Op::ArgReduce (argmax / argmin): I64 index of the first strict maximum / minimum along an axis, as
kurumi_core/src/interp/reduce.rs:16-66 computes it (ties keep the lowest index; a NaN never replaces the best,
and a leading NaN is never replaced), on the oracle and on the device, plus the blob tag (29)."""
import numpy as np
import pytest

from kurumi_b200 import api


def reference(v: np.ndarray, axis: int, arg_min: bool) -> np.ndarray:
    m = np.moveaxis(v, axis, -1)
    out = np.zeros(m.shape[:-1], np.int64)
    for idx in np.ndindex(*m.shape[:-1]):
        best, bk = m[idx][0], 0
        for k in range(1, m.shape[-1]):
            x = m[idx][k]
            if (x < best) if arg_min else (x > best):
                best, bk = x, k
        out[idx] = bk
    return out


CASES = [
    (api.F32, np.array([[1.0, 3.0, 3.0, -2.0], [np.nan, 5.0, 1.0, 0.0], [0.0, np.nan, 7.0, 7.0], [-np.inf, -np.inf, -1.0, np.inf]], np.float32)),
    (api.I32, np.array([[5, -7, 5, 2], [-3, -3, -9, -9], [0, 0, 0, 0]], np.int32)),
    (api.U8, np.array([[200, 13, 255, 255], [0, 0, 1, 0]], np.uint8)),
    (api.I64, np.array([[-2 ** 62, 2 ** 62, 2 ** 62 + 1, -2 ** 62 - 1]], np.int64)),
    (api.U64, np.array([[2 ** 63 + 5, 2 ** 63 + 6, 3, 2 ** 63 + 6]], np.uint64)),
]


@pytest.mark.parametrize("dtype,values", CASES)
def test_oracle_matches_the_reference_rule(oracle_lib, cpu, cpu64, dtype, values):
    for axis in range(values.ndim):
        for arg_min in (False, True):
            g = api.Graph(oracle_lib)
            x = g.constant(values, dtype)
            out = (g.argmin if arg_min else g.argmax)(x, axis)
            assert g.dtype(out) == api.I64
            want = reference(values, axis, arg_min)
            assert g.shape(out) == want.shape
            np.testing.assert_array_equal(cpu.eval(g, out).numpy(), want)
            if dtype == api.F32:
                np.testing.assert_array_equal(cpu64.eval(g, out).numpy(), want)


def test_checks_blob_and_device_compile(oracle_lib, cuda_lib, cpu):
    g = api.Graph(oracle_lib)
    x = g.input([3, 4], api.F32)
    with pytest.raises(api.Error):
        g.argmax(x, 2)
    with pytest.raises(api.Error, match="numeric"):
        g.argmax(g.input([3], api.BOOL), 0)
    out = g.argmin(g.mul(x, x), 1)
    blob = g.serialize([out], [(x, 1, "x")], reachable=True)
    rg, entries = api.deserialize(oracle_lib, blob)
    assert rg.serialize(entries[0][1], entries[0][2]) == blob
    v = np.array([[3, -1, 1, 2], [0, 5, 0, 5], [-4, 4, 9, 2]], np.float32)
    f = api.Feeds(oracle_lib).set(entries[0][2][0][0], v)
    np.testing.assert_array_equal(cpu.eval_with(rg, entries[0][1][0], f).numpy(), np.array([1, 0, 3], np.int64))
    bad_kind = blob.replace(bytes([29]) + (1).to_bytes(8, "little") + bytes([1]), bytes([29]) + (1).to_bytes(8, "little") + bytes([2]))
    assert bad_kind != blob
    with pytest.raises(api.Error, match="argkind"):
        api.deserialize(oracle_lib, bad_kind)
    cg, ce = api.deserialize(cuda_lib, blob)
    assert api.compile_check(cuda_lib, cg, ce[0][1]) == ["arg_fold"]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [api.F32, api.BF16, api.I32, api.U64])
def test_device_matches_the_oracle(oracle_lib, cuda_lib, cpu, gpu, dtype):
    rng = np.random.default_rng(4)
    shape = (37, 130, 9)
    if dtype == api.F32:
        v = rng.integers(-5, 6, shape).astype(np.float32)          # many ties
        v[3, 7, :] = np.nan; v[5, :, 2] = np.nan; v[6, 0, 0] = np.nan
    elif dtype == api.BF16:
        v = api.f32_to_bf16(rng.integers(-5, 6, shape).astype(np.float32))
    elif dtype == api.I32:
        v = rng.integers(-3, 4, shape).astype(np.int32)
    else:
        v = rng.integers(0, 4, shape).astype(np.uint64) + np.uint64(2 ** 63)
    for axis in range(3):
        for arg_min in (False, True):
            outs = []
            for lib, be in ((oracle_lib, cpu), (cuda_lib, gpu)):
                g = api.Graph(lib)
                x = g.input(list(shape), dtype)
                y = g.permute(x, [0, 1, 2]) if dtype != api.F32 else g.add(x, x)   # through a fused expression as well
                out = (g.argmin if arg_min else g.argmax)(y, axis)
                outs.append(be.eval_with(g, out, api.Feeds(lib).set(x, v, dtype)).numpy())
            np.testing.assert_array_equal(outs[0], outs[1])


@pytest.mark.gpu
@pytest.mark.parametrize("n", [3001, 4100, 10240])
@pytest.mark.parametrize("dtype", [api.F32, api.F64, api.BF16, api.I32, api.I8, api.U64])
def test_long_innermost_lines_take_a_cta_per_line(oracle_lib, cuda_lib, cpu, gpu, dtype, n):
    """A long innermost axis (the sampling head: argmax over the vocabulary) runs one CTA per line; partial results merge by
    value and then by lower index, which must equal the interpreter's first-maximum walk: ties everywhere, NaNs at the
    start, in the middle and at the end of a line, a line of NaNs, a line of one repeated value, +-inf and +-0. An odd
    length is read element by element; 4100 and 10240 in 128-bit pieces, eight turns of loads at a time (4100 ends inside a
    batch of turns, 10240 takes more than one batch)."""
    rng = np.random.default_rng(6)
    lines = 9
    if dtype in (api.F32, api.F64, api.BF16):
        v = rng.integers(-4, 5, (lines, n)).astype(np.float64)      # many ties
        v[1, 0] = np.nan                                            # a leading NaN is never replaced
        v[2, 1500] = np.nan; v[2, n - 1] = np.nan
        v[3, :] = np.nan
        v[4, :] = 2.0
        v[5, 17] = np.inf; v[5, 2900] = np.inf; v[5, 40] = -np.inf
        v[6, :] = 0.0; v[6, 5] = -0.0; v[6, 2000] = -0.0              # -0 == +0: the first position wins either way
        v[7, 1:] = np.nan                                           # only position 0 is a number
        carrier = v.astype(np.float32) if dtype == api.F32 else v if dtype == api.F64 else api.f32_to_bf16(v.astype(np.float32))
    elif dtype == api.U64:
        carrier = rng.integers(0, 3, (lines, n)).astype(np.uint64) + np.uint64(2 ** 63)
    else:
        carrier = rng.integers(-3, 4, (lines, n)).astype(np.int32 if dtype == api.I32 else np.int8)
    for arg_min in (False, True):
        outs = []
        for lib, be in ((oracle_lib, cpu), (cuda_lib, gpu)):
            g = api.Graph(lib)
            x = g.input([lines, n], dtype)
            out = (g.argmin if arg_min else g.argmax)(x, 1)
            if lib is cuda_lib:
                assert api.compile_check(lib, g, [out]) == ["arg_rows"]
            outs.append(be.eval_with(g, out, api.Feeds(lib).set(x, carrier, dtype)).numpy())
        np.testing.assert_array_equal(outs[0], outs[1])
        if dtype == api.F32:
            np.testing.assert_array_equal(outs[0], reference(carrier, 1, arg_min))


@pytest.mark.gpu
def test_more_lines_than_ctas_in_flight(oracle_lib, cuda_lib, cpu, gpu):
    """12000 lines are more than eight residencies of CTAs: the grid stays resident and its CTAs loop over the lines."""
    rng = np.random.default_rng(9)
    v = rng.integers(-50, 50, (12000, 256)).astype(np.float32)
    outs = []
    for lib, be in ((oracle_lib, cpu), (cuda_lib, gpu)):
        g = api.Graph(lib)
        x = g.input([12000, 256], api.F32)
        out = g.argmax(x, 1)
        outs.append(be.eval_with(g, out, api.Feeds(lib).set(x, v, api.F32)).numpy())
    np.testing.assert_array_equal(outs[0], outs[1])
    np.testing.assert_array_equal(outs[1], reference(v, 1, False))
