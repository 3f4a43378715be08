"""Helpers shared by the parity tests: build one graph in two libraries, compare results."""
import numpy as np

from kurumi_b200 import api


class Pair:
    """Records the same builder calls into an oracle graph and a CUDA graph. Node ids are arena
    indices, so identical call sequences give identical ids; every call checks that."""

    def __init__(self, oracle_lib, cuda_lib):
        self.go, self.gc = api.Graph(oracle_lib), api.Graph(cuda_lib)
        self.olib, self.clib = oracle_lib, cuda_lib
        self.feeds = {}

    def __getattr__(self, name):
        fo, fc = getattr(self.go, name), getattr(self.gc, name)

        def call(*a, **k):
            ro, rc = fo(*a, **k), fc(*a, **k)
            assert ro == rc, f"{name}: oracle {ro} vs cuda {rc}"
            return ro
        return call

    def feed(self, shape, dtype, values: np.ndarray):
        """An Input node bound to `values` (raw carrier array for bf16 / fp8)."""
        n = self.input(list(shape), dtype)
        self.feeds[n] = (np.ascontiguousarray(values).reshape(shape), dtype)
        return n

    def _feeds(self, lib):
        f = api.Feeds(lib)
        for n, (v, dt) in self.feeds.items():
            f.set(n, v, dt)
        return f

    def run(self, cpu, gpu, nodes):
        """(oracle results, cuda results) as numpy carrier arrays, one per node."""
        o = cpu.eval_many_with(self.go, nodes, self._feeds(self.olib))
        c = gpu.eval_many_with(self.gc, nodes, self._feeds(self.clib))
        for a, b in zip(o, c):
            assert a.dtype == b.dtype or a.dtype == api.F64, (a.dtype, b.dtype)
            assert a.shape == b.shape, (a.shape, b.shape)
        return [t.numpy() for t in o], [t.numpy() for t in c], [t.dtype for t in c]


def to_f64(arr: np.ndarray, dtype: int) -> np.ndarray:
    if dtype == api.BF16:
        return api.bf16_to_f32(arr).astype(np.float64)
    if dtype == api.F8E4M3:
        return api.e4m3_to_f32(arr).astype(np.float64)
    if dtype == api.F8E5M2:
        import torch
        return torch.from_numpy(arr.copy()).view(torch.float8_e5m2).to(torch.float64).numpy()
    return arr.astype(np.float64)


def assert_exact(o, c, what=""):
    assert o.dtype == c.dtype and o.shape == c.shape, (what, o.dtype, c.dtype, o.shape, c.shape)
    if not np.array_equal(o, c):
        bad = np.flatnonzero(o.reshape(-1) != c.reshape(-1))
        raise AssertionError(f"{what}: {bad.size} of {o.size} differ; first at {bad[0]}: oracle {o.reshape(-1)[bad[0]]} vs cuda {c.reshape(-1)[bad[0]]}")


def ulp_diff_f32(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Distance in units in the last place between two f32 arrays (NaN == NaN counts as 0)."""
    ai = a.astype(np.float32).view(np.int32).astype(np.int64)
    bi = b.astype(np.float32).view(np.int32).astype(np.int64)
    ai = np.where(ai < 0, np.int64(-(2 ** 31)) - ai, ai)
    bi = np.where(bi < 0, np.int64(-(2 ** 31)) - bi, bi)
    d = np.abs(ai - bi)
    both_nan = np.isnan(a) & np.isnan(b)
    return np.where(both_nan, 0, d)


def assert_ulp(o, c, max_ulp, what=""):
    d = ulp_diff_f32(o, c)
    assert d.max(initial=0) <= max_ulp, f"{what}: max ulp distance {d.max()} > {max_ulp} at {int(d.argmax())}: oracle {o.reshape(-1)[d.argmax()]!r} cuda {c.reshape(-1)[d.argmax()]!r}"


def assert_close(o, c, rel, abs_=0.0, what=""):
    o, c = np.asarray(o, np.float64), np.asarray(c, np.float64)
    nan_o, nan_c = np.isnan(o), np.isnan(c)
    assert np.array_equal(nan_o, nan_c), f"{what}: NaN pattern differs"
    inf = np.isinf(o)
    assert np.array_equal(o[inf], c[inf]), f"{what}: infinities differ"
    ok = ~(nan_o | inf)
    err = np.abs(o[ok] - c[ok])
    tol = abs_ + rel * np.abs(o[ok])
    assert (err <= tol).all(), f"{what}: max err {err.max():.3e} (rel {np.max(err / np.maximum(np.abs(o[ok]), 1e-30)):.3e}), {int((err > tol).sum())} of {err.size} outside rel {rel} abs {abs_}"


PARITY_LOG = []   # (what, max relative error outside the floor, max error in units of the row scale), printed at session end


def assert_band(o, c, rel, step, what=""):
    """The stated band for narrow-format contractions and attention: |got - want| <= rel * |want| for every element, with
    the format's own resolution as the floor near zero: `step` (2^-8 for bf16: one unit in the last place of a value at
    the row's scale) times the largest |want| of the element's row (last axis). Records the achieved errors."""
    o, c = np.asarray(o, np.float64), np.asarray(c, np.float64)
    assert o.shape == c.shape, (what, o.shape, c.shape)
    assert np.isfinite(o).all() and np.isfinite(c).all(), f"{what}: non-finite values"
    scale = np.abs(o).max(axis=-1, keepdims=True)
    floor = step * scale
    err = np.abs(o - c)
    tol = np.maximum(rel * np.abs(o), floor)
    above = np.abs(o) * rel > floor            # elements whose relative band is the wider one
    max_rel = float((err[above] / np.abs(o)[above]).max()) if above.any() else 0.0
    max_scaled = float((err / np.maximum(scale, 1e-300)).max())
    PARITY_LOG.append((what, max_rel, max_scaled))
    bad = err > tol
    assert not bad.any(), f"{what}: {int(bad.sum())} of {err.size} outside rel {rel} / floor {step} x row scale; max rel {max_rel:.3e}, max err / row scale {max_scaled:.3e}"


def threefry_np(key: int, ctr: np.ndarray) -> np.ndarray:
    """threefry2x32-20 (kurumi_core/src/rng.rs:10-26) over an array of 64-bit counters -> u64."""
    rot = [13, 15, 26, 6, 17, 29, 16, 24]
    k0, k1 = np.uint32(key & 0xFFFFFFFF), np.uint32((key >> 32) & 0xFFFFFFFF)
    ks = [k0, k1, np.uint32(0x1BD11BDA) ^ k0 ^ k1]
    ctr = ctr.astype(np.uint64)
    with np.errstate(over="ignore"):
        x0 = (ctr & np.uint64(0xFFFFFFFF)).astype(np.uint32) + ks[0]
        x1 = (ctr >> np.uint64(32)).astype(np.uint32) + ks[1]
        for r in range(20):
            x0 = x0 + x1
            s = rot[r % 8]
            x1 = (x1 << np.uint32(s)) | (x1 >> np.uint32(32 - s))
            x1 = x1 ^ x0
            if r % 4 == 3:
                inj = r // 4 + 1
                x0 = x0 + ks[inj % 3]
                x1 = x1 + ks[(inj + 1) % 3] + np.uint32(inj)
    return x0.astype(np.uint64) | (x1.astype(np.uint64) << np.uint64(32))


def split_key(seed: int, n: int) -> list:
    """Key::new(seed).split_n(n) (kurumi_core/src/rng.rs:51-53)."""
    return [int(v) for v in threefry_np(seed, np.arange(n, dtype=np.uint64))]
