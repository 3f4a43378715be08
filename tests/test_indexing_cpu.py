"""Gather / GatherAlong / Scatter / ScatterAlong / Argsort on the CPU oracle against numpy statements of the
reference's definitions (kurumi_core/src/interp/indexing/{gather,scatter}.rs, interp/sort.rs) and the values its own
tests hold: out-of-range indices are clamped by the gathers and dropped by the scatters, updates fold in index order,
sorting is stable."""
import numpy as np
import pytest

from kurumi_b200 import api


def ev(oracle_lib, cpu, build, *arrays):
    g = api.Graph(oracle_lib)
    nodes = [g.constant(a, {np.dtype(np.float32): api.F32, np.dtype(np.int64): api.I64, np.dtype(np.int32): api.I32}[a.dtype]) for a in arrays]
    return cpu.eval(g, build(g, *nodes)).numpy()


def test_gather_clamps_and_inserts_the_index_shape(oracle_lib, cpu):
    x = np.arange(24, dtype=np.float32).reshape(2, 4, 3)
    idx = np.array([[3, 0], [9, -2]], np.int64)                      # 9 -> 3, -2 -> 0
    got = ev(oracle_lib, cpu, lambda g, a, i: g.gather(a, i, 1), x, idx)
    want = np.take(x, np.clip(idx, 0, 3), axis=1)
    assert got.shape == (2, 2, 2, 3) and np.array_equal(got, want)
    # kurumi_core/tests/ops.rs: take rows [2, 0] of a [3, 2] matrix
    m = np.array([[1, 2], [3, 4], [5, 6]], np.float32)
    assert np.array_equal(ev(oracle_lib, cpu, lambda g, a, i: g.gather(a, i, 0), m, np.array([2, 0], np.int32)), m[[2, 0]])


def test_gather_along_takes_one_index_per_position(oracle_lib, cpu):
    rng = np.random.default_rng(0)
    x = rng.standard_normal((3, 5, 4)).astype(np.float32)
    idx = rng.integers(-2, 7, (3, 2, 4)).astype(np.int64)
    got = ev(oracle_lib, cpu, lambda g, a, i: g.gather_along(a, i, 1), x, idx)
    assert np.array_equal(got, np.take_along_axis(x, np.clip(idx, 0, 4), axis=1))


@pytest.mark.parametrize("combine", [0, 1, 2, 3])
def test_scatter_folds_updates_in_index_order(oracle_lib, cpu, combine):
    rng = np.random.default_rng(1)
    x = rng.standard_normal((2, 5, 3)).astype(np.float32)
    idx = np.array([4, 1, 4, 7, -1, 1], np.int64)                    # duplicates, two out of range
    up = rng.standard_normal((2, 6, 3)).astype(np.float32)
    want = x.copy()
    for p in range(2):
        for k, j in enumerate(idx):
            if 0 <= j < 5:
                old, new = want[p, j], up[p, k]
                want[p, j] = [new, old + new, np.maximum(old, new), np.minimum(old, new)][combine]
    got = ev(oracle_lib, cpu, lambda g, a, i, u: g.scatter(a, i, u, 1, combine), x, idx, up)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("combine", [0, 1, 2, 3])
def test_scatter_along(oracle_lib, cpu, combine):
    rng = np.random.default_rng(2)
    x = rng.standard_normal((4, 6)).astype(np.float32)
    idx = rng.integers(-1, 8, (4, 9)).astype(np.int64)
    up = rng.standard_normal((4, 9)).astype(np.float32)
    want = x.copy()
    for r in range(4):
        for c in range(9):
            j = idx[r, c]
            if 0 <= j < 6:
                old, new = want[r, j], up[r, c]
                want[r, j] = [new, old + new, max(old, new), min(old, new)][combine]
    got = ev(oracle_lib, cpu, lambda g, a, i, u: g.scatter_along(a, i, u, 1, combine), x, idx, up)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("descending", [False, True])
def test_argsort_is_stable_and_sort_follows_it(oracle_lib, cpu, descending):
    rng = np.random.default_rng(3)
    x = rng.integers(0, 6, (5, 40)).astype(np.float32)              # many ties
    x[0, :4] = [0.0, -0.0, 0.0, -0.0]                               # the two zeros compare equal
    perm = ev(oracle_lib, cpu, lambda g, a: g.argsort(a, 1, descending), x)
    want = np.argsort(-x if descending else x, axis=1, kind="stable")
    assert perm.dtype == np.int64 and np.array_equal(perm, want)
    srt = ev(oracle_lib, cpu, lambda g, a: g.sort(a, 1, descending), x)
    assert np.array_equal(srt, np.take_along_axis(x, want, axis=1))
    col = ev(oracle_lib, cpu, lambda g, a: g.argsort(a, 0, descending), x)
    assert np.array_equal(col, np.argsort(-x if descending else x, axis=0, kind="stable"))


def test_record_time_checks(oracle_lib):
    g = api.Graph(oracle_lib)
    x, f = g.input([4, 5], api.F32), g.input([3], api.F32)
    i = g.input([3], api.I64)
    with pytest.raises(api.Error, match="indices must be integer"):
        g.gather(x, f, 0)
    with pytest.raises(api.Error, match="axis 2 out of range"):
        g.gather(x, i, 2)
    with pytest.raises(api.Error, match="updates shape"):
        g.scatter(x, i, x, 0)
    with pytest.raises(api.Error, match="must match operand"):
        g.gather_along(x, g.input([3, 6], api.I64), 0)
    with pytest.raises(api.Error, match="bad combine"):
        g.scatter(x, i, g.input([3, 5], api.F32), 0, 9)


def test_blob_round_trip(oracle_lib, cpu):
    """Tags 50..54 of the KGPH v2 format (kurumi_core/src/graph/serialize/encode/op.rs:146-169)."""
    g = api.Graph(oracle_lib)
    x, i = g.input([4, 5], api.F32), g.input([4, 2], api.I64)
    root = g.scatter_along(g.sort(x, 1, True), i, g.gather_along(x, i, 1), 1, 1)
    root = g.add(root, g.gather(g.scatter(x, g.argmax(x, 1), x, 0, 2), g.argmin(x, 1), 0))
    blob = g.serialize([root], [(x, 1, "x"), (i, 1, "i")])
    g2, entries = api.deserialize(oracle_lib, blob)
    _, outs, ins = entries[0]
    rng = np.random.default_rng(4)
    xv, iv = rng.standard_normal((4, 5)).astype(np.float32), rng.integers(0, 5, (4, 2)).astype(np.int64)
    a = cpu.eval_with(g, root, api.Feeds(oracle_lib).set(x, xv).set(i, iv)).numpy()
    by_name = {name: node for node, _, name in ins}
    b = cpu.eval_with(g2, outs[0], api.Feeds(oracle_lib).set(by_name["x"], xv).set(by_name["i"], iv)).numpy()
    assert np.array_equal(a, b)


def test_known_answers_of_the_reference_tests(oracle_lib, cpu):
    """Values held by kurumi_core/tests/ops.rs:127-170 and kurumi_core/tests/dtype.rs:154-192."""
    f32 = lambda *v: np.array(v, np.float32)
    g = api.Graph(oracle_lib)
    w = g.constant(f32(10, 11, 20, 21, 30, 31).reshape(3, 2), api.F32)
    ids = g.constant(np.array([[2, 0], [1, 2]], np.int32), api.I32)
    y = g.gather(w, ids, 0)
    assert g.shape(y) == (2, 2, 2)
    assert np.array_equal(cpu.eval(g, y).numpy().reshape(-1), f32(30, 31, 10, 11, 20, 21, 30, 31))          # embedding lookup
    a = g.constant(f32(5, 6, 7), api.F32)
    assert np.array_equal(cpu.eval(g, g.gather(a, g.constant(np.array([-1, 1, 9], np.int32), api.I32), 0)).numpy(), f32(5, 6, 7))   # clamped
    ix = g.constant(np.array([1, 3], np.int32), api.I32)
    up = g.constant(f32(9, 7), api.F32)
    assert np.array_equal(cpu.eval(g, g.scatter(g.constant(f32(0, 0, 0, 0), api.F32), ix, up, 0, 0)).numpy(), f32(0, 9, 0, 7))
    assert np.array_equal(cpu.eval(g, g.scatter(g.constant(f32(1, 1, 1, 1), api.F32), ix, up, 0, 1)).numpy(), f32(1, 10, 1, 8))
    drop = g.scatter(g.constant(f32(0, 0, 0), api.F32), g.constant(np.array([5, 1], np.int32), api.I32), g.constant(f32(9, 4), api.F32), 0, 0)
    assert np.array_equal(cpu.eval(g, drop).numpy(), f32(0, 4, 0))                                           # out of range dropped
    for np_t, tag in ((np.uint8, api.U8), (np.uint16, api.U16), (np.uint32, api.U32), (np.uint64, api.U64), (np.int8, api.I8), (np.int16, api.I16),
                      (np.int32, api.I32), (np.int64, api.I64)):
        idx = g.constant(np.array([2, 0], np_t), tag)
        assert np.array_equal(cpu.eval(g, g.gather(g.constant(f32(10, 20, 30), api.F32), idx, 0)).numpy(), f32(30, 10))
    for np_t, tag in ((np.int8, api.I8), (np.int16, api.I16), (np.uint16, api.U16), (np.uint64, api.U64)):
        op = g.constant(np.array([1, 1, 1], np_t), tag)
        idx = g.constant(np.array([0, 0, 2], np.int64), api.I64)
        upd = g.constant(np.array([5, 3, 7], np_t), tag)
        assert np.array_equal(cpu.eval(g, g.scatter(op, idx, upd, 0, 1)).numpy(), np.array([9, 1, 8], np_t))
