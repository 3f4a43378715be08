"""Gather / GatherAlong / Scatter / ScatterAlong / Argsort / sort on the device against the CPU oracle, bit for bit
(indices and data movement are integer work; the scatter combiners fold in index order on both sides), over dtypes,
axes, out-of-range indices, duplicates and ties."""
import numpy as np
import pytest

from kurumi_b200 import api
from tests import util
from tests.util import Pair

pytestmark = pytest.mark.gpu


def test_gathers(oracle_lib, cuda_lib, cpu, gpu):
    rng = np.random.default_rng(50)
    p = Pair(oracle_lib, cuda_lib)
    x = p.feed((6, 9, 5), api.F32, rng.standard_normal((6, 9, 5)).astype(np.float32))
    xb = p.feed((6, 9, 5), api.BF16, api.f32_to_bf16(rng.standard_normal((6, 9, 5)).astype(np.float32)))
    xi = p.feed((6, 9, 5), api.I16, rng.integers(-300, 300, (6, 9, 5)).astype(np.int16))
    i0 = p.feed((4, 3), api.I32, rng.integers(-3, 12, (4, 3)).astype(np.int32))
    i1 = p.feed((7,), api.U8, rng.integers(0, 12, 7).astype(np.uint8))
    ia = p.feed((6, 4, 5), api.I64, rng.integers(-2, 11, (6, 4, 5)).astype(np.int64))
    nodes = [p.gather(x, i0, 0), p.gather(x, i0, 1), p.gather(xb, i1, 2), p.gather(xi, i1, 1), p.gather_along(x, ia, 1), p.gather_along(xb, ia, 1),
             p.gather(p.mul(x, x), p.add(i1, i1), 1),                       # fused producers on both operands
             p.gather_along(p.permute(x, [0, 2, 1]), p.permute(ia, [0, 2, 1]), 2)]
    o, c, _ = p.run(cpu, gpu, nodes)
    for k, (a, b) in enumerate(zip(o, c)):
        util.assert_exact(a, b, f"gather node {k}")


@pytest.mark.parametrize("combine", [0, 1, 2, 3])
def test_scatters(oracle_lib, cuda_lib, cpu, gpu, combine):
    rng = np.random.default_rng(51 + combine)
    p = Pair(oracle_lib, cuda_lib)
    x = p.feed((5, 8, 6), api.F32, rng.standard_normal((5, 8, 6)).astype(np.float32))
    xb = p.feed((5, 8, 6), api.BF16, api.f32_to_bf16(rng.standard_normal((5, 8, 6)).astype(np.float32)))
    xi = p.feed((5, 8, 6), api.I8, rng.integers(-100, 100, (5, 8, 6)).astype(np.int8))
    idx = p.feed((11,), api.I32, rng.integers(-2, 10, 11).astype(np.int32))            # duplicates and out-of-range entries
    up = p.feed((5, 11, 6), api.F32, rng.standard_normal((5, 11, 6)).astype(np.float32))
    upb = p.feed((5, 11, 6), api.BF16, api.f32_to_bf16(rng.standard_normal((5, 11, 6)).astype(np.float32)))
    upi = p.feed((5, 11, 6), api.I8, rng.integers(-100, 100, (5, 11, 6)).astype(np.int8))
    ia = p.feed((5, 13, 6), api.I64, rng.integers(-1, 10, (5, 13, 6)).astype(np.int64))
    ua = p.feed((5, 13, 6), api.F32, rng.standard_normal((5, 13, 6)).astype(np.float32))
    vec = p.feed((40,), api.F32, rng.standard_normal(40).astype(np.float32))
    vi = p.feed((100,), api.I64, rng.integers(0, 40, 100).astype(np.int64))
    vu = p.feed((100,), api.F32, rng.standard_normal(100).astype(np.float32))
    nodes = [p.scatter(x, idx, up, 1, combine), p.scatter(xb, idx, upb, 1, combine), p.scatter(xi, idx, upi, 1, combine), p.scatter_along(x, ia, ua, 1, combine),
             p.scatter(vec, vi, vu, 0, combine),                                 # one thread owns the whole vector: index order
             p.scatter(p.mul(x, x), idx, p.neg(up), 1, combine)]
    o, c, _ = p.run(cpu, gpu, nodes)
    for k, (a, b) in enumerate(zip(o, c)):
        util.assert_exact(a, b, f"scatter combine {combine} node {k}")


@pytest.mark.parametrize("descending", [False, True])
def test_argsort_and_sort(oracle_lib, cuda_lib, cpu, gpu, descending):
    rng = np.random.default_rng(60)
    p = Pair(oracle_lib, cuda_lib)
    ties = rng.integers(0, 7, (9, 300)).astype(np.float32)
    ties[0, :4] = [0.0, -0.0, 0.0, -0.0]
    x = p.feed((9, 300), api.F32, ties)
    xl = p.feed((3, 5000), api.F32, rng.standard_normal((3, 5000)).astype(np.float32))
    xb = p.feed((4, 33, 6), api.BF16, api.f32_to_bf16(rng.standard_normal((4, 33, 6)).astype(np.float32)))
    xi = p.feed((4, 17), api.I64, rng.integers(-2 ** 62, 2 ** 62, (4, 17)).astype(np.int64))
    xu = p.feed((4, 17), api.U8, rng.integers(0, 256, (4, 17)).astype(np.uint8))
    one = p.feed((5, 1), api.F32, rng.standard_normal((5, 1)).astype(np.float32))
    nodes = [p.argsort(x, 1, descending), p.argsort(x, 0, descending), p.argsort(xl, 1, descending), p.argsort(xb, 1, descending), p.argsort(xi, 1, descending),
             p.argsort(xu, 1, descending), p.argsort(one, 1, descending), p.sort(x, 1, descending), p.sort(xb, 1, descending)]
    o, c, _ = p.run(cpu, gpu, nodes)
    for k, (a, b) in enumerate(zip(o, c)):
        util.assert_exact(a, b, f"argsort descending={descending} node {k}")
    assert np.array_equal(c[0], np.argsort(-ties if descending else ties, axis=1, kind="stable"))


def test_embedding_lookup_and_its_gradient_shape(oracle_lib, cuda_lib, cpu, gpu):
    """The two uses the reference's frontends make of these ops: rows of a table by token id, and the scatter-add of
    the rows' gradients back into the table."""
    rng = np.random.default_rng(70)
    p = Pair(oracle_lib, cuda_lib)
    table = p.feed((1000, 64), api.F32, rng.standard_normal((1000, 64)).astype(np.float32))
    ids = p.feed((8, 128), api.I32, rng.integers(0, 1000, (8, 128)).astype(np.int32))
    rows = p.gather(table, ids, 0)
    grad = p.scatter(p.mul(table, p.scalar(table, 0.0)), p.reshape(ids, [1024]), p.reshape(rows, [1024, 64]), 0, 1)
    o, c, _ = p.run(cpu, gpu, [rows, grad])
    util.assert_exact(o[0], c[0], "embedding rows")
    util.assert_exact(o[1], c[1], "embedding gradient (scatter-add in index order)")
    assert api.compile_check(cuda_lib, p.gc, [rows]) == ["gather"]


@pytest.mark.parametrize("combine", [0, 1, 3])
def test_scatter_with_many_indices_and_few_columns(oracle_lib, cuda_lib, cpu, gpu, combine):
    """Few destination columns and thousands of indices: the device cuts the destination axis into blocks (a thread per
    column and block scans all indices, four at a time, and applies its own in order). Still bit for bit the
    interpreter's index-order fold: duplicates pile up on some rows, out-of-range indices are skipped, the index count is
    not a multiple of four, float sums depend on the order."""
    rng = np.random.default_rng(60 + combine)
    rows, cols, k = 1003, 24, 5003
    p = Pair(oracle_lib, cuda_lib)
    x = p.feed((rows, cols), api.F32, rng.standard_normal((rows, cols)).astype(np.float32))
    iv = rng.integers(-5, rows + 5, k).astype(np.int64)
    iv[:200] = 17; iv[-3:] = rows - 1                                    # a hot row, and the tail of the last group of four
    idx = p.feed((k,), api.I64, iv)
    up = p.feed((k, cols), api.F32, (rng.standard_normal((k, cols)) * 100).astype(np.float32))
    xa = p.feed((cols, rows), api.BF16, api.f32_to_bf16(rng.standard_normal((cols, rows)).astype(np.float32)))
    ia = p.feed((cols, k), api.I32, rng.integers(-3, rows + 3, (cols, k)).astype(np.int32))
    ua = p.feed((cols, k), api.BF16, api.f32_to_bf16(rng.standard_normal((cols, k)).astype(np.float32)))
    nodes = [p.scatter(x, idx, up, 0, combine), p.scatter_along(xa, ia, ua, 1, combine)]
    o, c, _ = p.run(cpu, gpu, nodes)
    for n, (a, b) in enumerate(zip(o, c)):
        util.assert_exact(a, b, f"scatter node {n}, combine {combine}")


@pytest.mark.parametrize("descending", [False, True])
def test_argsort_of_lines_longer_than_shared_memory(oracle_lib, cuda_lib, cpu, gpu, descending):
    """Lines of more than 16384 elements (a vocabulary) do not fit one CTA's shared memory: the same bitonic network runs over
    a padded copy in global scratch, 4096-pair chunks and the narrow steps in shared memory, the wide steps one launch
    each. Same stable permutation as the oracle: many ties, a length that is no power of two, an axis that is not the
    last one, 64-bit keys, and sort() through the gather that follows."""
    rng = np.random.default_rng(61)
    p = Pair(oracle_lib, cuda_lib)
    ties = rng.integers(0, 50, (2, 40000)).astype(np.float32)          # 3 steps above the chunk size, 16384 < 40000 < 65536
    x = p.feed((2, 40000), api.F32, ties)
    xm = p.feed((17001, 3), api.F32, rng.standard_normal((17001, 3)).astype(np.float32))       # sorted along axis 0, inner stride 3
    xi = p.feed((1, 16400), api.I64, rng.integers(-2 ** 62, 2 ** 62, (1, 16400)).astype(np.int64))
    xb = p.feed((3, 20000), api.BF16, api.f32_to_bf16(rng.integers(-9, 9, (3, 20000)).astype(np.float32)))
    nodes = [p.argsort(x, 1, descending), p.argsort(xm, 0, descending), p.argsort(xi, 1, descending), p.argsort(xb, 1, descending), p.sort(x, 1, descending)]
    # padded to 65536: the chunk sort, then for k = 8192, 16384, 32768, 65536 the 1, 2, 3, 4 wide steps and a local pass each, then the copy out
    assert api.compile_check(cuda_lib, p.gc, [nodes[0]]).count("argsort") == 1 + (1 + 2 + 3 + 4) + 4 + 1
    o, c, _ = p.run(cpu, gpu, nodes)
    for k, (a, b) in enumerate(zip(o, c)):
        util.assert_exact(a, b, f"long argsort descending={descending} node {k}")
    assert np.array_equal(c[0], np.argsort(-ties if descending else ties, axis=1, kind="stable"))
