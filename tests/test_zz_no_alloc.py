"""ku_cuda_softmax_lines_f32_noalloc: the strided-line softmax for callers that cannot allocate device
memory at call time. Its scratch is a fixed array in the library's device image; the result must equal
what ku_cuda_softmax_lines_f32 (pool-allocated scratch, same kernels) produces. Collected last on
purpose: a failure here stops nothing else under `pytest -x`."""
import numpy as np
import pytest

from kurumi_b200 import api

pytestmark = pytest.mark.gpu


def run_both(gpu, L, bias, lines, length, ld):
    d_in = gpu.upload(L)
    d_bias = gpu.upload(bias) if bias is not None else None
    d_a, d_b = gpu.upload(np.zeros((lines, length), np.float32)), gpu.upload(np.full((lines, length), -1, np.float32))
    gpu.softmax_lines(d_in, d_bias, d_a, lines, length, ld)                                           # existing entry point
    gpu.softmax_lines(d_in, d_bias, d_b, lines, length, ld, entry="ku_cuda_softmax_lines_f32_noalloc")  # no allocation
    return d_a.numpy(), d_b.numpy()


def test_no_alloc_entry_matches_the_allocating_one_twice_in_a_row(gpu):
    rng = np.random.default_rng(50)
    # two calls in a row with different shapes: the second must not see anything of the first in the shared scratch
    for lines, length, ld, with_bias in ((1024, 2048, 1024, True), (300, 700, 333, False)):
        L = (rng.standard_normal((length, ld)) * 2).astype(np.float32)
        bias = rng.uniform(-1, 1, length).astype(np.float32) if with_bias else None
        want, got = run_both(gpu, L, bias, lines, length, ld)
        assert np.isfinite(got).all() and np.abs(got.sum(axis=1) - 1).max() < 1e-4
        np.testing.assert_allclose(got, want, rtol=1e-6, atol=0)   # same kernels, same order: in fact bit-identical
        assert np.array_equal(got, want)


def test_no_alloc_entry_rejects_sizes_beyond_its_fixed_scratch(gpu):
    d = gpu.upload(np.zeros(16, np.float32))
    with pytest.raises(api.Error, match="exceed the fixed"):
        gpu.softmax_lines(d, None, d, 16384, 16384, 16384, entry="ku_cuda_softmax_lines_f32_noalloc")
    with pytest.raises(api.Error, match="ld"):
        gpu.softmax_lines(d, None, d, 64, 64, 32, entry="ku_cuda_softmax_lines_f32_noalloc")
    # one line of 100 M positions would fit the scratch (6.25 MB) but not the launch grid: refused before anything is queued
    with pytest.raises(api.Error, match="65535"):
        gpu.softmax_lines(d, None, d, 1, 100_000_000, 1, entry="ku_cuda_softmax_lines_f32_noalloc")
    with pytest.raises(api.Error, match="65535"):
        gpu.softmax_lines(d, None, d, 1, 100_000_000, 1)


def test_calls_after_the_warm_up_leave_device_memory_alone(gpu):
    """The first call on a device places the kernels and the scratch array (lazy loading); from then on a call changes
    nothing about the device's free memory."""
    from cuda.bindings import runtime as cudart
    rng = np.random.default_rng(51)
    L = rng.standard_normal((512, 256)).astype(np.float32)
    d_in, d_out = gpu.upload(L), gpu.upload(np.zeros((256, 512), np.float32))
    gpu.softmax_lines(d_in, None, d_out, 256, 512, 256, entry="ku_cuda_softmax_lines_f32_noalloc")   # the warm-up call
    gpu.sync()
    err, free0, _ = cudart.cudaMemGetInfo()
    assert int(err) == 0
    for _ in range(3):
        gpu.softmax_lines(d_in, None, d_out, 256, 512, 256, entry="ku_cuda_softmax_lines_f32_noalloc")
    gpu.sync()
    err, free1, _ = cudart.cudaMemGetInfo()
    assert int(err) == 0 and free1 == free0
