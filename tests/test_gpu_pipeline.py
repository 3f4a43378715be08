"""Chunked host-buffer evaluation (kurumi_b200/pipeline.py): the result assembled from chunks of output rows,
with uploads, kernels and downloads overlapped, equals the single evaluation."""
import numpy as np
import pytest
import torch

from kurumi_b200 import api, configs, pipeline

pytestmark = pytest.mark.gpu


def pinned(arr: np.ndarray) -> torch.Tensor:
    t = torch.from_numpy(np.ascontiguousarray(arr).view(np.uint8).reshape(-1)).pin_memory()
    return t


@pytest.mark.parametrize("case", ["softmax_columns", "reduce_rows", "gemm_rows"])
def test_chunked_equals_single(cuda_lib, gpu, case):
    rng = np.random.default_rng(11)
    chunks = 4
    if case == "softmax_columns":
        n = 1024
        make = lambda g, c: configs.transposed_softmax(g, n=n, lines=n // c)
        arrays = [(rng.standard_normal((n, n)).astype(np.float32), api.F32, 1), (rng.uniform(-1, 1, n).astype(np.float32), api.F32, None)]
    elif case == "reduce_rows":
        make = lambda g, c: configs.fused_reduce(g, rows=512 // c, cols=768)
        arrays = [(rng.uniform(-1, 1, (512, 768)).astype(np.float32), api.F32, 0), (rng.uniform(-1, 1, (512, 768)).astype(np.float32), api.F32, 0)]
    else:
        make = lambda g, c: configs.gemm_bias_gelu(g, m=1024 // c, n=256, kdim=384)
        arrays = [(api.f32_to_bf16(rng.standard_normal((1024, 384)).astype(np.float32) * 0.05), api.BF16, 0),
                  (api.f32_to_bf16(rng.standard_normal((384, 256)).astype(np.float32) * 0.05), api.BF16, None),
                  (api.f32_to_bf16(rng.uniform(-0.1, 0.1, 256).astype(np.float32)), api.BF16, None)]
    # the single evaluation
    g1 = api.Graph(cuda_lib)
    root1, gens1 = make(g1, 1)
    feeds = api.Feeds(cuda_lib)
    for node, (a, dt, _) in zip(gens1, arrays):
        feeds.set(node, a, dt)
    whole = gpu.eval_with(g1, root1, feeds)
    want = whole.numpy()
    # the chunked evaluation from pinned host buffers
    gc = api.Graph(cuda_lib)
    rootc, gensc = make(gc, chunks)
    hosts = [pinned(a) for (a, _, _) in arrays]
    inputs = [pipeline.HostInput(node, h.data_ptr(), tuple(a.shape), dt, axis) for node, h, (a, dt, axis) in zip(gensc, hosts, arrays)]
    out_host = torch.zeros(want.nbytes, dtype=torch.uint8).pin_memory()
    rows = want.shape[0]
    pipe = pipeline.RowPipeline(gpu, gc, rootc, inputs, out_host.data_ptr(), rows, want.nbytes // rows, chunks)
    try:
        for _ in range(3):   # buffers, events and the compiled program are reused from step to step
            out_host.zero_()
            pipe.step()
            got = out_host.numpy().view(want.dtype).reshape(want.shape)
            if case == "softmax_columns":   # the slab and the square problem may select different softmax kernels
                np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-12)
            else:
                assert np.array_equal(got, want), case
    finally:
        pipe.close()


def test_uneven_split_is_refused(cuda_lib, gpu):
    g = api.Graph(cuda_lib)
    root, gens = configs.fused_reduce(g, rows=100, cols=64)
    x = torch.zeros(300 * 64 * 4, dtype=torch.uint8).pin_memory()
    inputs = [pipeline.HostInput(n, x.data_ptr(), (300, 64), api.F32, 0) for n in gens]
    out = torch.zeros(1200, dtype=torch.uint8).pin_memory()
    with pytest.raises(api.Error):
        pipeline.RowPipeline(gpu, g, root, inputs, out.data_ptr(), 300, 4, 7)
