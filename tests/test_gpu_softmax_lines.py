"""ku_cuda_softmax_lines_f32 (the two-pass strided-line softmax on raw device pointers) against the
CPU oracle's evaluation of the same thing recorded as a graph: softmax(permute(L) + bias)."""
import numpy as np
import pytest

from kurumi_b200 import api
from tests import util

pytestmark = pytest.mark.gpu


def oracle_softmax_lines(oracle_lib, backend, L, bias):
    n_pos, ld = L.shape
    g = api.Graph(oracle_lib)
    Ln = g.input([n_pos, ld], api.F32)
    x = g.permute(Ln, [1, 0])
    f = api.Feeds(oracle_lib).set(Ln, L)
    if bias is not None:
        bn = g.input([n_pos], api.F32)
        x = g.add(x, g.broadcast_to(bn, [ld, n_pos]))
        f.set(bn, bias)
    return backend.eval_with(g, g.softmax(x, 1), f).numpy()


@pytest.mark.parametrize("lines,length,ld,with_bias", [(256, 512, 256, True), (100, 300, 100, True), (64, 1000, 96, False), (1024, 2048, 1024, True), (130, 257, 133, True)])
def test_softmax_lines_entry_point(oracle_lib, cpu, cpu64, gpu, lines, length, ld, with_bias):
    rng = np.random.default_rng(30)
    L = (rng.standard_normal((length, ld)) * 2).astype(np.float32)
    bias = rng.uniform(-1, 1, length).astype(np.float32) if with_bias else None
    d_in, d_out = gpu.upload(L), gpu.upload(np.zeros((lines, length), np.float32))
    d_bias = gpu.upload(bias) if with_bias else None
    gpu.softmax_lines(d_in, d_bias, d_out, lines, length, ld)
    got = d_out.numpy()
    want64 = oracle_softmax_lines(oracle_lib, cpu64, L, bias)[:lines]
    want32 = oracle_softmax_lines(oracle_lib, cpu, L, bias)[:lines]
    util.assert_close(want64, got, 1e-5, 1e-12, "vs f64 run")
    util.assert_close(want32, got, max(1e-5, length * 2.0 ** -24), 1e-9, "vs f32 oracle")
    assert np.abs(got.sum(axis=1) - 1).max() < 1e-4


def test_softmax_lines_special_values_and_errors(oracle_lib, cpu, gpu, cuda_lib):
    L = np.zeros((512, 64), np.float32)
    L[:, 0] = -np.inf; L[5, 0] = 0.0        # one finite entry in the line
    L[:, 1] = -np.inf                       # nothing finite: NaN, as the interpreter computes
    L[7, 2] = np.nan                        # NaN poisons its line
    L[:, 3] = np.linspace(-100, 80, 512)
    L[9, 4] = np.inf
    d_in, d_out = gpu.upload(L), gpu.upload(np.zeros((64, 512), np.float32))
    gpu.softmax_lines(d_in, None, d_out, 64, 512, 64)
    got = d_out.numpy()
    want = oracle_softmax_lines(oracle_lib, cpu, L, None)
    util.assert_close(want, got, 1e-5, 1e-30, "special values")
    with pytest.raises(api.Error, match="ld"):
        gpu.softmax_lines(d_in, None, d_out, 64, 512, 32)
