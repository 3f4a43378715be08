"""A graph that arrives as a KGPH v2 blob runs on the device like one recorded through the builders."""
import os

import numpy as np
import pytest

from kurumi_b200 import api, configs
from tests import util

pytestmark = pytest.mark.gpu

GOLDEN = bytes.fromhex(open(os.path.join(os.path.dirname(__file__), "golden", "graph_v2.kgph.hex")).read().strip())


def test_golden_blob_on_the_device(cuda_lib, gpu):
    g, entries = api.deserialize(cuda_lib, GOLDEN)
    np.testing.assert_array_equal(gpu.eval(g, entries[0][1][0]).numpy(), np.array([12.0, 21.0], np.float32))


def test_transposed_softmax_from_a_blob(oracle_lib, cuda_lib, cpu64, gpu):
    go = api.Graph(oracle_lib)
    root, gens = configs.transposed_softmax(go, n=1024)
    blob = go.serialize([root], [(n, 1, f"in{i}") for i, n in enumerate(gens)], reachable=True)
    gc, entries = api.deserialize(cuda_lib, blob)
    (_, outs, ins) = entries[0]
    fo, fc = api.Feeds(oracle_lib), api.Feeds(cuda_lib)
    cpu32 = api.Backend(oracle_lib, 0)
    for (node, _, _), (onode, mk) in zip(ins, gens.items()):
        h = api.Graph(oracle_lib)
        t = cpu32.eval(h, mk(h))
        fo.set(onode, t.numpy(), t.dtype)
        fc.set(node, t.numpy(), t.dtype)
    got = gpu.eval_with(gc, outs[0], fc).numpy()
    want = cpu64.eval_with(go, root, fo).numpy()
    util.assert_close(want, got, 1e-5, 1e-12, "softmax from a blob")
