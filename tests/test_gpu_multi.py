"""One evaluation sharded over two GPUs: each rank (a process of its own, one GPU each) evaluates the part graph of
ku_graph_row_split on its slices, the shards are assembled with the library's NCCL all-gather
(ku_cuda_all_gather_rows), and the assembled tensor equals the one-GPU evaluation bit for bit. Skipped when the box
shows fewer than two GPUs."""
import os
import subprocess
import sys
import time

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import os, sys, time
import numpy as np
sys.path.insert(0, sys.argv[1])
from kurumi_b200 import api, build, configs
rank, world, tmp = int(sys.argv[2]), int(sys.argv[3]), sys.argv[4]
lib = api.Library(build.LIB)
gpu = api.CudaBackend(lib, rank)
id_file = os.path.join(tmp, "nccl_id")
if rank == 0:
    uid = gpu.comm_unique_id()
    with open(id_file + ".tmp", "wb") as f:
        f.write(uid)
    os.replace(id_file + ".tmp", id_file)
else:
    t0 = time.time()
    while not os.path.exists(id_file):
        if time.time() - t0 > 60:
            raise SystemExit("no communicator id after 60 s")
        time.sleep(0.05)
    uid = open(id_file, "rb").read()
gpu.comm_init(uid, rank, world)
cases = [(configs.fused_reduce, dict(rows=512, cols=1024)), (configs.transposed_softmax, dict(n=1024)),
         (configs.gemm_bias_gelu, dict(m=512, n=512, kdim=256)), (configs.causal_attention, dict(batch=2, heads=2, seq=256, dh=128, fused=True)),
         (configs.fp8_weight_gemm, dict(m=512, kdim=256, n=512, amp=True))]
for i, (make, kw) in enumerate(cases):
    g = api.Graph(lib)
    root, gens = make(g, **kw)
    full = {}
    for node, mk in gens.items():            # the seeded inputs, generated whole on every rank
        h = api.Graph(lib)
        full[node] = gpu.eval_device(h, [mk(h)])[0]
    pg, proot, inputs = api.row_split(g, root, world)
    feeds = {}
    for orig, part, axis in inputs:          # this rank's slices, cut on the device
        t = full[orig]
        if axis is None:
            feeds[part] = t
        else:
            step = t.shape[axis] // world
            gs = api.Graph(lib)
            x = gs.input(list(t.shape), t.dtype)
            rng = [(0, d) for d in t.shape]
            rng[axis] = (rank * step, (rank + 1) * step)
            feeds[part] = gpu.eval_device(gs, [gs.slice(x, rng)], None, {x: t})[0]
    shard = gpu.eval_device(pg, [proot], None, feeds)[0]
    whole = gpu.all_gather_rows(shard)
    got = whole.numpy()
    if rank == 0:
        want = gpu.eval_device(g, [root], None, full)[0].numpy()
        assert got.shape == want.shape, (i, got.shape, want.shape)
        assert got.tobytes() == want.tobytes(), f"case {i}: the gathered result differs from the one-GPU evaluation"
    np.save(os.path.join(tmp, f"case{i}_rank{rank}.npy"), got.view(np.uint8) if got.dtype.itemsize == 1 else got)
gpu.sync()
gpu.comm_free()
print("rank", rank, "ok")
'''


def test_two_gpus_produce_one_result(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_DEBUG="WARN")
    procs = [subprocess.Popen([sys.executable, "-c", WORKER, ROOT, str(r), "2", str(tmp_path)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
             for r in range(2)]
    outs = []
    deadline = time.time() + 600
    for p in procs:
        try:
            o, _ = p.communicate(timeout=max(1, deadline - time.time()))
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        outs.append(o)
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {r} failed:\n{o[-3000:]}"
    for i in range(5):   # every rank holds the same assembled tensor
        a, b = np.load(tmp_path / f"case{i}_rank0.npy"), np.load(tmp_path / f"case{i}_rank1.npy")
        assert a.tobytes() == b.tobytes()
