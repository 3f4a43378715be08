"""One evaluation sharded over two GPUs: each rank (a process of its own, one GPU each) evaluates the part graph of
ku_graph_row_split on its slices, the shards are assembled with the library's NCCL all-gather
(ku_cuda_all_gather_rows), and the assembled tensor equals the one-GPU evaluation bit for bit (within the f32 band
for the softmax, whose shard may run another kernel). Skipped when the box
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
import torch   # brings the NCCL that torch ships into the process; the library uses the copy already loaded
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
print("rank", rank, "has the id", flush=True)
gpu.comm_init(uid, rank, world)
print("rank", rank, "joined", flush=True)
import traceback
def _die(kind, value, tb):
    traceback.print_exception(kind, value, tb)
    sys.stdout.flush(); sys.stderr.flush()
    os._exit(1)      # no teardown: the communicator's peers are still inside a collective
sys.excepthook = _die
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
        if make is configs.transposed_softmax:   # half the lines may take another softmax kernel (another summation order): the f32 band
            assert np.allclose(got, want, rtol=1e-5, atol=1e-12), f"case {i}: the gathered result is outside the f32 band of the one-GPU evaluation"
        else:
            assert got.tobytes() == want.tobytes(), f"case {i}: the gathered result differs from the one-GPU evaluation"
    np.save(os.path.join(tmp, f"case{i}_rank{rank}.npy"), got.view(np.uint8) if got.dtype.itemsize == 1 else got)
    print("rank", rank, "case", i, "done", flush=True)
gpu.sync()
gpu.comm_free()
print("rank", rank, "ok")
'''


def test_two_gpus_produce_one_result(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_DEBUG="WARN")
    logs = [open(tmp_path / f"rank{r}.log", "w+") for r in range(2)]
    procs = [subprocess.Popen([sys.executable, "-c", WORKER, ROOT, str(r), "2", str(tmp_path)], env=env, stdout=logs[r], stderr=subprocess.STDOUT, text=True)
             for r in range(2)]
    deadline = time.time() + 180
    while any(p.poll() is None for p in procs) and time.time() < deadline:
        if any(p.poll() not in (None, 0) for p in procs):   # a rank failed: its peers would wait for it in the next collective
            break
        time.sleep(0.2)
    late = [r for r, p in enumerate(procs) if p.poll() is None]
    for r in late:          # the exact processes started above
        procs[r].kill()
        procs[r].wait()
    outs = []
    for f in logs:
        f.seek(0)
        outs.append(f.read())
        f.close()
    failed = [r for r, p in enumerate(procs) if r not in late and p.returncode != 0]
    assert not failed and not late, f"ranks {failed} failed, ranks {late} were stopped:\n" + "\n----\n".join(o[-2000:] for o in outs)
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {r} failed:\n{o[-3000:]}"
    for i in range(5):   # every rank holds the same assembled tensor
        a, b = np.load(tmp_path / f"case{i}_rank0.npy"), np.load(tmp_path / f"case{i}_rank1.npy")
        assert a.tobytes() == b.tobytes()
