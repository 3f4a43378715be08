"""The N > 1 path on CPU: two gloo ranks each evaluate the part graph of ku_graph_row_split on their slices (the
CPU oracle stands in for the device: the host-side sharding logic is under test), assemble with an all-gather and
compare with the unsharded evaluation, bit for bit."""
import os
import socket

import numpy as np
import pytest

from kurumi_b200 import shard


def test_slices_cover_without_overlap():
    a = np.arange(8 * 6).reshape(8, 6)
    for axis in (0, 1):
        for world in (1, 2):
            parts = [shard.slice_of(a, axis, r, world) for r in range(world)]
            assert np.array_equal(np.concatenate(parts, axis), a)
    assert shard.slice_of(a, None, 1, 2) is a
    with pytest.raises(ValueError):
        shard.slice_of(a, 0, 0, 3)


def _graphs(g, api, rows, cols):
    """Two row-separable graphs over (x [rows, cols], y [cols, rows], bias [cols]): a fused reduce, and a softmax read
    through a transpose with a replicated bias."""
    x, y, bias = g.input([rows, cols], api.F32), g.input([cols, rows], api.F32), g.input([cols], api.F32)
    r1 = g.sum(g.relu(g.add(g.mul(x, g.permute(y, [1, 0])), g.mul(g.scalar(x, 0.5), x))), 1)
    r2 = g.softmax(g.add(g.permute(y, [1, 0]), g.broadcast_to(bias, [rows, cols])), 1)
    return (x, y, bias), (r1, r2)


def _worker(rank, world, port, rows, cols, out_dir):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from kurumi_b200 import api, build
    olib = api.Library(build.ORACLE_LIB)
    cpu = api.Backend(olib, 0)
    rng = np.random.default_rng(7)   # same draw on every rank
    vals = [rng.uniform(-1, 1, (rows, cols)).astype(np.float32), rng.uniform(-1, 1, (cols, rows)).astype(np.float32), rng.uniform(-1, 1, cols).astype(np.float32)]
    g = api.Graph(olib)
    nodes, roots = _graphs(g, api, rows, cols)
    arrays = {n: (v, api.F32) for n, v in zip(nodes, vals)}
    for i, root in enumerate(roots):
        pg, proot, inputs = api.row_split(g, root, world)
        used = {o: arrays[o] for o, _, _ in inputs}
        local = cpu.eval_with(pg, proot, shard.part_feeds(olib, inputs, used, rank, world)).numpy().copy()
        full = shard.assemble_cpu(torch.from_numpy(local))
        if rank == 0:
            np.save(os.path.join(out_dir, f"root{i}.npy"), full.numpy())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("rows", [64, 38])
def test_two_rank_sharded_evaluation_equals_unsharded(tmp_path, oracle_lib, cpu, rows):
    import torch.multiprocessing as mp
    from kurumi_b200 import api
    cols, world = 48, 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(world, port, rows, cols, str(tmp_path)), nprocs=world, join=True)
    rng = np.random.default_rng(7)
    vals = [rng.uniform(-1, 1, (rows, cols)).astype(np.float32), rng.uniform(-1, 1, (cols, rows)).astype(np.float32), rng.uniform(-1, 1, cols).astype(np.float32)]
    g = api.Graph(oracle_lib)
    nodes, roots = _graphs(g, api, rows, cols)
    f = api.Feeds(oracle_lib)
    for n, v in zip(nodes, vals):
        f.set(n, v)
    for i, root in enumerate(roots):
        want = cpu.eval_with(g, root, f).numpy()
        got = np.load(tmp_path / f"root{i}.npy")
        assert got.shape == want.shape and got.tobytes() == want.tobytes()
