"""The N > 1 path on CPU: two gloo ranks each evaluate their row shard (with the CPU oracle standing in
for the device, since only the host-side sharding logic is under test), assemble with an all-gather
and compare with the unsharded evaluation."""
import os
import socket

import numpy as np
import pytest

from kurumi_b200 import shard


def test_row_ranges_cover_without_overlap():
    for n in (0, 1, 7, 8, 4096, 4097):
        for world in (1, 2, 3, 8):
            spans = [shard.row_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard.row_range(10, 2, 2)


def _worker(rank, world, port, rows, cols, out_dir):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from kurumi_b200 import api, build, configs
    olib = api.Library(build.ORACLE_LIB)
    cpu = api.Backend(olib, 0)
    rng = np.random.default_rng(7)
    x, y = (rng.uniform(-1, 1, (rows, cols)).astype(np.float32) for _ in range(2))   # same draw on every rank
    lo, hi = shard.row_range(rows, rank, world)
    g = api.Graph(olib)
    root, gens = configs.fused_reduce(g, hi - lo, cols)
    xn, yn = list(gens)
    f = api.Feeds(olib).set(xn, shard.shard_rows(x, rank, world)).set(yn, shard.shard_rows(y, rank, world))
    local = torch.from_numpy(cpu.eval_with(g, root, f).numpy().copy())
    full = shard.assemble(local, rows)
    # a 2-D result as well (softmax rows), with a bias replicated on every rank
    g2 = api.Graph(olib)
    xs = g2.input([hi - lo, cols], api.F32)
    bias = g2.input([cols], api.F32)
    sm = g2.softmax(g2.add(xs, g2.broadcast_to(bias, [hi - lo, cols])), 1)
    f2 = api.Feeds(olib).set(xs, shard.shard_rows(x, rank, world)).set(bias, y[0])
    full2 = shard.assemble(torch.from_numpy(cpu.eval_with(g2, sm, f2).numpy().copy()), rows)
    if rank == 0:
        np.save(os.path.join(out_dir, "sum.npy"), full.numpy())
        np.save(os.path.join(out_dir, "softmax.npy"), full2.numpy())
        np.save(os.path.join(out_dir, "x.npy"), x)
        np.save(os.path.join(out_dir, "y.npy"), y)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("rows", [64, 37])
def test_two_rank_sharded_evaluation_equals_unsharded(tmp_path, oracle_lib, cpu, rows):
    import torch.multiprocessing as mp
    from kurumi_b200 import api, configs
    cols = 96
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, rows, cols, str(tmp_path)), nprocs=2, join=True)
    x, y = np.load(tmp_path / "x.npy"), np.load(tmp_path / "y.npy")
    g = api.Graph(oracle_lib)
    root, gens = configs.fused_reduce(g, rows, cols)
    xn, yn = list(gens)
    want = cpu.eval_with(g, root, api.Feeds(oracle_lib).set(xn, x).set(yn, y)).numpy()
    assert np.array_equal(np.load(tmp_path / "sum.npy"), want)       # row shards are independent: bit-equal
    g2 = api.Graph(oracle_lib)
    xs, bias = g2.input([rows, cols], api.F32), g2.input([cols], api.F32)
    sm = g2.softmax(g2.add(xs, g2.broadcast_to(bias, [rows, cols])), 1)
    want2 = cpu.eval_with(g2, sm, api.Feeds(oracle_lib).set(xs, x).set(bias, y[0])).numpy()
    assert np.array_equal(np.load(tmp_path / "softmax.npy"), want2)


def test_chunk_plans_of_the_bench_build_row_slices(oracle_lib):
    """The end-to-end measurement cuts every workload into chunks of independent output rows: the chunk graph's
    result is exactly one chunk of rows of the full result, and its sharded inputs are one chunk of theirs."""
    import bench
    from kurumi_b200 import api
    for name, plan in bench.CHUNKING.items():
        builder, kw, _ = bench.WORKLOADS[name]
        small = {k: (v // 8 if isinstance(v, int) and v >= 1024 else v) for k, v in kw.items()}   # same structure, cheaper to record
        c = plan["chunks"]
        gf, gc = api.Graph(oracle_lib), api.Graph(oracle_lib)
        rf, gens_f = builder(gf, **small)
        rc, gens_c = builder(gc, **plan["chunk_kw"](small, c))
        sf, sc = gf.shape(rf), gc.shape(rc)
        assert sc[0] * c == sf[0] and sc[1:] == sf[1:], name
        assert len(plan["axes"]) == len(gens_f) == len(gens_c)
        for (nf, nc, axis) in zip(gens_f, gens_c, plan["axes"]):
            a, b = gf.shape(nf), gc.shape(nc)
            if axis is None:
                assert a == b, name
            else:
                assert b[axis] * c == a[axis] and all(x == y for i, (x, y) in enumerate(zip(a, b)) if i != axis), name
