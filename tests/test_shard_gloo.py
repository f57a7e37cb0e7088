"""The data-parallel driver logic on CPU: two gloo ranks shard a batch by sample index, each
runs the (oracle) forward on its shard, the per-row outputs are gathered, and the result must
equal the unsharded forward row for row."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port_no, tmp):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port_no)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import runner
    from sparseconvnet_b200 import shard
    from tests.golden import cases
    inp, net, head = cases.net_modules("net_unet3d")
    coords, feats = cases.net_inputs("net_unet3d")
    order = np.argsort(coords[:, -1], kind="stable")      # rows in batch order
    coords, feats = coords[order], feats[order]
    be = runner.PortBackend()
    c, f, (lo, hi) = shard.shard_batch(coords, feats, rank, world)
    assert c[:, -1].min() == 0 and set(np.unique(c[:, -1])) == set(range(hi - lo))
    y = runner.run_module(head, runner.run_module(net, runner.run_module(inp, [c, f], be), be), be)
    gathered, counts = shard.gather_rows(torch.from_numpy(y))
    assert counts[rank] == y.shape[0]
    # the same with the counts exchanged through a host group of their own (what the GPU driver uses)
    gathered2, counts2 = shard.gather_rows(torch.from_numpy(y), count_group=shard.host_group())
    assert counts2 == counts and torch.equal(gathered2, gathered)
    gathered3, counts3 = shard.gather_rows(torch.from_numpy(y), count_group=shard.host_group(), async_op=True).result()
    assert counts3 == counts and torch.equal(gathered3, gathered)
    # the copy-free form: the result is written straight into this rank's block of a preallocated buffer
    yt = torch.from_numpy(y)
    for dst in (None, 0, 1):
        rg = shard.RowGather(yt.shape[1], max(counts) + 3, "cpu", count_group=shard.host_group(), dst=dst)
        for _ in range(3):  # more steps than buffers
            rg.block(yt.shape[0]).copy_(yt)
            rows, counts4 = rg.start(yt.shape[0]).result()
            assert counts4 == counts
            if dst is None or dst == rank:
                assert torch.equal(rows, gathered)
            else:
                assert rows is None
    # a shard larger than the capacity is refused on every rank, before anything is enqueued
    small = shard.RowGather(yt.shape[1], min(counts), "cpu", count_group=shard.host_group())
    try:
        if yt.shape[0] <= small.capacity:
            small.block(yt.shape[0])
        small.start(yt.shape[0])
        refused = max(counts) <= min(counts)
    except ValueError:
        refused = True
    assert refused
    if rank == 0:
        full = runner.run_module(head, runner.run_module(net, runner.run_module(inp, [coords, feats], be), be), be)
        np.save(os.path.join(tmp, "ok.npy"), np.array([np.abs(gathered.numpy() - full).max(), full.shape[0],
                                                        gathered.shape[0]]))
    dist.barrier()
    dist.destroy_process_group()


def test_shard_ranges():
    sys.path.insert(0, ROOT)
    from sparseconvnet_b200 import shard
    assert [shard.shard_range(100, r, 8) for r in range(8)] == [(0, 13), (13, 26), (26, 39), (39, 52), (52, 64),
                                                                  (64, 76), (76, 88), (88, 100)]
    assert [shard.shard_range(8, r, 8) for r in range(8)] == [(r, r + 1) for r in range(8)]
    assert shard.shard_range(3, 5, 8) == (3, 3)      # more ranks than samples: empty shard


def test_two_rank_sharded_forward_equals_unsharded(tmp_path):
    port_no = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(2, port_no, str(tmp_path)), nprocs=2, join=True)
    err, n_full, n_gathered = np.load(os.path.join(str(tmp_path), "ok.npy"))
    assert n_full == n_gathered
    assert err <= 1e-6


def _failing_worker(rank, world, port_no, tmp):
    """Rank 1 raises before the gather; rank 0 must get a clean error from the count exchange within
    the group's timeout instead of waiting forever."""
    import datetime
    import time
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port_no)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    from sparseconvnet_b200 import shard
    rg = shard.RowGather(4, 16, "cpu", count_group=shard.host_group())
    rg.block(8).fill_(float(rank))
    rows, counts = rg.start(8).result()          # one healthy step
    assert counts == [8, 8]
    if rank == 1:
        os._exit(3)                               # the rank dies between steps, nothing in flight
    t0 = time.time()
    try:
        rg.block(8).fill_(1.0)
        rg.start(8).result()
        outcome = "no error"
    except Exception as e:                        # noqa: BLE001 -- any clean Python exception counts
        outcome = "error after %.1f s: %s" % (time.time() - t0, type(e).__name__)
    with open(os.path.join(tmp, "rank0.txt"), "w") as f:
        f.write(outcome)
    os._exit(0)


def test_rank_that_dies_gives_a_clean_error(tmp_path):
    port_no = 31500 + os.getpid() % 2000
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_failing_worker, args=(r, 2, port_no, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
        assert p.exitcode is not None, "a rank hung"
    assert procs[1].exitcode == 3
    with open(os.path.join(str(tmp_path), "rank0.txt")) as f:
        outcome = f.read()
    assert outcome.startswith("error after"), outcome
    assert float(outcome.split()[2]) < 30.0


def _gradient_worker(rank, world, port_no, tmp):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port_no)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from sparseconvnet_b200 import shard
    shapes = [(7, 5), (3,), (4, 4, 2), (11,), (2, 3)]
    params = [torch.nn.Parameter(torch.zeros(s)) for s in shapes]
    params[3].requires_grad_(False)                       # skipped altogether
    for i, p in enumerate(params):
        if p.requires_grad and not (rank == 1 and i == 1):  # rank 1 has no gradient for parameter 1 (empty shard)
            p.grad = torch.full(p.shape, float(10 * (rank + 1) + i))
    n = shard.sum_gradients(params, bucket_bytes=100)     # several buckets
    assert n >= 2
    for i, p in enumerate(params):
        if not p.requires_grad:
            assert p.grad is None
            continue
        want = (10 + i) + (0 if i == 1 else 20 + i)
        assert torch.equal(p.grad, torch.full(p.shape, float(want))), (i, p.grad)
    shard.sum_gradients(params, scale=0.5)                # one bucket, averaged
    assert torch.equal(params[0].grad, torch.full((7, 5), 30.0))
    if rank == 0:
        np.save(os.path.join(tmp, "grads_ok.npy"), np.array([1.0]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_sum_their_gradients(tmp_path):
    port_no = 31500 + os.getpid() % 2000
    mp.spawn(_gradient_worker, args=(2, port_no, str(tmp_path)), nprocs=2, join=True)
    assert os.path.exists(os.path.join(str(tmp_path), "grads_ok.npy"))
