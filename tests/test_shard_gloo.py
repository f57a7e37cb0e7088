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
