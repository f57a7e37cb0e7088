"""Data-parallel training on two GPUs (one process each, NCCL): a training step whose batch is split by sample
over the ranks -- BatchNorm statistics shared (shard.share_batchnorm_statistics), parameter gradients summed
(shard.sum_gradients) -- gives the gradients and running statistics of the same step on the whole batch on one
device.  Needs two GPUs; skipped otherwise.

Tolerance: 1e-4 of the largest magnitude per tensor (fp32; the sums over rows are formed in another order)."""
import os
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOL = 1e-4


def _net(scn, cuda):
    torch.manual_seed(11)
    net = scn.Sequential().add(scn.SubmanifoldConvolution(3, 3, 8, 3, False)).add(
        scn.UNet(3, 1, [8, 16, 24], residual_blocks=True)).add(scn.BatchNormReLU(8)).to(cuda)
    head = torch.nn.Linear(8, 5).to(cuda)
    return net, head


def _step(scn, net, head, coords, feats, n_total, cuda):
    inp = scn.InputLayer(3, 64, mode=4)
    x = inp([torch.from_numpy(coords), torch.from_numpy(feats).to(cuda)])
    logits = head(net(x).features)
    sites = x.metadata.getSpatialLocations(x.spatial_size)
    labels = (sites[:, :3].sum(1) % 5).to(cuda)
    if n_total is None:
        n_total = logits.size(0)
    loss = torch.nn.functional.cross_entropy(logits, labels, reduction="sum") / n_total
    loss.backward()
    return logits.size(0), loss.detach()


def _rel(a, b):
    return (a - b).abs().max().item() / max(b.abs().max().item(), 1e-12)


def _worker(rank, world, port_no, tmp):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port_no)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    cuda = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=cuda)
    import sparseconvnet_b200 as scn
    from sparseconvnet_b200 import shard
    from tests.golden import cases
    coords, feats = cases.net_inputs("net_unet3d")
    order = np.argsort(coords[:, -1], kind="stable")
    coords, feats = coords[order], feats[order]
    n_samples = int(coords[:, -1].max()) + 1
    assert n_samples >= 2

    net, head = _net(scn, cuda)
    shard.share_batchnorm_statistics(net)
    net.train()
    c, f, _ = shard.shard_batch(coords, feats, rank, world, n_samples)
    # the number of sites of the whole batch: every rank's count, added
    inp = scn.InputLayer(3, 64, mode=4)
    mine = inp([torch.from_numpy(c), torch.from_numpy(f).to(cuda)]).features.size(0)
    count = torch.tensor([mine], dtype=torch.int64, device=cuda)
    dist.all_reduce(count)
    n_total = int(count.item())
    _step(scn, net, head, c, f, n_total, cuda)
    params = list(net.parameters()) + list(head.parameters())
    assert shard.sum_gradients(params) >= 1
    stats = [b.clone() for name, b in net.named_buffers() if "running" in name]

    # every rank ends with the same gradients and running statistics
    for t in [p.grad for p in params] + stats:
        other = t.clone()
        dist.broadcast(other, src=0)
        assert torch.equal(other, t)

    if rank == 0:
        one, one_head = _net(scn, cuda)
        one.train()
        n_one, _ = _step(scn, one, one_head, coords, feats, None, cuda)
        assert n_one == n_total
        worst = 0.0
        for p, q in zip(params, list(one.parameters()) + list(one_head.parameters())):
            assert q.grad is not None and p.grad is not None
            worst = max(worst, _rel(p.grad, q.grad))
        worst_stat = max(_rel(a, b) for a, b in zip(stats, [b for name, b in one.named_buffers() if "running" in name]))
        np.save(os.path.join(tmp, "two_ranks.npy"), np.array([worst, worst_stat, float(len(stats))]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_training_step_equals_one_device(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    port_no = 33500 + os.getpid() % 2000
    mp.spawn(_worker, args=(2, port_no, str(tmp_path)), nprocs=2, join=True)
    worst, worst_stat, n_stats = np.load(os.path.join(str(tmp_path), "two_ranks.npy"))
    assert n_stats > 0
    assert worst <= TOL and worst_stat <= TOL, (worst, worst_stat)
