"""Data-parallel inference: the minibatch shards by batch index, one process per GPU.

Each rank keeps a contiguous range of samples, builds its own Metadata (site hash and
rulebooks never cross ranks: no operator mixes rows of different samples, and inference-mode
BatchNorm uses running statistics), and the per-row results are gathered at the end with one
collective.  The reference has no multi-GPU path; this follows its per-sample structure
(one hash map per sample, sparseconvnet/SCN/Metadata/Metadata.h:34)."""
import torch
import torch.distributed as dist


def shard_range(n_samples, rank, world):
    """Contiguous sample range [lo, hi) of `rank`: the first n % world ranks get one extra."""
    base, extra = divmod(int(n_samples), int(world))
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_batch(coords, features, rank, world, n_samples=None):
    """Rows of this rank's samples, batch index renumbered from 0.  coords [n, D+1] (last
    column = batch index) and features [n, C] are torch tensors or numpy arrays."""
    b = coords[:, -1]
    if n_samples is None:
        n_samples = int(b.max()) + 1 if len(b) else 0
    lo, hi = shard_range(n_samples, rank, world)
    keep = (b >= lo) & (b < hi)
    c = coords[keep].copy() if hasattr(coords, "copy") else coords[keep].clone()
    c[:, -1] -= lo
    return c, features[keep], (lo, hi)


_host_groups = {}


def host_group(group=None):
    """A gloo group over the ranks of `group`, made on first use (every rank must call this at the
    same point): row counts are exchanged through it, on the host."""
    key = id(group)
    if key not in _host_groups:
        ranks = None if group is None else dist.get_process_group_ranks(group)
        _host_groups[key] = dist.new_group(ranks=ranks, backend="gloo")
    return _host_groups[key]


class PendingGather(object):
    """A gather_rows(..., async_op=True) in flight: `result()` makes the current stream wait for the
    collective and returns what gather_rows returns."""

    def __init__(self, out, keep, counts, biggest, work):
        self.out, self.keep, self.counts, self.biggest, self.work = out, keep, counts, biggest, work

    def result(self):
        if self.work is not None:
            self.work.wait()
            self.work = None
        counts, biggest, out = self.counts, self.biggest, self.out
        if all(c == biggest for c in counts):
            return out, counts
        return torch.cat([out[r * biggest:r * biggest + counts[r]] for r in range(len(counts))]), counts


def gather_rows(rows, group=None, count_group=None, async_op=False):
    """All ranks' row blocks concatenated in rank order (= batch order when every rank's rows
    are in batch order).  Blocks may have different row counts: counts are exchanged first,
    blocks padded to the largest, gathered with one all_gather, and trimmed.
    `count_group` (see host_group): the counts, which every rank knows on the host, travel through
    this CPU group; nothing then waits for the GPU, so the launches of the next step keep running
    ahead.  Without it the counts go through `group` itself and are read back from the device,
    which waits for the stream.
    `async_op`: returns a PendingGather right after the collective has been enqueued; kernels
    launched afterwards (the next batch) run beside it.
    Returns (gathered [sum n_r, C], counts list)."""
    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        done = (rows, [rows.shape[0]])
        return PendingGather(rows, None, done[1], rows.shape[0], None) if async_op else done
    world = dist.get_world_size(group)
    if count_group is not None:
        n = torch.tensor([rows.shape[0]], dtype=torch.int64)
        parts = [torch.empty(1, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(parts, n, group=count_group)
        counts = torch.cat(parts)
    else:
        n = torch.tensor([rows.shape[0]], dtype=torch.int64, device=rows.device)
        counts = torch.empty(world, dtype=torch.int64, device=rows.device)
        dist.all_gather_into_tensor(counts, n, group=group)
    counts = counts.tolist()
    width = rows.shape[1:]
    biggest = max(counts)
    padded = rows
    if rows.shape[0] < biggest:
        padded = rows.new_zeros((biggest,) + tuple(width))
        padded[:rows.shape[0]] = rows
    padded = padded.contiguous()
    out = rows.new_empty((world * biggest,) + tuple(width))
    work = dist.all_gather_into_tensor(out, padded, group=group, async_op=async_op)
    pending = PendingGather(out, padded, counts, biggest, work if async_op else None)
    return pending if async_op else pending.result()
