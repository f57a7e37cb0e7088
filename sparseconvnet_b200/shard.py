"""Data-parallel inference (and, at the end of this file, training): the minibatch shards by batch index, one
process per GPU.

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


class RowGather(object):
    """Gather of per-row results without staging copies: a preallocated buffer of
    ``world x capacity`` rows per step in flight; the last operator of the step (the linear head)
    writes this rank's rows straight into its own block (``block(n)``), and ``start(n)`` enqueues
    one collective on that buffer in place -- no padding copy, no zero fill.  Row counts travel on
    the host through `count_group` (see host_group) before anything is enqueued, so every rank sees
    the same counts and decides the same way: a count above the capacity raises ``ValueError`` on
    every rank instead of corrupting a neighbour's block, and a rank that never arrives ends the
    others' count exchange with the group's timeout, not with a hang on the GPU.

    `dst` = None: every rank receives all blocks (all_gather); `dst` = r: only rank r does (gather),
    the other ranks send their block and receive nothing.  `depth` buffers rotate, so a gather may
    still be running while the next step fills the next buffer."""

    def __init__(self, width, capacity, device, dtype=torch.float32, group=None, count_group=None, dst=None,
                 depth=2):
        self.group, self.count_group, self.dst = group, count_group, dst
        self.distributed = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
        self.world = dist.get_world_size(group) if self.distributed else 1
        self.rank = dist.get_rank(group) if self.distributed else 0
        self.capacity, self.width = int(capacity), int(width)
        receives = dst is None or dst == self.rank
        rows = self.world * self.capacity if receives else self.capacity
        self.buffers = [torch.empty(rows, self.width, dtype=dtype, device=device) for _ in range(depth)]
        self.receives = receives
        self.turn = 0

    def block(self, n):
        """View of this rank's block in the current buffer: write the step's `n` result rows here."""
        if n > self.capacity:
            raise ValueError("%d rows exceed the gather capacity of %d rows per rank" % (n, self.capacity))
        base = self.rank * self.capacity if self.receives else 0
        return self.buffers[self.turn][base:base + n]

    def start(self, n):
        """Enqueues the gather of the current buffer (this rank wrote `n` rows) and moves on to the next
        buffer.  Returns a PendingGather whose result() is (rows in rank order or None, counts)."""
        buf = self.buffers[self.turn]
        self.turn = (self.turn + 1) % len(self.buffers)
        if not self.distributed:
            return _Done(buf[:n], [n])
        if self.count_group is not None:
            parts = [torch.empty(1, dtype=torch.int64) for _ in range(self.world)]
            dist.all_gather(parts, torch.tensor([n], dtype=torch.int64), group=self.count_group)
            counts = torch.cat(parts).tolist()
        else:
            c = torch.empty(self.world, dtype=torch.int64, device=buf.device)
            dist.all_gather_into_tensor(c, torch.tensor([n], dtype=torch.int64, device=buf.device), group=self.group)
            counts = c.tolist()
        if max(counts) > self.capacity:  # every rank sees the same counts and raises together
            raise ValueError("a rank reported %d rows, the gather capacity is %d rows per rank"
                             % (max(counts), self.capacity))
        cap = self.capacity
        if self.dst is None:
            mine = buf[self.rank * cap:(self.rank + 1) * cap]
            work = dist.all_gather_into_tensor(buf, mine, group=self.group, async_op=True)
        elif self.receives:
            work = dist.gather(buf[self.rank * cap:(self.rank + 1) * cap],
                               [buf[r * cap:(r + 1) * cap] for r in range(self.world)],
                               dst=dist.get_global_rank(self.group, self.dst) if self.group is not None else self.dst,
                               group=self.group, async_op=True)
        else:
            work = dist.gather(buf, None,
                               dst=dist.get_global_rank(self.group, self.dst) if self.group is not None else self.dst,
                               group=self.group, async_op=True)
        return _PendingBlocks(buf if self.receives else None, counts, cap, work)


class _Done(object):
    def __init__(self, rows, counts):
        self.rows, self.counts = rows, counts

    def result(self):
        return self.rows, self.counts

    def blocks(self):
        return [self.rows], self.counts


class _PendingBlocks(object):
    def __init__(self, buf, counts, cap, work):
        self.buf, self.counts, self.cap, self.work = buf, counts, cap, work

    def wait(self):
        if self.work is not None:
            self.work.wait()
            self.work = None

    def blocks(self):
        """(list of per-rank views [n_r, width] or None on a rank that receives nothing, counts):
        no copy at all."""
        self.wait()
        if self.buf is None:
            return None, self.counts
        return [self.buf[r * self.cap:r * self.cap + c] for r, c in enumerate(self.counts)], self.counts

    def result(self):
        """(all ranks' rows concatenated in rank order, counts); one concatenation copy unless every
        block is full."""
        views, counts = self.blocks()
        if views is None:
            return None, counts
        if all(c == self.cap for c in counts):
            return self.buf, counts
        return torch.cat(views), counts


# ---- data-parallel training ----------------------------------------------------------------------
#
# Every rank runs forward and backward on its own samples.  Two things cross ranks: the training-mode
# BatchNorm statistics (share_batchnorm_statistics: one all-reduce of 2 x planes + 1 doubles per layer and
# direction) and the parameter gradients (sum_gradients: a few large all-reduces after the backward pass).
# With a loss that every rank divides by the TOTAL number of rows (or samples), the summed gradients are those
# of the whole batch on one device.  The reference has no multi-GPU path.

def share_batchnorm_statistics(module, group=None):
    """Every BatchNormalization layer under `module` takes its training-mode statistics over the rows of all
    ranks of `group` from now on (eval mode is unchanged: running statistics).  Returns `module`."""
    from .layers import BatchNormalization
    for m in module.modules():
        if isinstance(m, BatchNormalization):
            m.across_ranks = True
            m.ranks_group = group
    return module


def sum_gradients(parameters, group=None, bucket_bytes=64 << 20, scale=None):
    """Adds the gradients of `parameters` over the ranks of `group`, in place, through flat buckets of at most
    `bucket_bytes` (one all-reduce each, all enqueued before the first result is unpacked).  A parameter without
    a gradient on this rank (a rank whose shard was empty) counts as zeros and receives the sum, so that every
    rank packs the same layout; parameters that need no gradient are skipped.  `scale` multiplies the sums
    (1 / world for an average).  Returns the number of all-reduces."""
    params = [p for p in parameters if p.requires_grad]
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        if scale is not None:
            for p in params:
                if p.grad is not None:
                    p.grad.mul_(scale)
        return 0
    buckets, current, size = [], [], 0
    for p in params:
        nbytes = p.numel() * p.element_size()
        if current and (size + nbytes > bucket_bytes or p.dtype != current[0].dtype or p.device != current[0].device):
            buckets.append(current)
            current, size = [], 0
        current.append(p)
        size += nbytes
    if current:
        buckets.append(current)
    pending = []
    for bucket in buckets:
        flat = torch.cat([(p.grad if p.grad is not None else torch.zeros_like(p)).reshape(-1) for p in bucket])
        pending.append((bucket, flat, dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group, async_op=True)))
    for bucket, flat, work in pending:
        work.wait()
        if scale is not None:
            flat.mul_(scale)
        at = 0
        for p in bucket:
            part = flat[at:at + p.numel()].view_as(p)
            at += p.numel()
            if p.grad is None:
                p.grad = part.clone()
            else:
                p.grad.copy_(part)
    return len(buckets)
