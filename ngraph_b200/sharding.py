"""Batch sharding across GPUs: one process per GPU, every process runs the same compiled Function on its own
slice of the batch, and the only exchange is the gather of the outputs (NCCL on GPUs, gloo in the CPU tests).

nGraph's own multi-device story is a distributed all-reduce for training (src/ngraph/distributed.hpp); inference on
the quantized path has no cross-sample dependency, so the batch is the unit that shards."""
import torch
import torch.distributed as dist


def shard_bounds(n_items, world):
    """(counts, offsets): n_items split over `world` ranks as evenly as possible, the first ranks take the remainder."""
    if world <= 0 or n_items < 0:
        raise ValueError("shard_bounds: world must be positive and n_items non-negative")
    base, rem = divmod(n_items, world)
    counts = [base + (1 if r < rem else 0) for r in range(world)]
    offsets = [sum(counts[:r]) for r in range(world)]
    return counts, offsets


def local_slice(n_items, rank, world):
    counts, offsets = shard_bounds(n_items, world)
    return slice(offsets[rank], offsets[rank] + counts[rank])


def gather_rows(local, counts, group=None, out=None):
    """Every rank contributes `local` (its counts[rank] rows); every rank gets the concatenation in rank order.

    Equal shards use one all_gather_into_tensor; ragged shards are padded to the largest shard for the exchange and
    trimmed afterwards.  A single-process group returns `local` unchanged."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if len(counts) != world:
        raise ValueError("gather_rows: one count per rank expected")
    rank = dist.get_rank(group) if world > 1 else 0
    if local.shape[0] != counts[rank]:
        raise ValueError("gather_rows: this rank holds %d rows, its shard has %d" % (local.shape[0], counts[rank]))
    if world == 1:
        return local
    total, biggest = sum(counts), max(counts)
    tail = tuple(local.shape[1:])
    if min(counts) == biggest:
        if out is None:
            out = torch.empty((total,) + tail, dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(out, local.contiguous(), group=group)
        return out
    padded = torch.zeros((biggest,) + tail, dtype=local.dtype, device=local.device)
    padded[:counts[rank]] = local
    buf = torch.empty((world * biggest,) + tail, dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(buf, padded, group=group)
    pieces = [buf[r * biggest:r * biggest + counts[r]] for r in range(world)]
    res = torch.cat(pieces, dim=0)
    if out is not None:
        out.copy_(res)
        return out
    return res
