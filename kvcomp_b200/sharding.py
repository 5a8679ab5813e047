"""Multi-GPU partitioning of the decode-attention path: one process per GPU, torch.distributed for the
plumbing.  Every (layer, sequence, KV head) stream is independent, so the path shards without any
exchange of cache data:

  * by batch sequence -- each rank owns whole sequences; nothing is exchanged on the data path;
  * by KV head        -- each rank owns Hkv / world heads of every sequence and computes the outputs of
                         its query heads; one all-gather per step assembles [B, Hq, 128].
    K/V units that span heads (BlockQuant, TokenQuant with shared units) are then per shard, i.e. a rank's
    min/scale come from its own heads only; per-channel K units are head-local and unaffected.
"""
import torch
import torch.distributed as dist


def split_even(total, world, rank):
    """(start, count) of rank's contiguous share of `total` items; the first total % world ranks get one more."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("bad world/rank %d/%d" % (world, rank))
    base, extra = divmod(total, world)
    count = base + (1 if rank < extra else 0)
    start = rank * base + min(rank, extra)
    return start, count


def shard_batch(batch, world, rank):
    return split_even(batch, world, rank)


def shard_heads(kv_heads, q_heads, world, rank):
    """KV heads and the query heads that read them: (kv_start, kv_count, q_start, q_count)."""
    if kv_heads % world:
        raise ValueError("%d KV heads do not split over %d ranks" % (kv_heads, world))
    group = q_heads // kv_heads
    s, c = split_even(kv_heads, world, rank)
    return s, c, s * group, c * group


def gather_head_outputs(local, world, out=None):
    """local: [L, B, Hq_local, 128] (all layers of a step) -> [L, B, Hq, 128] on every rank (one all-gather)."""
    if world == 1:
        return local
    if dist.get_backend() == "nccl":
        L, B, Hl, D = local.shape
        buf = torch.empty((world, L, B, Hl, D), dtype=local.dtype, device=local.device) if out is None else out
        dist.all_gather_into_tensor(buf, local.contiguous())
        return buf.permute(1, 2, 0, 3, 4).reshape(L, B, world * Hl, D)
    parts = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(parts, local.contiguous())
    return torch.cat(parts, dim=2)


def max_over_ranks(values, device):
    """Element-wise maximum of a list of floats over all ranks (timings are the slowest rank's)."""
    t = torch.tensor(values, dtype=torch.float64, device=device)
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(x) for x in t]
