"""Multi-GPU partitioning of the decode-attention path: one process per GPU, torch.distributed for the
plumbing.  Every (layer, sequence, KV head) stream is independent, so the path shards without any
exchange of cache data:

  * by batch sequence -- each rank owns whole sequences; nothing is exchanged on the data path;
  * by KV head        -- each rank owns Hkv / world heads of every sequence and computes the outputs of
                         its query heads; one all-gather per step assembles [B, Hq, 128].
    The sharded cache is the single-GPU cache cut by head: BlockQuant / TokenQuant units span the heads
    (models/cache/kvcomp_encode.py:10-13, utils/compute.py:138-143), so at compression time the ranks
    exchange each unit's extremes (all-reduce min / max of one fp16 pair per unit) before they quantise,
    and the 256-bin code histogram (all-reduce sum, 2 KiB) before they build the codebook: every rank
    derives the same scale, min_int and book as one GPU holding all heads, and its stream holds that
    GPU's blocks for its columns.  Per-channel and per-vector units are head-local and need no exchange.
    Nothing of this is on the decode path.
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


def _world(group=None):
    return dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1


def reduce_extremes(mn, mx, group=None):
    """In place: the elementwise minimum of `mn` and maximum of `mx` over all ranks (per-unit extremes of a
    tensor whose heads are split over the ranks).  Exact: fp16 values are compared, never rounded."""
    if _world(group) == 1:
        return mn, mx
    if dist.get_backend(group) == "nccl":
        dist.all_reduce(mn, op=dist.ReduceOp.MIN, group=group)
        dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=group)
    else:                                   # gloo: reduce in fp32, which holds every fp16 value
        a, b = mn.float(), mx.float()
        dist.all_reduce(a, op=dist.ReduceOp.MIN, group=group)
        dist.all_reduce(b, op=dist.ReduceOp.MAX, group=group)
        mn.copy_(a.to(mn.dtype)); mx.copy_(b.to(mx.dtype))
    return mn, mx


def reduce_histogram(hist, group=None):
    """In place: the sum of the ranks' 256-bin code histograms, so that every rank builds the same codebook."""
    if _world(group) > 1:
        dist.all_reduce(hist, op=dist.ReduceOp.SUM, group=group)
    return hist


def quantize_head_shard(x, mode, block, rel, batch_shared, min_dtype, hist=None, group=None):
    """Quantise this rank's heads of a tensor (fp16 [T, B, H_local, D]) so that the result is the single-GPU
    result cut by head.  Returns what ops.quantize returns; `hist` receives this rank's code counts only
    (reduce_histogram joins them)."""
    from . import ops
    if mode in (ops.MODE_BLOCK, ops.MODE_TOKEN) and _world(group) > 1:
        mn, mx, _ = ops.quant_minmax(x, mode, block, batch_shared)
        reduce_extremes(mn, mx, group)
        return ops.quantize_ranged(x, mode, block, rel, mn, mx, batch_shared, min_dtype=min_dtype, hist=hist)
    return ops.quantize(x, mode, block, rel, batch_shared, min_dtype=min_dtype, hist=hist)


def build_shared_codebook(hist, group=None):
    """One codebook for all head shards of a (layer, K|V): joint histogram, same tree on every rank."""
    from . import ops
    return ops.build_codebook(reduce_histogram(hist, group))
