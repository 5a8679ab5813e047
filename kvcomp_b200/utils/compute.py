"""Host-side counterparts of the reference's utils/compute.py that the cache classes need: the
QuantMode enum, RoPE on one tensor, None-tolerant concatenation and the block cutter.  The
quantiser itself is a CUDA kernel (kvcomp_b200.ops.quantize), not torch ops."""
from enum import Enum

import torch


class QuantMode(Enum):          # utils/compute.py:5-10
    BlockQuant = "BlockQuant"
    ChannelQuant = "ChannelQuant"
    TokenQuant = "TokenQuant"
    VectorQuant = "VectorQuant"


def rotate_half(x):             # utils/compute.py:12-16
    x1 = x[..., : x.shape[-1] // 2]
    x2 = x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


def apply_rotary_pos_emb_single(t, cos, sin, position_ids=None, unsqueeze_dim=1):   # utils/compute.py:25-33
    cos = cos.unsqueeze(unsqueeze_dim)
    sin = sin.unsqueeze(unsqueeze_dim)
    return (t * cos) + (rotate_half(t) * sin)


def safe_cat(t1, t2, dim):      # utils/compute.py:35-42
    if t1 is None and t2 is None:
        return None
    if t1 is None:
        return t2.clone()
    if t2 is None:
        return t1.clone()
    return torch.cat([t1, t2], dim=dim)


def cut_len(length, block_size, recent_size):
    """How many leading tokens of `length` buffered tokens get compressed
    (utils/compute.py:44-72: n = (len + blk - len % blk - recent) // blk blocks, clipped by the slice)."""
    n = (length + block_size - length % block_size - recent_size) // block_size
    return min(n * block_size, length) if n > 0 else 0


def cut_tensor_ctx_len_0(buffer, new_tensor, block_size, recent_size, dim=0):
    """utils/compute.py:59-72 for token-major tensors: returns (to_compress or None, remaining buffer)."""
    buffer = safe_cat(buffer, new_tensor, dim)
    n = cut_len(buffer.shape[0], block_size, recent_size)
    if n == 0:
        return None, buffer
    return buffer[:n], buffer[n:]
