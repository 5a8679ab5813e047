"""On-disk form of a compressed K or V cache (the reference only dumps raw fp16 tensors with torch.save,
evaluation/evaluation.py:248-273): one file holds everything a KVCompCtx needs to continue -- the
codebook blob, the stream with its block and vector tables, the quantisation metadata and the
uncompressed recent window.

    file := magic "KVCB200\\0" | u32 version | u64 header bytes | header (JSON, utf-8) | sections
    every section starts on a 64-byte boundary; the header lists them as name -> (offset, bytes, dtype)
"""
import json
import struct

import numpy as np
import torch

from ..ops import Book
from ..utils.compute import QuantMode
from ..utils.config import KVCompCacheConfig, KVCompCacheConfigStatic

MAGIC = b"KVCB200\0"
VERSION = 1
_SECTIONS = (("book", "book"), ("encoded", "_enc"), ("block_info", "_bi"), ("thread_info", "_ti"),
             ("min_int", "_mi"), ("scale", "_sc"))


def _np(t):
    return t.detach().cpu().contiguous().view(torch.uint8).numpy()


def save_ctx(ctx, path):
    """Write a KVCompCtx to `path`.  Synchronises (device -> host copies)."""
    arrays = {}
    if ctx.book is not None:
        arrays["book"] = (_np(ctx.book.blob), "uint8")
    for name, attr in _SECTIONS[1:]:
        used = getattr(ctx, attr).used()
        if used is not None and used.numel():
            arrays[name] = (_np(used), str(used.dtype).replace("torch.", ""))
    if ctx.buffer is not None and ctx.buffer.shape[0]:
        arrays["buffer"] = (_np(ctx.buffer), "float16")
    cfg = KVCompCacheConfigStatic.config
    header = {
        "is_k": ctx.is_k, "batch_size": ctx.batch_size, "head_num": ctx.head_num, "head_dim": ctx.head_dim,
        "quant_scale_rel": ctx.quant_scale_rel, "quant_mode": ctx.quant_mode.value, "block_size": ctx.block_size,
        "recent_size": ctx.recent_size, "batch_shared": ctx.batch_shared,
        "min_dtype": str(ctx.min_dtype).replace("torch.", ""), "ctx_len": ctx.ctx_len,
        "compressed_ctx_len": ctx.compressed_ctx_len, "max_block_bytes": ctx.max_block_bytes,
        "buffer_tokens": 0 if ctx.buffer is None else int(ctx.buffer.shape[0]), "config": str(cfg), "sections": {},
    }
    # two passes: the header's own length moves the section offsets
    for _ in range(2):
        blob = json.dumps(header).encode()
        off = (len(MAGIC) + 4 + 8 + len(blob) + 256 + 63) // 64 * 64      # slack for the offsets' digits
        for name, (a, dt) in arrays.items():
            header["sections"][name] = [off, int(a.size), dt]
            off = (off + a.size + 63) // 64 * 64
    blob = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(MAGIC + struct.pack("<IQ", VERSION, len(blob)) + blob)
        for name, (a, _) in arrays.items():
            f.seek(header["sections"][name][0])
            a.tofile(f)
    return header


def load_ctx(path, device="cuda"):
    """Rebuild a KVCompCtx from a file written by save_ctx (the global config is taken from the file when
    none is set)."""
    from .kvcomp_encode import KVCompCtx
    with open(path, "rb") as f:
        if f.read(8) != MAGIC:
            raise ValueError("%s is not a kvcomp_b200 cache file" % path)
        version, n = struct.unpack("<IQ", f.read(12))
        if version != VERSION:
            raise ValueError("unsupported file version %d" % version)
        h = json.loads(f.read(n).decode())
        raw = {}
        for name, (off, size, dt) in h["sections"].items():
            f.seek(off)
            raw[name] = (np.fromfile(f, dtype=np.uint8, count=size), dt)
    if KVCompCacheConfigStatic.config is None:
        KVCompCacheConfigStatic.config = KVCompCacheConfig.from_str(h["config"])
    cfg = KVCompCacheConfigStatic.config
    mode = cfg.k_quant_mode if h["is_k"] else cfg.v_quant_mode
    if mode != QuantMode(h["quant_mode"]):
        raise ValueError("the active configuration quantises %s with %s, the file holds %s" %
                         ("K" if h["is_k"] else "V", mode.value, h["quant_mode"]))
    ctx = KVCompCtx(h["is_k"], h["batch_size"], h["head_num"], h["head_dim"], h["quant_scale_rel"])
    ctx.device = torch.device(device)
    if ctx.device.type == "cuda" and ctx.device.index is None:
        ctx.device = torch.device("cuda", torch.cuda.current_device())
    ctx.batch_shared = h["batch_shared"]
    ctx.ctx_len, ctx.compressed_ctx_len, ctx.max_block_bytes = h["ctx_len"], h["compressed_ctx_len"], h["max_block_bytes"]

    def dev(name):
        a, dt = raw[name]
        return torch.from_numpy(a.copy()).to(ctx.device).view(getattr(torch, dt))
    if "book" in raw:
        ctx.book = Book(dev("book"))
    for name, attr in _SECTIONS[1:]:
        if name in raw:
            t = dev(name)
            arena = getattr(ctx, attr)
            arena.buf, arena.n = t, t.numel()
    if "buffer" in raw:
        ctx.buffer = dev("buffer").view(h["buffer_tokens"], h["batch_size"], h["head_num"], h["head_dim"])
    return ctx
