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

from .._lib import BOOK_BYTES
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
    if ctx._pending is not None:
        arrays["pending"] = (_np(ctx._pending), "uint8")
    cfg = KVCompCacheConfigStatic.config
    header = {
        "is_k": ctx.is_k, "batch_size": ctx.batch_size, "head_num": ctx.head_num, "head_dim": ctx.head_dim,
        "quant_scale_rel": ctx.quant_scale_rel, "quant_mode": ctx.quant_mode.value, "block_size": ctx.block_size,
        "recent_size": ctx.recent_size, "batch_shared": ctx.batch_shared,
        "min_dtype": str(ctx.min_dtype).replace("torch.", ""), "ctx_len": ctx.ctx_len,
        "compressed_ctx_len": ctx.compressed_ctx_len, "encoded_ctx_len": ctx.encoded_ctx_len,
        "max_block_bytes": ctx.max_block_bytes,
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
    min_dtype = getattr(torch, h["min_dtype"])
    # unit layout and min_int width are the file's, whatever the active configuration would pick
    ctx = KVCompCtx(h["is_k"], h["batch_size"], h["head_num"], h["head_dim"], h["quant_scale_rel"],
                    batch_shared=h["batch_shared"], min_dtype=min_dtype)
    if ctx.block_size != h["block_size"]:
        raise ValueError("the active configuration uses blocks of %d tokens, the file %d" % (ctx.block_size, h["block_size"]))
    ctx.device = torch.device(device)
    if ctx.device.type == "cuda" and ctx.device.index is None:
        ctx.device = torch.device("cuda", torch.cuda.current_device())
    ctx.ctx_len, ctx.compressed_ctx_len, ctx.max_block_bytes = h["ctx_len"], h["compressed_ctx_len"], h["max_block_bytes"]
    ctx.encoded_ctx_len = h.get("encoded_ctx_len", h["compressed_ctx_len"])

    # every section must hold what the header's token counts imply: a truncated or foreign file would
    # otherwise make the kernels index the tables out of bounds
    cols = h["batch_size"] * h["head_num"]
    Te, Tq = ctx.encoded_ctx_len, ctx.compressed_ctx_len
    nblk = (Te // 64) * cols if h["is_k"] else (Te // 128) * cols * 2
    row = cols * h["head_dim"]
    want = {"block_info": nblk * 8, "thread_info": nblk * 128,
            "min_int": ctx.spec.units(Tq, h["batch_size"], h["head_num"], h["head_dim"]) * min_dtype.itemsize,
            "scale": ctx.spec.units(Tq, h["batch_size"], h["head_num"], h["head_dim"]) * 2,
            "pending": (Tq - Te) * row, "buffer": h["buffer_tokens"] * row * 2}
    for name, size in want.items():
        have = raw[name][0].size if name in raw else 0
        if have != size:
            raise ValueError("%s: section %s holds %d bytes, the header implies %d" % (path, name, have, size))
    if Te and ("book" not in raw or raw["book"][0].size != BOOK_BYTES or "encoded" not in raw):
        raise ValueError("%s: codebook or stream missing" % path)
    if Te % (64 if h["is_k"] else 128) or Te > Tq or Tq + h["buffer_tokens"] != h["ctx_len"]:
        raise ValueError("%s: inconsistent token counts" % path)
    if nblk:
        rec = raw["block_info"][0].reshape(-1, 8)
        off = rec[:, 0:4].copy().view("<u4").reshape(-1).astype(np.int64)
        num = rec[:, 4:6].copy().view("<u2").reshape(-1).astype(np.int64)
        if int((off + num).max()) > raw["encoded"][0].size or int(num.max()) > max(int(h["max_block_bytes"]), 0):
            raise ValueError("%s: block_info points outside the stream" % path)

    def dev(name):
        a, dt = raw[name]
        return torch.from_numpy(a.copy()).to(ctx.device).view(getattr(torch, dt))
    if "book" in raw:
        ctx.book = Book(dev("book"))
    for name, attr in _SECTIONS[1:]:
        if name in raw:
            t = dev(name)
            arena = getattr(ctx, attr)
            if t.dtype != arena.dtype:
                raise ValueError("%s: section %s is %s, expected %s" % (path, name, t.dtype, arena.dtype))
            arena.buf, arena.n = t, t.numel()
    if "buffer" in raw:
        ctx.buffer = dev("buffer").view(h["buffer_tokens"], h["batch_size"], h["head_num"], h["head_dim"])
    if "pending" in raw:
        ctx._pending = dev("pending").view(Tq - Te, h["batch_size"], h["head_num"], h["head_dim"])
    return ctx
