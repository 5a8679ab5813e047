"""torch-facing wrappers over the C ABI: tensors in, tensors out, launches on the current stream.

PyTorch is only the carrier of device memory and streams here; every computation is a kernel of
libkvcomp_b200.so.  Every function raises when the tensors are not CUDA tensors: there is no CPU path.
"""
import ctypes as C
from dataclasses import dataclass

import torch

from . import _lib
from ._lib import (BOOK_BYTES, BOOK_OFF_ENC, BOOK_OFF_REFTREE, MODE_BLOCK, MODE_CHANNEL, MODE_TOKEN,
                   MODE_VECTOR, Cache, KvcError, QMeta)

MODES = {"BlockQuant": MODE_BLOCK, "ChannelQuant": MODE_CHANNEL, "TokenQuant": MODE_TOKEN,
         "VectorQuant": MODE_VECTOR}


# The current device and stream are asked for at every call (a caller may switch either), through the
# interpreter's direct entries where this torch has them: the public context manager and stream object cost
# some ten microseconds per call, as much as the rest of a call's host work.
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_get_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    if _raw_stream is not None and _get_device is not None:
        return C.c_void_p(_raw_stream(_get_device()))
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


class _on:
    """`with _on(device):` makes the tensor's device current for the call, switching only when it is not."""
    __slots__ = ("idx", "prev")

    def __init__(self, device):
        self.idx = device.index if isinstance(device, torch.device) else torch.device(device).index

    def __enter__(self):
        self.prev = _get_device() if _get_device is not None else torch.cuda.current_device()
        if self.idx is not None and self.idx != self.prev:
            torch.cuda.set_device(self.idx)
        return self

    def __exit__(self, *exc):
        if self.idx is not None and self.idx != self.prev:
            torch.cuda.set_device(self.prev)
        return False


def _cuda(t, dtype, name):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KvcError("%s must be a CUDA tensor (kvcomp_b200 has no CPU path)" % name)
    if dtype is not None and t.dtype != dtype:
        raise KvcError("%s must be %s, got %s" % (name, dtype, t.dtype))
    if not t.is_contiguous():
        raise KvcError("%s must be contiguous" % name)
    return t


def _p(t):
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)


def new_status(device):
    """A zeroed device status word; kernels OR KVC_FLAG_* bits into it."""
    return torch.zeros(1, dtype=torch.int32, device=device)


def read_status(status, raise_on_fatal=True, what="kvcomp_b200"):
    """Synchronising read of a status word."""
    v = int(status.item())
    if raise_on_fatal and (v & _lib.FATAL_FLAGS):
        raise KvcError("%s: device reported %s" % (what, "|".join(_lib.flag_names(v))))
    return v


@dataclass
class QSpec:
    """Unit layout of a (min_int, scale) pair: unit = (t // tok_div)*sj + b*sb + h*sh + c*sc."""
    mode: int
    batch_shared: bool
    block: int
    tok_div: int
    sj: int
    sb: int
    sh: int
    sc: int

    def units(self, T, B, H, D):
        """Number of units of T tokens."""
        return (T // self.tok_div) * self.sj if self.sj else 0

    def qmeta(self, min_int, scale):
        return QMeta(min_int.data_ptr(), scale.data_ptr(), min_int.element_size(), self.tok_div,
                     self.sj, self.sb, self.sh, self.sc)


def qspec(mode, batch_shared, B, H, D, block):
    lib = _lib.load()
    q = QMeta()
    n = C.c_int64(0)
    T = block if mode in (MODE_BLOCK, MODE_CHANNEL) else 1
    _lib.check(lib.kvc_qmeta_make(mode, int(batch_shared), T, B, H, D, block, C.byref(q), C.byref(n)), "kvc_qmeta_make")
    return QSpec(mode, bool(batch_shared), int(block), q.tok_div, q.sj, q.sb, q.sh, q.sc)


def buffer_sizes(tokens, hidden, is_k):
    out = (C.c_int64 * 4)()
    _lib.check(_lib.load().kvc_buffer_sizes(tokens, hidden, int(is_k), out), "kvc_buffer_sizes")
    return tuple(int(v) for v in out)


def quantize(x, mode, block, rel, batch_shared=True, min_dtype=torch.int8, hist=None, status=None,
             codes=None, min_int=None, scale=None):
    """x: fp16 [T,B,H,D] -> (codes u8 [T,B,H,D], min_int [units], scale fp16 [units], QSpec, status)."""
    lib = _lib.load()
    _cuda(x, torch.float16, "x")
    if x.dim() != 4:
        raise KvcError("x must be [T,B,H,D]")
    T, B, H, D = x.shape
    spec = qspec(mode, batch_shared, B, H, D, block)
    if mode in (MODE_BLOCK, MODE_CHANNEL) and T % block:
        raise KvcError("T=%d is not a multiple of block=%d" % (T, block))
    n = spec.units(T, B, H, D)
    dev = x.device
    codes = torch.empty((T, B, H, D), dtype=torch.uint8, device=dev) if codes is None else _cuda(codes, torch.uint8, "codes")
    min_int = torch.empty(n, dtype=min_dtype, device=dev) if min_int is None else _cuda(min_int, None, "min_int")
    scale = torch.empty(n, dtype=torch.float16, device=dev) if scale is None else _cuda(scale, torch.float16, "scale")
    if min_int.dtype not in (torch.int8, torch.int16) or min_int.numel() < n or scale.numel() < n:
        raise KvcError("min_int must be int8/int16 and hold %d units" % n)
    status = new_status(dev) if status is None else status
    ws_bytes = lib.kvc_quantize_workspace(mode, int(batch_shared), T, B, block)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)
    if hist is not None:
        _cuda(hist, torch.int64, "hist")
    with _on(dev):
        _lib.check(lib.kvc_quantize(_p(x), T, B, H, D, mode, int(batch_shared), block, float(rel), _p(codes),
                                    _p(min_int), min_int.element_size(), _p(scale), _p(hist), _p(ws), ws.numel(),
                                    _p(status), _stream()), "kvc_quantize")
    return codes, min_int, scale, spec, status


def quant_minmax(x, mode, block, batch_shared=True):
    """Per-unit extremes of x (fp16 [T,B,H,D]) for BlockQuant / TokenQuant units: (min fp16 [units], max
    fp16 [units], QSpec).  First half of the two-call quantiser (kvc_quant_minmax)."""
    lib = _lib.load()
    _cuda(x, torch.float16, "x")
    T, B, H, D = x.shape
    spec = qspec(mode, batch_shared, B, H, D, block)
    n = spec.units(T, B, H, D)
    mn = torch.empty(n, dtype=torch.float16, device=x.device)
    mx = torch.empty(n, dtype=torch.float16, device=x.device)
    ws = torch.empty(max(8 * n, 16), dtype=torch.uint8, device=x.device)
    with _on(x.device):
        _lib.check(lib.kvc_quant_minmax(_p(x), T, B, H, D, mode, int(batch_shared), block, _p(mn), _p(mx), _p(ws),
                                        ws.numel(), _stream()), "kvc_quant_minmax")
    return mn, mx, spec


def quantize_ranged(x, mode, block, rel, mn, mx, batch_shared=True, min_dtype=torch.int8, hist=None, status=None):
    """Second half: quantise x with the given per-unit extremes (the joint ones of all head shards).
    Returns what quantize returns."""
    lib = _lib.load()
    _cuda(x, torch.float16, "x")
    _cuda(mn, torch.float16, "mn")
    _cuda(mx, torch.float16, "mx")
    T, B, H, D = x.shape
    spec = qspec(mode, batch_shared, B, H, D, block)
    n = spec.units(T, B, H, D)
    if mn.numel() != n or mx.numel() != n:
        raise KvcError("extremes must hold %d units" % n)
    dev = x.device
    codes = torch.empty((T, B, H, D), dtype=torch.uint8, device=dev)
    min_int = torch.empty(n, dtype=min_dtype, device=dev)
    scale = torch.empty(n, dtype=torch.float16, device=dev)
    status = new_status(dev) if status is None else status
    ws = torch.empty(max(8 * n, 16), dtype=torch.uint8, device=dev)
    if hist is not None:
        _cuda(hist, torch.int64, "hist")
    with _on(dev):
        _lib.check(lib.kvc_quantize_ranged(_p(x), T, B, H, D, mode, int(batch_shared), block, float(rel), _p(mn), _p(mx),
                                           _p(codes), _p(min_int), min_int.element_size(), _p(scale), _p(hist), _p(ws),
                                           ws.numel(), _p(status), _stream()), "kvc_quantize_ranged")
    return codes, min_int, scale, spec, status


def rope_store(x, cos, sin, out=None):
    """New keys x fp16 [B, H, t, D] rotated (t * cos + rotate_half(t) * sin in fp16, as torch evaluates it) and
    laid out token-major: fp16 [t, B, H, D].  cos / sin: fp16 [B, t, D] or [1, t, D]; both None: no rotation,
    the transposition alone (new values).  out: where the rows go (a row range of the recent window)."""
    lib = _lib.load()
    _cuda(x, torch.float16, "key_states")
    B, H, t, D = x.shape
    stride = 0
    if cos is not None:
        cos, sin = _cuda(cos.contiguous(), torch.float16, "cos"), _cuda(sin.contiguous(), torch.float16, "sin")
        if cos.shape != sin.shape or cos.dim() != 3 or cos.shape[1:] != (t, D) or cos.shape[0] not in (1, B):
            raise KvcError("cos / sin must be [B, t, D] or [1, t, D], got %s" % (tuple(cos.shape),))
        stride = 0 if cos.shape[0] == 1 and B > 1 else t * D
    out = torch.empty((t, B, H, D), dtype=torch.float16, device=x.device) if out is None else _cuda(out, torch.float16, "out")
    if tuple(out.shape) != (t, B, H, D):
        raise KvcError("out must be [t, B, H, D] = %s, got %s" % ((t, B, H, D), tuple(out.shape)))
    with _on(x.device):
        _lib.check(lib.kvc_rope_store(_p(x), _p(cos), _p(sin), _p(out), B, H, t, D, stride, _stream()), "kvc_rope_store")
    return out


def kv_store(k, v, cos, sin, kout, vout):
    """rope_store for the new keys (rotated) and the new values (not rotated) in one launch: k, v fp16
    [B, H, t, D] -> kout, vout fp16 [t, B, H, D] (row ranges of the recent windows)."""
    lib = _lib.load()
    _cuda(k, torch.float16, "key_states")
    _cuda(v, torch.float16, "value_states")
    B, H, t, D = k.shape
    cos, sin = _cuda(cos.contiguous(), torch.float16, "cos"), _cuda(sin.contiguous(), torch.float16, "sin")
    if cos.shape != sin.shape or cos.dim() != 3 or cos.shape[1:] != (t, D) or cos.shape[0] not in (1, B):
        raise KvcError("cos / sin must be [B, t, D] or [1, t, D], got %s" % (tuple(cos.shape),))
    if tuple(v.shape) != (B, H, t, D) or tuple(kout.shape) != (t, B, H, D) or tuple(vout.shape) != (t, B, H, D):
        raise KvcError("kv_store: k, v must be [B, H, t, D] and kout, vout [t, B, H, D]")
    _cuda(kout, torch.float16, "kout")
    _cuda(vout, torch.float16, "vout")
    with _on(k.device):
        _lib.check(lib.kvc_kv_store(_p(k), _p(v), _p(cos), _p(sin), _p(kout), _p(vout), B, H, t, D,
                                    0 if cos.shape[0] == 1 and B > 1 else t * D, _stream()), "kvc_kv_store")


def dequant(codes, min_int, scale, spec, out=None):
    lib = _lib.load()
    _cuda(codes, torch.uint8, "codes")
    T, B, H, D = codes.shape
    out = torch.empty((T, B, H, D), dtype=torch.float16, device=codes.device) if out is None else out
    q = spec.qmeta(_cuda(min_int, None, "min_int"), _cuda(scale, torch.float16, "scale"))
    with _on(codes.device):
        _lib.check(lib.kvc_dequant(_p(codes), C.byref(q), T, B, H, D, _p(out), _stream()), "kvc_dequant")
    return out


def histogram(codes, hist=None):
    """hist (int64[256], device) += bincount(codes)."""
    lib = _lib.load()
    _cuda(codes, torch.uint8, "codes")
    hist = torch.zeros(256, dtype=torch.int64, device=codes.device) if hist is None else _cuda(hist, torch.int64, "hist")
    with _on(codes.device):
        _lib.check(lib.kvc_histogram(_p(codes), codes.numel(), _p(hist), _stream()), "kvc_histogram")
    return hist


class Book:
    """A device codebook blob (encode table, reference-format decode tree, decode tables)."""

    def __init__(self, blob):
        self.blob = blob
        self._host = None

    @property
    def device(self):
        return self.blob.device

    def host(self):
        """Synchronising copy of the blob to the host (cached)."""
        if self._host is None:
            self._host = self.blob.cpu()
        return self._host

    def header(self):
        h = self.host()[:32].view(torch.int32).tolist()
        return dict(n_symbols=h[0], min_sym=h[1], max_sym=h[2], max_len=h[3], n_nodes=h[4], flags=h[5], lut_bits=h[6],
                    escape=h[7])

    def encode_table(self):
        """uint8 view of the 256-entry symbol-indexed {u32 code, u32 length} table (device)."""
        return self.blob[BOOK_OFF_ENC:BOOK_OFF_ENC + 2048]

    def ref_encode_tensor(self):
        """(shift, CPU uint8 tensor): the encode tensor of the reference's build_codebook."""
        hd = self.header()
        lo, hi = hd["min_sym"], hd["max_sym"]
        return lo, self.host()[BOOK_OFF_ENC + 8 * lo: BOOK_OFF_ENC + 8 * (hi + 1)].clone()

    def ref_decode_tensor(self):
        """CPU uint8 tensor: the decode tensor of the reference's build_codebook (3-byte nodes)."""
        n = self.header()["n_nodes"]
        return self.host()[BOOK_OFF_REFTREE: BOOK_OFF_REFTREE + 3 * n].clone()


def build_codebook(hist):
    lib = _lib.load()
    _cuda(hist, torch.int64, "hist")
    blob = torch.empty(BOOK_BYTES, dtype=torch.uint8, device=hist.device)
    with _on(hist.device):
        _lib.check(lib.kvc_build_codebook(_p(hist), _p(blob), _stream()), "kvc_build_codebook")
    return Book(blob)


def book_from_tree(ref_tree):
    lib = _lib.load()
    _cuda(ref_tree, torch.uint8, "decode_code_book")
    blob = torch.empty(BOOK_BYTES, dtype=torch.uint8, device=ref_tree.device)
    with _on(ref_tree.device):
        _lib.check(lib.kvc_book_from_tree(_p(ref_tree), ref_tree.numel(), _p(blob), _stream()), "kvc_book_from_tree")
    return Book(blob)


def encode(codes, is_k, enc_table, block_info, thread_info, encoded, base_offset=0, status=None, total=None):
    """codes u8 [T,B,H,128] -> writes block_info (u8, 8 B per block), thread_info (2 B per vector) and
    encoded (u8) in place; returns (total, status) where total is a device int64[2]: [0] the byte count
    of this call, [1] the largest block byte count (a running maximum when `total` is passed in again).
    enc_table: device uint8 tensor of {u32 code, u32 length} entries indexed by symbol."""
    lib = _lib.load()
    _cuda(codes, torch.uint8, "codes")
    T, B, H, D = codes.shape
    if D != 128:
        raise KvcError("head_dim must be 128")
    cols = B * H
    dev = codes.device
    status = new_status(dev) if status is None else status
    total = torch.zeros(2, dtype=torch.int64, device=dev) if total is None else total
    ws = torch.empty(max(lib.kvc_encode_workspace(T, cols, int(is_k)), 16), dtype=torch.uint8, device=dev)
    _cuda(enc_table, torch.uint8, "encode_code_book")
    for t, n in ((block_info, "block_infos"), (thread_info, "thread_infos"), (encoded, "encoded_data")):
        _cuda(t, None, n)
    nblk = (T // 64) * cols if is_k else (T // 128) * cols * 2
    if block_info.numel() * block_info.element_size() < nblk * 8 or \
            thread_info.numel() * thread_info.element_size() < nblk * 128:
        raise KvcError("block_infos / thread_infos too small for %d blocks" % nblk)
    with _on(dev):
        _lib.check(lib.kvc_encode(_p(codes), T, cols, int(is_k), _p(enc_table), enc_table.numel() // 8,
                                  int(base_offset), _p(block_info), _p(thread_info), _p(encoded),
                                  encoded.numel(), _p(total), _p(ws), ws.numel(), _p(status), _stream()), "kvc_encode")
    return total, status


def decode(encoded, block_info, thread_info, book, T, B, H, is_k, out=None, status=None, max_block=0):
    """Huffman-decode a stream to its uint8 codes [T,B,H,128].  max_block: the stream's largest block in
    bytes as the encoder reported it (0 = unknown); a known bound lets more CTAs share an SM."""
    lib = _lib.load()
    _cuda(encoded, torch.uint8, "encoded")
    dev = encoded.device
    out = torch.empty((T, B, H, 128), dtype=torch.uint8, device=dev) if out is None else _cuda(out, torch.uint8, "out")
    status = new_status(dev) if status is None else status
    with _on(dev):
        _lib.check(lib.kvc_decode_bounded(_p(encoded), encoded.numel(), _p(block_info), _p(thread_info), _p(book.blob),
                                          T, B * H, int(is_k), int(max_block), _p(out), _p(status), _stream()), "kvc_decode")
    return out, status


def make_cache(encoded, block_info, thread_info, book, min_int, scale, spec, encoded_bytes=None, max_block_bytes=0):
    """The kvc_cache argument of the fused kernels.  The tensors must stay alive during the call."""
    n = encoded.numel() if encoded_bytes is None else int(encoded_bytes)
    return Cache(encoded.data_ptr(), n, block_info.data_ptr(), thread_info.data_ptr(), book.blob.data_ptr(),
                 spec.qmeta(min_int, scale), int(max_block_bytes), 0)


def fused_qk(cache, T, B, Hkv, q, out=None, out_dtype=torch.float16, status=None):
    """q fp16 [B,Hq,128] -> raw scores [B,Hq,T]."""
    lib = _lib.load()
    _cuda(q, torch.float16, "q")
    Hq = q.shape[1]
    out = torch.empty((B, Hq, T), dtype=out_dtype, device=q.device) if out is None else _cuda(out, None, "C")
    if out.dtype not in (torch.float16, torch.float32):
        raise KvcError("scores must be fp16 or fp32")
    status = new_status(q.device) if status is None else status
    with _on(q.device):
        _lib.check(lib.kvc_fused_qk(C.byref(cache), T, B, Hkv, Hq, _p(q), _p(out), int(out.dtype == torch.float32),
                                    _p(status), _stream()), "kvc_fused_qk")
    return out, status


def fused_pv(cache, T, B, Hkv, P, out=None, status=None):
    """P fp16 [B,Hq,T] -> per-group partials fp16 [T/128, B, Hq, 128]."""
    lib = _lib.load()
    _cuda(P, torch.float16, "P")
    Hq = P.shape[1]
    out = torch.empty((T // 128, B, Hq, 128), dtype=torch.float16, device=P.device) if out is None else _cuda(out, torch.float16, "C")
    status = new_status(P.device) if status is None else status
    with _on(P.device):
        _lib.check(lib.kvc_fused_pv(C.byref(cache), T, B, Hkv, Hq, _p(P), _p(out), _p(status), _stream()), "kvc_fused_pv")
    return out, status


def attn_splits(T, B, Hkv):
    return int(_lib.load().kvc_attn_splits(T, B, Hkv, 0))


def attn_workspace(B, Hq, splits, device):
    """Zeroed workspace for attn_decode with up to `splits` splits (reusable across calls)."""
    n = _lib.load().kvc_attn_workspace(B, Hq, splits)
    return torch.zeros(n, dtype=torch.uint8, device=device)


def attn_decode(kcache, vcache, T, B, Hkv, q, scaling, ktail=None, vtail=None, out=None, splits=0,
                workspace=None, status=None):
    """One decode step: q fp16 [B,Hq,128] -> out fp16 [B,Hq,128] over T compressed (+ tail) tokens."""
    lib = _lib.load()
    _cuda(q, torch.float16, "q")
    Hq = q.shape[1]
    dev = q.device
    out = torch.empty((B, Hq, 128), dtype=torch.float16, device=dev) if out is None else _cuda(out, torch.float16, "out")
    status = new_status(dev) if status is None else status
    Tr = 0
    if ktail is not None and ktail.shape[0] > 0:
        _cuda(ktail, torch.float16, "ktail")
        _cuda(vtail, torch.float16, "vtail")
        Tr = ktail.shape[0]
    else:
        ktail = vtail = None
    # splits <= 0: the tiles of all (sequence, KV head) columns are shared evenly among the CTAs that
    # fit the device (attn_splits = partial results per head to leave room for); splits > 0: every
    # column is cut into that many equal parts.
    if workspace is None:
        workspace = attn_workspace(B, Hq, splits if splits > 0 else attn_splits(T, B, Hkv), dev)
    elif workspace is False:        # no workspace at all (splits must be 1): the CTAs take fixed shares of the columns
        workspace = torch.empty(0, dtype=torch.uint8, device=dev)
    with _on(dev):
        _lib.check(lib.kvc_attn_decode(C.byref(kcache) if kcache is not None else None,
                                       C.byref(vcache) if vcache is not None else None, T, B, Hkv, Hq, _p(q), float(scaling),
                                       _p(ktail), _p(vtail), Tr, _p(out), int(splits),
                                       _p(workspace if workspace.numel() else None), workspace.numel(),
                                       _p(status), _stream()), "kvc_attn_decode")
    return out, status


def encode_debug(wait_limit=0, starve=False):
    """Diagnostics of the encoder's bounded waits between blocks (kvc_encode_debug); (0, False) restores the
    defaults."""
    _lib.load().kvc_encode_debug(int(wait_limit), int(bool(starve)))


def attn_debug(wait_limit=0, starve=False):
    """Diagnostics of the attention kernel's bounded staging waits (kvc_attn_debug); (0, False) restores
    the defaults."""
    _lib.load().kvc_attn_debug(int(wait_limit), int(bool(starve)))


def attn_decode_static(kcache, vcache, T, B, Hkv, q, scaling, out, ktail=None, vtail=None, splits=0, status=None):
    """attn_decode for callers that must not allocate: the split-KV scratch is the library's built-in
    array, `out` and `status` are the caller's tensors, and this wrapper creates no tensor either.
    Calls that overlap on the GPU share the scratch and race; keep them on one stream."""
    lib = _lib.load()
    _cuda(q, torch.float16, "q")
    _cuda(out, torch.float16, "out")
    if status is None:
        raise KvcError("attn_decode_static: pass a status tensor (ops.new_status) made beforehand")
    Tr = 0
    if ktail is not None and ktail.shape[0] > 0:
        _cuda(ktail, torch.float16, "ktail")
        _cuda(vtail, torch.float16, "vtail")
        Tr = ktail.shape[0]
    else:
        ktail = vtail = None
    with _on(q.device):
        _lib.check(lib.kvc_attn_decode_static(C.byref(kcache), C.byref(vcache), T, B, Hkv, q.shape[1], _p(q),
                                              float(scaling), _p(ktail), _p(vtail), Tr, _p(out), int(splits),
                                              _p(status), _stream()), "kvc_attn_decode_static")
    return out


def k_matvec(k, q, out):
    lib = _lib.load()
    for t, n in ((k, "A"), (q, "B"), (out, "C")):
        _cuda(t, torch.float16, n)
    ctx, bsz, H, D = k.shape
    if bsz != 1 or D != 128:
        raise KvcError("Batch size must be 1 for now")
    with _on(k.device):
        _lib.check(lib.kvc_k_matvec(_p(k), _p(q), _p(out), ctx, H, _stream()), "kvc_k_matvec")
    return out
