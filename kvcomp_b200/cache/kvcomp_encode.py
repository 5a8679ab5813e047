"""KVCompCtx: the compressed store of one layer's K or V (models/cache/kvcomp_encode.py:15-326).

Same constructor, methods and bookkeeping as the reference class, with the work moved into the CUDA
library: the quantiser is one kernel instead of ~8 torch ops, histogram and codebook are built on the
device, and the stream grows inside pre-reserved arenas instead of torch.cat on every store
(kvcomp_encode.py:129-133).  Beyond the reference: ChannelQuant / VectorQuant for K, per-sequence
units, any batch size in the fused kernels, and `cache()` for the one-pass decode attention.

Tokens are quantised in whole blocks of the configured block size, exactly where the reference cuts
(utils/compute.py:44-72), and encoded in whole Huffman blocks (64 tokens for K, 128 for V).  When a V
block size is not a multiple of 128 (the reference's CUDA path forbids that, kvcomp_encode.py:52-54; its
model path allows it), up to 127 quantised tokens wait as plain codes for their vector to fill.
"""
import torch

from .. import ops
from .._lib import KvcError
from ..utils.compute import QuantMode, cut_len, cut_tensor_ctx_len_0
from ..utils.config import KVCompCacheConfigStatic

_MODE = {QuantMode.BlockQuant: ops.MODE_BLOCK, QuantMode.ChannelQuant: ops.MODE_CHANNEL,
         QuantMode.TokenQuant: ops.MODE_TOKEN, QuantMode.VectorQuant: ops.MODE_VECTOR}


class _Arena:
    """A 1-D device buffer that grows geometrically; `n` elements are in use."""

    def __init__(self, dtype):
        self.dtype, self.buf, self.n = dtype, None, 0

    def reserve(self, extra, device):
        need = self.n + extra
        if self.buf is None or self.buf.numel() < need:
            cap = max(need, int((self.buf.numel() if self.buf is not None else 0) * 1.5), 1024)
            new = torch.empty(cap, dtype=self.dtype, device=device)
            if self.buf is not None and self.n:
                new[:self.n] = self.buf[:self.n]
            self.buf = new
        return self.buf[self.n:need]

    def used(self):
        return self.buf[:self.n] if self.buf is not None else None


class _RecentRows:
    """The rows behind the compressed stream, fp16 [r, B, H, D], kept in place in one buffer:

        [ kept | recent )      kept:   dequantised values of quantised tokens that a reader still wants as rows
                               recent: the uncompressed recent window (the reference's `buffer`)

    New rows are written behind the recent ones; when the front of the window is compressed its rows are
    overwritten with their dequantised values and join the kept ones (or are given up), so that both parts
    always form one contiguous range and nothing is concatenated at a decode step (the reference's
    torch.cat, models/cache/kvcomp_encode.py:80, copies the whole window, some ten megabytes per tensor and
    layer, at every store).  The rows move to the front only when the end of the buffer is reached."""

    def __init__(self):
        self.buf, self.q, self.lo, self.hi = None, 0, 0, 0

    def __len__(self):                      # recent rows
        return self.hi - self.lo

    @property
    def kept(self):
        return self.lo - self.q

    def view(self):
        return None if self.buf is None else self.buf[self.lo:self.hi]

    def rows_from_kept(self, k):
        """The last k kept rows followed by the recent ones; earlier kept rows are given up."""
        self.q = self.lo - k
        if self.q == self.hi:
            self.q = self.lo = self.hi = 0
            return None
        return self.buf[self.q:self.hi]

    def consume(self, n):
        """The first n recent rows were compressed: their places now belong to the kept rows."""
        self.lo += n

    def reserve(self, t, room, shape, dtype, device):
        """Room for t more rows; returns the rows' place [t, B, H, D] without making them live (commit does)."""
        held = self.hi - self.q
        if self.buf is None or self.hi + t > self.buf.shape[0]:
            if self.buf is not None and held + t <= self.buf.shape[0] and self.q >= held:
                self.buf[:held] = self.buf[self.q:self.hi]          # the two ranges do not overlap
            else:
                new = torch.empty((held + t + room,) + tuple(shape), dtype=dtype, device=device)
                if held:
                    new[:held] = self.buf[self.q:self.hi]
                self.buf = new
            self.lo, self.hi, self.q = self.lo - self.q, held, 0
        return self.buf[self.hi:self.hi + t]

    def commit(self, t):
        self.hi += t

    def append(self, rows, room):
        """Add rows [t, B, H, D]; `room`: rows to leave space for beyond what is needed now."""
        t = rows.shape[0]
        self.reserve(t, room, rows.shape[1:], rows.dtype, rows.device)[:] = rows
        self.commit(t)

    def rebuild(self, kept, recent, room):
        """Start over with the given kept rows and recent rows (either may be None)."""
        parts = [p for p in (kept, recent) if p is not None and p.shape[0]]
        nk = 0 if kept is None else kept.shape[0]
        if not parts:
            self.q = self.lo = self.hi = 0
            return
        n = sum(p.shape[0] for p in parts)
        self.buf = torch.empty((n + room,) + tuple(parts[0].shape[1:]), dtype=parts[0].dtype, device=parts[0].device)
        torch.cat(parts, dim=0, out=self.buf[:n])
        self.q, self.lo, self.hi = 0, nk, n

    def set(self, rows):
        self.buf, self.q, self.lo, self.hi = rows, 0, 0, (0 if rows is None else rows.shape[0])


class KVCompCtx:
    def __init__(self, is_k, batch_size, head_num, head_dim, quant_scale_rel,
                 encode_codebook_path=None, decode_codebook_path=None, batch_shared=None, min_dtype=None,
                 keep_dequantised=False):
        """batch_shared / min_dtype: None takes the configuration's quant_per_sequence / wide_min_ints, and
        where those are None too the reference's CUDA-path conventions (units span the batch, int8 min_ints).
        keep_dequantised: keep the fp16 values of freshly quantised tokens until trim_dequantised() drops
        them, so that a decode loop can hand the tokens behind the fused kernel's range over without decoding."""
        cfg = KVCompCacheConfigStatic.config
        assert cfg is not None, "KVCompCacheConfigStatic.config is None"
        assert head_dim == 128, "head_dim must be equal to K_VEC_LEN and V_VEC_LEN for cuda kernel implementation"
        self.is_k = is_k
        self.batch_size, self.head_num, self.head_dim = batch_size, head_num, head_dim
        self.quant_scale_rel = quant_scale_rel
        self.quant_mode = cfg.k_quant_mode if is_k else cfg.v_quant_mode
        self.block_size = cfg.k_block_size if is_k else cfg.v_block_size
        self.recent_size = cfg.k_recent_size if is_k else cfg.v_recent_size
        if batch_shared is None:
            per_seq = getattr(cfg, "quant_per_sequence", None)
            batch_shared = True if per_seq is None else not per_seq
        if min_dtype is None:
            wide = getattr(cfg, "wide_min_ints", None)
            min_dtype = torch.int16 if wide else torch.int8
        self.batch_shared, self.min_dtype = bool(batch_shared), min_dtype
        self.cut_block = self.block_size                     # tokens are quantised where the reference cuts
        if is_k:
            assert self.block_size % 64 == 0, "for K, block size must be divisible by VEC_PER_BLK"
            assert self.quant_mode in _MODE
            self.enc_block = 64
        else:
            assert self.quant_mode in (QuantMode.TokenQuant, QuantMode.VectorQuant, QuantMode.BlockQuant), \
                "V units must not depend on the channel"
            self.enc_block = 128                             # whole 128-token vectors
        if self.quant_mode in (QuantMode.BlockQuant, QuantMode.ChannelQuant) and not is_k:
            assert self.block_size % 128 == 0 or 128 % self.block_size == 0
        self.spec = ops.qspec(_MODE[self.quant_mode], self.batch_shared, batch_size, head_num, head_dim,
                              self.block_size)
        self.ctx_len = 0
        self.compressed_ctx_len = 0              # quantised tokens
        self.encoded_ctx_len = 0                 # of those, the tokens in the stream (whole Huffman blocks)
        self._pending = None                     # codes of quantised tokens whose Huffman block is not full yet
        self.keep_dequantised = keep_dequantised
        self.device = None
        self._recent = _RecentRows()             # uncompressed recent tokens, fp16 [r, B, H, D] (self.buffer)
        self.book = None
        self.max_block_bytes = 0
        self._enc = _Arena(torch.uint8)
        self._bi = _Arena(torch.uint8)
        self._ti = _Arena(torch.int16)
        self._mi = _Arena(self.min_dtype)
        self._sc = _Arena(torch.float16)
        self._hist = None

    # ---- views with the reference's attribute names --------------------------------------------
    @property
    def buffer(self):
        return self._recent.view()

    @buffer.setter
    def buffer(self, rows):
        self._recent.set(rows)

    @property
    def encoded_data(self):
        return self._enc.used()

    @property
    def block_infos(self):
        return self._bi.used()

    @property
    def thread_infos(self):
        u = self._ti.used()
        return None if u is None else u.view(torch.uint8)

    def _unit_shape(self):
        s = self.spec
        B, H, D = self.batch_size, self.head_num, self.head_dim
        nb = 1 if (s.sb == 0) else B
        nh = 1 if (s.sh == 0) else H
        nc = 1 if (s.sc == 0) else D
        per_blk = self.block_size // s.tok_div if s.tok_div <= self.block_size else 1
        return (-1, per_blk, nb, nh, nc)

    @property
    def quant_min_ints(self):
        u = self._mi.used()
        return None if u is None else u.view(*self._unit_shape())

    @property
    def quant_scales(self):
        u = self._sc.used()
        return None if u is None else u.view(*self._unit_shape())

    @property
    def encode_codebook(self):
        return None if self.book is None else self.book.encode_table()

    @property
    def decode_codebook(self):
        return None if self.book is None else self.book.ref_decode_tensor().to(self.device)

    @property
    def shape(self):
        return torch.Size([self.compressed_ctx_len, self.batch_size, self.head_num, self.head_dim])

    # ---- store ------------------------------------------------------------------------------------
    def _room(self):
        return self.recent_size // 2 + self.cut_block          # rows to spare when the window's buffer has to grow

    def recent_place(self, t, device):
        """Where the next t tokens would lie in the recent window, fp16 [t, B, H, D], when storing them compresses
        nothing (the usual decode step), else None.  A caller that can produce the rows there (the rotation and
        transposition kernel) does so and calls recent_commit(t) instead of store(rows)."""
        if self.device is None:
            self.device = device
        if self.device != device or cut_len(len(self._recent) + t, self.cut_block, self.recent_size) // self.cut_block * self.cut_block:
            return None
        return self._recent.reserve(t, self._room(), (self.batch_size, self.head_num, self.head_dim), torch.float16, device)

    def recent_commit(self, t):
        self._recent.commit(t)
        self.ctx_len += t

    def _check(self, cache):
        assert cache.dtype == torch.float16, "cache must be float16"
        assert cache.shape[1] == self.batch_size, "batch size mismatch"
        assert cache.shape[2] == self.head_num, "head num mismatch"
        assert cache.shape[3] == self.head_dim, "head dim mismatch"
        if self.device is None:
            self.device = cache.device
        assert self.device == cache.device, "device mismatch"

    def _quantize(self, x, hist):
        T = x.shape[0]
        n = self.spec.units(T, self.batch_size, self.head_num, self.head_dim)
        mi = self._mi.reserve(n, self.device)
        sc = self._sc.reserve(n, self.device)
        codes, _, _, _, st = ops.quantize(x, _MODE[self.quant_mode], self.block_size, self.quant_scale_rel,
                                          self.batch_shared, min_dtype=self.min_dtype, hist=hist, min_int=mi, scale=sc)
        return codes, n, st

    def store(self, cache):
        """Append tokens [t, B, H, D]; whole blocks beyond the recent window are quantised and encoded.
        Returns the uint8 codes of the newly compressed tokens as [n_blocks, block, B, H, D] (or None)."""
        self._check(cache)
        self.ctx_len += cache.shape[0]
        # utils/compute.py:59-72: the first n tokens of (recent window + new tokens) are compressed.  With
        # recent_size = 0 and a ragged length the reference's slice clips to the length and its .view then
        # fails (kvcomp_encode.py:83); here the ragged rest simply stays in the window.
        live, t = len(self._recent), cache.shape[0]
        n = min(cut_len(live + t, self.cut_block, self.recent_size), live + t) // self.cut_block * self.cut_block
        room = self._room()
        if n == 0:
            self._recent.append(cache, room)                  # the usual decode step: the new rows, nothing else moves
            return None
        if live == 0:
            x, rest = cache[:n].contiguous(), cache[n:]       # a prefill: compressed from where it lies
        elif n <= live:
            x, rest = self._recent.view()[:n].clone(), cache  # the window's front
        else:
            x, rest = torch.cat([self._recent.view(), cache[:n - live]], dim=0), cache[n - live:]
        T = x.shape[0]
        hist = None
        if self.book is None:
            hist = torch.zeros(256, dtype=torch.int64, device=self.device)
        codes, n_units, st_q = self._quantize(x, hist)
        if self.book is None:
            self.book = ops.build_codebook(hist)
        flags = ops.read_status(st_q, what="quantize")
        if flags & ops._lib.FLAG_MIN_OVERFLOW:
            # int8 is the reference's CUDA path, which wraps silently (kvcomp_encode.py:97); its model path
            # keeps min_ints in floating point (utils/compute.py:89).  Wrapped values dequantise wrongly.
            if self.min_dtype == torch.int16:
                raise KvcError("a min_int does not fit 16 bits: the data lies too far from zero for its range")
            import warnings
            warnings.warn("a min_int wrapped in int8 as in the reference's CUDA path; set wide_min_ints to keep it")
        # the window: the compressed rows leave it, or stay as dequantised rows for a reader of the rows behind
        # the fused kernel's range (tail_from); the rest of the new tokens joins the recent rows
        mi = self._mi.buf[self._mi.n:self._mi.n + n_units]
        sc = self._sc.buf[self._sc.n:self._sc.n + n_units]
        if 0 < live and n <= live:
            if self.keep_dequantised:
                ops.dequant(codes, mi, sc, self.spec, out=self._recent.view()[:n])     # in place of the rows themselves
                self._recent.consume(n)
            else:
                self._recent.consume(n)
                self._recent.rows_from_kept(0)
            if rest.shape[0]:
                self._recent.append(rest, room)
        else:
            kept = None
            if self.keep_dequantised:
                k = min(n, max(self.KEEP_ROWS // self.cut_block, 1) * self.cut_block)    # a long prefill keeps its last rows only
                first = (n - k) // self.spec.tok_div * self.spec.sj                      # unit of the first kept token
                xh = ops.dequant(codes[n - k:], mi[first:], sc[first:], self.spec)
                old = self._recent.rows_from_kept(self._recent.kept if k == n else 0)
                old = None if old is None else old[:self._recent.kept]
                kept = xh if old is None or not old.shape[0] else torch.cat([old, xh], dim=0)
            self._recent.rebuild(kept, rest if rest.shape[0] else None, room)
        self._mi.n += n_units
        self._sc.n += n_units
        self.compressed_ctx_len += T
        pend = codes if self._pending is None else torch.cat([self._pending, codes], dim=0)
        n_enc = pend.shape[0] // self.enc_block * self.enc_block
        if n_enc:
            part = pend[:n_enc].contiguous()
            if not self._encode(part):
                # A symbol the frozen book has no code for.  The reference drops such symbols silently
                # (kernels.cu:197-205: a table entry of length 0 adds no bits), which corrupts the stream.
                # Here the book is rebuilt over everything stored so far plus every reachable code, and the
                # cache is re-encoded once; this cannot happen again for this context.
                self._rebook(part)
            self.encoded_ctx_len += n_enc
        self._pending = pend[n_enc:].contiguous() if pend.shape[0] > n_enc else None
        return codes.view(-1, self.block_size, self.batch_size, self.head_num, self.head_dim)

    def _encode(self, codes):
        """Append the stream of `codes` [T, B, H, D] to the arenas.  False if the book lacks a symbol."""
        T = codes.shape[0]
        cols = self.batch_size * self.head_num
        bsz, tsz, _, cap = ops.buffer_sizes(T, cols * self.head_dim, self.is_k)
        bi = self._bi.reserve(bsz, self.device)
        ti = self._ti.reserve(tsz // 2, self.device)
        # The reference reserves one byte per symbol (numel) for every store (kernels.cu:903); the stream
        # needs a fraction of that, so room is reserved from the density seen so far (8 bits per symbol at
        # first) with a quarter on top, and the store is repeated with the full reserve in the rare case
        # that the encoder reports the room as exceeded.
        seen = self.encoded_ctx_len * cols * self.head_dim
        est = cap if seen == 0 else min(cap, int(1.25 * self._enc.n / seen * codes.numel()) + 4096)
        for room in (est, cap):
            enc = self._enc.reserve(room, self.device)
            total = torch.tensor([0, self.max_block_bytes], dtype=torch.int64, device=self.device)
            total, st_e = ops.encode(codes, self.is_k, self.book.encode_table(), bi, ti, enc,
                                     base_offset=self._enc.n, total=total)
            n_bytes, max_block = (int(v) for v in total.tolist())      # synchronises, as the reference does
            flags = ops.read_status(st_e, raise_on_fatal=False)
            if not (flags & ops._lib.FLAG_STREAM_FULL) or room == cap:
                break
            self.stream_retries = getattr(self, "stream_retries", 0) + 1
        if flags & ops._lib.FLAG_SYMBOL_MISSING:
            return False
        ops.read_status(st_e, what="entropy_encode")
        self._enc.n += n_bytes
        self._bi.n += bsz
        self._ti.n += tsz // 2
        self.max_block_bytes = max_block
        return True

    def _rebook(self, new_codes):
        old = None
        if self.encoded_ctx_len:
            old, st = ops.decode(self._enc.used(), self._bi.used(), self._ti.used(), self.book,
                                 self.encoded_ctx_len, self.batch_size, self.head_num, self.is_k,
                                 max_block=self.max_block_bytes)
            ops.read_status(st, what="entropy_decode")
        hist = ops.histogram(new_codes.view(-1))
        if old is not None:
            hist = ops.histogram(old.view(-1), hist)
        reach = min(255, int(1.0 / self.quant_scale_rel) + 3)      # codes are 0 .. about 1/rel + 1
        hist[:reach + 1] += 1
        self.book = ops.build_codebook(hist)
        self._enc.n = self._bi.n = self._ti.n = 0
        self.max_block_bytes = 0
        self.rebooks = getattr(self, "rebooks", 0) + 1
        for part in (old, new_codes):
            if part is not None and not self._encode(part):
                raise KvcError("a code outside 0..%d appeared; the quantiser settings cannot produce it" % reach)

    def build_codebook(self, tensors):
        """Freeze the codebook from sample tensors before the first store (kvcomp_encode.py:282-306)."""
        assert len(tensors) > 0, "tensors must not be empty"
        hist = None
        for cache in tensors:
            self._check(cache)
            blocked = cache.shape[0] // self.block_size * self.block_size
            if blocked == 0:
                continue
            x = cache[:blocked].contiguous()
            if hist is None:
                hist = torch.zeros(256, dtype=torch.int64, device=self.device)
            mi = torch.empty(self.spec.units(blocked, self.batch_size, self.head_num, self.head_dim),
                             dtype=self.min_dtype, device=self.device)
            ops.quantize(x, _MODE[self.quant_mode], self.block_size, self.quant_scale_rel, self.batch_shared,
                         min_dtype=self.min_dtype, hist=hist, min_int=mi)
        if hist is None:
            raise KvcError("build_codebook: no whole block in the sample tensors")
        self.book = ops.build_codebook(hist)
        hd = self.book.header()
        assert hd["min_sym"] == 0, "shift must be 0"

    # ---- read back --------------------------------------------------------------------------------
    def _require(self):
        assert self.compressed_ctx_len > 0 and self.book is not None, "nothing has been compressed yet"

    def get_decode_quant_ints(self):
        """Decoded uint8 codes [n_blocks, block, B, H, D] and the kernel time in ms."""
        self._require()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        out = None
        if self.encoded_ctx_len:
            out, st = ops.decode(self._enc.used(), self._bi.used(), self._ti.used(), self.book,
                                 self.encoded_ctx_len, self.batch_size, self.head_num, self.is_k,
                                 max_block=self.max_block_bytes)
        stop.record()
        stop.synchronize()
        if out is not None:
            ops.read_status(st, what="entropy_decode")
        if self._pending is not None:
            out = self._pending if out is None else torch.cat([out, self._pending], dim=0)
        return out.view(-1, self.block_size, self.batch_size, self.head_num, self.head_dim), start.elapsed_time(stop)

    def get_only_compressed(self):
        """Dequantised compressed part [T, B, H, D] and the time of decode + dequantisation in ms."""
        codes, t = self.get_decode_quant_ints()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        x = ops.dequant(codes.view(self.compressed_ctx_len, self.batch_size, self.head_num, self.head_dim),
                        self._mi.used(), self._sc.used(), self.spec)
        stop.record()
        stop.synchronize()
        return x, t + start.elapsed_time(stop)

    def get(self):
        """Whole cache [ctx_len, B, H, D]: dequantised compressed part followed by the recent window."""
        if self.compressed_ctx_len == 0:
            return self.buffer, 0.0
        x, t = self.get_only_compressed()
        return (torch.cat([x, self.buffer], dim=0) if self.buffer is not None and self.buffer.shape[0] else x), t

    def cache(self):
        """The kvc_cache argument of the fused kernels over the encoded_ctx_len tokens of the stream (valid
        until the next store)."""
        assert self.encoded_ctx_len > 0 and self.book is not None, "nothing has been encoded yet"
        return ops.make_cache(self._enc.buf, self._bi.buf, self._ti.buf, self.book, self._mi.buf, self._sc.buf,
                              self.spec, self._enc.n, self.max_block_bytes)

    def mat_vec_mul(self, B):
        """K: scores [batch, heads, ctx] = q . K^T; V: [1, batch, heads, 128] = P . V over the compressed
        tokens (kvcomp_encode.py:209-280).  Returns (tensor, ms)."""
        self._require()
        if self._pending is not None:
            raise KvcError("mat_vec_mul: %d quantised tokens are not in the stream yet (V block sizes that are "
                           "no multiple of 128 leave such a rest)" % self._pending.shape[0])
        assert B.dtype == torch.float16, "B must be float16"
        assert len(B.shape) == 3, "B must be 3D tensor"
        assert B.shape[0] == self.batch_size, "batch size mismatch"
        hq = B.shape[1]
        assert hq % self.head_num == 0, "head num mismatch"
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if self.is_k:
            assert B.shape[2] == self.head_dim, "head dim mismatch"
            start.record()
            C, st = ops.fused_qk(self.cache(), self.compressed_ctx_len, self.batch_size, self.head_num, B)
        else:
            assert B.shape[2] == self.compressed_ctx_len, "ctx len mismatch"
            start.record()
            part, st = ops.fused_pv(self.cache(), self.compressed_ctx_len, self.batch_size, self.head_num, B)
            C = part.float().sum(dim=0, keepdim=True).half()
        stop.record()
        stop.synchronize()
        ops.read_status(st, what="mat_vec_mul")
        return C, start.elapsed_time(stop)

    def save(self, path):
        """Write this cache to a file (kvcomp_b200.cache.storage describes the format)."""
        from .storage import save_ctx
        return save_ctx(self, path)

    @staticmethod
    def load(path, device="cuda"):
        from .storage import load_ctx
        return load_ctx(path, device)

    def get_cr(self):
        """Compression ratio with the reference's accounting (kvcomp_encode.py:317-326)."""
        compressed = (self._bi.n + self._ti.n * 2 + self._enc.n + self._mi.n * self._mi.used().element_size() +
                      self._sc.n * 2)
        pending = 0 if self._pending is None else self._pending.numel()
        original = 2 * self.batch_size * self.compressed_ctx_len * self.head_num * self.head_dim
        return original / (compressed + pending)

    # ---- the tokens behind the fused kernel's range ---------------------------------------------------
    KEEP_ROWS = 512       # dequantised rows a long store keeps at most (tail_from decodes when it needs more)

    def tail_from(self, T):
        """fp16 [n, B, H, D]: the quantised tokens from index T on (dequantised) followed by the recent
        window, as one range of the window's buffer.  Dequantised rows before T are given up."""
        need = max(0, self.compressed_ctx_len - T)
        if need > self._recent.kept:
            # not kept (keep_dequantised off, a cache read from a file, a prefill longer than KEEP_ROWS whose
            # other tensor lags far behind): decode the stream once, keep the rows from T on
            x, _ = self.get_only_compressed()
            kept = x[T:].contiguous()
            if not self.keep_dequantised:
                return kept if not len(self._recent) else torch.cat([kept, self._recent.view()], dim=0)
            self._recent.rebuild(kept, self._recent.view(), self._room())
        return self._recent.rows_from_kept(need)

    def trim_dequantised(self, T):
        self._recent.rows_from_kept(min(self._recent.kept, max(0, self.compressed_ctx_len - T)))
