"""KVCompCache: the KV-cache object the patched model files construct and call
(models/cache/kvcomp_cache.py:22-38, models/cache/kvcomp_quant.py:14-123; call sites
models/llama.py:279-283,848-852, models/mistral.py:168-171,840-844, models/phi3.py:197-201,916-920).

    cache = KVCompCache(batch_size, head_num, head_dim, layer_num)
    k, v = cache.update(key_states, value_states, layer_idx, {"cos": cos, "sin": sin})   # drop-in
    out = cache.attend(query_states, layer_idx, scaling)                                 # fused path

`update` keeps the reference's contract and returns the reference's values: RoPE is applied to the new
keys inside, the tokens are appended, and the whole cache comes back as fp16 [B, H, T, D] for eager
attention -- compressed blocks dequantised (what the reference's simulated path returns,
kvcomp_quant.py:70-75), recent tokens as they are.  Like that path, quant units never span the batch
(utils/compute.py:138-143) and min_ints are not narrowed to int8, unless the configuration's
quant_per_sequence / wide_min_ints say otherwise.  `append` + `attend` is the path that never
materialises K/V: the tokens go into the compressed store and one kernel computes
softmax(q K^T * scaling) V straight from the streams.
"""
import inspect
import math

import torch

from .. import ops
from .._lib import KvcError
from ..utils.compute import apply_rotary_pos_emb_single, safe_cat
from ..utils.config import KVCompCacheConfigStatic
from .kvcomp_encode import KVCompCtx

try:                                    # transformers 4.50's Cache takes no constructor arguments
    from transformers import Cache as _HFCache
    _BASE = _HFCache if not [p for p in list(inspect.signature(_HFCache.__init__).parameters.values())[1:]
                             if p.default is inspect.Parameter.empty and p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD)] else object
except Exception:                       # pragma: no cover
    _BASE = object


class KVCompCache(_BASE):
    def __init__(self, batch_size, head_num, head_dim, layer_num):
        if _BASE is not object:
            try:
                super().__init__()
            except Exception:
                pass
        if KVCompCacheConfigStatic.config is None:
            raise ValueError("KVCompCacheConfigStatic.config is not set. Please set it before using KVCompCache.")
        self.batch_size, self.head_num, self.head_dim, self.layer_num = batch_size, head_num, head_dim, layer_num
        self.k_ctx = [None] * layer_num       # created at the first update: the KV head count is only known then
        self.v_ctx = [None] * layer_num
        self.k_plain = [None] * layer_num     # enable_quant = False: plain fp16 concatenation [B, H, T, D]
        self.v_plain = [None] * layer_num
        self.coss = [None] * layer_num
        self.sins = [None] * layer_num
        self._ws = {}
        self._status = {}

    # ---- appending --------------------------------------------------------------------------------
    def _ctx(self, layer_idx, kv_heads):
        cfg = KVCompCacheConfigStatic.config
        if self.k_ctx[layer_idx] is None:
            kw = dict(batch_shared=getattr(cfg, "quant_per_sequence", None) is False,
                      min_dtype=torch.int8 if getattr(cfg, "wide_min_ints", None) is False else torch.int16,
                      keep_dequantised=True)
            self.k_ctx[layer_idx] = KVCompCtx(True, self.batch_size, kv_heads, self.head_dim, cfg.k_quant_scale_rel, **kw)
            self.v_ctx[layer_idx] = KVCompCtx(False, self.batch_size, kv_heads, self.head_dim, cfg.v_quant_scale_rel, **kw)
        return self.k_ctx[layer_idx], self.v_ctx[layer_idx]

    def append(self, key_states, value_states, layer_idx, cache_kwargs=None):
        """Add new tokens (key/value_states: [B, Hkv, t, D]); keys get RoPE here unless pre-RoPE is on."""
        cfg = KVCompCacheConfigStatic.config
        cos, sin = cache_kwargs["cos"], cache_kwargs["sin"]
        k_rows = None                       # the new keys token-major [t, B, H, D], when one kernel made them so
        if cfg.enable_pre_rope:
            self.coss[layer_idx] = safe_cat(self.coss[layer_idx], cos, dim=1)
            self.sins[layer_idx] = safe_cat(self.sins[layer_idx], sin, dim=1)
        elif cfg.enable_quant and key_states.is_cuda and key_states.dtype == torch.float16 and key_states.is_contiguous() \
                and cos.dtype == torch.float16 and key_states.shape[3] % 16 == 0:
            kc0, vc0 = self._ctx(layer_idx, key_states.shape[1])
            t = key_states.shape[2]
            if value_states.is_cuda and value_states.dtype == torch.float16 and value_states.is_contiguous() \
                    and value_states.shape == key_states.shape:
                kplace, vplace = kc0.recent_place(t, key_states.device), vc0.recent_place(t, key_states.device)
                if kplace is not None and vplace is not None:   # the usual decode step: one launch, straight into both windows
                    ops.kv_store(key_states, value_states, cos, sin, kplace, vplace)
                    kc0.recent_commit(t)
                    vc0.recent_commit(t)
                    return
            place = kc0.recent_place(key_states.shape[2], key_states.device)
            if place is not None:                               # the usual decode step: straight into the recent window
                ops.rope_store(key_states, cos, sin, out=place)
                kc0.recent_commit(key_states.shape[2])
                k_rows = False                                  # stored already
            else:
                k_rows = ops.rope_store(key_states, cos, sin)  # rotation and transposition in one pass, torch's bits
        else:
            key_states = apply_rotary_pos_emb_single(key_states, cos, sin)
        if not cfg.enable_quant:
            self.k_plain[layer_idx] = safe_cat(self.k_plain[layer_idx], key_states, dim=2)
            self.v_plain[layer_idx] = safe_cat(self.v_plain[layer_idx], value_states, dim=2)
            return
        kc, vc = self._ctx(layer_idx, key_states.shape[1])
        if k_rows is not False:
            kc.store(k_rows if k_rows is not None else key_states.permute(2, 0, 1, 3).contiguous().half())
        t = value_states.shape[2]
        place = None
        if value_states.is_cuda and value_states.dtype == torch.float16 and value_states.is_contiguous() and value_states.shape[3] % 16 == 0:
            place = vc.recent_place(t, value_states.device)
        if place is not None:                                   # the transposition writes straight into the window
            ops.rope_store(value_states, None, None, out=place)
            vc.recent_commit(t)
        else:
            vc.store(value_states.permute(2, 0, 1, 3).contiguous().half())

    def update(self, key_states, value_states, layer_idx, cache_kwargs=None):
        """The reference's Cache.update: append, then return the whole K and V as [B, Hkv, T, D]."""
        cfg = KVCompCacheConfigStatic.config
        self.append(key_states, value_states, layer_idx, cache_kwargs)
        if not cfg.enable_quant:
            k, v = self.k_plain[layer_idx], self.v_plain[layer_idx]
        else:
            k = self.k_ctx[layer_idx].get()[0].permute(1, 2, 0, 3)
            v = self.v_ctx[layer_idx].get()[0].permute(1, 2, 0, 3)
        if cfg.enable_pre_rope:
            k = apply_rotary_pos_emb_single(k, self.coss[layer_idx], self.sins[layer_idx])
        return k, v

    def get_seq_length(self, layer_idx=0):
        layer_idx = 0 if layer_idx is None else layer_idx
        if not KVCompCacheConfigStatic.config.enable_quant:
            return 0 if self.k_plain[layer_idx] is None else self.k_plain[layer_idx].shape[2]
        return 0 if self.k_ctx[layer_idx] is None else self.k_ctx[layer_idx].ctx_len

    # ---- fused decode attention -------------------------------------------------------------------
    def _tails(self, kc, vc):
        """Length of the range the fused kernel reads from the streams and the fp16 tails behind it.  K and V
        cut their recent windows with different block and window sizes and fill Huffman blocks of
        different length, so either may have quantised tokens beyond that range: their dequantised values
        (kept since they were quantised) go in front of the recent window."""
        T = min(kc.encoded_ctx_len, vc.encoded_ctx_len) // 128 * 128
        return T, kc.tail_from(T), vc.tail_from(T)

    def check(self):
        """Raise if a fused launch since the last check reported a fatal condition (a stream that does not
        decode, a staging wait that ran out).  Synchronises; attend() itself never does."""
        for st in self._status.values():
            flags = ops.read_status(st, what="attend")
            if flags:
                st.zero_()

    def attend(self, query_states, layer_idx, scaling=None):
        """One decode step: query_states [B, Hq, 1, D] (or [B, Hq, D]), already rotated -> attention
        output of the same shape, computed straight from the compressed K and V of the layer; tokens
        that are not in the streams yet (the recent window) are read as fp16 rows by the same kernel.
        With pre-RoPE keys the stored keys are not rotated, every token would need its own rotation of
        the query, and the step goes through the dequantised cache instead (the slow way)."""
        cfg = KVCompCacheConfigStatic.config
        q = query_states
        squeeze = q.dim() == 4
        if squeeze:
            if q.shape[2] != 1:
                raise KvcError("attend handles one query token (decode); use update() for prefill")
            q = q[:, :, 0, :]
        q = q.contiguous().half()
        B, Hq, D = q.shape
        scaling = 1.0 / math.sqrt(D) if scaling is None else scaling
        if not cfg.enable_quant or cfg.enable_pre_rope:
            out = self._attend_dense(q, layer_idx, scaling)
            return out.unsqueeze(2) if squeeze else out
        kc, vc = self.k_ctx[layer_idx], self.v_ctx[layer_idx]
        if kc is None:
            raise KvcError("attend before any update")
        T, ktail, vtail = self._tails(kc, vc)
        if T == 0 and ktail is None:
            raise KvcError("empty cache")
        parts = ops.attn_splits(T, B, kc.head_num)          # partial results per head of the balanced split
        key = (q.device, B, Hq, parts)
        if key not in self._ws:
            self._ws[key] = ops.attn_workspace(B, Hq, parts, q.device)
        if q.device not in self._status:
            self._status[q.device] = ops.new_status(q.device)
        out, _ = ops.attn_decode(kc.cache() if T else None, vc.cache() if T else None, T, B, kc.head_num, q, scaling,
                                 ktail, vtail, splits=0, workspace=self._ws[key], status=self._status[q.device])
        return out.unsqueeze(2) if squeeze else out

    def _attend_dense(self, q, layer_idx, scaling):
        """softmax(q K^T * scaling) V over the materialised cache: plain fp16 caches (enable_quant off) and
        pre-RoPE caches."""
        cfg = KVCompCacheConfigStatic.config
        if not cfg.enable_quant:
            k, v = self.k_plain[layer_idx], self.v_plain[layer_idx]
        else:
            k = self.k_ctx[layer_idx].get()[0].permute(1, 2, 0, 3)
            v = self.v_ctx[layer_idx].get()[0].permute(1, 2, 0, 3)
        if k is None:
            raise KvcError("attend before any update")
        if cfg.enable_pre_rope:
            k = apply_rotary_pos_emb_single(k, self.coss[layer_idx], self.sins[layer_idx])
        g = q.shape[1] // k.shape[1]
        kf, vf = k.float().repeat_interleave(g, dim=1), v.float().repeat_interleave(g, dim=1)
        w = torch.softmax(torch.einsum("bhd,bhtd->bht", q.float(), kf) * scaling, dim=-1)
        return torch.einsum("bht,bhtd->bhd", w, vf).half()
