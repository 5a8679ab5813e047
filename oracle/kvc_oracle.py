"""numpy front end of the CPU checker (oracle/kvc_oracle.c) -- TEST INFRASTRUCTURE ONLY.

The product (kvcomp_b200) never imports this module.  It exists so that tests, the
smoke entry and the benchmark's CPU-baseline leg can compare the CUDA library with
a plain-C restatement of the reference's algorithm.  Every function here forwards to
the C function of the same name; the reference file:line each one follows is cited
in the C source.
"""
import ctypes as C
import os

import numpy as np

from . import build_oracle

MODE_BLOCK, MODE_CHANNEL, MODE_TOKEN, MODE_VECTOR = 0, 1, 2, 3
MODES = {"BlockQuant": MODE_BLOCK, "ChannelQuant": MODE_CHANNEL, "TokenQuant": MODE_TOKEN,
         "VectorQuant": MODE_VECTOR}


class QMeta(C.Structure):
    _fields_ = [("tok_div", C.c_int64), ("sj", C.c_int64), ("sb", C.c_int64),
                ("sh", C.c_int64), ("sc", C.c_int64)]


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(build_oracle.build())
        _lib.orc_qmeta_make.restype = C.c_int64
        _lib.orc_quant.restype = C.c_int64
        _lib.orc_encode.restype = C.c_int64
        _lib.orc_decode.restype = C.c_int64
        _lib.orc_cut_len.restype = C.c_int64
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def _i64(v):
    return C.c_int64(int(v))


def num_threads():
    return lib().orc_num_threads()


def qmeta(mode, batch_shared, T, B, H, D, block):
    m = QMeta()
    n = lib().orc_qmeta_make(C.c_int(mode), C.c_int(int(batch_shared)), _i64(T), _i64(B), _i64(H),
                             _i64(D), _i64(block), C.byref(m))
    assert n >= 0
    return m, int(n)


def quant(x, mode, block, rel, batch_shared=True, raw=False):
    """x: float16 [T,B,H,D].  Returns codes u8 [T,B,H,D], min_int i16 [units], scale f16 [units],
    the qmeta, the count of zero-scale units (+ un-narrowed fp16 codes / min_int when raw)."""
    x = np.ascontiguousarray(x, dtype=np.float16)
    T, B, H, D = x.shape
    m, n = qmeta(mode, batch_shared, T, B, H, D, block)
    codes = np.empty((T, B, H, D), np.uint8)
    mi = np.empty(n, np.int16)
    sc = np.empty(n, np.float16)
    cf = np.empty((T, B, H, D), np.float16) if raw else None
    mf = np.empty(n, np.float16) if raw else None
    deg = lib().orc_quant(_p(x), _i64(T), _i64(B), _i64(H), _i64(D), C.c_int(mode),
                          C.c_int(int(batch_shared)), _i64(block), C.c_float(rel),
                          _p(codes), _p(mi), _p(sc), _p(cf), _p(mf))
    if raw:
        return codes, mi, sc, m, int(deg), cf, mf
    return codes, mi, sc, m, int(deg)


def narrow_i8(mi):
    """The int8 the reference stores (models/cache/kvcomp_encode.py:97): two's-complement wrap."""
    return np.asarray(mi).astype(np.int16).astype(np.int8)


def _mi16(mi):
    return np.ascontiguousarray(mi, dtype=np.int16)


def dequant(codes, mi, sc, m):
    T, B, H, D = codes.shape
    out = np.empty((T, B, H, D), np.float16)
    lib().orc_dequant(_p(codes), _p(_mi16(mi)), _p(sc), _i64(T), _i64(B), _i64(H), _i64(D), C.byref(m), _p(out))
    return out


def cut_len(length, block, recent):
    return int(lib().orc_cut_len(_i64(length), _i64(block), _i64(recent)))


def histogram(codes, counts=None):
    codes = np.ascontiguousarray(codes, dtype=np.uint8).reshape(-1)
    if counts is None:
        counts = np.zeros(256, np.int64)
    lib().orc_histogram(_p(codes), _i64(codes.size), _p(counts))
    return counts


ENC_DT = np.dtype([("code", "<u4"), ("length", "<u4")])


def gen_codes(counts):
    """counts: int64[256] -> structured array [256] of (code, length), symbol-indexed."""
    counts = np.ascontiguousarray(counts, dtype=np.int64)
    enc = np.zeros(256, ENC_DT)
    n = lib().orc_gen_codes(_p(counts), _p(enc))
    return enc, int(n)


def ref_encode_table(enc):
    """The uint8 encode tensor the reference's build_codebook returns, and its shift."""
    out = np.zeros(256, ENC_DT)
    shift = C.c_int(0)
    n = lib().orc_ref_encode_table(_p(enc), _p(out), C.byref(shift))
    return out[:n].view(np.uint8).copy(), shift.value


def ref_decode_tree(enc):
    """The uint8 decode tensor the reference's build_codebook returns (3-byte nodes)."""
    out = np.zeros(3 * 512, np.uint8)
    n = lib().orc_ref_decode_tree(_p(enc), _p(out))
    return out[:3 * n].copy()


def code_strings(enc):
    return {int(s): format(int(enc[s]["code"]), "0%db" % int(enc[s]["length"]))
            for s in range(256) if enc[s]["length"]}


def encode(codes, is_k, enc, base_offset=0, cap=None):
    """codes: u8 [T,B,H,128].  Returns (encoded u8[n], block_info u8[8*nblk], thread_info u16[nvec],
    overflow int64[3])."""
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    T, B, H, D = codes.shape
    assert D == 128
    cols = B * H
    nblk = (T // 64) * cols if is_k else (T // 128) * cols * 2
    bi = np.zeros(8 * nblk, np.uint8)
    ti = np.zeros(64 * nblk, np.uint16)
    cap = codes.size * 4 if cap is None else cap
    out = np.zeros(cap, np.uint8)
    ov = np.zeros(3, np.int64)
    n = lib().orc_encode(_p(codes), _i64(T), _i64(cols), C.c_int(int(is_k)), _p(enc),
                         C.c_uint32(base_offset), _p(bi), _p(ti), _p(out), _i64(cap), _p(ov))
    assert n >= 0, "encoded capacity too small"
    return out[:n].copy(), bi, ti, ov


def decode(encoded, bi, ti, enc, T, B, H, is_k):
    out = np.zeros((T, B, H, 128), np.uint8)
    encoded = np.ascontiguousarray(encoded, dtype=np.uint8)
    bad = lib().orc_decode(_p(encoded), _p(bi), _p(ti), _p(enc), _i64(T), _i64(B * H),
                           C.c_int(int(is_k)), _p(out))
    return out, int(bad)


def block_infos(bi):
    """Split the 8-byte block_info records into (offset u32[], byte_num u16[])."""
    rec = np.ascontiguousarray(bi, dtype=np.uint8).reshape(-1, 8)
    off = rec[:, 0:4].copy().view("<u4").reshape(-1)
    num = rec[:, 4:6].copy().view("<u2").reshape(-1)
    return off, num


def qk(codes, mi, sc, m, q):
    """q: f16 [B,Hq,D] -> raw scores f32 [B,Hq,T]."""
    T, B, Hkv, D = codes.shape
    q = np.ascontiguousarray(q, dtype=np.float16)
    Hq = q.shape[1]
    S = np.empty((B, Hq, T), np.float32)
    lib().orc_qk(_p(codes), _p(_mi16(mi)), _p(sc), C.byref(m), _i64(T), _i64(B), _i64(Hkv), _i64(Hq), _i64(D),
                 _p(q), _p(S))
    return S


def qk_fp16chain(codes, mi, sc, m, q, fused=False):
    """The reference's fp16 accumulation chain of the fused K kernel; fused: mul + add as one fp16 fma."""
    T, B, H, D = codes.shape
    q = np.ascontiguousarray(q, dtype=np.float16)
    S = np.empty((B, H, T), np.float16)
    lib().orc_qk_fp16chain(_p(codes), _p(_mi16(mi)), _p(sc), C.byref(m), _i64(T), _i64(B), _i64(H), _i64(D),
                           _p(q), _p(S), C.c_int(int(fused)))
    return S


def pv_fp16chain(codes, mi, sc, m, P, fused=False):
    """The fused V kernel's per-group fp16 partials [T/128, B, H, D] for P fp16 [B, H, T]."""
    T, B, H, D = codes.shape
    P = np.ascontiguousarray(P, dtype=np.float16)
    out = np.empty((T // 128, B, H, D), np.float16)
    lib().orc_pv_fp16chain(_p(codes), _p(_mi16(mi)), _p(sc), C.byref(m), _i64(T), _i64(B), _i64(H), _i64(D),
                           _p(P), _p(out), C.c_int(int(fused)))
    return out


def pv(codes, mi, sc, m, P):
    """P: f32 [B,Hq,T] -> f32 [B,Hq,D]."""
    T, B, Hkv, D = codes.shape
    P = np.ascontiguousarray(P, dtype=np.float32)
    Hq = P.shape[1]
    O = np.empty((B, Hq, D), np.float32)
    lib().orc_pv(_p(codes), _p(_mi16(mi)), _p(sc), C.byref(m), _i64(T), _i64(B), _i64(Hkv), _i64(Hq), _i64(D),
                 _p(P), _p(O))
    return O


def attention(kc, kmi, ksc, km, vc, vmi, vsc, vm, q, scaling, ktail=None, vtail=None):
    """One decode step over the dequantised cache (+ optional fp16 tail [Tr,B,Hkv,D])."""
    T, B, Hkv, D = kc.shape
    q = np.ascontiguousarray(q, dtype=np.float16)
    Hq = q.shape[1]
    Tr = 0
    if ktail is not None:
        ktail = np.ascontiguousarray(ktail, dtype=np.float16)
        vtail = np.ascontiguousarray(vtail, dtype=np.float16)
        Tr = ktail.shape[0]
    O = np.empty((B, Hq, D), np.float32)
    lib().orc_attention(_p(kc), _p(_mi16(kmi)), _p(ksc), C.byref(km), _p(vc), _p(_mi16(vmi)), _p(vsc), C.byref(vm),
                        _i64(T), _i64(B), _i64(Hkv), _i64(Hq), _i64(D), _p(ktail), _p(vtail), _i64(Tr),
                        _p(q), C.c_float(scaling), _p(O))
    return O


def k_matvec(k, q):
    """k: f16 [ctx,1,H,D], q: f16 [1,H,D] -> f32 [ctx,1,H]."""
    k = np.ascontiguousarray(k, dtype=np.float16)
    q = np.ascontiguousarray(q, dtype=np.float16)
    ctx, _, H, D = k.shape
    out = np.empty((ctx, 1, H), np.float32)
    lib().orc_k_matvec(_p(k), _p(q), _i64(ctx), _i64(H), _i64(D), _p(out))
    return out
