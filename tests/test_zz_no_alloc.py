"""The allocation-free attention entry point (kvc_attn_decode_static), called through the C ABI.

It exists for hosts that are not allowed to allocate device memory themselves -- a serving process
whose memory pool owns the whole device, a plugin that must stay inside a fixed memory budget -- so its
split-KV scratch is a fixed array inside the library.  The test checks that it gives exactly the result
of kvc_attn_decode (which takes a caller workspace) on two calls in a row, that the shared scratch does
not leak state from one call into the next, and that sizes beyond the built-in array are refused.
This file sorts last on purpose: a run that stops at the first failure has then run every other test."""
import ctypes as C
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _cache(ops, x, is_k, mode, rel):
    T, B, H, _ = x.shape
    hist = torch.zeros(256, dtype=torch.int64, device="cuda")
    codes, mi, sc, spec, st = ops.quantize(x, mode, 64 if is_k else 128, rel, False, min_dtype=torch.int16, hist=hist)
    book = ops.build_codebook(hist)
    bsz, tsz, _, cap = ops.buffer_sizes(T, B * H * 128, is_k)
    bi = torch.zeros(bsz, dtype=torch.uint8, device="cuda")
    ti = torch.zeros(tsz // 2, dtype=torch.int16, device="cuda")
    enc = torch.zeros(cap, dtype=torch.uint8, device="cuda")
    total, st2 = ops.encode(codes, is_k, book.encode_table(), bi, ti, enc)
    n, maxb = (int(v) for v in total.tolist())
    ops.read_status(st); ops.read_status(st2)
    keep = (enc, bi, ti, book, mi, sc)
    return ops.make_cache(enc, bi, ti, book, mi, sc, spec, n, maxb), keep


def test_static_scratch_entry_point_matches_workspace_entry_point():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from kvcomp_b200 import _lib, ops
    from kvcomp_b200.synth import make_kv
    lib = _lib.load()
    T, B, Hkv, Hq, Tr, splits = 1024, 2, 2, 8, 70, 3
    k, v, q = make_kv(T + Tr, B, Hkv, 128, seed=77, device="cpu", Hq=Hq)
    k, v = k.cuda(), v.cuda()
    kc, keep_k = _cache(ops, k[:T].contiguous(), True, ops.MODE_CHANNEL, 0.05)
    vc, keep_v = _cache(ops, v[:T].contiguous(), False, ops.MODE_TOKEN, 0.1)
    ktail, vtail = k[T:].contiguous(), v[T:].contiguous()
    scaling = 1.0 / math.sqrt(128)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: C.c_void_p(t.data_ptr())
    status = ops.new_status("cuda")
    assert lib.kvc_attn_static_capacity() == 4 << 20
    for call in range(2):                         # two calls in a row, different queries
        qd = (q * (1 + call)).cuda().contiguous()
        want, st = ops.attn_decode(kc, vc, T, B, Hkv, qd, scaling, ktail, vtail, splits=splits)
        assert ops.read_status(st) == 0
        got = torch.full((B, Hq, 128), float("nan"), dtype=torch.float16, device="cuda")
        rc = lib.kvc_attn_decode_static(C.byref(kc), C.byref(vc), T, B, Hkv, Hq, p(qd), scaling, p(ktail), p(vtail), Tr,
                                        p(got), splits, p(status), stream)
        assert rc == 0, lib.kvc_last_error()
        assert ops.read_status(status) == 0
        assert torch.equal(got, want)             # same kernel, same split count: the same bits
        # through the Python wrapper as well, with the split count left to the library
        got2 = torch.empty_like(got)
        ops.attn_decode_static(kc, vc, T, B, Hkv, qd, scaling, got2, ktail, vtail, status=status)
        want2, _ = ops.attn_decode(kc, vc, T, B, Hkv, qd, scaling, ktail, vtail)
        assert ops.read_status(status) == 0 and torch.equal(got2, want2)
    # against the CPU checker as well, not only against the library's other entry point
    import numpy as np
    from oracle import kvc_oracle as orc
    kq = orc.quant(k[:T].cpu().numpy(), orc.MODE_CHANNEL, 64, 0.05, False)[:4]
    vq = orc.quant(v[:T].cpu().numpy(), orc.MODE_TOKEN, 128, 0.1, False)[:4]
    O = orc.attention(*kq, *vq, qd.cpu().numpy(), scaling, ktail.cpu().numpy(), vtail.cpu().numpy())
    assert np.abs(got.float().cpu().numpy() - O).max() <= 1e-3 * np.abs(O).max()
    # more splits than a column has tiles: the split count is clamped before the scratch is sized, so a
    # request like 256 heads x 64 splits over 4 tiles fits (it needs about 1 MB, not 17)
    Tb, Bb, Hb = 1024, 8, 32
    kb, vb, qb = make_kv(Tb, Bb, Hb, 128, seed=78, device="cpu")
    kcb, keep_kb = _cache(ops, kb.cuda(), True, ops.MODE_CHANNEL, 0.05)
    vcb, keep_vb = _cache(ops, vb.cuda(), False, ops.MODE_TOKEN, 0.1)
    gotb = torch.empty((Bb, Hb, 128), dtype=torch.float16, device="cuda")
    qbd = qb.cuda()
    rc = lib.kvc_attn_decode_static(C.byref(kcb), C.byref(vcb), Tb, Bb, Hb, Hb, p(qbd), scaling, None, None, 0,
                                    p(gotb), 64, p(status), stream)
    assert rc == 0, lib.kvc_last_error()
    wantb, _ = ops.attn_decode(kcb, vcb, Tb, Bb, Hb, qbd, scaling, splits=64)
    assert ops.read_status(status) == 0 and torch.equal(gotb, wantb)
    # a request whose scratch does not fit the built-in array is refused with a clear error
    rc = lib.kvc_attn_decode_static(C.byref(kc), C.byref(vc), T, 4096, Hkv, 4096 * 4, p(qd), scaling, None, None, 0,
                                    p(got), 4, p(status), stream)
    assert rc == 3 and b"built-in" in lib.kvc_last_error()
