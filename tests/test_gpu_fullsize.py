"""Size-independent properties at the sizes the benchmark configurations name, where the CPU checker would
take minutes: exact encode -> decode round trips, the bookkeeping of the stream (offsets are the prefix sums of
the block sizes, the histogram counts every symbol, the codes satisfy Kraft's equality), the quantiser's error
bound, and the fused attention against a plain fp32 torch evaluation of the same attention over the
dequantised cache (tolerance 1e-3 of the largest output magnitude, the bound the path's specification states;
2e-3 per element plus a floor, as for the small cases)."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from kvcomp_b200 import ops as _ops
    return _ops


def _store(ops, x, is_k, mode, block, rel, may_overflow=False):
    T, B, H, D = x.shape
    hist = torch.zeros(256, dtype=torch.int64, device=x.device)
    codes, mi, sc, spec, st = ops.quantize(x, mode, block, rel, False, min_dtype=torch.int16, hist=hist)
    assert ops.read_status(st) & 0x4 == 0
    book = ops.build_codebook(hist)
    bsz, tsz, _, cap = ops.buffer_sizes(T, B * H * D, is_k)
    bi = torch.zeros(bsz, dtype=torch.uint8, device=x.device)
    ti = torch.zeros(tsz // 2, dtype=torch.int16, device=x.device)
    enc = torch.empty(cap, dtype=torch.uint8, device=x.device)
    total, st = ops.encode(codes, is_k, book.encode_table(), bi, ti, enc)
    flags = ops.read_status(st, raise_on_fatal=False)
    if may_overflow and flags & 0x20:              # a block beyond the 8191 bytes the format can describe
        return None
    assert flags & ~0x10 == 0                      # a vector beyond the reference's scratch size is only reported
    n, maxb = (int(t) for t in total.tolist())
    return dict(codes=codes, mi=mi, sc=sc, spec=spec, hist=hist, book=book, bi=bi, ti=ti, enc=enc, n=n, maxb=maxb)


def _check_stream_bookkeeping(r, is_k):
    codes = r["codes"]
    T, B, H, D = codes.shape
    nblk = (T // 64) * B * H if is_k else (T // 128) * B * H * 2
    rec = r["bi"].cpu().numpy().view(np.dtype([("off", "<u4"), ("n", "<u2"), ("pad", "<u2")]))
    assert rec.size == nblk and not rec["pad"].any()
    sizes = rec["n"].astype(np.int64)
    assert int(sizes.sum()) == r["n"] and int(sizes.max()) == r["maxb"]
    assert np.array_equal(rec["off"].astype(np.int64), np.concatenate(([0], np.cumsum(sizes)[:-1])))
    # thread_info: (end byte << 3) | pad bits, ends ascending inside a block, the last one the block's size
    tinfo = r["ti"].cpu().numpy().view(np.uint16).reshape(nblk, 64)
    ends = (tinfo >> 3).astype(np.int64)
    assert (np.diff(ends, axis=1) >= 16).all() and np.array_equal(ends[:, -1], sizes)
    # the histogram counts every symbol once; the book's code lengths give the stream's bit count exactly
    hist = r["hist"].cpu().numpy()
    assert int(hist.sum()) == codes.numel()
    assert np.array_equal(hist, torch.bincount(codes.view(-1).int(), minlength=256).cpu().numpy())
    lens = r["book"].host()[64:64 + 2048].numpy().view(np.uint32).reshape(256, 2)[:, 1].astype(np.int64)
    assert ((lens > 0) == (hist > 0)).all()
    if (hist > 0).sum() > 1:
        assert abs(sum(2.0 ** -int(l) for l in lens if l) - 1.0) < 1e-12        # Kraft: a full binary tree
    bits = int((hist * lens).sum())
    pad_bits = int((tinfo & 7).astype(np.int64).sum())
    assert bits + pad_bits == 8 * r["n"]


def _check_error_bound(ops, x, r, rel):
    """|x - x_hat| <= scale / 2 up to fp16 rounding of the quotient and of the product."""
    xh = ops.dequant(r["codes"], r["mi"], r["sc"], r["spec"])
    err = (xh.float() - x.float()).abs().max().item()
    top_scale = r["sc"].float().max().item()
    assert err <= 0.5 * top_scale * 1.01 + 2.0 ** -10 * x.float().abs().max().item()
    return xh


CONFIGS = {  # the layer shapes of the benchmark's configurations (one layer each)
    "c1": dict(T=4096, B=8, Hkv=32, Hq=32, kblock=64, krel=0.05, vrel=0.1),
    "c2": dict(T=32768, B=16, Hkv=8, Hq=32, kblock=64, krel=0.05, vrel=0.1),
    "c3": dict(T=16384, B=32, Hkv=10, Hq=40, kblock=128, krel=0.02, vrel=0.15),
}


@pytest.mark.parametrize("name", ["c1", "c2", "c3"])
def test_full_size_layer_round_trip_and_attention(ops, name):
    from kvcomp_b200.synth import make_kv
    c = CONFIGS[name]
    T, B, Hkv, Hq = c["T"], c["B"], c["Hkv"], c["Hq"]
    k, v, q = make_kv(T, B, Hkv, 128, seed=31, layer=0, device="cuda", Hq=Hq)
    rk = _store(ops, k, True, ops.MODE_CHANNEL, c["kblock"], c["krel"])
    rv = _store(ops, v, False, ops.MODE_TOKEN, 128, c["vrel"])
    for r, is_k in ((rk, True), (rv, False)):
        _check_stream_bookkeeping(r, is_k)
        back, st = ops.decode(r["enc"][:r["n"]], r["bi"], r["ti"], r["book"], T, B, Hkv, is_k, max_block=r["maxb"])
        assert ops.read_status(st) == 0 and torch.equal(back, r["codes"])
        del back
    kh = _check_error_bound(ops, k, rk, c["krel"])
    vh = _check_error_bound(ops, v, rv, c["vrel"])
    del k, v
    kc = ops.make_cache(rk["enc"], rk["bi"], rk["ti"], rk["book"], rk["mi"], rk["sc"], rk["spec"], rk["n"], rk["maxb"])
    vc = ops.make_cache(rv["enc"], rv["bi"], rv["ti"], rv["book"], rv["mi"], rv["sc"], rv["spec"], rv["n"], rv["maxb"])
    scaling = 1.0 / math.sqrt(128)
    out, st = ops.attn_decode(kc, vc, T, B, Hkv, q, scaling)
    assert ops.read_status(st) == 0
    # plain torch, fp32, one sequence at a time: softmax(q K^T * scaling) V over the dequantised cache
    g = Hq // Hkv
    worst, worst_elem = 0.0, 0.0
    for b in range(B):
        kb = kh[:, b].float().permute(1, 0, 2)                       # [Hkv, T, 128]
        vb = vh[:, b].float().permute(1, 0, 2)
        qb = q[b].float().view(Hkv, g, 128)
        s = torch.einsum("hgd,htd->hgt", qb, kb) * scaling
        o = torch.einsum("hgt,htd->hgd", torch.softmax(s, dim=-1), vb).reshape(Hq, 128)
        err = (out[b].float() - o).abs()
        top = o.abs().max().item()
        worst = max(worst, err.max().item() / top)
        worst_elem = max(worst_elem, ((err - 2e-4 * top) / (o.abs() + 1e-30)).max().item())
    assert worst <= 1e-3, worst
    assert worst_elem <= 2e-3, worst_elem
    # the split of the work among CTAs does not change the result beyond rounding
    out2, st = ops.attn_decode(kc, vc, T, B, Hkv, q, scaling, splits=2)
    assert ops.read_status(st) == 0
    assert (out2.float() - out.float()).abs().max().item() <= 2e-3 * out.float().abs().max().item()


@pytest.mark.parametrize("rel", [0.01, 0.05, 0.2])
def test_full_size_codec_chunk_round_trip(ops, rel):
    """The prefill-side chunk: 32 heads x 128, batch 32, 4096 tokens (1 GiB of fp16 per tensor)."""
    from kvcomp_b200.synth import make_kv
    T, B, H = 4096, 32, 32
    k, v, _ = make_kv(T, B, H, 128, seed=5, layer=0, device="cuda")
    for x, is_k, mode, blk in ((k, True, ops.MODE_CHANNEL, 64), (v, False, ops.MODE_TOKEN, 128)):
        r = _store(ops, x, is_k, mode, blk, rel)
        _check_stream_bookkeeping(r, is_k)
        back, st = ops.decode(r["enc"][:r["n"]], r["bi"], r["ti"], r["book"], T, B, H, is_k, max_block=r["maxb"])
        assert ops.read_status(st) == 0 and torch.equal(back, r["codes"])
        del back
        _check_error_bound(ops, x, r, rel)
        # a second store of the same chunk with the frozen book writes the same stream (the encoder is deterministic)
        bi2, ti2, enc2 = torch.zeros_like(r["bi"]), torch.zeros_like(r["ti"]), torch.empty_like(r["enc"])
        total, st = ops.encode(r["codes"], is_k, r["book"].encode_table(), bi2, ti2, enc2)
        assert ops.read_status(st) == 0 and int(total[0]) == r["n"]
        assert torch.equal(enc2[:r["n"]], r["enc"][:r["n"]]) and torch.equal(bi2, r["bi"]) and torch.equal(ti2, r["ti"])
        del r, bi2, ti2, enc2


def _exact(codes, mi, sc, spec):
    """(code + min_int) * scale in float64, unit of element (t, b, h, c) = (t / tok_div) sj + b sb + h sh + c sc."""
    T, B, H, D = codes.shape
    dev = codes.device
    t = torch.arange(T, device=dev).view(T, 1, 1, 1) // spec.tok_div
    u = (t * spec.sj + torch.arange(B, device=dev).view(1, B, 1, 1) * spec.sb
         + torch.arange(H, device=dev).view(1, 1, H, 1) * spec.sh + torch.arange(D, device=dev).view(1, 1, 1, D) * spec.sc)
    return (codes.double() + mi.view(-1)[u].double()) * sc.view(-1)[u].double()


def test_attention_random_shapes_against_float64(ops):
    """Random context lengths (with and without compressed part and fp16 tail), batch, KV heads, query heads per
    KV head, quantiser modes, error bounds and work splits: the fused attention against float64 torch attention
    over the exact dequantised values, 1e-3 of the largest output magnitude."""
    from kvcomp_b200.synth import make_kv
    rng = np.random.default_rng(99)
    worst, checked = 0.0, 0
    for case in range(64):
        T = int(rng.integers(0, 24)) * 128
        Tr = int(rng.integers(0, 300)) if T else int(rng.integers(1, 300))
        B, Hkv = int(rng.integers(1, 5)), int(rng.integers(1, 6))
        G = [1, 1, 2, 3, 4, 5, 8][case % 7]
        Hq = Hkv * G
        krel, vrel = float(rng.choice([0.02, 0.05, 0.1])), float(rng.choice([0.05, 0.1, 0.15]))
        kmode, kblock = [(ops.MODE_CHANNEL, 64), (ops.MODE_CHANNEL, 128), (ops.MODE_BLOCK, 64), (ops.MODE_TOKEN, 64)][case % 4]
        k, v, q = make_kv(T + Tr, B, Hkv, 128, seed=1000 + case, layer=0, device="cuda", Hq=Hq)
        kc = vc = None
        ke, ve = k[:0].double(), v[:0].double()
        if T:
            rk = _store(ops, k[:T].contiguous(), True, kmode, kblock, krel, may_overflow=True)
            rv = _store(ops, v[:T].contiguous(), False, ops.MODE_TOKEN, 128, vrel, may_overflow=True)
            if rk is None or rv is None:
                continue
            kc = ops.make_cache(rk["enc"], rk["bi"], rk["ti"], rk["book"], rk["mi"], rk["sc"], rk["spec"], rk["n"], rk["maxb"])
            vc = ops.make_cache(rv["enc"], rv["bi"], rv["ti"], rv["book"], rv["mi"], rv["sc"], rv["spec"], rv["n"], rv["maxb"])
            ke, ve = _exact(rk["codes"], rk["mi"], rk["sc"], rk["spec"]), _exact(rv["codes"], rv["mi"], rv["sc"], rv["spec"])
        kt = k[T:].contiguous() if Tr else None
        vt = v[T:].contiguous() if Tr else None
        scaling = 1.0 / math.sqrt(128)
        out, st = ops.attn_decode(kc, vc, T, B, Hkv, q, scaling, kt, vt, splits=[0, 0, 1, 2, 3][case % 5])
        assert ops.read_status(st) == 0, case
        checked += 1
        ke, ve = torch.cat([ke, k[T:].double()], 0), torch.cat([ve, v[T:].double()], 0)
        for b in range(B):
            s = torch.einsum("hgd,htd->hgt", q[b].double().view(Hkv, G, 128), ke[:, b].permute(1, 0, 2)) * scaling
            o = torch.einsum("hgt,htd->hgd", torch.softmax(s, -1), ve[:, b].permute(1, 0, 2)).reshape(Hq, 128)
            e = ((out[b].double() - o).abs().max() / o.abs().max()).item()
            worst = max(worst, e)
            assert e <= 1e-3, (case, e, T, Tr, B, Hkv, G)
    assert checked >= 48 and worst > 0.0
