"""GPU tests of the reference-facing layers: the `kvcomp_cuda` operator module and the cache classes
(KVCompCtx, KVCompCache), written the way the reference's own scripts exercise them
(kvcomp_cuda_extension/scripts/test_py_ctx_k_2d_load.py, test_py_ctx_v.py, twice_get.py,
accuracy/reproduce_cuda_error.py), with the CPU checker as the referee."""
import hashlib
import json
import math
import os

import numpy as np
import pytest
import torch

from oracle import kvc_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def kc():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import kvcomp_b200.kvcomp_cuda as m
    return m


@pytest.fixture()
def cfg():
    from kvcomp_b200.utils.compute import QuantMode
    from kvcomp_b200.utils.config import KVCompCacheConfig, KVCompCacheConfigStatic

    def make(kmode="BlockQuant", vmode="TokenQuant", kblk=64, vblk=128, krec=0, vrec=0, krel=0.05, vrel=0.1, **kw):
        c = KVCompCacheConfig("synthetic", QuantMode(kmode), QuantMode(vmode), kblk, vblk, krec, vrec, krel, vrel, **kw)
        KVCompCacheConfigStatic.config = c
        return c
    yield make
    KVCompCacheConfigStatic.config = None


def synth(T, B, H, seed=0, Hq=None):
    from kvcomp_b200.synth import make_kv
    k, v, q = make_kv(T, B, H, 128, seed=seed, device="cpu", Hq=Hq)
    return k, v, q


def check_error(a, b, percentage):          # evaluation/cr_throughput_eval.py:18-20
    assert ((a - b).abs() < a.abs().max() * percentage).all(), "Error too large"


# ---- the operator module, called as models/cache/kvcomp_encode.py calls it ---------------------------
@pytest.mark.parametrize("is_k", [True, False])
def test_operator_module_roundtrip(kc, is_k):
    T, B, H = 256, 1, 4
    k, v, _ = synth(T, B, H, seed=1)
    x = (k if is_k else v).numpy()
    codes, mi, sc, m, _ = orc.quant(x, orc.MODE_BLOCK if is_k else orc.MODE_TOKEN, 64, 0.05, True)
    blk = 64 if is_k else 128
    quant_ints = torch.from_numpy(codes).cuda().view(-1, blk, B, H, 128)
    bsz, tsz, isz, cap = kc.calculate_buffer_size(quant_ints, is_k, H, 128)
    assert (bsz, tsz, isz, cap) == (T * B * H * 128 // 128 // 64 * 8, T * B * H * 128 // 128 * 2, 8, T * B * H * 128)
    shift, enc_book, dec_book = kc.build_codebook([quant_ints])
    assert shift == 0 and not enc_book.is_cuda and not dec_book.is_cuda
    oenc, _ = orc.gen_codes(orc.histogram(codes))
    otab, oshift = orc.ref_encode_table(oenc)
    assert np.array_equal(enc_book.numpy(), otab) and np.array_equal(dec_book.numpy(), orc.ref_decode_tree(oenc))
    bufs = [torch.zeros(n, dtype=torch.uint8, device="cuda") for n in (bsz, tsz, isz, cap)]
    encode = kc.k_entropy_encode_cuda_export if is_k else kc.v_entropy_encode_cuda_export
    enc_d, bi_d, ti_d = encode(quant_ints, enc_book.cuda(), bufs[0], bufs[1], bufs[2], bufs[3], 0, H, 128)
    odata, obi, oti, _ = orc.encode(codes, is_k, oenc)
    assert np.array_equal(enc_d.cpu().numpy(), odata)
    assert np.array_equal(bi_d.cpu().numpy(), obi) and np.array_equal(ti_d.cpu().numpy().view(np.uint16), oti)
    assert enc_d.data_ptr() == bufs[3].data_ptr()            # views into the caller's scratch, as in the reference
    out = torch.empty_like(quant_ints)
    decode = kc.k_entropy_decode_cuda_export if is_k else kc.v_entropy_decode_cuda_export
    ms = decode(enc_d, bi_d, ti_d, dec_book.cuda(), out, H, 128)
    assert ms > 0 and torch.equal(out, quant_ints)
    # fused half against the dense product over the dequantised tensor (the reference's own check)
    xh = torch.from_numpy(orc.dequant(codes, mi, sc, m).astype(np.float32)).cuda()
    mi8 = torch.from_numpy(orc.narrow_i8(mi)).cuda()
    scd = torch.from_numpy(sc).cuda()
    if is_k:
        q = torch.empty(B, H, 128, dtype=torch.float16, device="cuda").uniform_(-1, 1)
        C = torch.empty(B, H, T, dtype=torch.float16, device="cuda")
        ms = kc.k_decode_and_mat_vec_mul_cuda_export(dec_book.cuda(), bi_d, ti_d, enc_d, mi8, scd, q, C, H, 128)
        ref = torch.einsum("tbhc,bhc->bht", xh, q.float())
        check_error(ref, C.float(), 0.01)
        assert (C.float() - ref).abs().max() <= 2e-3 * ref.abs().max()
    else:
        P = torch.softmax(torch.randn(B, H, T, device="cuda") * 2.5, dim=-1).half()
        C = torch.empty(T // 128, B, H, 128, dtype=torch.float16, device="cuda")
        ms = kc.v_decode_and_mat_vec_mul_cuda_export(dec_book.cuda(), bi_d, ti_d, enc_d, mi8, scd, P, C, H, 128)
        ref = torch.einsum("bht,tbhc->bhc", P.float(), xh)
        check_error(ref, C.float().sum(0), 0.01)
    assert ms > 0


def test_operator_module_dense_matvec_and_errors(kc):
    from kvcomp_b200._lib import KvcError
    k = torch.randn(128, 1, 8, 128, device="cuda").half()
    q = torch.randn(1, 8, 128, device="cuda").half()
    out = torch.empty(128, 1, 8, dtype=torch.float16, device="cuda")
    assert kc.k_mat_vec_mul_cuda_export(k, q, out) > 0
    ref = torch.einsum("tbhc,bhc->tbh", k.float(), q.float())
    check_error(ref, out.float(), 0.01)
    with pytest.raises(KvcError):
        kc.k_mat_vec_mul_cuda_export(torch.cat([k, k], 1), q, out)            # "Batch size must be 1 for now"
    with pytest.raises(KvcError):
        kc.calculate_buffer_size(torch.zeros(1, 100, 1, 1, 128, dtype=torch.uint8, device="cuda"), True, 1, 128)
    with pytest.raises(KvcError):
        kc.build_codebook([torch.zeros(4, dtype=torch.float16, device="cuda")])
    assert (kc.K_VEC_LEN, kc.K_VEC_PER_BLK, kc.V_VEC_LEN, kc.V_VEC_PER_BLK) == (128, 64, 128, 64)


# ---- KVCompCtx ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("is_k", [True, False])
def test_ctx_twice_store_and_reads(cfg, is_k):
    """test_py_ctx_k_2d_load.py:77-84 / test_py_ctx_v.py:41-48: build the codebook from both chunks, store
    twice, the decoded codes equal the stored ones; then get(), mat_vec_mul() and get_cr()."""
    from kvcomp_b200.cache import KVCompCtx
    cfg()
    T, B, H = 512, 1, 4
    k, v, _ = synth(T, B, H, seed=3)
    x = (k if is_k else v).cuda()
    ctx = KVCompCtx(is_k, B, H, 128, 0.05 if is_k else 0.1)
    ctx.build_codebook([x[:256], x[256:]])
    q1 = ctx.store(x[:256])
    q2 = ctx.store(x[256:])
    stored = torch.cat([q1, q2], dim=0)
    decoded, ms = ctx.get_decode_quant_ints()
    assert ms > 0 and torch.equal(decoded, stored)
    # the codes are the reference's: same op sequence per store call
    rel = 0.05 if is_k else 0.1
    mode = orc.MODE_BLOCK if is_k else orc.MODE_TOKEN
    oc = np.concatenate([orc.quant(x[i:i + 256].cpu().numpy(), mode, 64 if is_k else 128, rel, True)[0] for i in (0, 256)])
    assert np.array_equal(stored.view(T, B, H, 128).cpu().numpy(), oc)
    full, _ = ctx.get()
    assert full.shape == (T, B, H, 128) and ctx.shape == torch.Size([T, B, H, 128])
    err = (full.float() - x.float()).abs()
    assert (err <= 0.53 * ctx.quant_scales.float().max()).all()               # src/compute.cpp:60-69
    if is_k:
        q = torch.empty(B, H, 128, dtype=torch.float16, device="cuda").uniform_(-1, 1)
        C, ms = ctx.mat_vec_mul(q)
        ref = torch.einsum("tbhc,bhc->bht", full.float(), q.float())
        assert C.shape == (B, H, T)
    else:
        P = torch.softmax(torch.randn(B, H, T, device="cuda") * 2.5, dim=-1).half()
        C, ms = ctx.mat_vec_mul(P)
        ref = torch.einsum("bht,tbhc->bhc", P.float(), full.float()).unsqueeze(0)
        assert C.shape == (1, B, H, 128)
    check_error(ref, C.float(), 0.01)
    # compression ratio accounting of kvcomp_encode.py:317-326
    comp = ctx.block_infos.numel() + ctx.thread_infos.numel() + ctx.encoded_data.numel() + \
        ctx.quant_min_ints.numel() + ctx.quant_scales.numel() * 2
    assert ctx.get_cr() == pytest.approx(2 * B * T * H * 128 / comp)
    assert 3.0 < ctx.get_cr() < 12.0
    assert ctx.quant_min_ints.shape[1:] == ((1, 1, 1, 1) if is_k else (128, 1, 1, 1))


def test_ctx_recent_window_and_token_by_token(cfg):
    """accuracy/reproduce_cuda_error.py:23-46: prefill 952 tokens, then one token at a time; the recent
    window stays uncompressed and get() always returns every token in order."""
    from kvcomp_b200.cache import KVCompCtx
    from kvcomp_b200.utils.compute import cut_len
    cfg(krec=128, vrec=256)
    B, H = 1, 2
    k, v, _ = synth(1100, B, H, seed=5)
    for is_k, x, blk, rec in ((True, k.cuda(), 64, 128), (False, v.cuda(), 128, 256)):
        ctx = KVCompCtx(is_k, B, H, 128, 0.05)
        ctx.store(x[:952])
        assert ctx.compressed_ctx_len == cut_len(952, blk, rec)
        n = 952
        for _ in range(140):
            ctx.store(x[n:n + 1])
            n += 1
        assert ctx.ctx_len == n and ctx.compressed_ctx_len + ctx.buffer.shape[0] == n
        assert ctx.buffer.shape[0] >= rec - blk and ctx.buffer.shape[0] < rec + blk
        full, _ = ctx.get()
        assert full.shape[0] == n
        assert torch.equal(full[ctx.compressed_ctx_len:], x[ctx.compressed_ctx_len:n])
        err = (full[:ctx.compressed_ctx_len].float() - x[:ctx.compressed_ctx_len].float()).abs().max()
        assert err <= 0.6 * ctx.quant_scales.float().max()


def test_ctx_channel_mode_per_sequence(cfg):
    """K per channel with per-sequence units and wide min_ints: what the benchmark configurations use."""
    from kvcomp_b200.cache import KVCompCtx
    cfg(kmode="ChannelQuant", quant_per_sequence=True, wide_min_ints=True)
    T, B, H = 256, 2, 2
    k, _, _ = synth(T, B, H, seed=6)
    ctx = KVCompCtx(True, B, H, 128, 0.05)
    stored = ctx.store(k.cuda())
    oc, omi, osc, om, _ = orc.quant(k.numpy(), orc.MODE_CHANNEL, 64, 0.05, False)
    assert np.array_equal(stored.view(T, B, H, 128).cpu().numpy(), oc)
    assert np.array_equal(ctx.quant_min_ints.view(-1).cpu().numpy(), omi)
    assert ctx.quant_min_ints.shape == (T // 64, 1, B, H, 128)
    full, _ = ctx.get()
    assert np.array_equal(full.cpu().numpy().view(np.uint16), orc.dequant(oc, omi, osc, om).view(np.uint16))


# ---- KVCompCache ------------------------------------------------------------------------------------------
def _rope(T, D=128):
    pos = torch.arange(T, dtype=torch.float32)
    inv = 1.0 / (10000 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    f = torch.outer(pos, inv)
    emb = torch.cat([f, f], dim=-1)
    return emb.cos()[None].half(), emb.sin()[None].half()            # [1, T, D]


@pytest.mark.parametrize("kmode,krec,vrec,Hkv,Hq", [("BlockQuant", 128, 256, 4, 4), ("ChannelQuant", 0, 0, 2, 8),
                                                     ("ChannelQuant", 128, 256, 2, 4)])
def test_cache_update_and_attend(cfg, kmode, krec, vrec, Hkv, Hq):
    """Prefill through update(), a few decode tokens through append() + attend(); the fused output equals
    eager attention (models/llama.py:211-234) over what update() returns."""
    from kvcomp_b200.cache import KVCompCache
    from kvcomp_b200.utils.compute import apply_rotary_pos_emb_single
    cfg(kmode=kmode, krec=krec, vrec=vrec, quant_per_sequence=True, wide_min_ints=True)
    B, T0, steps = 2, 700, 3
    k, v, _ = synth(T0 + steps, B, Hkv, seed=9, Hq=Hq)
    kk = k.permute(1, 2, 0, 3).contiguous().cuda()                   # [B, Hkv, T, D], as the model hands them over
    vv = v.permute(1, 2, 0, 3).contiguous().cuda()
    cos, sin = _rope(T0 + steps)
    cos, sin = cos.cuda(), sin.cuda()
    cache = KVCompCache(B, Hq, 128, layer_num=2)
    K, V = cache.update(kk[:, :, :T0], vv[:, :, :T0], 1, {"cos": cos[:, :T0], "sin": sin[:, :T0]})
    assert K.shape == (B, Hkv, T0, 128) and V.shape == (B, Hkv, T0, 128) and cache.get_seq_length(1) == T0
    assert cache.get_seq_length(0) == 0
    k_rot = apply_rotary_pos_emb_single(kk, cos, sin)
    # lossy, but the same tokens in the same order
    assert (K.float() - k_rot[:, :, :T0].float()).abs().max() <= 0.6 * cache.k_ctx[1].quant_scales.float().max() + 1e-3
    scaling = 1.0 / math.sqrt(128)
    for i in range(steps):
        t = T0 + i
        cache.append(kk[:, :, t:t + 1], vv[:, :, t:t + 1], 1, {"cos": cos[:, t:t + 1], "sin": sin[:, t:t + 1]})
        q = (torch.randn(B, Hq, 1, 128, device="cuda") / math.sqrt(128)).half()
        out = cache.attend(q, 1, scaling)
        assert out.shape == (B, Hq, 1, 128)
        # eager attention over the dequantised cache
        Kf = cache.k_ctx[1].get()[0].permute(1, 2, 0, 3).float().repeat_interleave(Hq // Hkv, dim=1)
        Vf = cache.v_ctx[1].get()[0].permute(1, 2, 0, 3).float().repeat_interleave(Hq // Hkv, dim=1)
        w = torch.softmax(torch.matmul(q.float(), Kf.transpose(2, 3)) * scaling, dim=-1)
        ref = torch.matmul(w, Vf)
        assert (out.float() - ref).abs().max() <= 1e-3 * ref.abs().max()
    assert cache.get_seq_length(1) == T0 + steps


def test_cache_disabled_quant_is_plain_concat(cfg):
    from kvcomp_b200.cache import KVCompCache
    cfg(enable_quant=False)
    B, H = 1, 2
    k = torch.randn(B, H, 10, 128, device="cuda").half()
    v = torch.randn(B, H, 10, 128, device="cuda").half()
    cos, sin = _rope(10)
    cache = KVCompCache(B, H, 128, 1)
    K, V = cache.update(k, v, 0, {"cos": cos.cuda(), "sin": sin.cuda()})
    assert torch.equal(V, v) and K.shape == k.shape and cache.get_seq_length(0) == 10


def test_ctx_save_load_roundtrip(cfg, tmp_path):
    """A cache written to disk and read back decodes to the same codes, keeps its recent window and
    accepts further stores."""
    from kvcomp_b200.cache import KVCompCtx
    cfg(kmode="ChannelQuant", krec=128, vrec=256, quant_per_sequence=True, wide_min_ints=True)
    B, H = 2, 2
    k, v, _ = synth(900, B, H, seed=12)
    for is_k, x in ((True, k.cuda()), (False, v.cuda())):
        ctx = KVCompCtx(is_k, B, H, 128, 0.05)
        ctx.store(x[:700])
        path = str(tmp_path / ("k.kvc" if is_k else "v.kvc"))
        hdr = ctx.save(path)
        assert hdr["compressed_ctx_len"] == ctx.compressed_ctx_len and "encoded" in hdr["sections"]
        back = KVCompCtx.load(path)
        assert back.compressed_ctx_len == ctx.compressed_ctx_len and back.ctx_len == 700
        assert torch.equal(back.get_decode_quant_ints()[0], ctx.get_decode_quant_ints()[0])
        assert torch.equal(back.get()[0], ctx.get()[0])
        ctx.store(x[700:])
        back.store(x[700:])
        assert torch.equal(back.get()[0], ctx.get()[0]) and back.get_cr() == pytest.approx(ctx.get_cr())


def test_evaluation_harness_keys(cfg):
    """The evaluation entry point of evaluation/cr_throughput_eval.py:128-240: same result keys, one value
    per layer, fused results within the reference's 1 % check."""
    from kvcomp_b200.evaluation import crs_throughputs_evaluation_with_data, quant_rel_to_bit_num
    c = cfg()
    B, H, T, L = 1, 4, 512, 2
    ks, vs = [], []
    for l in range(L):
        k, v, _ = synth(T, B, H, seed=40 + l)
        ks.append(k.permute(1, 2, 0, 3).contiguous().cuda())
        vs.append(v.permute(1, 2, 0, 3).contiguous().cuda())
    r = crs_throughputs_evaluation_with_data(c, ks, vs)
    for key in ("k_quant_crs", "v_quant_crs", "k_huffman_crs", "v_huffman_crs", "k_time_multi_kernels",
                "v_time_multi_kernels", "k_pytorch_mat_vec_mul_times", "v_pytorch_mat_vec_mul_times",
                "k_fused_mat_vec_mul_times", "v_fused_mat_vec_mul_times", "k_throughput_multi_kernels",
                "k_throughput_fused_kernels", "v_throughput_multi_kernels", "v_throughput_fused_kernels"):
        assert len(r[key]) == L, key
    assert all(x > 1.0 for x in r["k_huffman_crs"] + r["v_huffman_crs"])
    assert all(h > q * 0.9 for h, q in zip(r["k_huffman_crs"], r["k_quant_crs"]))
    assert quant_rel_to_bit_num(0.05) == 5 and quant_rel_to_bit_num(0.1) == 4


# ---- the model-facing cache against the reference's own update() ------------------------------------------
def _golden_inputs(meta):
    s, cuts = meta["shape"], meta["cuts"]
    g = torch.Generator().manual_seed(s["seed"])
    H, D, B, T = s["H"], s["D"], s["B"], cuts[-1]
    mu = 0.5 * torch.randn(H, D, generator=g)
    sd = torch.exp(0.5 * torch.randn(H, D, generator=g))
    sd = torch.where(torch.rand(H, D, generator=g) < 0.02, 8 * sd, sd)
    k = (mu + sd * torch.randn(T, B, H, D, generator=g)).half()
    r = torch.exp(0.25 * torch.randn(T, B, generator=g))
    v = (r[..., None, None] * torch.randn(T, B, H, D, generator=g)).half()
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    f = torch.outer(torch.arange(T, dtype=torch.float32), inv)
    emb = torch.cat((f, f), dim=-1)
    cos = emb.cos().half()[None].expand(B, -1, -1).contiguous()
    sin = emb.sin().half()[None].expand(B, -1, -1).contiguous()
    return k.permute(1, 2, 0, 3).contiguous().cuda(), v.permute(1, 2, 0, 3).contiguous().cuda(), cos.cuda(), sin.cuda()


def test_cache_update_returns_the_reference_values(cfg, golden_dir):
    """KVCompCache.update() with a reference-style configuration (no extra fields) at batch 2: after the
    prefill and after each of 45 single-token steps, K and V equal bit for bit what the reference's
    update() returned (tests/golden/update_golden.npz: models/cache/kvcomp_quant.py:29-75 run on the CPU),
    for five mode / block / recent-window / pre-RoPE settings.  V blocks of 64 tokens leave quantised
    tokens waiting for their 128-token Huffman vector."""
    from kvcomp_b200.cache import KVCompCache
    z = np.load(os.path.join(golden_dir, "update_golden.npz"))
    meta = json.loads(bytes(z["cases_json"]).decode())
    kk, vv, cos, sin = _golden_inputs(meta)
    s, cuts = meta["shape"], meta["cuts"]
    for c in meta["cases"]:
        cfg(kmode=c["k_mode"], vmode=c["v_mode"], kblk=c["k_block"], vblk=c["v_block"], krec=c["k_recent"],
            vrec=c["v_recent"], krel=c["k_rel"], vrel=c["v_rel"], enable_pre_rope=c["pre_rope"])
        cache = KVCompCache(s["B"], s["H"], s["D"], layer_num=1)
        for i, (a, b) in enumerate(zip(cuts[:-1], cuts[1:])):
            K, V = cache.update(kk[:, :, a:b], vv[:, :, a:b], 0, {"cos": cos[:, a:b], "sin": sin[:, a:b]})
            if i in (0, 1, 20, len(cuts) - 2) or i % 7 == 0:
                assert hashlib.sha256(K.contiguous().cpu().numpy().tobytes()).hexdigest() == c["sha"][i][0], (c["name"], "K", i)
                assert hashlib.sha256(V.contiguous().cpu().numpy().tobytes()).hexdigest() == c["sha"][i][1], (c["name"], "V", i)
        assert cache.k_ctx[0].compressed_ctx_len == c["k_compressed"] and cache.v_ctx[0].compressed_ctx_len == c["v_compressed"]
        assert cache.get_seq_length(0) == cuts[-1]
        if c["name"] + "_K" in z:
            assert np.array_equal(K.contiguous().cpu().numpy().view(np.uint16), z[c["name"] + "_K"].view(np.uint16))
            assert np.array_equal(V.contiguous().cpu().numpy().view(np.uint16), z[c["name"] + "_V"].view(np.uint16))


def test_ctx_rebook_when_a_frozen_book_meets_new_symbols(cfg):
    """A book frozen on a narrow sample, then data with symbols it has no code for: the reference drops them
    (kernels.cu:197-205), this context re-encodes once.  Codes, get() and the fused kernels still agree with
    the checker."""
    from kvcomp_b200.cache import KVCompCtx
    cfg(kmode="BlockQuant", vmode="TokenQuant", krec=0, vrec=0, krel=0.05, vrel=0.1)
    T, B, H = 512, 1, 2
    k, v, q = synth(T, B, H, seed=14)
    for is_k, x, mode, blk, rel in ((True, k, orc.MODE_BLOCK, 64, 0.05), (False, v, orc.MODE_TOKEN, 128, 0.1)):
        xd = x.cuda()
        ctx = KVCompCtx(is_k, B, H, 128, rel)
        narrow = (xd[:128] * 0.0 + xd[:128].mean()).half()
        narrow[::2] += 0.5                                            # two levels only: a book of very few symbols
        ctx.build_codebook([narrow])
        few = ctx.book.header()["n_symbols"]
        ctx.store(xd[:256])                                           # unseen symbols at the first store
        assert getattr(ctx, "rebooks", 0) == 1 and ctx.book.header()["n_symbols"] > few
        ctx.store(xd[256:])                                           # the rebuilt book covers every reachable code
        assert ctx.rebooks == 1
        oc = np.concatenate([orc.quant(x[i:i + 256].numpy(), mode, blk, rel, True)[0] for i in (0, 256)])
        decoded, _ = ctx.get_decode_quant_ints()
        assert np.array_equal(decoded.reshape(T, B, H, 128).cpu().numpy(), oc)
        full, _ = ctx.get()
        parts = [orc.quant(x[i:i + 256].numpy(), mode, blk, rel, True) for i in (0, 256)]
        want = np.concatenate([orc.dequant(p[0], p[1], p[2], p[3]) for p in parts])
        assert np.array_equal(full.cpu().numpy().view(np.uint16), want.view(np.uint16))
        if is_k:
            C, _ = ctx.mat_vec_mul(q.cuda())
            ref = torch.einsum("tbhc,bhc->bht", full.float(), q.cuda().float())
            check_error(ref, C.float(), 0.01)


class _TinyAttention(torch.nn.Module):
    """A minimal decoder attention layer in the shape of models/llama.py:236-308: q/k/v/o projections, rotary
    embedding on q here and on k inside the cache, grouped-query heads, and the cache hook."""

    def __init__(self, hidden, Hq, Hkv, layer_idx, seed):
        super().__init__()
        g = torch.Generator().manual_seed(seed)
        self.Hq, self.Hkv, self.D, self.layer_idx = Hq, Hkv, 128, layer_idx
        mk = lambda o, i: torch.nn.Parameter((torch.randn(o, i, generator=g) / math.sqrt(i)).half().cuda(), requires_grad=False)
        self.wq, self.wk, self.wv, self.wo = mk(Hq * 128, hidden), mk(Hkv * 128, hidden), mk(Hkv * 128, hidden), mk(hidden, Hq * 128)
        self.scaling = 1.0 / math.sqrt(128)

    def forward(self, x, cos, sin, cache, fused):
        from kvcomp_b200.utils.compute import apply_rotary_pos_emb_single
        B, t, _ = x.shape
        q = (x @ self.wq.T).view(B, t, self.Hq, 128).transpose(1, 2)
        k = (x @ self.wk.T).view(B, t, self.Hkv, 128).transpose(1, 2)
        v = (x @ self.wv.T).view(B, t, self.Hkv, 128).transpose(1, 2)
        q = apply_rotary_pos_emb_single(q, cos, sin)                    # models/llama.py:281
        kw = {"cos": cos, "sin": sin}
        if fused and t == 1:
            # the hook: two lines instead of update() + eager attention (models/llama.py:283-297)
            cache.append(k, v, self.layer_idx, kw)
            a = cache.attend(q, self.layer_idx, self.scaling)           # [B, Hq, 1, D]
        else:
            K, V = cache.update(k, v, self.layer_idx, kw)               # models/llama.py:283
            # eager_attention_forward, models/llama.py:211-234 (causal mask for the prefill)
            g = self.Hq // self.Hkv
            Kr, Vr = K.repeat_interleave(g, dim=1), V.repeat_interleave(g, dim=1)      # repeat_kv, :199-208
            w = torch.matmul(q, Kr.transpose(2, 3)) * self.scaling
            if t > 1:
                T = K.shape[2]
                mask = torch.full((t, T), float("-inf"), device=x.device).triu(T - t + 1)
                w = w + mask.to(w.dtype)
            w = torch.softmax(w, dim=-1, dtype=torch.float32).to(q.dtype)
            a = torch.matmul(w, Vr)
        return a.transpose(1, 2).reshape(B, t, self.Hq * 128) @ self.wo.T


def test_two_layer_decode_loop_through_the_hook(cfg):
    """A two-layer model decodes 600 tokens from an empty cache through append() + attend(), crossing K blocks,
    V vectors and both recent windows, starting before anything is compressed; a twin model with the same
    weights takes the reference's route (update() + eager attention).  The hidden states fed to both are the
    same, so every step compares one attention layer output: fused against eager over the dequantised cache."""
    from kvcomp_b200.cache import KVCompCache
    cfg(kmode="ChannelQuant", vmode="TokenQuant", kblk=64, vblk=64, krec=128, vrec=256, krel=0.05, vrel=0.1)
    B, hidden, Hq, Hkv, steps = 2, 256, 8, 2, 600
    layers = [_TinyAttention(hidden, Hq, Hkv, i, 100 + i) for i in range(2)]
    fused_cache, eager_cache = KVCompCache(B, Hq, 128, 2), KVCompCache(B, Hq, 128, 2)
    cos_all, sin_all = _rope(steps + 8)
    cos_all, sin_all = cos_all.cuda().expand(B, -1, -1), sin_all.cuda().expand(B, -1, -1)
    g = torch.Generator().manual_seed(7)
    worst = 0.0
    pos = 0
    for step in range(steps):
        t = 5 if step == 0 else 1                                        # a short prompt, then one token at a time
        x = torch.randn(B, t, hidden, generator=g).half().cuda()
        cos, sin = cos_all[:, pos:pos + t], sin_all[:, pos:pos + t]
        hf = he = x
        for layer in layers:
            of = layer(hf, cos, sin, fused_cache, fused=True)
            oe = layer(he, cos, sin, eager_cache, fused=False)
            err = (of.float() - oe.float()).abs().max().item() / max(oe.float().abs().max().item(), 1e-6)
            worst = max(worst, err)
            assert err <= 4e-3, (step, layer.layer_idx, err)             # two fp16 matmuls sit on top of the attention's 1e-3
            hf = he = (x + oe).half()                                    # both models continue from the same state
        pos += t
    fused_cache.check()
    for l in range(2):
        assert fused_cache.get_seq_length(l) == eager_cache.get_seq_length(l) == pos
        assert fused_cache.k_ctx[l].encoded_ctx_len >= 384 and fused_cache.v_ctx[l].encoded_ctx_len >= 256
    assert worst > 0.0


def test_attend_pre_rope_and_plain(cfg):
    """attend() also answers for caches the fused kernel cannot read directly: pre-RoPE keys (stored
    unrotated, rotated on the way out) and caches with quantisation switched off."""
    from kvcomp_b200.cache import KVCompCache
    B, Hkv, Hq, T = 1, 2, 4, 300
    k, v, q = synth(T, B, Hkv, seed=15, Hq=Hq)
    kk, vv = k.permute(1, 2, 0, 3).contiguous().cuda(), v.permute(1, 2, 0, 3).contiguous().cuda()
    cos, sin = _rope(T)
    kw = {"cos": cos.cuda(), "sin": sin.cuda()}
    qd = q.cuda().unsqueeze(2)
    for kwargs in (dict(enable_pre_rope=True, krec=64, vrec=64), dict(enable_quant=False)):
        cfg(kmode="ChannelQuant", **kwargs)
        cache = KVCompCache(B, Hq, 128, 1)
        K, V = cache.update(kk, vv, 0, kw)
        out = cache.attend(qd, 0)
        g = Hq // Hkv
        w = torch.softmax(torch.matmul(qd.float(), K.float().repeat_interleave(g, 1).transpose(2, 3)) / math.sqrt(128), dim=-1)
        ref = torch.matmul(w, V.float().repeat_interleave(g, 1))
        assert out.shape == (B, Hq, 1, 128) and (out.float() - ref).abs().max() <= 2e-3 * ref.abs().max()


def test_rope_store_equals_torch_ops():
    """kvc_rope_store against the reference's op sequence (utils/compute.py:25-33) evaluated by torch on
    CUDA fp16 tensors, followed by the transposition to token-major: the same bits, for batch-wide and
    broadcast cos / sin."""
    from kvcomp_b200 import ops
    from kvcomp_b200.utils.compute import apply_rotary_pos_emb_single
    g = torch.Generator().manual_seed(2)
    for B, H, t in ((2, 3, 37), (1, 8, 1), (3, 2, 200)):
        x = (torch.randn(B, H, t, 128, generator=g) * 3).half().cuda()
        cos, sin = _rope(t + 11)
        cos, sin = cos[:, 11:].cuda(), sin[:, 11:].cuda()
        want = apply_rotary_pos_emb_single(x, cos, sin).permute(2, 0, 1, 3).contiguous()
        assert torch.equal(ops.rope_store(x, cos, sin), want)
        assert torch.equal(ops.rope_store(x, cos.expand(B, -1, -1).contiguous(), sin.expand(B, -1, -1).contiguous()), want)
        # without cos / sin: the transposition alone (new values), into a row range of a larger buffer
        big = torch.zeros(t + 5, B, H, 128, dtype=torch.float16, device="cuda")
        ops.rope_store(x, None, None, out=big[3:3 + t])
        assert torch.equal(big[3:3 + t], x.permute(2, 0, 1, 3)) and not big[:3].any() and not big[3 + t:].any()
        # keys (rotated) and values (not rotated) in one launch
        y = (torch.randn(B, H, t, 128, generator=g) * 2).half().cuda()
        kout, vout = torch.zeros_like(want), torch.zeros_like(want)
        ops.kv_store(x, y, cos, sin, kout, vout)
        assert torch.equal(kout, want) and torch.equal(vout, y.permute(2, 0, 1, 3))


def test_ctx_stream_room_follows_the_density_seen(cfg):
    """The stream's arena grows by what the data needs (estimated from the density so far), not by one byte
    per symbol as the reference reserves; when a store is denser than the estimate allows, the encoder
    reports the room as exceeded and the store is repeated with the full reserve.  Same codes either way."""
    from kvcomp_b200.cache import KVCompCtx
    cfg(kmode="ChannelQuant", krec=0, vrec=0, quant_per_sequence=True, wide_min_ints=True)
    T, B, H = 512, 1, 4
    k, _, _ = synth(T, B, H, seed=16)
    wide = k.cuda()
    narrow = wide.clone()
    # every channel at its centre, two tokens per block keep the channel's range: nearly all codes are the
    # book's shortest (3 bits against 4.2 on average)
    narrow[:256] = ((wide.amin(dim=0, keepdim=True).float() + wide.amax(dim=0, keepdim=True).float()) / 2).half()
    narrow[0:256:64] = wide.amin(dim=0, keepdim=True)
    narrow[1:256:64] = wide.amax(dim=0, keepdim=True)
    ctx = KVCompCtx(True, B, H, 128, 0.05)
    ctx.build_codebook([wide])
    ctx.store(narrow[:256])
    low = ctx.encoded_data.numel()
    assert ctx._enc.buf.numel() == 256 * B * H * 128             # the first store cannot know better
    ctx.store(wide[256:])                                          # denser than the estimate allows: stored on the second try
    assert ctx.encoded_data.numel() > 2.3 * low and getattr(ctx, "rebooks", 0) == 0 and ctx.stream_retries == 1
    decoded, _ = ctx.get_decode_quant_ints()
    want = np.concatenate([orc.quant(x.cpu().numpy(), orc.MODE_CHANNEL, 64, 0.05, False)[0] for x in (narrow[:256], wide[256:])])
    assert np.array_equal(decoded.reshape(T, B, H, 128).cpu().numpy(), want)
    # a third store of the usual density fits the estimate: the arena grows by far less than a byte per symbol
    before = ctx._enc.buf.numel()
    ctx.store(wide[:256])
    assert ctx._enc.buf.numel() - before < 256 * B * H * 128
    assert ctx.compressed_ctx_len == 768


@pytest.mark.parametrize("is_k,rec", [(True, 128), (False, 128), (True, 0), (False, 300)])
def test_rows_behind_the_fused_range_come_from_one_buffer(cfg, is_k, rec):
    """tail_from(T): the dequantised values of the quantised tokens from T on followed by the recent window,
    kept in place in one buffer (appends of every size, compressions from the window's front, from a prefill
    and across both, the buffer's moves to its front, a reader that falls back behind the kept rows and a
    cache without kept rows)."""
    from kvcomp_b200.cache import KVCompCtx
    cfg(kmode="ChannelQuant", krec=rec, vrec=rec, quant_per_sequence=True, wide_min_ints=True)
    B, H = 2, 2
    total = 1500
    k, v, _ = synth(total, B, H, seed=71)
    x = (k if is_k else v).cuda()
    rng = np.random.default_rng(5)
    for keep in (True, False):
        ctx = KVCompCtx(is_k, B, H, 128, 0.05 if is_k else 0.1, keep_dequantised=keep)
        n, T = 0, 0
        sizes = [700] + [int(s) for s in rng.choice([1, 1, 1, 1, 2, 7, 64, 130, 200], size=400)]
        for step, t in enumerate(sizes):
            if n + t > total:
                break
            ctx.store(x[n:n + t].contiguous())
            n += t
            if step % 3 and keep:
                continue                                  # not every store is followed by a read
            top = ctx.encoded_ctx_len // 128 * 128
            if step % 17 == 5:
                T = max(0, top - 256)                     # a reader that falls back behind what was kept
            else:
                T = max(T, top - (128 if step % 2 else 0)) if top else 0
            T = min(T, top)
            got = ctx.tail_from(T)
            want = ctx.get()[0][T:]
            assert (got is None and want.shape[0] == 0) or torch.equal(got, want), (keep, step, n, T)
            if got is not None and keep:
                assert got.data_ptr() % 16 == 0 and got.is_contiguous()
        assert n > 1200
