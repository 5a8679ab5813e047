"""GPU tests of the reference-facing layers: the `kvcomp_cuda` operator module and the cache classes
(KVCompCtx, KVCompCache), written the way the reference's own scripts exercise them
(kvcomp_cuda_extension/scripts/test_py_ctx_k_2d_load.py, test_py_ctx_v.py, twice_get.py,
accuracy/reproduce_cuda_error.py), with the CPU checker as the referee."""
import math

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
