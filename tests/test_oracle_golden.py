"""Pins the CPU checker (oracle/) against golden vectors produced by the reference itself
(tests/golden/make_golden.py): utils/compute.py for the quantiser and block cutter,
utils/huffman.py and src/huffman.cpp for the code assignment and tables."""
import json
import os

import numpy as np
import pytest

from oracle import kvc_oracle as orc

MODE = {"BlockQuant": orc.MODE_BLOCK, "ChannelQuant": orc.MODE_CHANNEL, "TokenQuant": orc.MODE_TOKEN,
        "VectorQuant": orc.MODE_VECTOR}


@pytest.fixture(scope="module")
def qg(golden_dir):
    z = np.load(os.path.join(golden_dir, "quant_golden.npz"))
    meta = json.loads(bytes(z["cases_json"]).decode())
    return z, meta


def _case_args(c):
    if c["api"] == "quant":      # the CUDA path's tables: the unit spans the batch
        mode = orc.MODE_BLOCK if c["dims"] == [1, 2, 3, 4] else orc.MODE_TOKEN
        return mode, True
    return MODE[c["mode"]], False


def test_quantiser_matches_reference(qg):
    z, meta = qg
    assert len(meta["cases"]) >= 10
    for c in meta["cases"]:
        mode, shared = _case_args(c)
        x = z[c["src"]]
        codes, mi, sc, m, deg, cf, mf = orc.quant(x, mode, c["block"], c["rel"], shared, raw=True)
        assert deg == 0
        name = c["name"]
        assert np.array_equal(sc.view(np.uint16), z[name + "_scale"].view(np.uint16)), name
        assert np.array_equal(mf.view(np.uint16), z[name + "_min"].view(np.uint16)), name
        assert np.array_equal(codes, z[name + "_codes"]), name
        assert np.array_equal(cf.astype(np.float32), codes.astype(np.float32)), name


def test_dequant_error_bound(qg):
    # src/compute.cpp:60-69: |x - x^| < 0.53 * scale.  x/scale is itself rounded to fp16, so at
    # small rel (quotients in the hundreds) the reference's own codes sit up to ~0.6 scale off.
    z, meta = qg
    for c in meta["cases"]:
        mode, shared = _case_args(c)
        x = z[c["src"]]
        codes, mi, sc, m, _ = orc.quant(x, mode, c["block"], c["rel"], shared)
        xh = orc.dequant(codes, mi, sc, m).astype(np.float32)
        T, B, H, D = x.shape
        t, b, h, d = np.meshgrid(np.arange(T), np.arange(B), np.arange(H), np.arange(D), indexing="ij")
        u = (t // m.tok_div) * m.sj + b * m.sb + h * m.sh + d * m.sc
        bound = (0.53 if c["rel"] >= 0.05 else 0.75) * sc.astype(np.float32)[u]
        assert (np.abs(x.astype(np.float32) - xh) < bound + 1e-6).all(), c["name"]


def test_cut_len(qg):
    _, meta = qg
    for ln, blk, recent, n in meta["cuts"]:
        assert orc.cut_len(ln, blk, recent) == n, (ln, blk, recent)


@pytest.fixture(scope="module")
def hg(golden_dir):
    with open(os.path.join(golden_dir, "huffman_golden.json")) as f:
        return json.load(f)


def _counts(case):
    h = np.zeros(256, np.int64)
    for k, v in case["counts"].items():
        h[int(k)] = v
    return h


def test_codes_match_python_and_cpp(hg):
    assert len(hg) >= 30
    n_cpp = 0
    for case in hg:
        h = _counts(case)
        enc, n = orc.gen_codes(h)
        assert n == len(case["counts"])
        assert orc.code_strings(enc) == {int(k): v for k, v in case["py_book"].items()}
        assert int((enc["length"].astype(np.int64) * h).sum()) == case["py_total_bits"]
        if case["cpp_encode"] is not None:
            n_cpp += 1
            tab, shift = orc.ref_encode_table(enc)
            assert shift == case["cpp_shift"]
            assert tab.tobytes().hex() == case["cpp_encode"]
            assert orc.ref_decode_tree(enc).tobytes().hex() == case["cpp_decode"]
    assert n_cpp >= 30


def test_flat_bitstream_matches_python(golden_dir):
    # utils/huffman.py concatenates the codes of the flattened tensor; K vectors in (token, column)
    # order are exactly that order, so stripping each vector's byte padding must give the same bits.
    z = np.load(os.path.join(golden_dir, "flat_golden.npz"))
    codes = z["codes"]
    enc, _ = orc.gen_codes(orc.histogram(codes))
    assert orc.code_strings(enc) == {int(k): v for k, v in json.loads(bytes(z["book_json"]).decode()).items()}
    data, bi, ti, ov = orc.encode(codes, True, enc)
    assert ov.sum() == 0
    off, num = orc.block_infos(bi)
    T, B, H, D = codes.shape
    cols = B * H
    bits = []
    for t in range(T):
        for col in range(cols):
            blk, v = (t // 64) * cols + col, t % 64
            start = (ti[blk * 64 + v - 1] >> 3) if v else 0
            end, pad = ti[blk * 64 + v] >> 3, ti[blk * 64 + v] & 7
            b = np.unpackbits(data[off[blk] + start: off[blk] + end])
            assert pad == 0 or not b[len(b) - pad:].any()
            bits.append(b[:len(b) - pad])
    bits = np.concatenate(bits)
    assert bits.size == int(z["nbits"])
    assert np.array_equal(np.packbits(bits), z["bits"])


@pytest.mark.parametrize("is_k", [True, False])
def test_roundtrip_and_layout(qg, is_k):
    z, _ = qg
    x = z["k" if is_k else "v"]
    codes, mi, sc, m, _ = orc.quant(x, orc.MODE_BLOCK if is_k else orc.MODE_TOKEN, 64, 0.05, True)
    enc, _ = orc.gen_codes(orc.histogram(codes))
    data, bi, ti, ov = orc.encode(codes, is_k, enc, base_offset=12345)
    off, num = orc.block_infos(bi)
    assert off[0] == 12345 and (np.diff(off.astype(np.int64)) == num[:-1]).all()
    assert num.sum() == data.size
    assert ((ti.reshape(-1, 64)[:, -1] >> 3) == num).all()
    bi0 = bi.copy()
    bi0.reshape(-1, 8)[:, :4] = (off - 12345).astype("<u4").view(np.uint8).reshape(-1, 4)
    T, B, H, D = codes.shape
    back, bad = orc.decode(data, bi0, ti, enc, T, B, H, is_k)
    assert bad == 0 and np.array_equal(back, codes)


def test_frozen_book_drops_unseen_symbols():
    # kernels.cu:197-205: a table entry of length 0 adds no bits (the reference drops the symbol)
    rng = np.random.default_rng(0)
    codes = rng.integers(0, 4, (64, 1, 1, 128)).astype(np.uint8)
    enc, _ = orc.gen_codes(orc.histogram(codes))
    codes2 = codes.copy()
    codes2[3, 0, 0, 7] = 9
    _, _, ti, ov = orc.encode(codes2, True, enc)
    assert ov[1] == 1


def test_attention_pieces_consistent(qg):
    # qk -> softmax -> pv assembled by hand equals the one-call attention of the checker
    z, _ = qg
    k, v = z["k"], z["v"]
    T, B, H, D = k.shape
    kc, kmi, ksc, km, _ = orc.quant(k, orc.MODE_CHANNEL, 64, 0.05, False)
    vc, vmi, vsc, vm, _ = orc.quant(v, orc.MODE_TOKEN, 64, 0.1, False)
    rng = np.random.default_rng(1)
    q = (rng.standard_normal((B, H, D)) / np.sqrt(D)).astype(np.float16)
    scaling = 1.0 / np.sqrt(D)
    S = orc.qk(kc, kmi, ksc, km, q).astype(np.float64) * scaling
    P = np.exp(S - S.max(-1, keepdims=True))
    P /= P.sum(-1, keepdims=True)
    O = orc.pv(vc, vmi, vsc, vm, P.astype(np.float32))
    O2 = orc.attention(kc, kmi, ksc, km, vc, vmi, vsc, vm, q, scaling)
    assert np.allclose(O, O2, rtol=1e-5, atol=1e-6)
    # against a numpy evaluation over the dequantised tensors
    kh = orc.dequant(kc, kmi, ksc, km).astype(np.float64)
    vh = orc.dequant(vc, vmi, vsc, vm).astype(np.float64)
    S3 = np.einsum("tbhd,bhd->bht", kh, q.astype(np.float64)) * scaling
    P3 = np.exp(S3 - S3.max(-1, keepdims=True)); P3 /= P3.sum(-1, keepdims=True)
    O3 = np.einsum("bht,tbhd->bhd", P3, vh)
    assert np.abs(O2 - O3).max() < 2e-3 * np.abs(O3).max()


def _rope_cpu(t, cos, sin):
    """utils/compute.py:25-33 on [B, H, t, D] fp16 tensors (torch on the CPU: every op rounds to fp16)."""
    import torch
    cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    half = t.shape[-1] // 2
    rot = torch.cat((-t[..., half:], t[..., :half]), dim=-1)
    return (t * cos) + (rot * sin)


def test_model_path_update_matches_reference(golden_dir):
    """What the reference's model-facing cache returns from update() (models/cache/kvcomp_quant.py:29-75 with
    utils/compute.py:quant_error) over a prefill and 45 single-token steps at batch 2, restated with the
    checker's quantiser, dequantiser and block cutter: units per sequence, min_ints not narrowed."""
    import hashlib
    import torch
    z = np.load(os.path.join(golden_dir, "update_golden.npz"))
    meta = json.loads(bytes(z["cases_json"]).decode())
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
    cos, sin = emb.cos().half()[None].expand(B, -1, -1), emb.sin().half()[None].expand(B, -1, -1)
    for c in meta["cases"]:
        kin = k.permute(1, 2, 0, 3)                                   # [B, H, T, D]
        if not c["pre_rope"]:
            kin = torch.cat([_rope_cpu(kin[:, :, a:b], cos[:, a:b], sin[:, a:b]) for a, b in zip(cuts[:-1], cuts[1:])], dim=2)
        streams = {}
        for tag, x, mode, blk, rec, rel in (("k", kin.permute(2, 0, 1, 3).contiguous().numpy(), c["k_mode"], c["k_block"], c["k_recent"], c["k_rel"]),
                                            ("v", v.numpy(), c["v_mode"], c["v_block"], c["v_recent"], c["v_rel"])):
            done, outs = 0, []                                        # tokens quantised so far
            xh = np.zeros_like(x)
            for b_ in cuts[1:]:
                n = orc.cut_len(b_ - done, blk, rec)
                if n:
                    codes, mi, sc, m, deg = orc.quant(x[done:done + n], MODE[mode], blk, rel, False)
                    assert deg == 0
                    xh[done:done + n] = orc.dequant(codes, mi, sc, m)
                    done += n
                outs.append(np.concatenate([xh[:done], x[done:b_]], axis=0))
            streams[tag] = outs
            assert done == c[tag + "_compressed"]
        for i, b_ in enumerate(cuts[1:]):
            K = torch.from_numpy(streams["k"][i]).permute(1, 2, 0, 3)
            V = torch.from_numpy(streams["v"][i]).permute(1, 2, 0, 3).contiguous()
            if c["pre_rope"]:
                K = _rope_cpu(K, cos[:, :b_], sin[:, :b_])
            K = K.contiguous()
            assert hashlib.sha256(K.numpy().tobytes()).hexdigest() == c["sha"][i][0], (c["name"], "K", i)
            assert hashlib.sha256(V.numpy().tobytes()).hexdigest() == c["sha"][i][1], (c["name"], "V", i)
        if c["name"] + "_K" in z:
            assert np.array_equal(K.numpy().view(np.uint16), z[c["name"] + "_K"].view(np.uint16))
