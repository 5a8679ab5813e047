"""Generate the golden fixtures in this folder from the reference itself.

Run once where the reference tree is at hand (REF=/path/to/reference):

    python tests/golden/make_golden.py

It imports the reference's Python CPU path unmodified (utils/compute.py,
utils/huffman.py) and the reference's own src/huffman.cpp compiled by
oracle/build_ref.py, runs them on small seeded inputs and stores inputs and outputs.
The fixtures travel with the repository; the reference tree does not have to exist
where the tests run.

Fixtures written:
  quant_golden.npz    inputs + (codes, min_int, scale) of utils/compute.py:quant (the CUDA
                      path's call, models/cache/kvcomp_encode.py:84) and :quant_ints
  huffman_golden.json per seeded histogram: the {symbol: bitstring} book of
                      utils/huffman.py:huffman_encode, its total bit count, and the
                      (shift, encode bytes, decode bytes) of src/huffman.cpp:build_codebook
  flat_golden.npz     a small code tensor and the flat bitstream utils/huffman.py makes of it
  update_golden.npz   what the model-facing cache returns (models/cache/kvcomp_quant.py:29-75: RoPE on the
                      new keys, utils/compute.py:quant_error for K and V) over a prefill followed by
                      single-token updates, batch 2, for five mode / block / pre-RoPE settings
"""
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, REPO)
from oracle import ref_root  # noqa: E402
REF = ref_root.require()
sys.path.insert(0, REF)

from utils.compute import (quant, quant_ints, QuantMode, cut_tensor_ctx_len_0, cut_tensor, quant_error,  # noqa: E402
                           apply_rotary_pos_emb_single, safe_cat)
from utils.huffman import huffman_encode  # noqa: E402
from oracle import build_ref  # noqa: E402


def synth_kv(T, B, H, D, seed):
    """Small K/V with the benchmark's distributions (per-channel outliers / per-token scale)."""
    g = torch.Generator().manual_seed(seed)
    mu = 0.5 * torch.randn(H, D, generator=g)
    s = torch.exp(0.5 * torch.randn(H, D, generator=g))
    s = torch.where(torch.rand(H, D, generator=g) < 0.02, 8 * s, s)
    k = mu + s * torch.randn(T, B, H, D, generator=g)
    r = torch.exp(0.25 * torch.randn(T, B, generator=g))
    v = r[..., None, None] * torch.randn(T, B, H, D, generator=g)
    return k.half(), v.half()


def narrow(qi):
    """fp16 code tensor -> uint8 as models/cache/kvcomp_encode.py:98 does, after checking that
    the narrowing loses nothing (integers in 0..255)."""
    f = qi.float()
    assert bool((f == f.round()).all()) and float(f.min()) >= 0 and float(f.max()) <= 255
    return qi.to(torch.uint8).numpy()


def make_quant():
    T, B, H, D = 256, 2, 2, 128
    k, v = synth_kv(T, B, H, D, 1234)
    out = {"k": k.numpy(), "v": v.numpy()}
    cases = []
    # the CUDA path's call: quant(x.view(-1, blk, B, H, D), dims, rel), kvcomp_encode.py:83-84
    for name, x, dims, blk, rel in (("cuda_block_k", k, [1, 2, 3, 4], 64, 0.05),
                                    ("cuda_block_k_02", k, [1, 2, 3, 4], 64, 0.02),
                                    ("cuda_token_v", v, [2, 3, 4], 128, 0.1),
                                    ("cuda_token_v_05", v, [2, 3, 4], 128, 0.05)):
        qi, mi, sc = quant(x.view(-1, blk, B, H, D).clone(), dims, rel)
        out[name + "_codes"] = narrow(qi.reshape(T, B, H, D))
        out[name + "_min"] = mi.reshape(-1).numpy()
        out[name + "_scale"] = sc.reshape(-1).numpy()
        cases.append({"name": name, "src": "k" if x is k else "v", "api": "quant", "dims": dims,
                      "block": blk, "rel": rel})
    # the simulated path's call: quant_ints(x[B,H,T,D], blk, rel, mode), utils/compute.py:74-91
    for name, x, mode, blk, rel in (("sim_channel_k", k, QuantMode.ChannelQuant, 64, 0.05),
                                    ("sim_channel_k_128", k, QuantMode.ChannelQuant, 128, 0.02),
                                    ("sim_channel_k_01", k, QuantMode.ChannelQuant, 64, 0.01),
                                    ("sim_block_k", k, QuantMode.BlockQuant, 64, 0.05),
                                    ("sim_token_v", v, QuantMode.TokenQuant, 64, 0.1),
                                    ("sim_token_v_015", v, QuantMode.TokenQuant, 128, 0.15),
                                    ("sim_vector_v", v, QuantMode.VectorQuant, 64, 0.2)):
        xb = x.permute(1, 2, 0, 3).contiguous()                     # [B,H,T,D]
        qi, mi, sc = quant_ints(xb, blk, rel, mode)                 # [B,H,nblk,blk,D], kept dims 1
        # back to token-major [T,B,H,D]; unit arrays to [nblk|T, B', H', D'] order
        out[name + "_codes"] = narrow(qi.reshape(B, H, T, D).permute(2, 0, 1, 3).contiguous())
        # unit tensors have shape [B,H,nblk,blk',D'] with 1s on reduced dims -> (nblk, blk', B, H, D')
        out[name + "_min"] = mi.permute(2, 3, 0, 1, 4).contiguous().reshape(-1).numpy()
        out[name + "_scale"] = sc.permute(2, 3, 0, 1, 4).contiguous().reshape(-1).numpy()
        cases.append({"name": name, "src": "k" if x is k else "v", "api": "quant_ints",
                      "mode": mode.value, "block": blk, "rel": rel})
    # block cutting, utils/compute.py:44-72
    cuts = []
    for ln, blk, recent in ((1024, 64, 128), (1000, 64, 128), (100, 64, 128), (1024, 64, 0), (953, 64, 128),
                            (1, 64, 128), (4096, 128, 256), (300, 128, 256), (129, 128, 0), (191, 64, 64)):
        to_c, buf = cut_tensor_ctx_len_0(None, torch.zeros(ln, 1, 1, 1), blk, recent, dim=0)
        to_c2, buf2 = cut_tensor(None, torch.zeros(1, 1, ln, 1), blk, recent, dim=2)
        n = 0 if to_c is None else to_c.shape[0]
        assert n == (0 if to_c2 is None else to_c2.shape[2])
        cuts.append([ln, blk, recent, n])
    out["cases_json"] = np.frombuffer(json.dumps({"cases": cases, "cuts": cuts}).encode(), dtype=np.uint8)
    np.savez_compressed(os.path.join(HERE, "quant_golden.npz"), **out)
    print("quant_golden.npz:", len(cases), "cases")


def histograms():
    rng = np.random.default_rng(7)
    hs = []
    # Gaussian-shaped code histograms like the quantiser produces (about 1/rel + 1 symbols)
    for nsym, sigma, total in ((22, 3.5, 20000), (12, 2.0, 12000), (7, 1.2, 9000), (52, 8.0, 30000),
                               (102, 16.0, 40000), (22, 3.0, 5000), (35, 6.0, 15000), (36, 6.0, 15000)):
        x = np.arange(nsym)
        p = np.exp(-0.5 * ((x - nsym / 2) / sigma) ** 2) + 1e-4
        c = rng.multinomial(total, p / p.sum())
        h = np.zeros(256, np.int64); h[:nsym] = c; hs.append(h)
    # tie-heavy: equal counts, powers of two, small integers
    for nsym in (2, 3, 4, 5, 8, 16, 17, 31, 64):
        h = np.zeros(256, np.int64); h[:nsym] = 10; hs.append(h)
    for nsym in (6, 11, 20):
        h = np.zeros(256, np.int64); h[:nsym] = 2 ** np.arange(nsym) % 97 + 1; hs.append(h)
    for _ in range(12):
        nsym = int(rng.integers(2, 40))
        h = np.zeros(256, np.int64); h[:nsym] = rng.integers(1, 6, nsym); hs.append(h)
    # gaps (symbols absent in the middle) and a non-zero smallest symbol
    h = np.zeros(256, np.int64); h[[0, 3, 4, 9, 200]] = [5, 1, 1, 7, 2]; hs.append(h)
    h = np.zeros(256, np.int64); h[[5, 6, 7, 9]] = [8, 4, 2, 2]; hs.append(h)
    # very skewed (long codes)
    h = np.zeros(256, np.int64); h[:18] = [2 ** max(0, 16 - i) for i in range(18)]; hs.append(h)
    return hs


def make_huffman():
    ref = build_ref.build()
    cases = []
    for h in histograms():
        sym = np.repeat(np.arange(256, dtype=np.uint8), h)
        t = torch.from_numpy(sym.copy())
        bits, book = huffman_encode(t)
        case = {"counts": {str(i): int(c) for i, c in enumerate(h) if c},
                "py_book": {str(k): v for k, v in book.items()},
                "py_total_bits": int(bits.numel()),
                "cpp_shift": None, "cpp_encode": None, "cpp_decode": None}
        # src/huffman.cpp keeps decode-tree child indices in int8 (include/huffman.h:18-22):
        # beyond 65 symbols (128 nodes) they wrap negative and build_decode_code_book writes
        # out of bounds (seen here as heap corruption), so the C++ twin is only run up to 65.
        if int((h > 0).sum()) <= 65:
            shift, enc, dec = ref.build_codebook([t])
            case.update(cpp_shift=int(shift), cpp_encode=enc.numpy().tobytes().hex(),
                        cpp_decode=dec.numpy().tobytes().hex())
        cases.append(case)
    # single distinct symbol: only the Python path defines it (the C++ path crashes)
    t = torch.full((100,), 3, dtype=torch.uint8)
    bits, book = huffman_encode(t)
    cases.append({"counts": {"3": 100}, "py_book": {str(k): v for k, v in book.items()},
                  "py_total_bits": int(bits.numel()), "cpp_shift": None, "cpp_encode": None, "cpp_decode": None})
    with open(os.path.join(HERE, "huffman_golden.json"), "w") as f:
        json.dump(cases, f)
    print("huffman_golden.json:", len(cases), "cases")


def make_flat():
    T, B, H, D = 128, 1, 2, 128
    k, _ = synth_kv(T, B, H, D, 99)
    qi, _, _ = quant(k.view(-1, 64, B, H, D).clone(), [1, 2, 3, 4], 0.05)
    codes = qi.to(torch.uint8).reshape(T, B, H, D)
    bits, book = huffman_encode(codes)
    np.savez_compressed(os.path.join(HERE, "flat_golden.npz"), codes=codes.numpy(),
                        bits=np.packbits(bits.numpy()), nbits=np.int64(bits.numel()),
                        book_json=np.frombuffer(json.dumps({str(k): v for k, v in book.items()}).encode(),
                                                dtype=np.uint8))
    print("flat_golden.npz:", bits.numel(), "bits")


UPDATE_CASES = (
    # name, K mode, K block, K recent, K rel, V mode, V block, V recent, V rel, pre-RoPE
    ("channel_token", "ChannelQuant", 64, 64, 0.05, "TokenQuant", 64, 32, 0.1, False),
    ("block_token", "BlockQuant", 64, 64, 0.05, "TokenQuant", 64, 32, 0.1, False),
    ("channel128_vector", "ChannelQuant", 128, 32, 0.02, "VectorQuant", 128, 64, 0.15, False),
    ("vector_block", "VectorQuant", 64, 32, 0.1, "BlockQuant", 64, 64, 0.05, False),
    ("channel_token_prerope", "ChannelQuant", 64, 64, 0.05, "TokenQuant", 64, 32, 0.1, True),
)
UPDATE_SHAPE = dict(B=2, H=2, D=128, prefill=150, steps=45, seed=4321)


def rope_tables(B, t0, t1, D):
    """cos / sin [B, t1 - t0, D] as a Llama rotary embedding hands them to the attention layers."""
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    pos = torch.arange(t0, t1, dtype=torch.float32)
    f = torch.outer(pos, inv)
    emb = torch.cat((f, f), dim=-1)
    return emb.cos().half()[None].expand(B, -1, -1).contiguous(), emb.sin().half()[None].expand(B, -1, -1).contiguous()


def update_inputs():
    """The key / value states [B, H, T, D] fed to the cache, chunk by chunk."""
    s = UPDATE_SHAPE
    T = s["prefill"] + s["steps"]
    k, v = synth_kv(T, s["B"], s["H"], s["D"], s["seed"])            # [T, B, H, D]
    k, v = k.permute(1, 2, 0, 3).contiguous(), v.permute(1, 2, 0, 3).contiguous()
    cuts = [0, s["prefill"]] + [s["prefill"] + i + 1 for i in range(s["steps"])]
    return k, v, cuts


def make_update():
    import hashlib
    s = UPDATE_SHAPE
    k, v, cuts = update_inputs()
    out = {}
    meta = []
    for name, km, kb, kr, krel, vm, vb, vr, vrel, pre in UPDATE_CASES:
        ck = cv = bk = bv = None
        coss = sins = None
        shas = []
        for a, b in zip(cuts[:-1], cuts[1:]):
            ks, vs = k[:, :, a:b], v[:, :, a:b]
            cos, sin = rope_tables(s["B"], a, b, s["D"])
            # models/cache/kvcomp_quant.py:43-75
            if pre:
                coss, sins = safe_cat(coss, cos, dim=1), safe_cat(sins, sin, dim=1)
            else:
                ks = apply_rotary_pos_emb_single(ks, cos, sin)
            ck, bk = quant_error(ck, bk, ks, kb, kr, krel, QuantMode(km))
            cv, bv = quant_error(cv, bv, vs, vb, vr, vrel, QuantMode(vm))
            K, V = safe_cat(ck, bk, dim=2), safe_cat(cv, bv, dim=2)
            if pre:
                K = apply_rotary_pos_emb_single(K, coss, sins)
            shas.append([hashlib.sha256(K.contiguous().numpy().tobytes()).hexdigest(),
                         hashlib.sha256(V.contiguous().numpy().tobytes()).hexdigest()])
        meta.append({"name": name, "k_mode": km, "k_block": kb, "k_recent": kr, "k_rel": krel, "v_mode": vm,
                     "v_block": vb, "v_recent": vr, "v_rel": vrel, "pre_rope": pre, "sha": shas,
                     "k_compressed": 0 if ck is None else int(ck.shape[2]), "v_compressed": 0 if cv is None else int(cv.shape[2])})
        if name in ("channel_token", "channel_token_prerope"):
            out[name + "_K"], out[name + "_V"] = K.contiguous().numpy(), V.contiguous().numpy()
    out["cases_json"] = np.frombuffer(json.dumps({"cases": meta, "shape": s, "cuts": cuts}).encode(), dtype=np.uint8)
    np.savez_compressed(os.path.join(HERE, "update_golden.npz"), **out)
    print("update_golden.npz:", len(meta), "cases,", [(m["k_compressed"], m["v_compressed"]) for m in meta])


if __name__ == "__main__":
    if "--update-only" in sys.argv:
        make_update()
        sys.exit(0)
    make_quant()
    make_huffman()
    make_flat()
    make_update()
