"""GPU parity against the reference's own CUDA kernels: streams, tables and fused outputs that the
unmodified kvcomp_cuda module produced on a B200 (tests/golden/ref_cuda_golden.npz) go through
libkvcomp_b200.so, and this library's encoder is held to the reference's blocks byte for byte."""
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
def ops():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from kvcomp_b200 import ops as _ops
    return _ops


@pytest.fixture(scope="module")
def rg(golden_dir):
    z = np.load(os.path.join(golden_dir, "ref_cuda_golden.npz"))
    return z, json.loads(bytes(z["cases_json"]).decode())["cases"]


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def inputs(c):
    from kvcomp_b200.synth import make_kv
    k, v, q = make_kv(c["T"], 1, c["H"], 128, seed=c["seed"], device="cpu")
    return k, v, q


def ref_cache(ops, z, p, spec, mi, sc):
    """A kvc_cache over the reference's stream and tables, with a book made from its decode tensor."""
    book = ops.book_from_tree(dev(z[p + "dec_book"]))
    enc = dev(np.concatenate([z[p + "encoded"], np.zeros(64, np.uint8)]))      # readable to the next 16-byte boundary
    bi, ti = dev(z[p + "block_info"]), dev(z[p + "thread_info"])
    keep = (book, enc, bi, ti, mi, sc)
    return ops.make_cache(enc, bi, ti, book, mi, sc, spec, z[p + "encoded"].size), keep


@pytest.mark.parametrize("tag", ["k", "v"])
def test_codec_against_reference_stream(ops, rg, tag):
    z, cases = rg
    is_k = tag == "k"
    for c in cases:
        T, H = c["T"], c["H"]
        k, v, _ = inputs(c)
        x = (k if is_k else v).cuda()
        p = "%s_%s_" % (c["name"], tag)
        mode, blk, rel = (ops.MODE_BLOCK, 64, c["rel_k"]) if is_k else (ops.MODE_TOKEN, 128, c["rel_v"])
        hist = torch.zeros(256, dtype=torch.int64, device="cuda")
        codes, mi, sc, spec, st = ops.quantize(x, mode, blk, rel, True, min_dtype=torch.int8, hist=hist)
        assert ops.read_status(st) == 0
        assert hashlib.sha256(codes.cpu().numpy().tobytes()).digest() == bytes(z[p + "codes_sha"])
        assert np.array_equal(sc.cpu().numpy().view(np.uint16), z[p + "scale"].view(np.uint16))
        assert np.array_equal(mi.cpu().numpy().astype(np.float32), z[p + "min"].astype(np.float32))
        # both book tensors equal the reference's build_codebook
        book = ops.build_codebook(hist)
        shift, tab = book.ref_encode_tensor()
        assert shift == 0 and np.array_equal(tab.numpy(), z[p + "enc_book"])
        assert np.array_equal(book.ref_decode_tensor().numpy(), z[p + "dec_book"])
        # this library's blocks equal the reference's, block by block (its block order is arbitrary)
        bsz, tsz, _, cap = ops.buffer_sizes(T, H * 128, is_k)
        bi = torch.zeros(bsz, dtype=torch.uint8, device="cuda")
        ti = torch.zeros(tsz // 2, dtype=torch.int16, device="cuda")
        enc = torch.zeros(cap, dtype=torch.uint8, device="cuda")
        total, st = ops.encode(codes, is_k, book.encode_table(), bi, ti, enc)
        assert ops.read_status(st) == 0
        n = int(total[0])
        rdata = z[p + "encoded"]
        assert n == rdata.size
        off, num = orc.block_infos(bi.cpu().numpy())
        roff, rnum = orc.block_infos(z[p + "block_info"])
        assert np.array_equal(num, rnum)
        assert np.array_equal(ti.cpu().numpy().view(np.uint16), z[p + "thread_info"].view("<u2"))
        data = enc[:n].cpu().numpy()
        for b in range(num.size):
            assert np.array_equal(data[off[b]: off[b] + num[b]], rdata[roff[b]: roff[b] + rnum[b]]), (c["name"], tag, b)
        # this library's decoder reads the reference's stream in the reference's block order, with a
        # book derived from the reference's decode tensor
        book2 = ops.book_from_tree(dev(z[p + "dec_book"]))
        out, st = ops.decode(dev(rdata), dev(z[p + "block_info"]), dev(z[p + "thread_info"]), book2, T, 1, H, is_k)
        assert ops.read_status(st) == 0 and torch.equal(out, codes)


def test_fused_kernels_against_reference_outputs(ops, rg):
    """kvc_fused_qk / kvc_fused_pv over the reference's streams: inside the reference's own 1 %-of-max rule
    against its fp16-chain outputs (scripts/test_py_ctx_k_2d_load.py:129-134, test_py_ctx_v.py:50-52),
    and much closer to the exact values than the reference is."""
    z, cases = rg
    for c in cases:
        T, H = c["T"], c["H"]
        k, v, q = inputs(c)
        # K
        p = "%s_k_" % c["name"]
        codes, mi, sc, spec, _ = ops.quantize(k.cuda(), ops.MODE_BLOCK, 64, c["rel_k"], True, min_dtype=torch.int8)
        kc, keep_k = ref_cache(ops, z, p, spec, mi, sc)
        S, st = ops.fused_qk(kc, T, 1, H, q.cuda(), out_dtype=torch.float32)
        assert ops.read_status(st) == 0
        ref = z[p + "fused"].astype(np.float32)
        m, _ = orc.qmeta(orc.MODE_BLOCK, True, T, 1, H, 128, 64)
        exact = orc.qk(codes.cpu().numpy(), mi.cpu().numpy(), sc.cpu().numpy(), m, q.numpy())
        got = S.cpu().numpy()
        assert np.abs(got - ref).max() < 0.01 * np.abs(ref).max()
        assert np.abs(got - exact).max() <= 5e-4 * np.abs(exact).max()
        assert np.abs(got - exact).max() < np.abs(ref - exact).max()
        # V
        p = "%s_v_" % c["name"]
        codes, mi, sc, spec, _ = ops.quantize(v.cuda(), ops.MODE_TOKEN, 128, c["rel_v"], True, min_dtype=torch.int8)
        vc, keep_v = ref_cache(ops, z, p, spec, mi, sc)
        P = z[c["name"] + "_P"]
        part, st = ops.fused_pv(vc, T, 1, H, dev(P))
        assert ops.read_status(st) == 0
        ref = z[p + "fused"].astype(np.float32)
        m, _ = orc.qmeta(orc.MODE_TOKEN, True, T, 1, H, 128, 128)
        exact = orc.pv(codes.cpu().numpy(), mi.cpu().numpy(), sc.cpu().numpy(), m, P.astype(np.float32))
        assert part.shape == ref.shape
        assert np.abs(part.float().cpu().numpy() - ref).max() < 0.01 * np.abs(ref).max()
        got = part.float().sum(0).cpu().numpy()
        assert np.abs(got - exact).max() <= 2e-3 * np.abs(exact).max()


def test_attention_over_reference_streams(ops, rg):
    """The one-pass attention kernel fed with K and V streams the reference encoded."""
    z, cases = rg
    for c in cases:
        T, H = c["T"], c["H"]
        k, v, q = inputs(c)
        kcodes, kmi, ksc, kspec, _ = ops.quantize(k.cuda(), ops.MODE_BLOCK, 64, c["rel_k"], True, min_dtype=torch.int8)
        vcodes, vmi, vsc, vspec, _ = ops.quantize(v.cuda(), ops.MODE_TOKEN, 128, c["rel_v"], True, min_dtype=torch.int8)
        kc, keep_k = ref_cache(ops, z, "%s_k_" % c["name"], kspec, kmi, ksc)
        vc, keep_v = ref_cache(ops, z, "%s_v_" % c["name"], vspec, vmi, vsc)
        scaling = 1.0 / math.sqrt(128)
        out, st = ops.attn_decode(kc, vc, T, 1, H, q.cuda(), scaling)
        assert ops.read_status(st) == 0
        km, _ = orc.qmeta(orc.MODE_BLOCK, True, T, 1, H, 128, 64)
        vm, _ = orc.qmeta(orc.MODE_TOKEN, True, T, 1, H, 128, 128)
        O = orc.attention(kcodes.cpu().numpy(), kmi.cpu().numpy(), ksc.cpu().numpy(), km,
                          vcodes.cpu().numpy(), vmi.cpu().numpy(), vsc.cpu().numpy(), vm, q.numpy(), scaling)
        assert np.abs(out.float().cpu().numpy() - O).max() <= 1e-3 * np.abs(O).max()
