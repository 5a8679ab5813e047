"""Pins the CPU checker against what the reference's own CUDA kernels produced on a B200
(tests/golden/ref_cuda_golden.npz, written by tests/golden/make_ref_cuda_golden.py from the unmodified
kvcomp_cuda module): book tensors, the blocked stream with block_info / thread_info, the decoded codes
and both fused decode + mat-vec outputs.

The reference places the blocks of one encode call through an atomic cursor (kernels.cu:472-479), so
its block order differs from run to run; every comparison of stream bytes goes block by block through
block_info, as the stream's own readers do."""
import hashlib
import json
import os

import numpy as np
import pytest

from oracle import kvc_oracle as orc


@pytest.fixture(scope="module")
def rg(golden_dir):
    z = np.load(os.path.join(golden_dir, "ref_cuda_golden.npz"))
    return z, json.loads(bytes(z["cases_json"]).decode())["cases"]


def case_inputs(c):
    from kvcomp_b200.synth import make_kv
    k, v, q = make_kv(c["T"], 1, c["H"], 128, seed=c["seed"], device="cpu")
    return k.numpy(), v.numpy(), q.numpy()


def tensors(c, z, tag, x):
    """The checker's codes / units for one tensor of a case, after holding them to the reference's."""
    is_k = tag == "k"
    mode, blk, rel = (orc.MODE_BLOCK, 64, c["rel_k"]) if is_k else (orc.MODE_TOKEN, 128, c["rel_v"])
    codes, mi, sc, m, deg = orc.quant(x, mode, blk, rel, True)
    p = "%s_%s_" % (c["name"], tag)
    assert deg == 0
    assert hashlib.sha256(codes.tobytes()).digest() == bytes(z[p + "codes_sha"]), "codes differ from torch's on CUDA"
    assert np.array_equal(sc.view(np.uint16), z[p + "scale"].view(np.uint16))
    assert np.array_equal(mi.astype(np.float32), z[p + "min"].astype(np.float32))
    return codes, mi, sc, m, p


def test_fixture_covers_the_reference_range(rg):
    z, cases = rg
    assert len(cases) >= 3
    for c in cases:
        for tag in "kv":
            p = "%s_%s_" % (c["name"], tag)
            assert bytes(z[p + "decoded_sha"]) == bytes(z[p + "codes_sha"])      # the reference's own round trip


@pytest.mark.parametrize("tag", ["k", "v"])
def test_books_and_blocked_stream_equal_the_reference_kernels(rg, tag):
    z, cases = rg
    for c in cases:
        k, v, _ = case_inputs(c)
        codes, mi, sc, m, p = tensors(c, z, tag, k if tag == "k" else v)
        is_k = tag == "k"
        enc, nsym = orc.gen_codes(orc.histogram(codes))
        tab, shift = orc.ref_encode_table(enc)
        assert shift == 0 and np.array_equal(tab, z[p + "enc_book"])
        assert np.array_equal(orc.ref_decode_tree(enc), z[p + "dec_book"])
        data, bi, ti, ov = orc.encode(codes, is_k, enc)
        assert ov.sum() == 0
        off, num = orc.block_infos(bi)
        roff, rnum = orc.block_infos(z[p + "block_info"])
        rdata = z[p + "encoded"]
        assert rdata.size == data.size
        assert np.array_equal(num, rnum), "block byte counts"
        assert np.array_equal(ti, z[p + "thread_info"].view("<u2")), "thread_info"
        # the reference's blocks tile its stream exactly once, in some order
        order = np.argsort(roff, kind="stable")
        assert roff[order[0]] == 0 and np.array_equal(roff[order][1:], np.cumsum(rnum[order].astype(np.int64))[:-1])
        for b in range(num.size):
            assert np.array_equal(data[off[b]: off[b] + num[b]], rdata[roff[b]: roff[b] + rnum[b]]), (c["name"], tag, b)
        # and the checker's decoder reads the reference's stream through the reference's tables
        back, bad = orc.decode(rdata, z[p + "block_info"], z[p + "thread_info"].view("<u2"), enc, c["T"], 1, c["H"], is_k)
        assert bad == 0 and np.array_equal(back, codes)


def _chain_matches(ref, plain, fused):
    """The reference's fp16 output equals the restated chain bit for bit, with the multiply-add either
    kept as two roundings or contracted into one fma by its compiler."""
    a = np.array_equal(ref.view(np.uint16), plain.view(np.uint16))
    b = np.array_equal(ref.view(np.uint16), fused.view(np.uint16))
    return a or b


def test_fused_k_scores_equal_the_reference_kernel(rg):
    z, cases = rg
    for c in cases:
        k, v, q = case_inputs(c)
        codes, mi, sc, m, p = tensors(c, z, "k", k)
        ref = z[p + "fused"]                                            # [1, H, T] fp16
        mi8 = orc.narrow_i8(mi)
        assert np.array_equal(mi8, mi), "min_int does not fit the reference's int8"
        plain = orc.qk_fp16chain(codes, mi, sc, m, q, fused=False)
        fused = orc.qk_fp16chain(codes, mi, sc, m, q, fused=True)
        assert _chain_matches(ref, plain, fused), c["name"]
        # the exact scores sit inside the reference's own 1 %-of-max rule (scripts/test_py_ctx_k_2d_load.py:129-134)
        S = orc.qk(codes, mi, sc, m, q)
        assert np.abs(ref.astype(np.float32) - S).max() < 0.01 * np.abs(S).max()


def test_fused_v_partials_equal_the_reference_kernel(rg):
    z, cases = rg
    for c in cases:
        k, v, q = case_inputs(c)
        codes, mi, sc, m, p = tensors(c, z, "v", v)
        ref = z[p + "fused"]                                            # [T/128, 1, H, 128] fp16
        P = z[c["name"] + "_P"]
        assert np.array_equal(orc.narrow_i8(mi), mi)
        plain = orc.pv_fp16chain(codes, mi, sc, m, P, fused=False)
        fused = orc.pv_fp16chain(codes, mi, sc, m, P, fused=True)
        assert _chain_matches(ref, plain, fused), c["name"]
        O = orc.pv(codes, mi, sc, m, P.astype(np.float32))
        got = ref.astype(np.float32).sum(0)
        assert np.abs(got - O).max() < 0.01 * np.abs(O).max()
