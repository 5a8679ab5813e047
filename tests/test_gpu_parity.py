"""GPU parity: every kernel of libkvcomp_b200.so (called through the C ABI) against the CPU checker
and the committed golden vectors.  Integer/byte results must be bit-exact; attention outputs must be
within 1e-3 of the exact (double precision) value relative to the largest output magnitude."""
import json
import math
import os

import numpy as np
import pytest
import torch

from oracle import kvc_oracle as orc

pytestmark = pytest.mark.gpu

ATTN_RTOL = 1e-3      # relative to max |out|: the 1e-3 relative error the path's specification states
ATTN_ELEM_RTOL = 2e-3  # per element, on top of a floor of 2e-4 of max |out| (the output is rounded to fp16: 2^-11)


def assert_attn_close(out, O, what=""):
    """out: the kernel's fp16 output; O: the checker's exact (double precision) attention over the
    dequantised values (code + min_int) * scale.  Two bounds: every element within ATTN_RTOL of the largest
    output magnitude, and every element within ATTN_ELEM_RTOL of its own magnitude plus a small floor."""
    got = out.float().cpu().numpy()
    err = np.abs(got - O)
    top = np.abs(O).max()
    assert err.max() <= ATTN_RTOL * top, (what, err.max() / top)
    assert (err <= ATTN_ELEM_RTOL * np.abs(O) + 2e-4 * top).all(), (what, (err / (np.abs(O) + 1e-30)).max())


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from kvcomp_b200 import ops as _ops
    return _ops


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def synth(T, B, H, seed=0, Hq=None):
    from kvcomp_b200.synth import make_kv
    k, v, q = make_kv(T, B, H, 128, seed=seed, device="cpu", Hq=Hq)
    return k.numpy(), v.numpy(), q.numpy()


MODE_CASES = [  # (tensor, mode, block, rel, batch_shared)
    ("k", orc.MODE_BLOCK, 64, 0.05, True), ("k", orc.MODE_BLOCK, 64, 0.03, False),
    ("k", orc.MODE_CHANNEL, 64, 0.05, False), ("k", orc.MODE_CHANNEL, 128, 0.02, False),
    ("k", orc.MODE_CHANNEL, 64, 0.01, False),
    ("v", orc.MODE_TOKEN, 128, 0.1, True), ("v", orc.MODE_TOKEN, 64, 0.05, False),
    ("v", orc.MODE_TOKEN, 128, 0.15, False), ("v", orc.MODE_VECTOR, 64, 0.2, False),
]


@pytest.mark.parametrize("which,mode,block,rel,shared", MODE_CASES)
def test_quantize_bit_exact(ops, which, mode, block, rel, shared):
    k, v, _ = synth(256, 2, 4, seed=3)
    x = k if which == "k" else v
    codes, mi, sc, m, deg = orc.quant(x, mode, block, rel, shared)
    hist = torch.zeros(256, dtype=torch.int64, device="cuda")
    c2, mi2, sc2, spec, st = ops.quantize(dev(x), mode, block, rel, shared, min_dtype=torch.int16, hist=hist)
    flags = ops.read_status(st)
    assert np.array_equal(sc2.cpu().numpy().view(np.uint16), sc.view(np.uint16))
    assert np.array_equal(mi2.cpu().numpy(), mi)
    assert np.array_equal(c2.cpu().numpy(), codes)
    assert np.array_equal(hist.cpu().numpy(), orc.histogram(codes))
    assert (spec.tok_div, spec.sj, spec.sb, spec.sh, spec.sc) == (m.tok_div, m.sj, m.sb, m.sh, m.sc)
    # int8 narrowing as the reference stores it
    c3, mi8, _, _, st8 = ops.quantize(dev(x), mode, block, rel, shared, min_dtype=torch.int8)
    assert np.array_equal(mi8.cpu().numpy(), orc.narrow_i8(mi))
    assert bool(ops.read_status(st8) & 0x2) == bool(((mi < -128) | (mi > 127)).any())
    assert flags & 0x4 == 0
    # dequantised values
    xh = ops.dequant(c2, mi2, sc2, spec).cpu().numpy()
    assert np.array_equal(xh.view(np.uint16), orc.dequant(codes, mi, sc, m).view(np.uint16))


@pytest.mark.parametrize("H,shared", [(2, False), (3, False), (16, False), (24, False), (32, False), (64, False), (8, True)])
def test_quantize_token_units_of_every_size(ops, H, shared):
    """Token units of 256 .. 8192 elements take the register-resident kernels (1, 2, 4 or 8 warps per
    unit), other lengths the generic one: same bits from all of them."""
    k, v, _ = synth(64, 2, H, seed=5)
    codes, mi, sc, m, _ = orc.quant(v, orc.MODE_TOKEN, 128, 0.07, shared)
    hist = torch.zeros(256, dtype=torch.int64, device="cuda")
    c2, mi2, sc2, spec, st = ops.quantize(dev(v), orc.MODE_TOKEN, 128, 0.07, shared, min_dtype=torch.int16, hist=hist)
    assert ops.read_status(st) & 0x4 == 0
    assert np.array_equal(sc2.cpu().numpy().view(np.uint16), sc.view(np.uint16))
    assert np.array_equal(mi2.cpu().numpy(), mi)
    assert np.array_equal(c2.cpu().numpy(), codes)
    assert np.array_equal(hist.cpu().numpy(), orc.histogram(codes))


def test_quantize_matches_reference_golden(ops, golden_dir):
    z = np.load(os.path.join(golden_dir, "quant_golden.npz"))
    meta = json.loads(bytes(z["cases_json"]).decode())
    MODE = {"BlockQuant": 0, "ChannelQuant": 1, "TokenQuant": 2, "VectorQuant": 3}
    for c in meta["cases"]:
        if c["api"] == "quant":
            mode, shared = (0 if c["dims"] == [1, 2, 3, 4] else 2), True
        else:
            mode, shared = MODE[c["mode"]], False
        codes, mi, sc, _, st = ops.quantize(dev(z[c["src"]]), mode, c["block"], c["rel"], shared, min_dtype=torch.int16)
        name = c["name"]
        assert np.array_equal(codes.cpu().numpy(), z[name + "_codes"]), name
        assert np.array_equal(sc.cpu().numpy().view(np.uint16), z[name + "_scale"].view(np.uint16)), name
        assert np.array_equal(mi.cpu().numpy().astype(np.float32), z[name + "_min"].astype(np.float32)), name


def test_quantize_matches_torch_ops_on_gpu(ops):
    """The op sequence of utils/compute.py:93-106 evaluated by torch on CUDA fp16 tensors."""
    k, v, _ = synth(128, 2, 4, seed=5)
    for x, dims, blk, rel, mode in ((k, [1, 2, 3, 4], 64, 0.05, 0), (v, [2, 3, 4], 128, 0.1, 2)):
        t = dev(x).view(-1, blk, 2, 4, 128)
        mn, mx = t, t
        for d in dims:
            mn = mn.min(dim=d, keepdim=True).values
            mx = mx.max(dim=d, keepdim=True).values
        scale = (mx - mn) * rel
        mi = (mn / scale).round_()
        qi = (t / scale).round_() - mi
        codes, mi2, sc2, _, _ = ops.quantize(dev(x), mode, blk, rel, True, min_dtype=torch.int16)
        assert torch.equal(codes.view(-1), qi.to(torch.uint8).view(-1))
        assert torch.equal(sc2.view(-1), scale.reshape(-1))
        assert torch.equal(mi2.view(-1).float(), mi.reshape(-1).float())


@pytest.mark.parametrize("mode,block,shared", [(orc.MODE_CHANNEL, 64, False), (orc.MODE_TOKEN, 128, False),
                                               (orc.MODE_VECTOR, 64, False), (orc.MODE_BLOCK, 64, True)])
def test_quantize_every_arithmetic_path(ops, mode, block, shared):
    """Units whose min_int is small take the packed fp16 path, units far from zero (min_int beyond +-255) the
    fp32 one, and single values that leave 0..255 are redone one by one: data that mixes all of them, fp16
    subnormals, magnitudes near the top of fp16 and constant units, against the checker."""
    rng = np.random.default_rng(77)
    T, B, H = 128, 2, 4
    # spread and centre are constant over a unit of the mode under test
    shape = {orc.MODE_CHANNEL: (1, B, H, 128), orc.MODE_TOKEN: (T, B, 1, 1), orc.MODE_VECTOR: (T, B, H, 1),
             orc.MODE_BLOCK: (T // block, 1, 1, 1)}[mode]
    lo = 1e-6 if mode == orc.MODE_CHANNEL else 1e-3
    spread = np.exp(rng.uniform(np.log(lo), np.log(50.0), shape)).astype(np.float32)
    centre = spread * rng.choice([0.0, 0.0, 3.0, -8.0, 40.0, -300.0], shape).astype(np.float32)
    if mode == orc.MODE_BLOCK:
        spread, centre = np.repeat(spread, block, axis=0), np.repeat(centre, block, axis=0)
    x = np.clip(rng.standard_normal((T, B, H, 128)).astype(np.float32) * spread + centre, -60000, 60000)
    x[:, 0, 1, 5] = x[0, 0, 1, 5] if mode == orc.MODE_CHANNEL else x[:, 0, 1, 5]      # a constant channel
    if mode in (orc.MODE_TOKEN, orc.MODE_VECTOR):
        x[5, 1] = 0.0                                        # constant units
    x = x.astype(np.float16)
    seen = set()
    for rel in (0.05, 0.011):
        codes, mi, sc, m, deg = orc.quant(x, mode, block, rel, shared)
        hist = torch.zeros(256, dtype=torch.int64, device="cuda")
        c2, mi2, sc2, spec, st = ops.quantize(dev(x), mode, block, rel, shared, min_dtype=torch.int16, hist=hist)
        ops.read_status(st, raise_on_fatal=False)
        assert np.array_equal(sc2.cpu().numpy().view(np.uint16), sc.view(np.uint16))
        assert np.array_equal(mi2.cpu().numpy(), mi)
        assert np.array_equal(c2.cpu().numpy(), codes)
        assert np.array_equal(hist.cpu().numpy(), orc.histogram(codes))
        seen |= {bool(v) for v in (np.abs(mi.astype(np.int64)) > 255).reshape(-1)}
    assert seen == {True, False}                             # both kinds of unit were met


def test_zero_scale_unit_is_flagged(ops):
    x = torch.ones(64, 1, 1, 128, dtype=torch.float16, device="cuda")
    codes, mi, sc, _, st = ops.quantize(x, 0, 64, 0.05, True)
    assert ops.read_status(st, raise_on_fatal=False) & 0x1
    assert int(codes.max()) == 0


def test_histogram(ops):
    rng = np.random.default_rng(0)
    for n in (1, 15, 16, 17, 4097, 1 << 20):
        a = rng.integers(0, 40, n).astype(np.uint8)
        h = ops.histogram(dev(a))
        assert np.array_equal(h.cpu().numpy(), np.bincount(a, minlength=256))
    # unaligned start, accumulation into an existing histogram
    a = rng.integers(0, 256, 100003).astype(np.uint8)
    t = dev(a)
    h = ops.histogram(t[3:])
    h = ops.histogram(t[:3], h)
    assert np.array_equal(h.cpu().numpy(), np.bincount(a, minlength=256))


def test_codebook_matches_reference_golden(ops, golden_dir):
    with open(os.path.join(golden_dir, "huffman_golden.json")) as f:
        cases = json.load(f)
    for case in cases:
        h = np.zeros(256, np.int64)
        for s, c in case["counts"].items():
            h[int(s)] = c
        book = ops.build_codebook(dev(h))
        hd = book.header()
        enc = book.host()[64:64 + 2048].numpy().view(orc.ENC_DT)
        assert orc.code_strings(enc) == {int(k): v for k, v in case["py_book"].items()}
        assert hd["n_symbols"] == len(case["counts"]) and hd["flags"] == 0
        oenc, _ = orc.gen_codes(h)
        assert np.array_equal(book.ref_decode_tensor().numpy(), orc.ref_decode_tree(oenc))
        if case["cpp_encode"] is not None:
            shift, tab = book.ref_encode_tensor()
            assert shift == case["cpp_shift"]
            assert tab.numpy().tobytes().hex() == case["cpp_encode"]
            assert book.ref_decode_tensor().numpy().tobytes().hex() == case["cpp_decode"]


def _pipeline(ops, x, is_k, mode, block, rel, shared, min_dtype=torch.int16):
    """quantise -> histogram -> book -> encode on the GPU; returns everything as device tensors."""
    T, B, H, D = x.shape
    hist = torch.zeros(256, dtype=torch.int64, device="cuda")
    codes, mi, sc, spec, st = ops.quantize(dev(x), mode, block, rel, shared, min_dtype=min_dtype, hist=hist)
    book = ops.build_codebook(hist)
    bsz, tsz, _, cap = ops.buffer_sizes(T, B * H * D, is_k)
    bi = torch.zeros(bsz, dtype=torch.uint8, device="cuda")
    ti = torch.zeros(tsz // 2, dtype=torch.int16, device="cuda")
    enc = torch.zeros(cap, dtype=torch.uint8, device="cuda")
    total, st2 = ops.encode(codes, is_k, book.encode_table(), bi, ti, enc)
    n, maxb = (int(x) for x in total.tolist())
    assert ops.read_status(st2) & ~0x10 == 0
    _, nb = orc.block_infos(bi.cpu().numpy())
    assert maxb == int(nb.max())
    return dict(codes=codes, mi=mi, sc=sc, spec=spec, book=book, bi=bi, ti=ti, enc=enc, n=n, hist=hist, maxb=maxb)


@pytest.mark.parametrize("is_k,mode,rel,T,B,H", [
    (True, orc.MODE_BLOCK, 0.05, 256, 1, 4), (True, orc.MODE_CHANNEL, 0.05, 192, 2, 3),
    (True, orc.MODE_CHANNEL, 0.01, 128, 1, 2), (False, orc.MODE_TOKEN, 0.1, 256, 1, 4),
    (False, orc.MODE_TOKEN, 0.05, 384, 2, 3), (False, orc.MODE_TOKEN, 0.02, 128, 1, 2),
])
def test_encode_decode_bit_exact(ops, is_k, mode, rel, T, B, H):
    k, v, _ = synth(T, B, H, seed=11)
    x = k if is_k else v
    shared = mode != orc.MODE_CHANNEL
    r = _pipeline(ops, x, is_k, mode, 64 if is_k else 128, rel, shared)
    codes = r["codes"].cpu().numpy()
    oenc, _ = orc.gen_codes(orc.histogram(codes))
    odata, obi, oti, ov = orc.encode(codes, is_k, oenc)
    assert r["n"] == odata.size
    assert np.array_equal(r["enc"][:r["n"]].cpu().numpy(), odata)
    assert np.array_equal(r["bi"].cpu().numpy(), obi)
    assert np.array_equal(r["ti"].cpu().numpy().view(np.uint16), oti)
    out, st = ops.decode(r["enc"][:r["n"]], r["bi"], r["ti"], r["book"], T, B, H, is_k)
    assert ops.read_status(st) == 0
    assert np.array_equal(out.cpu().numpy(), codes)
    # a stream written by the checker decodes on the GPU too
    out2, st = ops.decode(dev(odata), dev(obi), dev(oti.view(np.int16)), r["book"], T, B, H, is_k)
    assert ops.read_status(st) == 0 and np.array_equal(out2.cpu().numpy(), codes)


@pytest.mark.parametrize("is_k", [True, False])
def test_codec_buffers_off_16_byte_boundaries(ops, is_k):
    """Codes that do not start on 16 bytes are staged with 4-byte loads and written back with 4-byte
    stores; a bound on the block size changes nothing but the launch; a bound that is too small is
    reported, not overrun."""
    T, B, H = 256, 2, 3
    k, v, _ = synth(T, B, H, seed=19)
    x = k if is_k else v
    r = _pipeline(ops, x, is_k, orc.MODE_CHANNEL if is_k else orc.MODE_TOKEN, 64 if is_k else 128, 0.05, False)
    n = T * B * H * 128
    shifted = torch.zeros(n + 32, dtype=torch.uint8, device="cuda")
    codes4 = shifted[4:4 + n].view(T, B, H, 128)
    codes4.copy_(r["codes"])
    bsz, tsz, _, cap = ops.buffer_sizes(T, B * H * 128, is_k)
    bi = torch.zeros(bsz, dtype=torch.uint8, device="cuda")
    ti = torch.zeros(tsz // 2, dtype=torch.int16, device="cuda")
    enc = torch.zeros(cap, dtype=torch.uint8, device="cuda")
    total, st = ops.encode(codes4, is_k, r["book"].encode_table(), bi, ti, enc)
    assert ops.read_status(st) & ~0x10 == 0 and int(total[0]) == r["n"]
    assert torch.equal(enc[:r["n"]], r["enc"][:r["n"]]) and torch.equal(bi, r["bi"]) and torch.equal(ti, r["ti"])
    out_buf = torch.zeros(n + 32, dtype=torch.uint8, device="cuda")
    out4 = out_buf[4:4 + n].view(T, B, H, 128)
    for bound in (0, r["maxb"], 8191):
        out4.zero_()
        _, st = ops.decode(r["enc"][:r["n"]], r["bi"], r["ti"], r["book"], T, B, H, is_k, out=out4, max_block=bound)
        assert ops.read_status(st) == 0 and torch.equal(out4, r["codes"])
    _, st = ops.decode(r["enc"][:r["n"]], r["bi"], r["ti"], r["book"], T, B, H, is_k, max_block=r["maxb"] - 1)
    assert ops.read_status(st, False) & 0x80           # KVC_FLAG_BAD_STREAM


def test_encode_base_offset_and_append(ops):
    """Two store calls into one stream: the second call's block offsets carry the base offset
    (kernels.cu:476) and the whole stream decodes as one cache."""
    k, _, _ = synth(256, 1, 4, seed=2)
    T, B, H = 256, 1, 4
    codes, mi, sc, spec, _ = ops.quantize(dev(k), 0, 64, 0.05, True)
    book = ops.build_codebook(ops.histogram(codes))
    bi = torch.zeros(8 * (T // 64) * B * H, dtype=torch.uint8, device="cuda")
    ti = torch.zeros(64 * (T // 64) * B * H, dtype=torch.int16, device="cuda")
    enc = torch.zeros(T * B * H * 128, dtype=torch.uint8, device="cuda")
    half = T // 2
    nb = (half // 64) * B * H
    t1, _ = ops.encode(codes[:half].contiguous(), True, book.encode_table(), bi[:8 * nb], ti[:64 * nb], enc)
    n1 = int(t1[0].item())
    t2, _ = ops.encode(codes[half:].contiguous(), True, book.encode_table(), bi[8 * nb:], ti[64 * nb:], enc[n1:], base_offset=n1)
    n2 = int(t2[0].item())
    out, st = ops.decode(enc[:n1 + n2], bi, ti, book, T, B, H, True)
    assert ops.read_status(st) == 0 and torch.equal(out, codes)
    off, _ = orc.block_infos(bi.cpu().numpy())
    assert off[nb] == n1


def test_encode_wait_between_blocks_runs_out_and_returns(ops):
    """A block's CTA learns its byte offset from the blocks before it, with bounded waits.  With the
    diagnostic that makes the first block keep its count to itself the waits run out after a few polls:
    the call returns, the status word carries KVC_FLAG_WAIT_TIMEOUT, and the next ordinary call writes
    the same stream as before."""
    T, B, H = 256, 2, 3
    k, _, _ = synth(T, B, H, seed=23)
    r = _pipeline(ops, k, True, orc.MODE_CHANNEL, 64, 0.05, False)
    bi, ti, enc = torch.zeros_like(r["bi"]), torch.zeros_like(r["ti"]), torch.zeros_like(r["enc"])
    try:
        ops.encode_debug(wait_limit=8, starve=True)
        total, st = ops.encode(r["codes"], True, r["book"].encode_table(), bi, ti, enc)
        torch.cuda.synchronize()
        assert ops.read_status(st, raise_on_fatal=False) & 0x400
    finally:
        ops.encode_debug()
    total, st = ops.encode(r["codes"], True, r["book"].encode_table(), bi, ti, enc)
    assert ops.read_status(st) & ~0x10 == 0 and int(total[0]) == r["n"]
    assert torch.equal(enc[:r["n"]], r["enc"][:r["n"]]) and torch.equal(bi, r["bi"]) and torch.equal(ti, r["ti"])


def test_encode_random_shapes_books_and_alignments(ops):
    """Random block counts, alphabets of 1 to 256 symbols (table in registers, in shared memory, codes beyond 16
    bits), destinations at every alignment: the stream, block_info and thread_info equal the checker's and the
    stream decodes to the codes."""
    rng = np.random.default_rng(2024)
    for case in range(32):
        is_k = bool(case & 1)
        T = int(rng.integers(1, 6)) * (64 if is_k else 128)
        B, H = int(rng.integers(1, 4)), int(rng.integers(1, 5))
        nsym = [1, 2, 5, 21, 32, 33, 60, 120, 256][case % 9]
        prob = rng.random(nsym) ** (6 if case % 4 == 3 else 3) + 1e-6      # every fourth case: long codes
        codes = rng.choice(nsym, size=(T, B, H, 128), p=prob / prob.sum()).astype(np.uint8)
        book = ops.build_codebook(ops.histogram(dev(codes).view(-1)))
        oenc, _ = orc.gen_codes(orc.histogram(codes))
        odata, obi, oti, ov = orc.encode(codes, is_k, oenc)
        bsz, tsz, _, cap = ops.buffer_sizes(T, B * H * 128, is_k)
        bi = torch.zeros(bsz, dtype=torch.uint8, device="cuda")
        ti = torch.zeros(tsz // 2, dtype=torch.int16, device="cuda")
        buf = torch.zeros(cap + 16, dtype=torch.uint8, device="cuda")
        off = case % 16
        total, st = ops.encode(dev(codes), is_k, book.encode_table(), bi, ti, buf[off:off + cap])
        flags = ops.read_status(st, raise_on_fatal=False)
        assert flags & ~0x30 == 0, (case, flags)
        if flags & 0x30:                       # a vector or block beyond what the format describes: nothing to compare
            continue
        n = int(total[0])
        assert n == odata.size, case
        assert np.array_equal(buf[off:off + n].cpu().numpy(), odata), case
        assert np.array_equal(bi.cpu().numpy(), obi) and np.array_equal(ti.cpu().numpy().view(np.uint16), oti), case
        assert int(buf[:off].sum()) == 0 and int(buf[off + n:].sum()) == 0, case      # nothing written outside the stream
        out, st = ops.decode(buf[off:off + n], bi, ti, book, T, B, H, is_k, max_block=int(total[1]))
        assert ops.read_status(st) == 0 and np.array_equal(out.cpu().numpy(), codes), case


def test_book_from_reference_decode_tensor(ops):
    k, _, _ = synth(128, 1, 2, seed=4)
    r = _pipeline(ops, k, True, 0, 64, 0.05, True)
    tree = r["book"].ref_decode_tensor().cuda()
    book2 = ops.book_from_tree(tree)
    assert torch.equal(book2.blob[64:], r["book"].blob[64:])
    out, st = ops.decode(r["enc"][:r["n"]], r["bi"], r["ti"], book2, 128, 1, 2, True)
    assert ops.read_status(st) == 0 and torch.equal(out, r["codes"])


def test_frozen_book_flags_unseen_symbol(ops):
    rng = np.random.default_rng(0)
    codes = rng.integers(0, 4, (64, 1, 1, 128)).astype(np.uint8)
    book = ops.build_codebook(ops.histogram(dev(codes)))
    codes[3, 0, 0, 7] = 9
    bi = torch.zeros(8, dtype=torch.uint8, device="cuda")
    ti = torch.zeros(64, dtype=torch.int16, device="cuda")
    enc = torch.zeros(8192, dtype=torch.uint8, device="cuda")
    total, st = ops.encode(dev(codes), True, book.encode_table(), bi, ti, enc)
    assert ops.read_status(st, raise_on_fatal=False) & 0x8
    # bytes equal the checker's (which drops the symbol like the reference does)
    enc_tab = book.host()[64:64 + 2048].numpy().view(orc.ENC_DT)
    odata, _, oti, ov = orc.encode(codes, True, enc_tab)
    assert ov[1] == 1
    assert np.array_equal(enc[:int(total[0].item())].cpu().numpy(), odata)


def test_single_symbol_book_meets_foreign_bits(ops):
    """A book of one symbol has the code '0' only: a 1 bit belongs to no code.  The decoders must report
    such a stream (their table says so in the book header) and still come to an end."""
    T, B, H = 128, 1, 2
    codes = torch.full((T, B, H, 128), 7, dtype=torch.uint8, device="cuda")
    book = ops.build_codebook(ops.histogram(codes.view(-1)))
    hd = book.header()
    assert hd["n_symbols"] == 1 and hd["max_len"] == 1 and hd["escape"] == 1
    bsz, tsz, _, cap = ops.buffer_sizes(T, B * H * 128, True)
    bi = torch.zeros(bsz, dtype=torch.uint8, device="cuda")
    ti = torch.zeros(tsz // 2, dtype=torch.int16, device="cuda")
    enc = torch.zeros(cap, dtype=torch.uint8, device="cuda")
    total, st = ops.encode(codes, True, book.encode_table(), bi, ti, enc)
    n = int(total[0])
    assert ops.read_status(st) == 0 and n == T * B * H * 16          # one bit per symbol
    out, st = ops.decode(enc[:n], bi, ti, book, T, B, H, True)
    assert ops.read_status(st) == 0 and torch.equal(out, codes)
    enc[5] = 0xFF; enc[n - 3] = 0x18
    out, st = ops.decode(enc[:n], bi, ti, book, T, B, H, True)
    assert ops.read_status(st, False) & 0x80                          # KVC_FLAG_BAD_STREAM


def test_long_codes_use_the_slow_path(ops):
    """A very skewed alphabet has codes longer than the decode window; the stream still round-trips."""
    rng = np.random.default_rng(1)
    p = np.array([2.0 ** -(i + 1) for i in range(20)]); p[-1] = p[-2]; p /= p.sum()
    p[12:] = p[12:].sum() / 8                       # keep the long codes frequent enough to occur often
    codes = rng.choice(20, size=(128, 1, 2, 128), p=p).astype(np.uint8)
    codes[5, 0, 1, :20] = np.arange(20)          # make sure every symbol occurs
    for is_k in (True, False):
        book = ops.build_codebook(ops.histogram(dev(codes)))
        assert book.header()["max_len"] > 12
        bi = torch.zeros(8 * 4, dtype=torch.uint8, device="cuda")
        ti = torch.zeros(64 * 4, dtype=torch.int16, device="cuda")
        enc = torch.zeros(codes.size, dtype=torch.uint8, device="cuda")
        total, st = ops.encode(dev(codes), is_k, book.encode_table(), bi, ti, enc)
        out, st2 = ops.decode(enc[:int(total[0].item())], bi, ti, book, 128, 1, 2, is_k)
        assert ops.read_status(st) == 0 and ops.read_status(st2) == 0
        assert np.array_equal(out.cpu().numpy(), codes)


def _caches(ops, k, v, kmode, vmode, krel, vrel, kblock=64, shared=True, min_dtype=torch.int16, tight=True):
    T, B, H, _ = k.shape
    rk = _pipeline(ops, k, True, kmode, kblock, krel, shared, min_dtype)
    rv = _pipeline(ops, v, False, vmode, 128, vrel, shared, min_dtype)
    kc = ops.make_cache(rk["enc"], rk["bi"], rk["ti"], rk["book"], rk["mi"], rk["sc"], rk["spec"], rk["n"], rk["maxb"] if tight else 0)
    vc = ops.make_cache(rv["enc"], rv["bi"], rv["ti"], rv["book"], rv["mi"], rv["sc"], rv["spec"], rv["n"], rv["maxb"] if tight else 0)
    return rk, rv, kc, vc


def _oracle_q(r, T, B, H, mode, block, shared):
    m, _ = orc.qmeta(mode, shared, T, B, H, 128, block)
    return r["codes"].cpu().numpy(), r["mi"].cpu().numpy(), r["sc"].cpu().numpy(), m


@pytest.mark.parametrize("kmode,shared,B,Hkv,Hq", [
    (orc.MODE_BLOCK, True, 1, 4, 4), (orc.MODE_CHANNEL, False, 2, 2, 2), (orc.MODE_CHANNEL, False, 1, 2, 8),
    (orc.MODE_BLOCK, False, 2, 2, 6), (orc.MODE_VECTOR, False, 1, 2, 2),
])
def test_fused_qk(ops, kmode, shared, B, Hkv, Hq):
    T = 320
    k, v, q = synth(T, B, Hkv, seed=7, Hq=Hq)
    hist = torch.zeros(256, dtype=torch.int64, device="cuda")
    r = _pipeline(ops, k, True, kmode, 64, 0.05, shared)
    kc = ops.make_cache(r["enc"], r["bi"], r["ti"], r["book"], r["mi"], r["sc"], r["spec"], r["n"])
    S, st = ops.fused_qk(kc, T, B, Hkv, dev(q), out_dtype=torch.float32)
    assert ops.read_status(st) == 0
    So = orc.qk(*_oracle_q(r, T, B, Hkv, kmode, 64, shared), q)
    # the shared weight vector is held in 16-bit block fixed point: errors of a few 1e-4 of max
    assert np.abs(S.cpu().numpy() - So).max() <= 5e-4 * np.abs(So).max()
    # fp16 output, the reference's C tensor; its own tolerance is 1 % of max (test_py_ctx_k_2d_load.py:129-134)
    S16, _ = ops.fused_qk(kc, T, B, Hkv, dev(q))
    assert np.abs(S16.float().cpu().numpy() - So).max() <= 2e-3 * np.abs(So).max()


@pytest.mark.parametrize("vmode,shared,B,Hkv,Hq", [
    (orc.MODE_TOKEN, True, 1, 4, 4), (orc.MODE_TOKEN, False, 2, 2, 8), (orc.MODE_VECTOR, False, 1, 2, 4),
])
def test_fused_pv(ops, vmode, shared, B, Hkv, Hq):
    T = 384
    k, v, q = synth(T, B, Hkv, seed=8, Hq=Hq)
    r = _pipeline(ops, v, False, vmode, 128, 0.1, shared)
    vc = ops.make_cache(r["enc"], r["bi"], r["ti"], r["book"], r["mi"], r["sc"], r["spec"], r["n"])
    rng = np.random.default_rng(3)
    logits = rng.standard_normal((B, Hq, T)) * 2.5          # as test_py_ctx_v.py:62-67
    P = np.exp(logits - logits.max(-1, keepdims=True)); P /= P.sum(-1, keepdims=True)
    P16 = P.astype(np.float16)
    part, st = ops.fused_pv(vc, T, B, Hkv, dev(P16))
    assert ops.read_status(st) == 0 and part.shape == (T // 128, B, Hq, 128)
    O = part.float().sum(0).cpu().numpy()
    Oo = orc.pv(*_oracle_q(r, T, B, Hkv, vmode, 128, shared), P16.astype(np.float32))
    assert np.abs(O - Oo).max() <= 2e-3 * np.abs(Oo).max()


ATTN_CASES = [  # kmode, vmode, shared, T, B, Hkv, Hq, Tr, splits, min_dtype
    (orc.MODE_CHANNEL, orc.MODE_TOKEN, False, 512, 1, 4, 4, 0, 0, torch.int16),
    (orc.MODE_CHANNEL, orc.MODE_TOKEN, False, 640, 2, 2, 8, 0, 2, torch.int16),
    (orc.MODE_BLOCK, orc.MODE_TOKEN, True, 1024, 1, 4, 4, 0, 3, torch.int8),
    (orc.MODE_BLOCK, orc.MODE_TOKEN, True, 384, 2, 2, 2, 100, 1, torch.int8),
    (orc.MODE_CHANNEL, orc.MODE_TOKEN, False, 896, 1, 2, 12, 300, 2, torch.int16),
    (orc.MODE_CHANNEL, orc.MODE_VECTOR, False, 128, 3, 1, 1, 1, 0, torch.int16),
    (orc.MODE_CHANNEL, orc.MODE_TOKEN, False, 1152, 3, 5, 15, 0, 0, torch.int16),     # 3 query heads per KV head: chunks of 2 + 1
    (orc.MODE_BLOCK, orc.MODE_TOKEN, False, 256, 1, 7, 35, 37, 9, torch.int16),       # 5 per KV head (4 + 1), more splits than tiles
    (orc.MODE_CHANNEL, orc.MODE_TOKEN, False, 2304, 1, 2, 4, 0, 4, torch.int16),      # 2 per KV head, 9 tiles in 3 runs
    (orc.MODE_CHANNEL, orc.MODE_TOKEN, False, 128, 2, 3, 6, 5, 0, torch.int16),       # half a tile and a tail
]


@pytest.mark.parametrize("kmode,vmode,shared,T,B,Hkv,Hq,Tr,splits,min_dtype", ATTN_CASES)
def test_attn_decode(ops, kmode, vmode, shared, T, B, Hkv, Hq, Tr, splits, min_dtype):
    k, v, q = synth(T + Tr, B, Hkv, seed=21, Hq=Hq)
    rk, rv, kc, vc = _caches(ops, k[:T], v[:T], kmode, vmode, 0.05, 0.1, 64, shared, min_dtype)
    scaling = 1.0 / math.sqrt(128)
    kt = dev(k[T:]) if Tr else None
    vt = dev(v[T:]) if Tr else None
    out, st = ops.attn_decode(kc, vc, T, B, Hkv, dev(q), scaling, kt, vt, splits=splits)
    assert ops.read_status(st) == 0
    ko = _oracle_q(rk, T, B, Hkv, kmode, 64, shared)
    vo = _oracle_q(rv, T, B, Hkv, vmode, 128, shared)
    O = orc.attention(*ko, *vo, q, scaling, k[T:] if Tr else None, v[T:] if Tr else None)
    assert_attn_close(out, O)
    # a second call reuses a caller-held workspace and must give the same bits
    ws = ops.attn_workspace(B, Hq, max(splits, ops.attn_splits(T, B, Hkv)), "cuda")
    o1, _ = ops.attn_decode(kc, vc, T, B, Hkv, dev(q), scaling, kt, vt, splits=splits, workspace=ws)
    o2, _ = ops.attn_decode(kc, vc, T, B, Hkv, dev(q), scaling, kt, vt, splits=splits, workspace=ws)
    assert torch.equal(o1, o2) and torch.equal(o1, out)
    # without any workspace (one run per column, fixed shares of the columns) the attention kernel writes the
    # output itself and reads the tail itself; with one the merge kernel adds the tail
    o3, st = ops.attn_decode(kc, vc, T, B, Hkv, dev(q), scaling, kt, vt, splits=1, workspace=False)
    assert ops.read_status(st) == 0
    assert_attn_close(o3, O)


@pytest.mark.parametrize("B,Hkv,Hq,T,Tr", [(2, 2, 8, 1024, 0), (1, 2, 10, 768, 45), (3, 10, 40, 256, 0)])
def test_attn_decode_phi3_settings(ops, B, Hkv, Hq, T, Tr):
    """The Phi-3-medium-shaped configuration's settings: K per channel in 128-token blocks at relative error
    bound 0.02 (about 52 symbols, 5.5 bits each), V per token at 0.15, four query heads per KV head -- and
    five per KV head, which the kernel handles as chunks of 4 + 1."""
    k, v, q = synth(T + Tr, B, Hkv, seed=33, Hq=Hq)
    rk, rv, kc, vc = _caches(ops, k[:T], v[:T], orc.MODE_CHANNEL, orc.MODE_TOKEN, 0.02, 0.15, 128, False)
    assert rk["book"].header()["n_symbols"] >= 45 and rk["book"].header()["escape"] in (0, 1)
    scaling = 1.0 / math.sqrt(128)
    kt = dev(k[T:]) if Tr else None
    vt = dev(v[T:]) if Tr else None
    out, st = ops.attn_decode(kc, vc, T, B, Hkv, dev(q), scaling, kt, vt)
    assert ops.read_status(st) == 0
    O = orc.attention(*_oracle_q(rk, T, B, Hkv, orc.MODE_CHANNEL, 128, False),
                      *_oracle_q(rv, T, B, Hkv, orc.MODE_TOKEN, 128, False), q, scaling,
                      k[T:] if Tr else None, v[T:] if Tr else None)
    assert_attn_close(out, O)


def test_attn_decode_llama7b_shape_small(ops):
    """The Llama-2-7B-shaped configuration with a short context: batch 8, 32 heads (MHA), K per channel
    at 0.05, V per token at 0.1, block 64."""
    T, B, H = 512, 8, 32
    k, v, q = synth(T, B, H, seed=44)
    rk, rv, kc, vc = _caches(ops, k, v, orc.MODE_CHANNEL, orc.MODE_TOKEN, 0.05, 0.1, 64, False)
    scaling = 1.0 / math.sqrt(128)
    out, st = ops.attn_decode(kc, vc, T, B, H, dev(q), scaling)
    assert ops.read_status(st) == 0
    O = orc.attention(*_oracle_q(rk, T, B, H, orc.MODE_CHANNEL, 64, False),
                      *_oracle_q(rv, T, B, H, orc.MODE_TOKEN, 128, False), q, scaling)
    assert_attn_close(out, O)


def _skewed_cache(ops, rng, is_k, T, B, H):
    """Codes drawn from a very skewed alphabet (a code longer than the 12-bit decode window exists), with
    made-up units: K per 64-token block and sequence, V per token and sequence."""
    p = np.array([2.0 ** -(i + 1) for i in range(20)]); p[-1] = p[-2]; p /= p.sum()
    p[12:] = p[12:].sum() / 8
    codes = rng.choice(20, size=(T, B, H, 128), p=p / p.sum()).astype(np.uint8)
    codes[1, 0, 0, :20] = np.arange(20)
    mode, blk = (orc.MODE_BLOCK, 64) if is_k else (orc.MODE_TOKEN, 128)
    m, n = orc.qmeta(mode, False, T, B, H, 128, blk)
    mi = rng.integers(-12, 3, n).astype(np.int16)
    sc = (0.02 + 0.1 * rng.random(n)).astype(np.float16)
    spec = ops.qspec(mode, False, B, H, 128, blk)
    cd = dev(codes)
    book = ops.build_codebook(ops.histogram(cd.view(-1)))
    bsz, tsz, _, cap = ops.buffer_sizes(T, B * H * 128, is_k)
    bi = torch.zeros(bsz, dtype=torch.uint8, device="cuda")
    ti = torch.zeros(tsz // 2, dtype=torch.int16, device="cuda")
    enc = torch.zeros(cap, dtype=torch.uint8, device="cuda")
    total, st = ops.encode(cd, is_k, book.encode_table(), bi, ti, enc)
    assert ops.read_status(st) & ~0x10 == 0
    n_bytes, maxb = (int(x) for x in total.tolist())
    mid, scd = dev(mi), dev(sc)
    cache = ops.make_cache(enc, bi, ti, book, mid, scd, spec, n_bytes, maxb)
    return cache, (enc, bi, ti, book, mid, scd), (codes, mi, sc, m), book


@pytest.mark.parametrize("G", [1, 2, 4, 3])
def test_attn_decode_books_with_long_codes(ops, G):
    """Books whose header says `escape`: the fused kernels take the decoder that tests every table entry and
    continues bit by bit from the tree, for one, two and four query heads per KV head (and 3 = 2 + 1)."""
    rng = np.random.default_rng(5 + G)
    T, B, Hkv = 512, 2, 2
    Hq = Hkv * G
    kc, keep_k, ko, kbook = _skewed_cache(ops, rng, True, T, B, Hkv)
    vc, keep_v, vo, vbook = _skewed_cache(ops, rng, False, T, B, Hkv)
    for b in (kbook, vbook):
        hd = b.header()
        assert hd["escape"] == 1 and hd["max_len"] > 12
    q = (rng.standard_normal((B, Hq, 128)) / math.sqrt(128)).astype(np.float16)
    scaling = 1.0 / math.sqrt(128)
    out, st = ops.attn_decode(kc, vc, T, B, Hkv, dev(q), scaling, splits=2)
    assert ops.read_status(st) == 0
    O = orc.attention(*ko, *vo, q, scaling)
    assert_attn_close(out, O)
    # the two-call kernels take the same path
    S, st = ops.fused_qk(kc, T, B, Hkv, dev(q), out_dtype=torch.float32)
    assert ops.read_status(st) == 0
    So = orc.qk(*ko, q)
    assert np.abs(S.cpu().numpy() - So).max() <= 5e-4 * np.abs(So).max()


def test_attn_decode_flags_a_vector_that_starts_outside_its_block(ops):
    """thread_info is input: an entry that points past its block's bytes (still inside the staging area) must
    be reported, not decoded."""
    T, B, Hkv, Hq = 512, 1, 2, 2
    k, v, q = synth(T, B, Hkv, seed=51, Hq=Hq)
    rk, rv, kc, vc = _caches(ops, k, v, orc.MODE_CHANNEL, orc.MODE_TOKEN, 0.05, 0.1, 64, False)
    scaling = 1.0 / math.sqrt(128)
    out, st = ops.attn_decode(kc, vc, T, B, Hkv, dev(q), scaling)
    assert ops.read_status(st) == 0
    for r, is_k in ((rk, True), (rv, False)):
        ti = r["ti"].clone()
        bad = r["ti"].clone()
        # vector 10 of block 3 would start 40 bytes past the largest block
        bad[64 * 3 + 9] = int(np.array([(r["maxb"] + 40) << 3], dtype=np.uint16).view(np.int16)[0])
        r["ti"].copy_(bad)
        out2, st = ops.attn_decode(kc, vc, T, B, Hkv, dev(q), scaling)
        assert ops.read_status(st, raise_on_fatal=False) & 0x80, "K" if is_k else "V"
        assert torch.isfinite(out2.float()).all()
        if is_k:
            S, st = ops.fused_qk(kc, T, B, Hkv, dev(q))
        else:
            P = torch.softmax(torch.randn(B, Hq, T, device="cuda"), dim=-1).half()
            S, st = ops.fused_pv(vc, T, B, Hkv, P)
        assert ops.read_status(st, raise_on_fatal=False) & 0x80
        r["ti"].copy_(ti)
    out3, st = ops.attn_decode(kc, vc, T, B, Hkv, dev(q), scaling)
    assert ops.read_status(st) == 0 and torch.equal(out3, out)


def test_attn_decode_staging_wait_runs_out_and_returns(ops):
    """The kernel's waits for its staged blocks are bounded.  With the diagnostic that announces bytes which
    are never copied, the first wait runs out after a few tries: the call returns, the status word carries
    KVC_FLAG_WAIT_TIMEOUT, nothing is left in flight, and the next ordinary call is correct."""
    T, B, Hkv, Hq = 512, 2, 2, 4
    k, v, q = synth(T, B, Hkv, seed=52, Hq=Hq)
    rk, rv, kc, vc = _caches(ops, k, v, orc.MODE_CHANNEL, orc.MODE_TOKEN, 0.05, 0.1, 64, False)
    scaling = 1.0 / math.sqrt(128)
    want, st = ops.attn_decode(kc, vc, T, B, Hkv, dev(q), scaling, splits=2)
    assert ops.read_status(st) == 0
    ws = ops.attn_workspace(B, Hq, 2, "cuda")
    try:
        ops.attn_debug(wait_limit=8, starve=True)
        out, st = ops.attn_decode(kc, vc, T, B, Hkv, dev(q), scaling, splits=2, workspace=ws)
        torch.cuda.synchronize()
        assert ops.read_status(st, raise_on_fatal=False) & 0x400
    finally:
        ops.attn_debug()
    assert int(ws[:256].view(torch.int32).abs().sum()) == 0          # the scheduling counters were left zeroed
    out, st = ops.attn_decode(kc, vc, T, B, Hkv, dev(q), scaling, splits=2, workspace=ws)
    assert ops.read_status(st) == 0 and torch.equal(out, want)


def test_attn_decode_tail_only(ops):
    """Nothing compressed yet (the first tokens of a sequence): T = 0, no streams, only fp16 rows."""
    B, Hkv, Hq, Tr = 2, 2, 6, 77
    k, v, q = synth(Tr, B, Hkv, seed=53, Hq=Hq)
    scaling = 1.0 / math.sqrt(128)
    out, st = ops.attn_decode(None, None, 0, B, Hkv, dev(q), scaling, dev(k), dev(v))
    assert ops.read_status(st) == 0
    kf, vf = torch.from_numpy(k).float(), torch.from_numpy(v).float()
    g = Hq // Hkv
    S = torch.einsum("bhd,tbhd->bht", torch.from_numpy(q).float(), kf.repeat_interleave(g, dim=2)) * scaling
    O = torch.einsum("bht,tbhd->bhd", torch.softmax(S.double(), -1).float(), vf.repeat_interleave(g, dim=2)).numpy()
    assert_attn_close(out, O)


def test_attn_decode_many_items(ops):
    """More items than two per resident CTA: the later ones are drawn from the workspace's counter.
    Every way of sharing the work gives the oracle's result, and the counters end at zero."""
    T, B, Hkv, Hq = 2048, 8, 16, 16
    k, v, q = synth(T, B, Hkv, seed=77, Hq=Hq)
    rk, rv, kc, vc = _caches(ops, k, v, orc.MODE_BLOCK, orc.MODE_TOKEN, 0.05, 0.1, 64, False)
    scaling = 1.0 / math.sqrt(128)
    O = orc.attention(*_oracle_q(rk, T, B, Hkv, orc.MODE_BLOCK, 64, False),
                      *_oracle_q(rv, T, B, Hkv, orc.MODE_TOKEN, 128, False), q, scaling)
    ws = ops.attn_workspace(B, Hq, 8, "cuda")
    outs = []
    for splits, w in ((8, ws), (8, ws), (1, False), (1, ws), (0, None), (3, None)):
        out, st = ops.attn_decode(kc, vc, T, B, Hkv, dev(q), scaling, splits=splits, workspace=w)
        assert ops.read_status(st) == 0
        assert_attn_close(out, O, splits)
        outs.append(out)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[2], outs[3])
    assert int(ws[:256].view(torch.int32).abs().sum()) == 0


def test_attn_decode_unaligned_stream_and_unknown_bound(ops):
    """Streams that do not start on a 16-byte boundary take the plain-load staging path; an unknown
    block bound falls back to the format's maximum.  Same bits either way."""
    T, B, Hkv, Hq = 512, 2, 2, 4
    k, v, q = synth(T, B, Hkv, seed=31, Hq=Hq)
    rk, rv, kc, vc = _caches(ops, k, v, orc.MODE_CHANNEL, orc.MODE_TOKEN, 0.05, 0.1, 64, False)
    scaling = 1.0 / math.sqrt(128)
    out, st = ops.attn_decode(kc, vc, T, B, Hkv, dev(q), scaling, splits=2)
    assert ops.read_status(st) == 0
    rk0, rv0, kc0, vc0 = _caches(ops, k, v, orc.MODE_CHANNEL, orc.MODE_TOKEN, 0.05, 0.1, 64, False, tight=False)
    out0, st = ops.attn_decode(kc0, vc0, T, B, Hkv, dev(q), scaling, splits=2)
    assert ops.read_status(st) == 0 and torch.equal(out, out0)
    # shift both streams by 3 bytes
    ek = torch.zeros(rk["n"] + 64, dtype=torch.uint8, device="cuda"); ek[3:3 + rk["n"]] = rk["enc"][:rk["n"]]
    ev = torch.zeros(rv["n"] + 64, dtype=torch.uint8, device="cuda"); ev[3:3 + rv["n"]] = rv["enc"][:rv["n"]]
    kc1 = ops.make_cache(ek[3:], rk["bi"], rk["ti"], rk["book"], rk["mi"], rk["sc"], rk["spec"], rk["n"], rk["maxb"])
    vc1 = ops.make_cache(ev[3:], rv["bi"], rv["ti"], rv["book"], rv["mi"], rv["sc"], rv["spec"], rv["n"], rv["maxb"])
    out1, st = ops.attn_decode(kc1, vc1, T, B, Hkv, dev(q), scaling, splits=2)
    assert ops.read_status(st) == 0 and torch.equal(out, out1)


def test_attn_decode_config0(ops):
    """Llama-2-7B single layer: 32 heads x 128, batch 1, 1024 tokens, K per channel / V per token in
    64-token blocks at relative error bound 0.05, one decode step."""
    T, B, H = 1024, 1, 32
    k, v, q = synth(T, B, H, seed=0)
    rk, rv, kc, vc = _caches(ops, k, v, orc.MODE_CHANNEL, orc.MODE_TOKEN, 0.05, 0.05, 64, False)
    scaling = 1.0 / math.sqrt(128)
    out, st = ops.attn_decode(kc, vc, T, B, H, dev(q), scaling)
    assert ops.read_status(st) == 0
    O = orc.attention(*_oracle_q(rk, T, B, H, orc.MODE_CHANNEL, 64, False),
                      *_oracle_q(rv, T, B, H, orc.MODE_TOKEN, 128, False), q, scaling)
    assert_attn_close(out, O)
    # the two-call path (scores -> softmax -> partials) agrees as well
    S, _ = ops.fused_qk(kc, T, B, H, dev(q), out_dtype=torch.float32)
    P = torch.softmax(S * scaling, dim=-1).half()
    part, _ = ops.fused_pv(vc, T, B, H, P)
    O2 = part.float().sum(0).cpu().numpy()
    assert np.abs(O2 - O).max() <= 2e-3 * np.abs(O).max()


@pytest.mark.parametrize("kmode,vmode,shared", [(orc.MODE_BLOCK, orc.MODE_TOKEN, True), (orc.MODE_BLOCK, orc.MODE_TOKEN, False),
                                                (orc.MODE_CHANNEL, orc.MODE_TOKEN, False)])
def test_head_shards_reproduce_the_single_gpu_cache(ops, kmode, vmode, shared):
    """The heads of a cache split in two, as two ranks would hold them, with the compression-time exchanges
    done by hand (elementwise min / max of the shards' unit extremes, sum of their histograms): scale,
    min_int, codes and books equal the unsharded run's, every block of a shard's stream equals the unsharded
    block of the same column, and the attention outputs equal the unsharded ones head by head."""
    T, B, Hkv, Hq = 512, 2, 4, 8
    k, v, q = synth(T, B, Hkv, seed=61, Hq=Hq)
    scaling = 1.0 / math.sqrt(128)
    full = {}
    for tag, x, is_k, mode, blk, rel in (("k", k, True, kmode, 64, 0.05), ("v", v, False, vmode, 128, 0.1)):
        full[tag] = _pipeline(ops, x, is_k, mode, blk, rel, shared)
    kc = ops.make_cache(*[full["k"][n] for n in ("enc", "bi", "ti", "book", "mi", "sc", "spec", "n", "maxb")])
    vc = ops.make_cache(*[full["v"][n] for n in ("enc", "bi", "ti", "book", "mi", "sc", "spec", "n", "maxb")])
    want, st = ops.attn_decode(kc, vc, T, B, Hkv, dev(q), scaling, splits=2)
    assert ops.read_status(st) == 0
    halves = [(0, 2), (2, 4)]
    shard = {}
    for tag, x, is_k, mode, blk, rel in (("k", k, True, kmode, 64, 0.05), ("v", v, False, vmode, 128, 0.1)):
        xs = [dev(x[:, :, a:b]) for a, b in halves]
        spans = mode in (orc.MODE_BLOCK, orc.MODE_TOKEN)
        hists = [torch.zeros(256, dtype=torch.int64, device="cuda") for _ in halves]
        if spans:
            ext = [ops.quant_minmax(xi, mode, blk, shared) for xi in xs]
            mn = torch.minimum(ext[0][0], ext[1][0]); mx = torch.maximum(ext[0][1], ext[1][1])
            qs = [ops.quantize_ranged(xi, mode, blk, rel, mn, mx, shared, min_dtype=torch.int16, hist=h) for xi, h in zip(xs, hists)]
        else:
            qs = [ops.quantize(xi, mode, blk, rel, shared, min_dtype=torch.int16, hist=h) for xi, h in zip(xs, hists)]
        book = ops.build_codebook(hists[0] + hists[1])
        assert torch.equal(book.blob[:32], full[tag]["book"].blob[:32]) and torch.equal(book.blob[64:], full[tag]["book"].blob[64:])
        f = full[tag]
        foff, fnum = orc.block_infos(f["bi"].cpu().numpy())
        fdata = f["enc"][:f["n"]].cpu().numpy()
        shard[tag] = []
        for (a, b), (codes, mi, sc, spec, st) in zip(halves, qs):
            assert ops.read_status(st) == 0
            assert torch.equal(codes, f["codes"][:, :, a:b])
            if spans:
                assert torch.equal(mi, f["mi"]) and torch.equal(sc, f["sc"])
            Hl = b - a
            bsz, tsz, _, cap = ops.buffer_sizes(T, B * Hl * 128, is_k)
            bi = torch.zeros(bsz, dtype=torch.uint8, device="cuda")
            ti = torch.zeros(tsz // 2, dtype=torch.int16, device="cuda")
            enc = torch.zeros(cap, dtype=torch.uint8, device="cuda")
            total, st = ops.encode(codes, is_k, book.encode_table(), bi, ti, enc)
            assert ops.read_status(st) & ~0x10 == 0
            n, maxb = (int(t_) for t_ in total.tolist())
            off, num = orc.block_infos(bi.cpu().numpy())
            data = enc[:n].cpu().numpy()
            # block (row r, local column c) of the shard <-> block (r, global column) of the full stream;
            # V has two blocks (channel halves) per column
            per = 1 if is_k else 2
            lc, gc = B * Hl * per, B * Hkv * per
            for blk_id in range(num.size):
                r, c = divmod(blk_id, lc)
                bb, rest = divmod(c, Hl * per)
                g_id = r * gc + bb * Hkv * per + a * per + rest
                assert num[blk_id] == fnum[g_id]
                assert np.array_equal(data[off[blk_id]: off[blk_id] + num[blk_id]], fdata[foff[g_id]: foff[g_id] + fnum[g_id]])
            shard[tag].append((ops.make_cache(enc, bi, ti, book, mi, sc, spec, n, maxb), (enc, bi, ti, book, mi, sc)))
    g = Hq // Hkv
    for i, (a, b) in enumerate(halves):
        out, st = ops.attn_decode(shard["k"][i][0], shard["v"][i][0], T, B, b - a, dev(q[:, a * g:b * g]), scaling, splits=2)
        assert ops.read_status(st) == 0
        assert torch.equal(out, want[:, a * g:b * g])


def test_k_matvec(ops):
    rng = np.random.default_rng(0)
    k = rng.standard_normal((192, 1, 8, 128)).astype(np.float16)
    q = rng.standard_normal((1, 8, 128)).astype(np.float16)
    out = torch.empty((192, 1, 8), dtype=torch.float16, device="cuda")
    ops.k_matvec(dev(k), dev(q), out)
    ref = orc.k_matvec(k, q)
    assert np.abs(out.float().cpu().numpy() - ref).max() <= 2e-3 * np.abs(ref).max()


def test_errors_are_reported_not_fatal(ops):
    from kvcomp_b200._lib import KvcError
    x = torch.zeros(100, 1, 1, 128, dtype=torch.float16, device="cuda")
    with pytest.raises(KvcError):
        ops.quantize(x, 0, 64, 0.05)                      # T not a multiple of the block
    with pytest.raises(KvcError):
        ops.quantize(x.cpu(), 2, 64, 0.05)                # no CPU path
    with pytest.raises(KvcError):
        ops.buffer_sizes(100, 128, True)
