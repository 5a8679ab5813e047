"""Generate ref_cuda_golden.npz by running the reference's own CUDA operator module.

Run on a machine with a B200 where baseline/_ref/kvcomp_cuda.so exists (built by
oracle/build_ref_cuda.py from the unmodified reference sources); the reference tree itself is
not needed:

    python tests/golden/make_ref_cuda_golden.py [out.npz]

For each small seeded case (batch 1, MHA, K per 64-token block, V per token) it quantises with
the reference's op sequence on CUDA tensors (utils/compute.py:93-106, models/cache/kvcomp_encode.py:83-98),
then calls the reference module for the codebook, both encoders, both decoders and both fused
decode + mat-vec kernels, and stores what they returned: book tensors, the stream with its
block_info / thread_info as the reference laid them out (block order comes from an atomic
cursor), whether decode(encode(x)) == x, and the fused outputs.

The reference's kernels are only run inside the range they are valid for (checked first with the
CPU checker): at most 35 symbols (the fused kernels copy 204 bytes of the decode book,
kernels.cu:740), every K vector at most 128 bytes and every V vector at most 255
(include/kernels.h:15,21; the decoder keeps a vector's byte count in 8 bits, kernels.cu:246),
every block at most 8192 bytes (kernels.cu:615,670), at most 65 535 blocks (kernels.cu:429).
The decode book is handed over inside a larger tensor because huffman_decode reads the node
before the first one (kernels.cu:255 with idx == -1) and the fused kernels always copy 204 bytes.
"""
import hashlib
import importlib.util
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, REPO)

from kvcomp_b200.synth import make_kv  # noqa: E402
from oracle import kvc_oracle as orc  # noqa: E402

CASES = (
    # name, T, H, seed, K rel, V rel
    ("a", 512, 4, 11, 0.05, 0.10),
    ("b", 256, 2, 12, 0.04, 0.07),
    ("c", 1024, 2, 13, 0.06, 0.14),
)


def load_reference():
    so = os.path.join(REPO, "baseline", "_ref", "kvcomp_cuda.so")
    spec = importlib.util.spec_from_file_location("kvcomp_cuda", so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def ref_quant(x5, dims, rel):
    """utils/compute.py:93-106 on a CUDA fp16 tensor [nblk, blk, B, H, D]: every op is torch's."""
    lo, hi = x5, x5
    for d in dims:
        lo = lo.min(dim=d, keepdim=True).values
        hi = hi.max(dim=d, keepdim=True).values
    scale = (hi - lo) * rel
    mi = (lo / scale).round_()
    q = (x5 / scale).round_() - mi
    return q, mi, scale


def guarded(t, front=512, back=512):
    """The bytes of `t` inside a larger device tensor, so that a few bytes before and after it are readable."""
    buf = torch.zeros(front + t.numel() + back, dtype=torch.uint8, device="cuda")
    buf[front:front + t.numel()] = t.to("cuda")
    return buf[front:front + t.numel()]


def check_valid_range(codes_np, is_k):
    """The CPU checker's encode of the same codes tells whether the reference's kernels may run."""
    enc, nsym = orc.gen_codes(orc.histogram(codes_np))
    assert 2 <= nsym <= 35, "book of %d symbols is outside the fused kernels' range" % nsym
    data, bi, ti, ov = orc.encode(codes_np, is_k, enc)
    off, num = orc.block_infos(bi)
    assert num.size <= 65535 and int(num.max()) <= 8192
    ends = (ti.reshape(-1, 64) >> 3).astype(np.int64)
    vec_bytes = np.diff(np.concatenate([np.zeros((ends.shape[0], 1), np.int64), ends], axis=1), axis=1)
    assert int(vec_bytes.max()) <= (128 if is_k else 255), "a vector is longer than the reference's scratch"
    return nsym, int(vec_bytes.max())


def run_case(ref, name, T, H, seed, rel_k, rel_v, out):
    B, D = 1, 128
    k, v, q = make_kv(T, B, H, D, seed=seed, device="cpu")
    g = torch.Generator().manual_seed(seed + 77)
    P = torch.softmax(2.5 * torch.randn(B, H, T, generator=g), dim=-1).half()
    for tag, x, is_k, dims, blk, rel in (("k", k, True, [1, 2, 3, 4], 64, rel_k), ("v", v, False, [2, 3, 4], 128, rel_v)):
        x5 = x.cuda().view(-1, blk, B, H, D)
        qf, mi, sc = ref_quant(x5, dims, rel)
        assert float(qf.min()) >= 0 and float(qf.max()) <= 255
        codes = qf.to(torch.uint8)
        mi8 = mi.to(torch.int8)
        codes_np = codes.reshape(T, B, H, D).cpu().numpy()
        nsym, longest = check_valid_range(codes_np, is_k)
        shift, enc_book, dec_book = ref.build_codebook([codes])
        assert shift == 0
        bsz, tsz, isz, cap = ref.calculate_buffer_size(codes, is_k, H, D)
        bi = torch.zeros(bsz, dtype=torch.uint8, device="cuda")
        ti = torch.zeros(tsz, dtype=torch.uint8, device="cuda")
        cur = torch.zeros(isz, dtype=torch.uint8, device="cuda")
        data = torch.zeros(cap, dtype=torch.uint8, device="cuda")
        enc_dev = enc_book.cuda()
        dec_dev = guarded(dec_book)
        torch.cuda.synchronize()
        encode = ref.k_entropy_encode_cuda_export if is_k else ref.v_entropy_encode_cuda_export
        e_, b_, t_ = encode(codes, enc_dev, bi, ti, cur, data, 0, H, D)
        torch.cuda.synchronize()
        e_, b_, t_ = e_.clone(), b_.clone(), t_.clone()
        back = torch.zeros_like(codes)
        decode = ref.k_entropy_decode_cuda_export if is_k else ref.v_entropy_decode_cuda_export
        decode(e_, b_, t_, dec_dev, back, H, D)
        torch.cuda.synchronize()
        same = bool(torch.equal(back, codes))
        if is_k:
            C = torch.zeros(B, H, T, dtype=torch.float16, device="cuda")
            ref.k_decode_and_mat_vec_mul_cuda_export(dec_dev, b_, t_, e_, mi8, sc, q.cuda(), C, H, D)
        else:
            C = torch.zeros(T // 128, B, H, D, dtype=torch.float16, device="cuda")
            ref.v_decode_and_mat_vec_mul_cuda_export(dec_dev, b_, t_, e_, mi8, sc, P.cuda(), C, H, D)
        torch.cuda.synchronize()
        p = "%s_%s_" % (name, tag)
        out[p + "codes_sha"] = np.frombuffer(hashlib.sha256(codes_np.tobytes()).digest(), dtype=np.uint8)
        out[p + "min"] = mi.reshape(-1).cpu().numpy()
        out[p + "scale"] = sc.reshape(-1).cpu().numpy()
        out[p + "enc_book"] = enc_book.numpy()
        out[p + "dec_book"] = dec_book.numpy()
        out[p + "encoded"] = e_.cpu().numpy()
        out[p + "block_info"] = b_.cpu().numpy()
        out[p + "thread_info"] = t_.cpu().numpy()
        out[p + "fused"] = C.cpu().numpy()
        out[p + "decoded_sha"] = np.frombuffer(hashlib.sha256(back.cpu().numpy().tobytes()).digest(), dtype=np.uint8)
        print("%s %s: %d symbols, longest vector %d B, stream %d B, decode==codes: %s"
              % (name, tag, nsym, longest, e_.numel(), same))
        assert same, "the reference's decoder did not return the codes it encoded"
    out[name + "_P"] = P.numpy()


def main():
    ref = load_reference()
    out = {}
    meta = []
    for name, T, H, seed, rel_k, rel_v in CASES:
        run_case(ref, name, T, H, seed, rel_k, rel_v, out)
        meta.append({"name": name, "T": T, "H": H, "seed": seed, "rel_k": rel_k, "rel_v": rel_v})
    out["cases_json"] = np.frombuffer(json.dumps({"cases": meta, "gpu": torch.cuda.get_device_name(0),
                                                  "torch": torch.__version__}).encode(), dtype=np.uint8)
    dst = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "ref_cuda_golden.npz")
    os.makedirs(os.path.dirname(os.path.abspath(dst)), exist_ok=True)
    np.savez_compressed(dst, **out)
    print("wrote", dst, os.path.getsize(dst), "bytes")


if __name__ == "__main__":
    main()
