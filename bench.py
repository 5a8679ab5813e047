#!/usr/bin/env python
"""Benchmark of the fused decompress-matvec decode attention and of the codec around it.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c1|c0|c2|c3|c4] [--impl reference]

One "step" = one decode step of the whole model: for every layer, one call of the fused kernel that
reads the layer's compressed K and V streams and produces the attention output of every sequence and
head (q.K^T -> softmax -> P.V, no fp16 K/V materialised).  value = tokens/s = sequences / step time,
summed over all ranks.  With N > 1 every rank holds its own batch of sequences of the same size (the
path shards by batch sequence without any exchange on the data path), so scaling is weak.

The timed region is a block of exactly K steps between two barriers; the block is repeated until a
second of device time has been measured and the median block is reported (ms_per_step is per step).

Prints ONE JSON line (rank 0).  Besides the headline it carries
  roofline       the attention kernel against the measured HBM copy peak
  e2e            the same step with q coming from and the output going back to pinned host memory
  codec          quantise + histogram + codebook + encode, and decode, of one 1 GiB fp16 chunk per
                 tensor at five error bounds: encode / decode GB/s, compression ratio, bits per symbol
  gpu_reference  (N = 1, when baseline/_ref/kvcomp_cuda.so is present) the reference's own fused K and
                 V kernels timed beside this library's on the reference's own shapes
  other_workloads (N = 1) the two grouped-query configurations, a few layers each: per-layer time and roofline
                 fraction; c1 with its newest 128 tokens as the uncompressed recent window; a decode loop
                 through the cache class the model files call (append + attend per layer)
  strong         (N > 1) the Mistral-shaped GQA cache with its KV heads split over the ranks and one NCCL
                 all-gather of the outputs per step, against the same layers on one GPU
  cpu_baseline   (N = 1) the CPU restatement of the reference's path on a bounded sample
--impl reference times that CPU restatement (oracle/, OpenMP over the host cores) instead.
Profiling helpers: --layers, --no-extras, --min-seconds, --codec-rels (c4: fewer error bounds), --side (one side record alone).
"""
import argparse
import importlib.util
import json
import math
import os
import re
import subprocess
import sys
import tempfile
import time

import numpy as np

REPO = os.path.dirname(os.path.abspath(__file__))
if REPO not in sys.path:
    sys.path.insert(0, REPO)

WORKLOADS = {
    # name: layers, T, B, Hkv, Hq, K mode/rel/block, V rel
    "c0": dict(desc="Llama-2-7B single layer, 32 heads x 128, batch 1, 1024 tokens, K per-channel 0.05 / V per-token 0.05, block 64",
               layers=1, T=1024, B=1, Hkv=32, Hq=32, kmode="ChannelQuant", krel=0.05, kblock=64, vrel=0.05),
    "c1": dict(desc="Llama-2-7B-shaped full cache: 32 layers x 32 heads (MHA) x 128, batch 8, 4096-token context, K per-channel 0.05 / V per-token 0.1, block 64",
               layers=32, T=4096, B=8, Hkv=32, Hq=32, kmode="ChannelQuant", krel=0.05, kblock=64, vrel=0.1),
    "c2": dict(desc="Mistral-7B-shaped GQA: 32 layers, 32 query / 8 KV heads x 128, batch 16, 32768-token context, K per-channel 0.05 / V per-token 0.1",
               layers=32, T=32768, B=16, Hkv=8, Hq=32, kmode="ChannelQuant", krel=0.05, kblock=64, vrel=0.1),
    "c3": dict(desc="Phi-3-medium-shaped GQA: 40 layers, 40 query / 10 KV heads x 128, batch 32, 16384-token context, K per-channel 0.02 block 128 / V per-token 0.15",
               layers=40, T=16384, B=32, Hkv=10, Hq=40, kmode="ChannelQuant", krel=0.02, kblock=128, vrel=0.15),
}
METRIC = "decode attn tokens/s (fused decomp-matvec)"
MIN_TIMED_SECONDS = 1.0
MAX_BLOCKS = 200


def make_config(args, cfg, heads_mode=False):
    """The `config` object of the JSON line: the same for this library's arm and for the CPU arm."""
    return {"workload": args.workload + ": " + cfg["desc"], "layers": cfg["layers"],
            "l2": "inputs larger than L2: every step reads every layer's compressed K and V streams once",
            "sharding": "KV heads split over the ranks, one NCCL all-gather of the outputs per step" if heads_mode
            else "batch sequences per rank, no collective on the data path"}


def peaks():
    """Measured HBM peak of this pool (driver-written file), else the stated fallback."""
    try:
        with open(os.path.join(REPO, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def profile_traffic(name="attn_decode_c1.md"):
    """DRAM bytes per algorithmic byte of the attention kernel, from the committed ncu summary: the lines
    `dram_bytes_per_launch:`, `algorithmic_bytes_per_launch:` and `commit:` of profiles/<name>."""
    try:
        with open(os.path.join(REPO, "profiles", name)) as f:
            text = f.read()
        dram = float(re.search(r"^\s*dram_bytes_per_launch:\s*([0-9.eE+]+)", text, re.M).group(1))
        alg = float(re.search(r"^\s*algorithmic_bytes_per_launch:\s*([0-9.eE+]+)", text, re.M).group(1))
        commit = re.search(r"^\s*commit:\s*(\S+)", text, re.M)
        return dram / alg, {"file": "profiles/" + name, "commit": commit.group(1) if commit else None,
                            "dram_bytes_per_launch": dram, "algorithmic_bytes_per_launch": alg}
    except Exception:
        return None, None


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.path = index, None, None

    def start(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            with open(self.path) as f:
                for line in f:
                    p = [x.strip() for x in line.split(",")]
                    if len(p) < 9:
                        continue
                    try:
                        sm.append(float(p[1])); mx.append(float(p[2]))
                    except ValueError:
                        continue
                    for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[5:9]):
                        if val.lower().startswith("active"):
                            reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out.update(sm_mhz=float(np.median(sm)), sm_max_mhz=float(max(mx)), reasons=sorted(reasons), samples=len(sm))
        return out


def compress(ops, torch, x, is_k, mode, rel, blk, device, batch_shared=False, head_sharded=False):
    """fp16 [T, B, H, 128] -> (cache, tensors that back it, byte accounting)."""
    T, B, H, _ = x.shape
    hist = torch.zeros(256, dtype=torch.int64, device=device)
    if head_sharded:
        from kvcomp_b200 import sharding
        codes, mi, sc, spec, st = sharding.quantize_head_shard(x, mode, blk, rel, batch_shared, torch.int16, hist)
        book = sharding.build_shared_codebook(hist)
    else:
        codes, mi, sc, spec, st = ops.quantize(x, mode, blk, rel, batch_shared, min_dtype=torch.int16, hist=hist)
        book = ops.build_codebook(hist)
    bsz, tsz, _, cap = ops.buffer_sizes(T, B * H * 128, is_k)
    bi = torch.empty(bsz, dtype=torch.uint8, device=device)
    ti = torch.empty(tsz // 2, dtype=torch.int16, device=device)
    enc = torch.empty(cap, dtype=torch.uint8, device=device)
    total, st2 = ops.encode(codes, is_k, book.encode_table(), bi, ti, enc)
    n, maxb = (int(v) for v in total.tolist())
    ops.read_status(st, what="quantize"); ops.read_status(st2, what="encode")
    enc = enc[:n].clone()
    keep = (enc, bi, ti, book, mi, sc)
    acct = dict(encoded=n, block_info=bsz, thread_info=tsz, quant_meta=mi.numel() * mi.element_size() + sc.numel() * 2,
                symbols=T * B * H * 128, max_block=maxb)
    return ops.make_cache(enc, bi, ti, book, mi, sc, spec, n, maxb), keep, acct


def build_layer(ops, torch, cfg, layer, seed, device, heads=None):
    """Synthetic K/V of one layer -> compressed caches resident in HBM.  heads = (start, count, q_start,
    q_count): this rank's KV heads of the full tensor (the compression-time exchanges of head sharding run
    inside).  Returns the cache pair, the tensors that back them, q and the byte accounting."""
    from kvcomp_b200.synth import make_kv
    T, B, Hkv, Hq = cfg["T"], cfg["B"], cfg["Hkv"], cfg["Hq"]
    k, v, q = make_kv(T, B, Hkv, 128, seed=seed, layer=layer, device=device, Hq=Hq)
    if heads is not None:
        s, c, qs, qc = heads
        k, v, q = k[:, :, s:s + c].contiguous(), v[:, :, s:s + c].contiguous(), q[:, qs:qs + qc].contiguous()
    keep, caches, acct = [], [], {}
    for name, x, is_k, mode, rel, blk in (("k", k, True, ops.MODES[cfg["kmode"]], cfg["krel"], cfg["kblock"]),
                                          ("v", v, False, ops.MODE_TOKEN, cfg["vrel"], 128)):
        cache, kp, a = compress(ops, torch, x, is_k, mode, rel, blk, device, head_sharded=heads is not None)
        caches.append(cache); keep.append(kp); acct[name] = a
    del k, v
    return caches, keep, q, acct


def algorithmic_bytes(acct, cfg):
    """Bytes one fused launch has to move: both compressed streams, their offset tables and quant
    metadata once, q in and the output once."""
    qo = 2 * cfg["B"] * cfg["Hq"] * 128 * 2
    return sum(a["encoded"] + a["block_info"] + a["thread_info"] + a["quant_meta"] for a in acct.values()) + qo


def cpu_sample(cfg, seed, min_seconds=8.0):
    """The CPU restatement on a bounded sample: one sequence of one layer (all heads, full context):
    Huffman-decode both streams, then one decode-attention step.  Returns seconds per sample."""
    # torch.distributed.run pins OMP_NUM_THREADS to 1; the CPU arm is meant to use every host core
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    from kvcomp_b200.synth import make_kv
    from oracle import kvc_oracle as orc
    T, Hkv, Hq = cfg["T"], cfg["Hkv"], cfg["Hq"]
    k, v, q = make_kv(T, 1, Hkv, 128, seed=seed, layer=0, device="cpu", Hq=Hq)
    k, v, q = k.numpy(), v.numpy(), q.numpy()
    kc, kmi, ksc, km, _ = orc.quant(k, orc.MODES[cfg["kmode"]], cfg["kblock"], cfg["krel"], False)
    vc, vmi, vsc, vm, _ = orc.quant(v, orc.MODE_TOKEN, 128, cfg["vrel"], False)
    kenc, _ = orc.gen_codes(orc.histogram(kc)); venc, _ = orc.gen_codes(orc.histogram(vc))
    kd, kbi, kti, _ = orc.encode(kc, True, kenc); vd, vbi, vti, _ = orc.encode(vc, False, venc)
    scaling = 1.0 / math.sqrt(128)
    reps, t0 = 0, time.perf_counter()
    while True:
        kc2, bad1 = orc.decode(kd, kbi, kti, kenc, T, 1, Hkv, True)
        vc2, bad2 = orc.decode(vd, vbi, vti, venc, T, 1, Hkv, False)
        orc.attention(kc2, kmi, ksc, km, vc2, vmi, vsc, vm, q, scaling)
        reps += 1
        el = time.perf_counter() - t0
        if el >= min_seconds or reps >= 64:
            break
    assert bad1 == 0 and bad2 == 0
    return el / reps, orc.num_threads()


CPU_NOTE = ("the reference has no CPU decoder or CPU attention (utils/huffman.py only encodes): this arm is the C/OpenMP "
            "restatement of its kernels; the reference's own Python CPU path (utils/compute.py quantiser, utils/huffman.py "
            "encoder, torch-CPU attention) is timed on config 0 where the reference tree is mounted, figures in the repository's baseline notes")


def cpu_baseline_record(cfg, seed, min_seconds):
    s, threads = cpu_sample(cfg, seed, min_seconds=min_seconds)
    samples = cfg["layers"] * cfg["B"]
    step_s = s * samples
    return {"value": cfg["B"] / step_s, "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": "1 sequence x 1 layer (%d heads, %d tokens) of the same workload: Huffman decode of K and V + attention, "
                      "%.2f s each; a step is %d such samples" % (cfg["Hkv"], cfg["T"], s, samples),
            "sample_fraction": 1.0 / samples, "extrapolated": True, "sample_seconds": s, "note": CPU_NOTE}, step_s


# ---- codec: quantise + histogram + codebook + encode, decode, compression ratio ------------------------
def codec_sweep(ops, torch, device, seed, rels=(0.01, 0.02, 0.05, 0.1, 0.2), T=4096, B=32, H=32, reps=2):
    """One 1 GiB fp16 chunk per tensor (32 heads x 128, batch 32, 4096 tokens: a chunk of the prefill-side
    configuration's 131072-token sequences), K per channel / V per token.  Per error bound:
      encode_GBps       fp16 bytes in per second over quantise + histogram + codebook + encode, K then V on one
                        stream: a sequence's first chunk, whose codes make the book (kvcomp_encode.py:99-103)
      encode_next_GBps  the same chunk stored with the books frozen, as every later chunk of a sequence is:
                        quantise + encode, the K and the V chain on two streams
      decode_GBps       fp16-equivalent bytes out per second, K then V (decode_2s_GBps: on two streams)
    plus compression ratio in the reference's accounting, bits per symbol, and an exact round-trip check of
    both stores.  Returns (per-rel results, launches, raw ms)."""
    from kvcomp_b200.synth import make_kv
    fp16_bytes = 2 * T * B * H * 128
    out, launches, raw = {}, 0, {}
    k, v, _ = make_kv(T, B, H, 128, seed=seed, layer=0, device=device)
    tensors = (("k", k, True, ops.MODE_CHANNEL, 64), ("v", v, False, ops.MODE_TOKEN, 128))
    side = [torch.cuda.Stream(device=device) for _ in range(2)]
    main = torch.cuda.current_stream()

    def on_two_streams(fk, fv):
        """ms for fk on one stream and fv on another, both starting after everything queued so far."""
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        done = [torch.cuda.Event() for _ in range(2)]
        ev[0].record(main)
        for st, f, d in zip(side, (fk, fv), done):
            st.wait_event(ev[0])
            with torch.cuda.stream(st):
                f()
                d.record(st)
        for d in done:
            main.wait_event(d)
        ev[1].record(main)
        torch.cuda.synchronize()
        return ev[0].elapsed_time(ev[1])

    for rel in rels:
        enc_ms, dec_ms, comp, bits, skipped = 0.0, 0.0, 0, {}, False
        st8 = {}
        for name, x, is_k, mode, blk in tensors:
            bsz, tsz, _, cap = ops.buffer_sizes(T, B * H * 128, is_k)
            bi = torch.empty(bsz, dtype=torch.uint8, device=device)
            ti = torch.empty(tsz // 2, dtype=torch.int16, device=device)
            enc = torch.empty(cap, dtype=torch.uint8, device=device)
            best_e, best_d = None, None
            for it in range(1 + reps):                       # one warm-up pass, then `reps` timed ones (the best counts)
                hist = torch.zeros(256, dtype=torch.int64, device=device)
                ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
                ev[0].record()
                codes, mi, sc, spec, st = ops.quantize(x, mode, blk, rel, False, min_dtype=torch.int16, hist=hist)
                book = ops.build_codebook(hist)
                total, st2 = ops.encode(codes, is_k, book.encode_table(), bi, ti, enc)
                ev[1].record()
                n, maxb = (int(t_) for t_ in total.tolist())
                flags = ops.read_status(st, False) | ops.read_status(st2, False)
                if flags & 0x20:                             # a block beyond 8191 bytes: the format's u16 fields cannot hold it
                    skipped = True
                    break
                ev[2].record()
                back, st3 = ops.decode(enc[:n], bi, ti, book, T, B, H, is_k, max_block=maxb)
                ev[3].record()
                torch.cuda.synchronize()
                assert torch.equal(back, codes), "round trip failed at rel %g" % rel
                if it:
                    e, d = ev[0].elapsed_time(ev[1]), ev[2].elapsed_time(ev[3])
                    best_e = e if best_e is None else min(best_e, e)
                    best_d = d if best_d is None else min(best_d, d)
                    launches += 4                            # quantise, codebook, encode, decode
                del back
            if skipped:
                break
            enc_ms += best_e; dec_ms += best_d
            comp += n + bsz + tsz + mi.numel() * mi.element_size() + sc.numel() * 2
            bits[name] = 8.0 * n / codes.numel()
            raw["%s_%g" % (name, rel)] = [best_e, best_d]
            st8[name] = dict(x=x, is_k=is_k, mode=mode, blk=blk, book=book, bi=bi, ti=ti, enc=enc, n=n, maxb=maxb,
                             codes=codes, mi=mi, sc=sc, status=ops.new_status(device), total=torch.zeros(2, dtype=torch.int64, device=device),
                             back=torch.empty_like(codes))
        if skipped:
            out[str(rel)] = {"skipped": "a block exceeds the 8191 bytes the stream format can describe"}
            continue

        # later chunks of a sequence: the books are frozen; nothing is read back inside the timed region
        def store_next(t):
            def f():
                ops.quantize(t["x"], t["mode"], t["blk"], rel, False, min_dtype=torch.int16, codes=t["codes"], min_int=t["mi"],
                             scale=t["sc"], status=t["status"])
                t["total"].zero_()
                ops.encode(t["codes"], t["is_k"], t["book"].encode_table(), t["bi"], t["ti"], t["enc"], status=t["status"], total=t["total"])
            return f

        def load(t):
            return lambda: ops.decode(t["enc"][:t["n"]], t["bi"], t["ti"], t["book"], T, B, H, t["is_k"], out=t["back"],
                                      status=t["status"], max_block=t["maxb"])
        next_ms = min(on_two_streams(store_next(st8["k"]), store_next(st8["v"])) for _ in range(1 + reps))
        dec2_ms = min(on_two_streams(load(st8["k"]), load(st8["v"])) for _ in range(1 + reps))
        launches += (1 + reps) * 6                       # (quantise, encode) x 2 and decode x 2
        for t in st8.values():
            assert ops.read_status(t["status"]) == 0 and int(t["total"][0]) == t["n"], "frozen-book store differs"
            assert torch.equal(t["back"], t["codes"]), "round trip of the frozen-book store failed at rel %g" % rel
        out[str(rel)] = {"encode_GBps": 2 * fp16_bytes / 1e9 / (enc_ms / 1e3), "decode_GBps": 2 * fp16_bytes / 1e9 / (dec_ms / 1e3),
                         "encode_next_GBps": 2 * fp16_bytes / 1e9 / (next_ms / 1e3), "decode_2s_GBps": 2 * fp16_bytes / 1e9 / (dec2_ms / 1e3),
                         "compression_ratio": 2 * fp16_bytes / comp, "bits_per_symbol": bits,
                         "encode_ms": enc_ms, "decode_ms": dec_ms, "encode_next_ms": next_ms, "decode_2s_ms": dec2_ms}
        del st8
    del k, v
    return out, launches, raw


# ---- the reference's own CUDA kernels beside this library's -------------------------------------------
def load_reference_cuda():
    so = os.path.join(REPO, "baseline", "_ref", "kvcomp_cuda.so")
    if not os.path.exists(so):
        return None
    import torch  # noqa: F401
    spec = importlib.util.spec_from_file_location("kvcomp_cuda", so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def gpu_reference(ops, torch, device, seed, ctxs=(2048, 4096, 8192, 16384), H=32, reps=5):
    """The unmodified reference module's fused kernels (kernels.cu:721-776 K, :778-861 V; its own cudaEvent
    milliseconds) beside kvc_fused_qk / kvc_fused_pv on the same data, on the reference's own benchmark
    shapes (kvcomp_cuda_extension/scripts/temp.py:4-8: 32 heads x 128, batch 1, ctx 2048..16384) and
    settings (K per 64-token block at 0.05, V per token at 0.1).  The reference only runs inside its valid
    range: at most 35 symbols, no vector beyond its per-thread scratch, at most 65 535 blocks."""
    ref = load_reference_cuda()
    if ref is None:
        return {"unavailable": "baseline/_ref/kvcomp_cuda.so is not present (built by oracle/build_ref_cuda.py where the reference tree is)"}
    from kvcomp_b200.synth import make_kv
    rows = []
    for T in ctxs:
        k, v, q = make_kv(T, 1, H, 128, seed=seed, layer=0, device=device)
        P = torch.softmax(2.5 * torch.randn(1, H, T, device=device), dim=-1).half()
        row = {"ctx": T}
        for tag, x, is_k, mode, blk, rel, B_ in (("k", k, True, ops.MODE_BLOCK, 64, 0.05, q), ("v", v, False, ops.MODE_TOKEN, 128, 0.1, P)):
            hist = torch.zeros(256, dtype=torch.int64, device=device)
            codes, mi, sc, spec, st = ops.quantize(x, mode, blk, rel, True, min_dtype=torch.int8, hist=hist)
            book = ops.build_codebook(hist)
            hd = book.header()
            # this library's encoder reports what the reference cannot hold: a vector beyond its per-thread scratch
            # (K 128 B, V 256 B, include/kernels.h:15,21) or a block beyond the format's 16-bit byte count
            bsz0, tsz0, _, cap0 = ops.buffer_sizes(T, H * 128, is_k)
            tmp = [torch.empty(bsz0, dtype=torch.uint8, device=device), torch.empty(tsz0 // 2, dtype=torch.int16, device=device),
                   torch.empty(cap0, dtype=torch.uint8, device=device)]
            tot, st_e = ops.encode(codes, is_k, book.encode_table(), tmp[0], tmp[1], tmp[2])
            del tmp
            if not (2 <= hd["n_symbols"] <= 35 and ops.read_status(st, False) == 0 and ops.read_status(st_e, False) == 0
                    and T // blk * H * (1 if is_k else 2) <= 65535):
                row[tag] = {"skipped": "outside the reference kernels' valid range (%d symbols, encoder flags %#x)" % (hd["n_symbols"], ops.read_status(st_e, False))}
                continue
            c5 = codes.view(-1, blk, 1, H, 128)
            shift, enc_book, dec_book = ref.build_codebook([c5])
            bsz, tsz, isz, cap = ref.calculate_buffer_size(c5, is_k, H, 128)
            bufs = [torch.zeros(n, dtype=torch.uint8, device=device) for n in (bsz, tsz, isz, cap)]
            guard = torch.zeros(1024 + dec_book.numel(), dtype=torch.uint8, device=device)     # readable bytes around the book
            guard[512:512 + dec_book.numel()] = dec_book.to(device)
            dec_dev = guard[512:512 + dec_book.numel()]
            torch.cuda.synchronize()
            encode = ref.k_entropy_encode_cuda_export if is_k else ref.v_entropy_encode_cuda_export
            e_, b_, t_ = encode(c5, enc_book.to(device), bufs[0], bufs[1], bufs[2], bufs[3], 0, H, 128)
            torch.cuda.synchronize()
            if is_k:
                C = torch.zeros(1, H, T, dtype=torch.float16, device=device)
                fused = lambda: ref.k_decode_and_mat_vec_mul_cuda_export(dec_dev, b_, t_, e_, mi, sc, B_, C, H, 128)
            else:
                C = torch.zeros(T // 128, 1, H, 128, dtype=torch.float16, device=device)
                fused = lambda: ref.v_decode_and_mat_vec_mul_cuda_export(dec_dev, b_, t_, e_, mi, sc, B_, C, H, 128)
            ref_ms = min(fused() for _ in range(reps + 1))
            torch.cuda.synchronize()
            # this library on the reference's stream, through the same tables
            mine_book = ops.book_from_tree(dec_dev.clone())
            encp = torch.cat([e_, torch.zeros(64, dtype=torch.uint8, device=device)])
            cache = ops.make_cache(encp, b_, t_, mine_book, mi, sc, spec, e_.numel())
            # outputs and the status word are made once: the timed region holds kernel launches only, ten per
            # measurement (the reference's figure is the cudaEvent time around its one launch)
            st = ops.new_status(device)
            out = torch.empty((1, H, T) if is_k else (T // 128, 1, H, 128), dtype=torch.float16, device=device)
            call = (lambda: ops.fused_qk(cache, T, 1, H, B_, out=out, status=st)) if is_k else \
                (lambda: ops.fused_pv(cache, T, 1, H, B_, out=out, status=st))
            call()
            best = None
            for _ in range(reps):
                ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
                torch.cuda.synchronize()
                ev[0].record()
                for _i in range(10):
                    call()
                ev[1].record()
                torch.cuda.synchronize()
                ms = ev[0].elapsed_time(ev[1]) / 10
                best = ms if best is None else min(best, ms)
            assert ops.read_status(st) == 0
            mine = out.float() if is_k else out.float().sum(0)
            theirs = C.float() if is_k else C.float().sum(0)
            agree = float((mine - theirs).abs().max() / theirs.abs().max())
            row[tag] = {"reference_ms": ref_ms, "kvcomp_b200_ms": best, "speedup": ref_ms / best,
                        "max_diff_of_max": agree, "fp16_GBps_reference": 2 * x.numel() / 1e6 / ref_ms,
                        "fp16_GBps_kvcomp_b200": 2 * x.numel() / 1e6 / best}
        rows.append(row)
        del k, v
    return {"shapes": "32 heads x 128, batch 1, K per 64-token block at 0.05 / V per token at 0.1 (the reference's own settings)",
            "timing": "reference: the milliseconds its export returns (cudaEvent around its launch); this library: CUDA events around 10 launches, best of %d" % reps,
            "rows": rows}


def side_workloads(ops, torch, device, seed, names=("c2", "c3"), layers=2):
    """The grouped-query configurations on one GPU, a few layers each (their full caches are for several GPUs):
    per-layer time of the fused kernel, its fraction of the HBM roofline on compressed bytes, fp16-equivalent
    bytes served."""
    out = {}
    peak, _ = peaks()
    for name in names:
        cfg = dict(WORKLOADS[name]); cfg["layers"] = layers
        T, B, Hkv, Hq = cfg["T"], cfg["B"], cfg["Hkv"], cfg["Hq"]
        built = [build_layer(ops, torch, cfg, l, seed, device) for l in range(layers)]
        ws = ops.attn_workspace(B, Hq, ops.attn_splits(T, B, Hkv), device)
        status = ops.new_status(device)
        outs = torch.empty((layers, B, Hq, 128), dtype=torch.float16, device=device)
        scaling = 1.0 / math.sqrt(128)

        def step():
            for i, (caches, _, q, _) in enumerate(built):
                ops.attn_decode(caches[0], caches[1], T, B, Hkv, q, scaling, out=outs[i], workspace=ws, status=status)
        for _ in range(3):
            step()
        blocks = timed_blocks(torch, step, 5, torch.cuda.synchronize, min_seconds=0.2)
        ops.read_status(status, what="attn_decode")
        ms_layer = float(np.median(blocks)) / 5 / layers
        alg = float(np.mean([algorithmic_bytes(b[3], cfg) for b in built]))
        out[name] = {"workload": name + ": " + cfg["desc"], "layers_timed": layers, "ms_per_layer": ms_layer,
                     "tokens_per_s_full_model": B / (ms_layer * WORKLOADS[name]["layers"] / 1e3),
                     "algorithmic_bytes_per_layer": alg, "achieved_GBps": alg / ms_layer / 1e6, "frac_of_hbm_peak": alg / ms_layer / 1e6 / peak,
                     "effective_fp16_GBps": 2 * 2 * T * B * Hkv * 128 / ms_layer / 1e6,
                     "launches_per_layer": sum(1 for _ in _chunks(Hq // Hkv)) + 1,
                     "bits_per_symbol": {k: float(np.mean([8.0 * b[3][k]["encoded"] / b[3][k]["symbols"] for b in built])) for k in ("k", "v")}}
        del built, ws, outs
        torch.cuda.empty_cache()
    out["c1_recent_window"] = recent_window_record(ops, torch, device, seed)
    out["c1_cache_class_loop"] = cache_class_loop_record(torch, device, seed)
    return out


def cache_class_loop_record(torch, device, seed, layers=8, steps=96):
    """A decode loop through the cache class the model files call (KVCompCache.append + attend per layer:
    models/llama.py:279-283 with the fused branch), c1's shape: a 4096-token prefill, then one token per step.
    Per-layer time including the rotation and transposition of the new token into the recent window, the
    compression of a block whenever the window overflows (every 64 / 128 steps), and the fused attention with
    the window as fp16 tail."""
    from kvcomp_b200.cache import KVCompCache
    from kvcomp_b200.synth import make_kv
    from kvcomp_b200.utils.compute import QuantMode
    from kvcomp_b200.utils.config import KVCompCacheConfig, KVCompCacheConfigStatic
    c = WORKLOADS["c1"]
    T, B, H = c["T"], c["B"], c["Hkv"]
    saved = KVCompCacheConfigStatic.config
    KVCompCacheConfigStatic.config = KVCompCacheConfig("synthetic", QuantMode.ChannelQuant, QuantMode.TokenQuant, c["kblock"], 128,
                                                      128, 128, c["krel"], c["vrel"])
    try:
        cache = KVCompCache(B, H, 128, layers)
        cos = torch.ones(1, T, 128, dtype=torch.float16, device=device)
        sin = torch.zeros(1, T, 128, dtype=torch.float16, device=device)
        for l in range(layers):
            k, v, _ = make_kv(T, B, H, 128, seed=seed, layer=l, device=device)
            cache.append(k.permute(1, 2, 0, 3).contiguous(), v.permute(1, 2, 0, 3).contiguous(), l, {"cos": cos, "sin": sin})
            del k, v
        k1, v1, q = make_kv(1, B, H, 128, seed=seed + 5, layer=0, device=device)
        kn, vn, qq = k1.permute(1, 2, 0, 3).contiguous(), v1.permute(1, 2, 0, 3).contiguous(), q.view(B, H, 1, 128)
        kw = {"cos": cos[:, :1], "sin": sin[:, :1]}
        scaling = 1.0 / math.sqrt(128)

        def step():
            for l in range(layers):
                cache.append(kn, vn, l, kw)
                cache.attend(qq, l, scaling)
        for _ in range(4):
            step()
        torch.cuda.synchronize()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        ev[0].record()
        for _ in range(steps):
            step()
        ev[1].record()
        torch.cuda.synchronize()
        cache.check()
        ms_layer = ev[0].elapsed_time(ev[1]) / steps / layers
        return {"workload": "KVCompCache.append + attend per layer, c1's shape, %d layers, %d decode steps after a %d-token prefill" % (layers, steps, T),
                "ms_per_layer": ms_layer, "tokens_per_s_full_model": B / (ms_layer * c["layers"] / 1e3),
                "recent_window": 128, "includes": "RoPE and transposition of the new token, block compression when the window overflows, fused attention with the window as fp16 tail"}
    finally:
        KVCompCacheConfigStatic.config = saved
        torch.cuda.empty_cache()


def recent_window_record(ops, torch, device, seed, layers=4, recent=128):
    """c1's 4096-token context as a cache class holds it during decoding: the newest `recent` tokens
    (models/cache/kvcomp_encode.py:80, k_recent_size) uncompressed as fp16 rows behind 4096 - recent compressed
    ones.  Per-layer time of the same launch pair as the headline."""
    from kvcomp_b200.synth import make_kv
    cfg = dict(WORKLOADS["c1"]); cfg["T"] = WORKLOADS["c1"]["T"] - recent
    T, B, Hkv, Hq = cfg["T"], cfg["B"], cfg["Hkv"], cfg["Hq"]
    built = [build_layer(ops, torch, cfg, l, seed, device) for l in range(layers)]
    tails = [make_kv(recent, B, Hkv, 128, seed=seed + 17, layer=l, device=device)[:2] for l in range(layers)]
    ws = ops.attn_workspace(B, Hq, ops.attn_splits(T, B, Hkv), device)
    status = ops.new_status(device)
    outs = torch.empty((layers, B, Hq, 128), dtype=torch.float16, device=device)
    scaling = 1.0 / math.sqrt(128)

    def step():
        for i, (caches, _, q, _) in enumerate(built):
            ops.attn_decode(caches[0], caches[1], T, B, Hkv, q, scaling, tails[i][0], tails[i][1], out=outs[i], workspace=ws, status=status)
    for _ in range(3):
        step()
    blocks = timed_blocks(torch, step, 5, torch.cuda.synchronize, min_seconds=0.2)
    ops.read_status(status, what="attn_decode")
    ms_layer = float(np.median(blocks)) / 5 / layers
    rec = {"workload": "c1 with the newest %d of its 4096 tokens as uncompressed fp16 rows (the recent window)" % recent,
           "layers_timed": layers, "compressed_tokens": T, "fp16_tail_tokens": recent, "ms_per_layer": ms_layer,
           "tokens_per_s_full_model": B / (ms_layer * WORKLOADS["c1"]["layers"] / 1e3)}
    del built, tails, ws, outs
    torch.cuda.empty_cache()
    return rec


def timed_blocks(torch, step, steps, barrier, min_seconds=MIN_TIMED_SECONDS, max_blocks=MAX_BLOCKS, world_reduce=None):
    """Blocks of exactly `steps` steps, each bracketed by barrier + synchronize on both sides and timed with
    CUDA events on the launching stream; repeated until `min_seconds` of device time are covered.  Every
    rank runs the same number of blocks (the count is agreed after the first).  Returns the per-block ms."""
    def one():
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        barrier()
        ev[0].record()
        for _ in range(steps):
            step()
        ev[1].record()
        barrier()
        ms = ev[0].elapsed_time(ev[1])
        return world_reduce(ms) if world_reduce else ms
    first = one()
    n = int(min(max_blocks, max(1, math.ceil(min_seconds * 1e3 / max(first, 1e-3)))))
    return [first] + [one() for _ in range(n - 1)]


def run_reference(args, cfg, rank, world):
    """CPU arm: the restated reference path on the host cores, a bounded sample per step."""
    if rank != 0:
        return
    per_step = []
    for i in range(args.warmup + args.steps):
        s, threads = cpu_sample(cfg, args.seed, min_seconds=2.0)
        if i >= args.warmup:
            per_step.append(s)
    s = float(np.mean(per_step))
    samples_per_step = cfg["layers"] * cfg["B"]
    step_s = s * samples_per_step
    val = cfg["B"] / step_s                       # one host: the CPU does every rank's work in turn
    sample = "1 sequence x 1 layer (%d heads, %d tokens): Huffman decode of K and V + attention; a step is %d such samples" % (
        cfg["Hkv"], cfg["T"], samples_per_step)
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8 codes -> f32 accumulate",
            "data": "synthetic", "config": make_config(args, cfg),
            "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample,
                             "sample_fraction": 1.0 / samples_per_step, "extrapolated": True, "sample_seconds": s,
                             "note": "ms_per_step is the measured sample time x %d; the run itself measures %d samples. " % (samples_per_step, args.steps) + CPU_NOTE},
            "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def strong_record(args, ops, torch, dist, device, rank, world, barrier, reduce_max):
    """Head sharding against one GPU: a few layers of the Mistral-shaped cache (4 query heads per KV head) and of
    the Llama-shaped one.  Rank 0 first runs the layers with all heads alone; then every rank runs its KV
    heads of the same caches (the shards are the single-GPU caches cut by head) and the step ends in one NCCL
    all-gather of the outputs.  The gather is also timed alone."""
    from kvcomp_b200 import sharding
    res = {}
    for name, L in (("c2", 4), ("c1", 8)):
        cfg = dict(WORKLOADS[name]); cfg["layers"] = L
        if cfg["Hkv"] % world:
            res[name] = {"skipped": "%d KV heads do not split over %d ranks" % (cfg["Hkv"], world)}
            continue
        T, B, Hkv, Hq = cfg["T"], cfg["B"], cfg["Hkv"], cfg["Hq"]
        scaling = 1.0 / math.sqrt(128)

        def stepper(layers, hkv, hq, gather):
            ws = ops.attn_workspace(B, hq, ops.attn_splits(T, B, hkv), device)
            status = ops.new_status(device)
            out_all = torch.empty((L, B, hq, 128), dtype=torch.float16, device=device)
            buf = torch.empty((world, L, B, hq, 128), dtype=torch.float16, device=device) if gather else None

            def step():
                for i, (caches, _, q, _) in enumerate(layers):
                    ops.attn_decode(caches[0], caches[1], T, B, hkv, q, scaling, out=out_all[i], workspace=ws, status=status)
                if gather:
                    dist.all_gather_into_tensor(buf, out_all)
            return step, status, out_all, buf

        one_ms = None
        if rank == 0:                                   # all heads on one GPU
            layers = [build_layer(ops, torch, cfg, l, args.seed, device) for l in range(L)]
            step, status, _, _ = stepper(layers, Hkv, Hq, False)
            for _ in range(3):
                step()
            torch.cuda.synchronize()
            blocks = timed_blocks(torch, step, 3, torch.cuda.synchronize, min_seconds=0.3)
            one_ms = float(np.median(blocks)) / 3
            ops.read_status(status, what="attn_decode")
            del layers, step
            torch.cuda.empty_cache()
        barrier()
        heads = sharding.shard_heads(Hkv, Hq, world, rank)
        scfg = dict(cfg)
        layers = []
        for l in range(L):                              # the exchanges inside need every rank at the same layer
            layers.append(build_layer(ops, torch, scfg, l, args.seed, device, heads=heads))
        step, status, out_all, buf = stepper(layers, heads[1], heads[3], True)
        for _ in range(3):
            step()
        blocks = timed_blocks(torch, step, 3, barrier, min_seconds=0.3, world_reduce=reduce_max)
        shard_ms = float(np.median(blocks)) / 3
        gather = lambda: dist.all_gather_into_tensor(buf, out_all)
        for _ in range(3):
            gather()
        gblocks = timed_blocks(torch, gather, 10, barrier, min_seconds=0.05, world_reduce=reduce_max)
        gather_ms = float(np.median(gblocks)) / 10
        ops.read_status(status, what="attn_decode")
        one = torch.tensor([one_ms if one_ms is not None else 0.0], dtype=torch.float64, device=device)
        dist.broadcast(one, 0)
        one_ms = float(one[0])
        cols_local = B * heads[1]
        res[name] = {"workload": name + ": " + cfg["desc"], "layers": L, "ms_per_step_1gpu": one_ms, "ms_per_step_sharded": shard_ms,
                     "speedup": one_ms / shard_ms, "efficiency": one_ms / shard_ms / world,
                     "allgather_ms_alone": gather_ms, "allgather_bytes_per_rank": L * B * heads[3] * 128 * 2,
                     "per_rank": {"kv_heads": heads[1], "query_heads": heads[3], "columns": cols_local, "tiles_per_column": (T + 255) // 256},
                     "limiter": ("the all-gather's latency is %.0f %% of the sharded step; the rest of the gap to linear is the kernel's fixed "
                                 "cost per launch (tables and first blocks loaded by every CTA, the merge launch per layer) spread over 1/%d of "
                                 "the tiles" % (100 * gather_ms / shard_ms, world))}
        del layers
        torch.cuda.empty_cache()
        barrier()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="c1", choices=sorted(WORKLOADS) + ["c4"])
    ap.add_argument("--impl", default="kvcomp_b200", choices=["kvcomp_b200", "reference"])
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (profiling small cases)")
    ap.add_argument("--codec-rels", default="", help="c4: comma-separated error bounds instead of the full sweep (profiling)")
    ap.add_argument("--side", default="", choices=["", "c1_recent_window"], help="run one side record alone and print it (profiling)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="leave out the codec, gpu_reference and strong sub-records")
    ap.add_argument("--min-seconds", type=float, default=MIN_TIMED_SECONDS, help="device time the repeated timed block has to cover")
    ap.add_argument("--shard", default="batch", choices=["batch", "heads"],
                    help="N > 1: every rank owns its own batch of sequences (weak scaling, default) or the KV heads "
                         "are split over the ranks and the outputs all-gathered once per step (strong scaling)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    codec_only = args.workload == "c4"
    if codec_only and args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "the CPU arm times the decode-attention workloads (c0-c3) only"}))
        return
    cfg = dict(WORKLOADS["c1" if codec_only else args.workload])
    if args.layers:
        cfg["layers"] = args.layers
    if args.impl == "reference":
        run_reference(args, cfg, rank, world)
        return

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: kvcomp_b200 has no CPU path")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    from kvcomp_b200 import ops
    if args.side == "c1_recent_window":
        print(json.dumps({"side": args.side, "record": recent_window_record(ops, torch, device, args.seed, layers=args.layers or 4)}), flush=True)
        return

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def reduce_max(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    if codec_only:
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        rels = tuple(float(r) for r in args.codec_rels.split(",")) if args.codec_rels else (0.01, 0.02, 0.05, 0.1, 0.2)
        sweep, launches, raw = codec_sweep(ops, torch, device, args.seed + 7919 * rank, rels=rels, reps=max(2, args.steps // 5))
        clocks = sampler.stop() if rank == 0 else None
        agg = {}
        for rel, r in sweep.items():
            if "skipped" in r:
                agg[rel] = r
                continue
            e, d = reduce_max(r["encode_ms"]), reduce_max(r["decode_ms"])
            e2, d2 = reduce_max(r["encode_next_ms"]), reduce_max(r["decode_2s_ms"])
            agg[rel] = dict(r, encode_GBps=world * r["encode_GBps"] * r["encode_ms"] / e, decode_GBps=world * r["decode_GBps"] * r["decode_ms"] / d,
                            encode_next_GBps=world * r["encode_next_GBps"] * r["encode_next_ms"] / e2,
                            decode_2s_GBps=world * r["decode_2s_GBps"] * r["decode_2s_ms"] / d2)
        if rank == 0:
            head = agg.get("0.05", next(iter(agg.values())))
            peak, kind = peaks()
            per = head.get("encode_GBps", 0) / world
            print(json.dumps({
                "metric": "encode GB/s (quantise + histogram + codebook + Huffman encode), fp16 bytes in", "value": head.get("encode_GBps"),
                "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "fp16 -> u8 codes -> bitstream", "data": "synthetic",
                "config": {"workload": "c4: KV blocks 32 heads x 128, batch 32, one 4096-token chunk (1 GiB of fp16) per tensor and rank, K per-channel / V per-token",
                           "l2": "inputs larger than L2 (1 GiB of fp16 per tensor)"},
                "codec": agg, "gpu_launches": launches, "clocks": clocks,
                "roofline": {"bound": "hbm", "achieved": per * 2.13, "peak": peak, "unit": "GB/s", "frac": per * 2.13 / peak, "peak_kind": kind,
                             "note": "bytes moved per fp16 byte in: 1 (read) + 0.5 (codes out) + 0.5 (codes read once by the encoder) + ~0.13 (stream)", "traffic": None}}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    heads_mode = args.shard == "heads" and world > 1
    heads = None
    Hq_total = cfg["Hq"]
    if heads_mode:
        from kvcomp_b200 import sharding
        heads = sharding.shard_heads(cfg["Hkv"], cfg["Hq"], world, rank)
    T, B, L = cfg["T"], cfg["B"], cfg["layers"]
    Hkv, Hq = (heads[1], heads[3]) if heads_mode else (cfg["Hkv"], cfg["Hq"])
    layers, accts = [], []
    for l in range(L):
        # head sharding: every rank cuts its heads out of the same tensors; batch sharding: own sequences
        caches, keep, q, acct = build_layer(ops, torch, cfg, l, args.seed + (0 if heads_mode else 7919 * rank), device, heads=heads)
        layers.append((caches, keep, q))
        accts.append(acct)
    torch.cuda.synchronize()
    lcfg = dict(cfg, Hkv=Hkv, Hq=Hq)
    splits = args.splits                      # 0: the library balances the tiles over the resident CTAs
    ws = ops.attn_workspace(B, Hq, splits or ops.attn_splits(T, B, Hkv), device)
    status = ops.new_status(device)
    out_all = torch.empty((L, B, Hq, 128), dtype=torch.float16, device=device)
    outs = [out_all[i] for i in range(L)]
    gather_buf = torch.empty((world, L, B, Hq, 128), dtype=torch.float16, device=device) if heads_mode else None
    scaling = 1.0 / math.sqrt(128)
    launches_per_call = sum(1 for _ in _chunks(Hq // Hkv))

    def step():
        for (caches, _, q), out in zip(layers, outs):
            ops.attn_decode(caches[0], caches[1], T, B, Hkv, q, scaling, out=out, splits=splits, workspace=ws, status=status)
        if heads_mode:      # the only exchange of the path: the step's outputs of every rank's query heads
            dist.all_gather_into_tensor(gather_buf, out_all)

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    blocks = timed_blocks(torch, step, args.steps, barrier, min_seconds=args.min_seconds, world_reduce=reduce_max)
    flags = ops.read_status(status, what="attn_decode")

    # end to end through the public call with host buffers: every layer's q comes from pinned host memory
    # and every layer's output goes back to pinned host memory, every step (the cache itself lives in HBM).
    # The copies run on a second stream, ordered against the kernels by events: layer i+1's q arrives and
    # layer i-1's output leaves while layer i computes.
    q_host = [q.cpu().pin_memory() for (_, _, q) in layers]
    o_host = [torch.empty((B, Hq, 128), dtype=torch.float16).pin_memory() for _ in range(L)]
    q_dev = [torch.empty_like(q) for (_, _, q) in layers]
    copy_stream = torch.cuda.Stream(device=device)
    q_ready = [torch.cuda.Event() for _ in range(L)]
    o_ready = [torch.cuda.Event() for _ in range(L)]
    step_done = torch.cuda.Event()

    def step_e2e():
        main_s = torch.cuda.current_stream()
        copy_stream.wait_event(step_done)               # the previous step's kernels are done with q_dev
        with torch.cuda.stream(copy_stream):
            for i in range(L):
                q_dev[i].copy_(q_host[i], non_blocking=True)
                q_ready[i].record(copy_stream)
        for i, ((caches, _, _), out) in enumerate(zip(layers, outs)):
            main_s.wait_event(q_ready[i])
            ops.attn_decode(caches[0], caches[1], T, B, Hkv, q_dev[i], scaling, out=out, splits=splits, workspace=ws, status=status)
            o_ready[i].record(main_s)
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(o_ready[i])
                o_host[i].copy_(out, non_blocking=True)
        if heads_mode:
            dist.all_gather_into_tensor(gather_buf, out_all)
        step_done.record(main_s)
        copy_stream.synchronize()                       # the caller needs the results of the step
        main_s.synchronize()

    step_done.record(torch.cuda.current_stream())
    for _ in range(3):
        step_e2e()
    blocks_e2e = timed_blocks(torch, step_e2e, args.steps, barrier, min_seconds=args.min_seconds, world_reduce=reduce_max)
    clocks = sampler.stop() if rank == 0 else None

    extras = {}
    if not args.no_extras:
        # the codec half of the metric, on every rank's GPU (its own sequences: weak scaling like the headline)
        sweep, codec_launches, _ = codec_sweep(ops, torch, device, args.seed + 7919 * rank)
        agg = {}
        for rel, r in sweep.items():
            if "skipped" in r:
                agg[rel] = r
                continue
            e, d = reduce_max(r["encode_ms"]), reduce_max(r["decode_ms"])
            e2, d2 = reduce_max(r["encode_next_ms"]), reduce_max(r["decode_2s_ms"])
            agg[rel] = dict(r, encode_GBps=world * r["encode_GBps"] * r["encode_ms"] / e, decode_GBps=world * r["decode_GBps"] * r["decode_ms"] / d,
                            encode_next_GBps=world * r["encode_next_GBps"] * r["encode_next_ms"] / e2,
                            decode_2s_GBps=world * r["decode_2s_GBps"] * r["decode_2s_ms"] / d2,
                            encode_ms=e, decode_ms=d, encode_next_ms=e2, decode_2s_ms=d2)
        extras["codec"] = {"workload": "one 1 GiB fp16 chunk per tensor and rank (32 heads x 128, batch 32, 4096 tokens), K per-channel / V per-token; "
                                       "GB/s = fp16 bytes in (encode: quantise + histogram + codebook + encode) or out (decode) per second, all ranks",
                           "by_error_bound": agg, "gpu_launches": codec_launches}
        if world == 1:
            extras["gpu_reference"] = gpu_reference(ops, torch, device, args.seed)
            if args.workload == "c1":
                extras["other_workloads"] = side_workloads(ops, torch, device, args.seed)
        elif not heads_mode:
            extras["strong"] = strong_record(args, ops, torch, dist, device, rank, world, barrier, reduce_max)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    ms_step = float(np.median(blocks)) / args.steps
    ms_e2e = float(np.median(blocks_e2e)) / args.steps
    seqs = B if heads_mode else B * world             # sequences the whole job advances by one token per step
    value = seqs / (ms_step / 1e3)
    e2e_value = seqs / (ms_e2e / 1e3)
    alg = float(np.mean([algorithmic_bytes(a, lcfg) for a in accts]))
    merge = 1 if (splits or ops.attn_splits(T, B, Hkv)) > 1 else 0
    launch_s = ms_step / 1e3 / (L * launches_per_call)
    peak, peak_kind = peaks()
    achieved = alg / launch_s / 1e9
    served = 2 * 2 * T * B * Hkv * 128
    line = {
        "metric": METRIC, "value": value, "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "strong" if heads_mode else "weak", "vs_baseline": None,
        "dtype": "u8 codes -> int32 dot products (16-bit fixed-point weights), f32 softmax, fp16 in/out", "data": "synthetic",
        "config": make_config(args, cfg, heads_mode),
        "timing": {"blocks": len(blocks), "steps_per_block": args.steps, "timed_seconds": float(np.sum(blocks)) / 1e3,
                   "block_ms_min_median_max": [float(np.min(blocks)), float(np.median(blocks)), float(np.max(blocks))],
                   "rule": "each block: barrier + synchronize, CUDA events around exactly `steps` steps, barrier + synchronize; max over ranks; the median block counts"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": peak_kind + " (STREAM-style copy)", "traffic": None,
                     "algorithmic_bytes_per_launch": alg, "launch_ms": launch_s * 1e3, "compressed_gb_per_step": alg * L / 1e9,
                     "effective_fp16_gbs": served / launch_s / 1e9,
                     "bits_per_symbol": {k: float(np.mean([8.0 * a[k]["encoded"] / a[k]["symbols"] for a in accts])) for k in ("k", "v")}},
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": L * B * Hq * 128 * 2,
                "d2h_bytes_per_step": L * B * Hq * 128 * 2, "ms_per_step": ms_e2e, "blocks": len(blocks_e2e)},
        # per layer: one attention kernel per chunk of query heads, then the merge of the partial results
        "gpu_launches": len(blocks) * args.steps * L * (launches_per_call + merge),
        "clocks": clocks, "status_flags": flags,
    }
    if Hq == Hkv:
        ratio, src = profile_traffic()
        if ratio is not None:
            line["roofline"]["traffic"] = ratio * alg
            line["roofline"]["traffic_source"] = dict(src, note="ncu dram__bytes_read.sum + dram__bytes_write.sum of the kernel on a 2-layer case, scaled by algorithmic bytes")
    line.update(extras)
    if not args.no_cpu_baseline and world == 1:
        line["cpu_baseline"], _ = cpu_baseline_record(cfg, args.seed, 10.0)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def _chunks(g):
    while g > 0:
        c = 4 if g >= 4 else (2 if g >= 2 else 1)
        yield c
        g -= c


if __name__ == "__main__":
    main()
