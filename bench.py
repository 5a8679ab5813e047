#!/usr/bin/env python
"""Benchmark of the fused decompress-matvec decode attention (the metric of BASELINE.json).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c1|c0|c2|c3] [--impl reference]

One "step" = one decode step of the whole model: for every layer, one call of the fused kernel that
reads the layer's compressed K and V streams and produces the attention output of every sequence and
head (q.K^T -> softmax -> P.V, no fp16 K/V materialised).  value = tokens/s = sequences / step time,
summed over all ranks.  With N > 1 every rank holds its own batch of sequences of the same size (the
path shards by batch sequence without any exchange on the data path), so scaling is weak.

Prints ONE JSON line (rank 0).  --impl reference times the CPU restatement of the reference's path
(oracle/, OpenMP over the host cores) on a bounded sample of the same workload instead.
"""
import argparse
import json
import math
import os
import subprocess
import sys
import tempfile
import threading
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


DRAM_TRAFFIC_PER_ALGORITHMIC_BYTE = 1.04


def peaks():
    """Measured HBM peak of this pool (driver-written file), else the stated fallback."""
    try:
        with open(os.path.join(REPO, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


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


def build_layer(ops, torch, cfg, layer, seed, device):
    """Synthetic K/V of one layer -> compressed caches resident in HBM.  Returns the cache pair, the
    tensors that back them, and the byte accounting of the layer."""
    from kvcomp_b200.synth import make_kv
    T, B, Hkv, Hq = cfg["T"], cfg["B"], cfg["Hkv"], cfg["Hq"]
    k, v, q = make_kv(T, B, Hkv, 128, seed=seed, layer=layer, device=device, Hq=Hq)
    keep, caches, acct = [], [], {}
    for name, x, is_k, mode, rel, blk in (("k", k, True, ops.MODES[cfg["kmode"]], cfg["krel"], cfg["kblock"]),
                                          ("v", v, False, ops.MODE_TOKEN, cfg["vrel"], 128)):
        hist = torch.zeros(256, dtype=torch.int64, device=device)
        codes, mi, sc, spec, st = ops.quantize(x, mode, blk, rel, False, min_dtype=torch.int16, hist=hist)
        book = ops.build_codebook(hist)
        bsz, tsz, _, cap = ops.buffer_sizes(T, B * Hkv * 128, is_k)
        bi = torch.empty(bsz, dtype=torch.uint8, device=device)
        ti = torch.empty(tsz // 2, dtype=torch.int16, device=device)
        enc = torch.empty(cap, dtype=torch.uint8, device=device)
        total, st2 = ops.encode(codes, is_k, book.encode_table(), bi, ti, enc)
        n, maxb = (int(x) for x in total.tolist())
        ops.read_status(st, what="quantize"); ops.read_status(st2, what="encode")
        enc = enc[:n].clone()
        keep.append((enc, bi, ti, book, mi, sc))
        caches.append(ops.make_cache(enc, bi, ti, book, mi, sc, spec, n, maxb))
        acct[name] = dict(encoded=n, block_info=bsz, thread_info=tsz,
                          quant_meta=mi.numel() * mi.element_size() + sc.numel() * 2,
                          symbols=T * B * Hkv * 128, min_flag=ops.read_status(st, False), max_block=maxb)
        del codes, x
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
    import torch
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


def run_codec(args, rank, world, local):
    """Prefill-side sweep (workload c4): quantise + histogram + codebook + Huffman encode of KV shaped
    32 heads x 128, batch 32, in chunks of 4096 tokens per sequence (the 131072-token sequences of the
    configuration are processed chunk by chunk: one chunk is 1 GiB of fp16 per tensor), then a full decode
    and an exact round-trip check.  Error bounds {0.01 .. 0.2}; GB/s counts fp16 bytes in (encode) or
    fp16-equivalent bytes out (decode).  With N > 1 every rank processes its own sequences."""
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    from kvcomp_b200 import ops
    from kvcomp_b200.synth import make_kv
    T, B, H = 4096, 32, 32
    chunks = max(1, args.layers or 2)            # chunks per step (default 2: K and V of each make 4 GiB of fp16)
    fp16_bytes = 2 * T * B * H * 128
    results, launches = {}, 0
    clocks = None
    for rel in (0.01, 0.02, 0.05, 0.1, 0.2):
        enc_ms, dec_ms, comp, orig, bits = 0.0, 0.0, 0, 0, {}
        sampler = ClockSampler(local)
        if rank == 0 and rel == 0.05:
            sampler.start()
        for it in range(args.warmup + args.steps):
            timed = it >= args.warmup
            for c in range(chunks):
                k, v, _ = make_kv(T, B, H, 128, seed=args.seed + 7919 * rank, layer=c, device=device)
                for name, x, is_k, mode, blk in (("k", k, True, ops.MODE_CHANNEL, 64), ("v", v, False, ops.MODE_TOKEN, 128)):
                    bsz, tsz, _, cap = ops.buffer_sizes(T, B * H * 128, is_k)
                    bi = torch.empty(bsz, dtype=torch.uint8, device=device)
                    ti = torch.empty(tsz // 2, dtype=torch.int16, device=device)
                    enc = torch.empty(cap, dtype=torch.uint8, device=device)
                    hist = torch.zeros(256, dtype=torch.int64, device=device)
                    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
                    ev[0].record()
                    codes, mi, sc, spec, st = ops.quantize(x, mode, blk, rel, False, min_dtype=torch.int16, hist=hist)
                    book = ops.build_codebook(hist)
                    total, st2 = ops.encode(codes, is_k, book.encode_table(), bi, ti, enc)
                    ev[1].record()
                    n, maxb = (int(x) for x in total.tolist())
                    flags = ops.read_status(st, False) | ops.read_status(st2, False)
                    ev[2].record()
                    back, st3 = ops.decode(enc[:n], bi, ti, book, T, B, H, is_k, max_block=maxb)
                    ev[3].record()
                    torch.cuda.synchronize()
                    if flags & 0x20:            # a block beyond 8191 bytes: the format's u16 fields cannot hold it
                        bits[name] = float("nan")
                        continue
                    assert torch.equal(back, codes), "round trip failed at rel %g" % rel
                    if timed:
                        enc_ms += ev[0].elapsed_time(ev[1]); dec_ms += ev[2].elapsed_time(ev[3])
                        comp += n + bsz + tsz + mi.numel() * 2 + sc.numel() * 2
                        orig += fp16_bytes
                        bits[name] = 8.0 * n / codes.numel()
                        launches += 7            # quantise, codebook, sizes, 2 scans, emit, decode
                    del codes, back, enc
                del k, v
        if rank == 0 and rel == 0.05:
            clocks = sampler.stop()
        vals = [enc_ms, dec_ms]
        if world > 1:
            t = torch.tensor(vals, dtype=torch.float64, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            vals = [float(t[0]), float(t[1])]
        if orig:
            results[str(rel)] = {"encode_GBps": world * orig / 1e9 / (vals[0] / 1e3), "decode_GBps": world * orig / 1e9 / (vals[1] / 1e3),
                                 "compression_ratio": orig / comp, "bits_per_symbol": bits}
        else:
            results[str(rel)] = {"skipped": "a block exceeds the 8191 bytes the stream format can describe"}
    if rank == 0:
        head = results.get("0.05", {})
        peak, kind = peaks()
        # encode reads fp16 (2 B/symbol), writes and re-reads the codes twice (1 B each) and writes the stream
        line = {"metric": "encode GB/s (quantise + histogram + codebook + Huffman encode), fp16 bytes in", "value": head.get("encode_GBps"),
                "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "fp16 -> u8 codes -> bitstream", "data": "synthetic",
                "config": {"workload": "c4: KV blocks 32 heads x 128, batch 32, %d-token chunks x %d per step, K per-channel / V per-token" % (T, chunks),
                           "l2": "inputs larger than L2 (1 GiB of fp16 per tensor and chunk)"},
                "sweep": results, "gpu_launches": launches, "clocks": clocks,
                "roofline": {"bound": "hbm", "achieved": head.get("encode_GBps", 0) * 2.75 if head else None, "peak": peak, "unit": "GB/s",
                             "frac": (head.get("encode_GBps", 0) * 2.75 / peak) if head else None, "peak_kind": kind,
                             "note": "bytes moved per fp16 byte in: 1 (read) + 0.5 (codes out) + 2 x 0.5 (codes re-read by sizes and emit) + ~0.25 (stream)", "traffic": None}}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_reference(args, cfg, rank, world):
    """CPU arm: the restated reference path on the host cores, bounded sample per step."""
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
    val = cfg["B"] * world / step_s / world      # one host: the CPU does every rank's work in turn
    sample = "1 sequence x 1 layer (%d heads, %d tokens): Huffman decode of K and V + attention; a step is %d such samples" % (
        cfg["Hkv"], cfg["T"], samples_per_step)
    line = {"impl": "reference", "metric": "decode attn tokens/s (fused decomp-matvec)", "value": val, "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8 codes -> f32 accumulate",
            "data": "synthetic", "config": {"workload": args.workload + ": " + cfg["desc"]},
            "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


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
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--shard", default="batch", choices=["batch", "heads"],
                    help="N > 1: every rank owns its own batch of sequences (weak scaling, default) or the KV heads "
                         "are split over the ranks and the outputs all-gathered once per step (strong scaling)")
    args = ap.parse_args()
    if args.workload == "c4":
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "the CPU arm times the decode-attention workloads (c0-c3) only"}))
            return
        run_codec(args, int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0")))
        return
    cfg = dict(WORKLOADS[args.workload])
    if args.layers:
        cfg["layers"] = args.layers
    if args.warmup < 3 and args.impl != "reference":
        args.warmup = max(args.warmup, 1)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

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

    heads_mode = args.shard == "heads" and world > 1
    Hq_total = cfg["Hq"]
    if heads_mode:
        from kvcomp_b200 import sharding
        _, kvc, _, qc = sharding.shard_heads(cfg["Hkv"], cfg["Hq"], world, rank)
        cfg["Hkv"], cfg["Hq"] = kvc, qc
    T, B, Hkv, Hq, L = cfg["T"], cfg["B"], cfg["Hkv"], cfg["Hq"], cfg["layers"]
    layers, accts = [], []
    for l in range(L):
        caches, keep, q, acct = build_layer(ops, torch, cfg, l, args.seed + 7919 * rank, device)
        layers.append((caches, keep, q))
        accts.append(acct)
    torch.cuda.synchronize()
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

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 1)):
        step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    barrier()
    ev[0].record()
    for _ in range(args.steps):
        step()
    ev[1].record()
    barrier()
    ms = ev[0].elapsed_time(ev[1])
    clocks = sampler.stop() if rank == 0 else None
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
        main = torch.cuda.current_stream()
        copy_stream.wait_event(step_done)               # the previous step's kernels are done with q_dev
        with torch.cuda.stream(copy_stream):
            for i in range(L):
                q_dev[i].copy_(q_host[i], non_blocking=True)
                q_ready[i].record(copy_stream)
        for i, ((caches, _, _), out) in enumerate(zip(layers, outs)):
            main.wait_event(q_ready[i])
            ops.attn_decode(caches[0], caches[1], T, B, Hkv, q_dev[i], scaling, out=out, splits=splits, workspace=ws, status=status)
            o_ready[i].record(main)
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(o_ready[i])
                o_host[i].copy_(out, non_blocking=True)
        if heads_mode:
            dist.all_gather_into_tensor(gather_buf, out_all)
        step_done.record(main)
        copy_stream.synchronize()                       # the caller needs the results of the step
        main.synchronize()

    step_done.record(torch.cuda.current_stream())
    for _ in range(2):
        step_e2e()
    barrier()
    e0 = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    t0 = time.perf_counter()
    e0[0].record()
    for _ in range(args.steps):
        step_e2e()
    e0[1].record()
    barrier()
    ms_e2e = e0[0].elapsed_time(e0[1])

    if world > 1:
        t = torch.tensor([ms, ms_e2e], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e = float(t[0]), float(t[1])
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    ms_step = ms / args.steps
    seqs = B if heads_mode else B * world             # sequences the whole job advances by one token per step
    value = seqs / (ms_step / 1e3)
    e2e_value = seqs / (ms_e2e / args.steps / 1e3)
    alg = float(np.mean([algorithmic_bytes(a, cfg) for a in accts]))
    launch_s = ms_step / 1e3 / (L * launches_per_call)
    peak, peak_kind = peaks()
    achieved = alg / launch_s / 1e9
    served = 2 * 2 * T * B * Hkv * 128
    line = {
        "metric": "decode attn tokens/s (fused decomp-matvec)", "value": value, "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "strong" if heads_mode else "weak", "vs_baseline": None,
        "dtype": "u8 codes -> int32 dot products (16-bit fixed-point weights), f32 softmax, fp16 in/out", "data": "synthetic",
        "config": {"workload": args.workload + ": " + cfg["desc"], "layers": L, "splits": splits or "auto: (column, run of tiles) items drawn by the resident CTAs",
                   "l2": "inputs larger than L2 (%.2f GB of compressed cache read per step)" % (alg * L / 1e9),
                   "sharding": ("KV heads split over ranks (%d of %d query heads each), one NCCL all-gather of the outputs per step" % (Hq, Hq_total))
                   if heads_mode else "batch sequences per rank, no collective on the data path"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": peak_kind + " (STREAM-style copy)", "traffic": None,
                     "algorithmic_bytes_per_launch": alg, "launch_ms": launch_s * 1e3,
                     "effective_fp16_gbs": served / launch_s / 1e9,
                     "bits_per_symbol": {k: float(np.mean([8.0 * a[k]["encoded"] / a[k]["symbols"] for a in accts])) for k in ("k", "v")}},
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": L * B * Hq * 128 * 2,
                "d2h_bytes_per_step": L * B * Hq * 128 * 2, "ms_per_step": ms_e2e / args.steps},
        # per layer: one attention kernel per chunk of query heads, then the merge of the partial results
        "gpu_launches": args.steps * L * (launches_per_call + (1 if (splits or ops.attn_splits(T, B, Hkv)) > 1 else 0)),
        "clocks": clocks, "status_flags": flags,
    }
    # DRAM traffic of the kernel from one ncu capture (profiles/attn_decode_c1.md): read + written bytes
    # were 1.035 x the algorithmic bytes of the launch on c1-shaped data; it grows with the bytes staged.
    if Hq == Hkv:
        line["roofline"]["traffic"] = DRAM_TRAFFIC_PER_ALGORITHMIC_BYTE * alg
        line["roofline"]["traffic_source"] = "ncu dram__bytes_read.sum + dram__bytes_write.sum on 2 layers of c1, scaled by algorithmic bytes"
    if not args.no_cpu_baseline and world == 1:
        s, threads = cpu_sample(cfg, args.seed, min_seconds=10.0)
        step_s = s * L * B
        line["cpu_baseline"] = {"value": B / step_s, "unit": "tokens/s", "cores": threads, "kind": "port",
                                "sample": "1 sequence x 1 layer (%d heads, %d tokens) of the same workload, Huffman decode of K and V + attention, %.2f s each; a step is %d such samples" % (Hkv, T, s, L * B)}
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
