"""Compression-ratio / kernel-time evaluation with the result keys of the reference's harness
(evaluation/cr_throughput_eval.py:128-240), so that its analysis and plotting scripts can read the
numbers produced here.

    crs_throughputs_evaluation_with_data(config, key_caches, value_caches) -> dict

key_caches / value_caches: one fp16 tensor [B, H, T, D] per layer (the layout the reference extracts
from a model run).  Throughput = original fp16 bytes / 2^30 / time, as there (:235-238).  "multi-kernel"
time = decode kernel + dequantisation (:58-71); "fused" time = fused kernel time minus the dense
mat-vec time over already-decompressed data (:90,125).
"""
import math

import torch

from .cache.kvcomp_encode import KVCompCtx
from .utils.compute import QuantMode
from .utils.config import KVCompCacheConfigStatic


def quant_rel_to_bit_num(quant_rel):            # cr_throughput_eval.py:13-16
    return math.ceil(math.log2(math.ceil(1 / quant_rel) + 1))


def check_error(a, b, percentage):              # cr_throughput_eval.py:18-20
    assert ((a - b).abs() < a.abs().max() * percentage).all(), "Error too large"


def _timed(fn):
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    out = fn()
    stop.record()
    torch.cuda.synchronize()
    return out, start.elapsed_time(stop)


def k_get_fused_kernel_time(ctx):
    """(fused - dense, dense ms, fused ms) for q.K^T; checks fused against dense at 1 % of max (:73-90)."""
    q = torch.empty((ctx.batch_size, ctx.head_num, ctx.head_dim), dtype=torch.float16, device=ctx.device).uniform_(-1, 1)
    k, _ = ctx.get_only_compressed()                              # [T, B, H, D]
    kt = k.permute(1, 2, 3, 0)                                    # [B, H, D, T]
    ref, t_dense = _timed(lambda: torch.matmul(q.unsqueeze(2), kt))
    out, t_fused = ctx.mat_vec_mul(q)
    check_error(ref.squeeze(2).float(), out.float(), 0.01)
    return t_fused - t_dense, t_dense, t_fused


def v_get_fused_kernel_time(ctx):
    """Same for P.V with softmaxed random weights (:108-125)."""
    w = torch.softmax(torch.randn((ctx.batch_size, ctx.head_num, ctx.compressed_ctx_len), dtype=torch.float16,
                                  device=ctx.device) * 2.5, dim=-1)
    v, _ = ctx.get_only_compressed()
    vt = v.permute(1, 2, 0, 3)                                    # [B, H, T, D]
    ref, t_dense = _timed(lambda: torch.matmul(w.unsqueeze(2), vt))
    out, t_fused = ctx.mat_vec_mul(w)
    check_error(ref.squeeze(2).float(), out[0].float(), 0.01)
    return t_fused - t_dense, t_dense, t_fused


def crs_throughputs_evaluation_with_data(config, key_caches, value_caches, warmup=2):
    KVCompCacheConfigStatic.config = config
    B, H, _, D = key_caches[0].shape
    L = len(key_caches)
    keys = ("k_original_sizes", "k_quant_sizes", "k_encode_sizes", "v_original_sizes", "v_quant_sizes", "v_encode_sizes",
            "k_multi", "k_fused", "v_multi", "v_fused", "k_dense", "k_fuse", "v_dense", "v_fuse")
    r = {k: [0] * L for k in keys}
    order = list(range(min(warmup, L))) + list(range(L))          # the first layers run twice: warm-up (:154-156)
    for i in order:
        ctxs = {}
        for name, caches, is_k, rel in (("k", key_caches, True, config.k_quant_scale_rel),
                                        ("v", value_caches, False, config.v_quant_scale_rel)):
            ctx = KVCompCtx(is_k, B, H, D, rel)
            ctx.store(caches[i].permute(2, 0, 1, 3).contiguous())
            n = ctx.compressed_ctx_len * B * H * D
            quant_meta = ctx.quant_min_ints.numel() * 8 + ctx.quant_scales.numel() * 16            # bits (:167)
            enc_meta = ctx.block_infos.numel() * 8 + ctx.thread_infos.numel() * 8
            r[name + "_original_sizes"][i] = n * 16
            r[name + "_quant_sizes"][i] = n * quant_rel_to_bit_num(rel) + quant_meta
            r[name + "_encode_sizes"][i] = ctx.encoded_data.numel() * 8 + enc_meta + quant_meta
            ctxs[name] = ctx
        r["k_multi"][i] = ctxs["k"].get_only_compressed()[1]
        r["v_multi"][i] = ctxs["v"].get_only_compressed()[1]
        r["k_fused"][i], r["k_dense"][i], r["k_fuse"][i] = k_get_fused_kernel_time(ctxs["k"])
        r["v_fused"][i], r["v_dense"][i], r["v_fuse"][i] = v_get_fused_kernel_time(ctxs["v"])
    gib = 8 * 1024 * 1024 * 1024

    def thr(sizes, times):
        return [s / gib / (t / 1000) if t > 0 else float("inf") for s, t in zip(sizes, times)]
    return {
        "k_quant_crs": [o / q for o, q in zip(r["k_original_sizes"], r["k_quant_sizes"])],
        "v_quant_crs": [o / q for o, q in zip(r["v_original_sizes"], r["v_quant_sizes"])],
        "k_huffman_crs": [o / e for o, e in zip(r["k_original_sizes"], r["k_encode_sizes"])],
        "v_huffman_crs": [o / e for o, e in zip(r["v_original_sizes"], r["v_encode_sizes"])],
        "k_time_multi_kernels": r["k_multi"], "v_time_multi_kernels": r["v_multi"],
        "k_pytorch_mat_vec_mul_times": r["k_dense"], "v_pytorch_mat_vec_mul_times": r["v_dense"],
        "k_fused_mat_vec_mul_times": r["k_fuse"], "v_fused_mat_vec_mul_times": r["v_fuse"],
        "k_throughput_multi_kernels": thr(r["k_original_sizes"], r["k_multi"]),
        "k_throughput_fused_kernels": thr(r["k_original_sizes"], r["k_fused"]),
        "v_throughput_multi_kernels": thr(r["v_original_sizes"], r["v_multi"]),
        "v_throughput_fused_kernels": thr(r["v_original_sizes"], r["v_fused"]),
    }
