"""Time the reference's own Python CPU path on the CPU-runnable configuration (one Llama-2-7B-shaped
layer: 32 heads x 128, batch 1, 1024 tokens, K per channel / V per token in 64-token blocks at 0.05).

    REF=/path/to/reference python oracle/time_reference_python.py

Runs where the reference tree is mounted; imports utils/compute.py and utils/huffman.py unmodified.
Stages: (i) the quantiser (utils/compute.py:74-91, torch fp16 ops on the CPU), (ii) the Huffman encoder
(utils/huffman.py:15-94: heapq tree, per-symbol Python loop; the reference has no CPU decoder),
(iii) dequantisation (utils/compute.py:130) and one decode-step attention in torch on the CPU over the
dequantised tensors (models/llama.py:211-234).  Prints one JSON object; the figures are quoted in the
baseline notes, the benchmark itself does not run this (the reference tree does not travel)."""
import json
import math
import os
import sys
import time

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
from oracle import ref_root  # noqa: E402
REF = ref_root.require()
sys.path.insert(0, REF)

from utils.compute import QuantMode, quant_ints  # noqa: E402
from utils.huffman import huffman_encode  # noqa: E402
from kvcomp_b200.synth import make_kv  # noqa: E402


def best(f, n=3):
    ts = []
    for _ in range(n):
        t0 = time.perf_counter(); r = f(); ts.append(time.perf_counter() - t0)
    return min(ts), r


def main():
    T, B, H, D = 1024, 1, 32, 128
    k, v, q = make_kv(T, B, H, D, seed=0, device="cpu")
    kb, vb = k.permute(1, 2, 0, 3).contiguous(), v.permute(1, 2, 0, 3).contiguous()      # [B, H, T, D]
    out = {"config": "32 heads x 128, batch 1, 1024 tokens, fp16, seed 0; K ChannelQuant / V TokenQuant, block 64, rel 0.05",
           "host_cores": os.cpu_count(), "torch_threads": torch.get_num_threads(), "symbols_per_tensor": T * B * H * D}
    tq_k, (kq, kmin, ksc) = best(lambda: quant_ints(kb, 64, 0.05, QuantMode.ChannelQuant))
    tq_v, (vq, vmin, vsc) = best(lambda: quant_ints(vb, 64, 0.05, QuantMode.TokenQuant))
    out["quantise_s"] = {"k": tq_k, "v": tq_v}
    te_k, (kbits, kbook) = best(lambda: huffman_encode(kq.to(torch.uint8)), n=1)
    te_v, (vbits, vbook) = best(lambda: huffman_encode(vq.to(torch.uint8)), n=1)
    out["huffman_encode_s"] = {"k": te_k, "v": te_v}
    out["bits_per_symbol"] = {"k": kbits.numel() / kq.numel(), "v": vbits.numel() / vq.numel()}
    out["symbols"] = {"k": len(kbook), "v": len(vbook)}

    def attend():
        kh = ((kq + kmin) * ksc).reshape(B, H, T, D).float()
        vh = ((vq + vmin) * vsc).reshape(B, H, T, D).float()
        w = torch.softmax(torch.matmul(q.float().unsqueeze(2), kh.transpose(2, 3)) / math.sqrt(D), dim=-1)
        return torch.matmul(w, vh)
    ta, _ = best(attend)
    out["dequant_plus_attention_s"] = ta
    out["encode_MBps_fp16_in"] = {"k": 2 * kq.numel() / 1e6 / (tq_k + te_k), "v": 2 * vq.numel() / 1e6 / (tq_v + te_v)}
    print(json.dumps(out, indent=1))


if __name__ == "__main__":
    main()
