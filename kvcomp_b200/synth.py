"""Seeded synthetic K/V/q tensors with the shapes and value distributions of the benchmark
configurations (stand-ins for KV dumped from real models, which the reference measures on).

    K[t,b,h,c] = mu[h,c] + s[h,c] * N(0,1),  mu ~ N(0, 0.5),  s ~ LogNormal(0, 0.5),
                 2 % of the (h,c) channels have s multiplied by 8 (outlier channels)
    V[t,b,h,c] = r[t,b] * N(0,1),            r ~ LogNormal(0, 0.25)
    q[b,hq,c]  = N(0,1) / sqrt(128)

Everything is drawn in fp32 from one torch.Generator seeded with seed + 1000*layer and cast to
fp16.  The generator lives on the device the tensors are made on, so CPU and GPU draws differ;
tests that compare against the CPU checker generate on the CPU and copy.
"""
import math

import torch


def make_kv(T, B, H, D=128, seed=0, layer=0, device="cpu", Hq=None):
    """Returns K, V as fp16 [T,B,H,D] and q as fp16 [B,Hq,D]."""
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(seed + 1000 * layer)
    f32 = dict(dtype=torch.float32, device=dev, generator=g)
    mu = 0.5 * torch.randn(H, D, **f32)
    s = torch.exp(0.5 * torch.randn(H, D, **f32))
    s = torch.where(torch.rand(H, D, **f32) < 0.02, 8 * s, s)
    k = (mu + s * torch.randn(T, B, H, D, **f32)).half()
    r = torch.exp(0.25 * torch.randn(T, B, **f32))
    v = (r[..., None, None] * torch.randn(T, B, H, D, **f32)).half()
    q = (torch.randn(B, Hq or H, D, **f32) / math.sqrt(D)).half()
    return k, v, q
