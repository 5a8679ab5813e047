"""CPU tests of the host-side logic: config object, block cutter against the reference-generated golden
cuts, sharding helpers (world_size-2 gloo processes), synthetic data generator and the benchmark's
accounting helpers."""
import json
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from kvcomp_b200 import sharding
from kvcomp_b200.utils.compute import QuantMode, cut_len, cut_tensor_ctx_len_0
from kvcomp_b200.utils.config import KVCompCacheConfig


def test_config_roundtrip_eq_hash():
    c = KVCompCacheConfig("llama", QuantMode.BlockQuant, QuantMode.TokenQuant, 64, 128, 128, 256, 0.05, 0.1)
    text = str(c)
    assert "'k_quant_mode': 'BlockQuant'" in text and "'v_recent_size': 256" in text
    d = KVCompCacheConfig.from_str(text)
    assert d == c and hash(d) == hash(c) and repr(c) == text
    assert d != KVCompCacheConfig("llama", QuantMode.ChannelQuant, QuantMode.TokenQuant, 64, 128, 128, 256, 0.05, 0.1)
    off = KVCompCacheConfig("llama", None, None, None, None, None, None, None, None, enable_quant=False)
    assert KVCompCacheConfig.from_str(str(off)) == off and "k_quant_mode" not in str(off)


def test_cut_len_matches_reference(golden_dir):
    z = np.load(os.path.join(golden_dir, "quant_golden.npz"))
    cuts = json.loads(bytes(z["cases_json"]).decode())["cuts"]
    assert len(cuts) >= 10
    for ln, blk, recent, n in cuts:
        assert cut_len(ln, blk, recent) == n, (ln, blk, recent)
        to_c, buf = cut_tensor_ctx_len_0(None, torch.zeros(ln, 1, 1, 1), blk, recent)
        assert (0 if to_c is None else to_c.shape[0]) == n and buf.shape[0] == ln - n


def test_split_even_and_heads():
    for total, world in ((8, 1), (8, 2), (8, 4), (32, 8), (10, 4), (3, 8)):
        got = [sharding.split_even(total, world, r) for r in range(world)]
        assert sum(c for _, c in got) == total
        assert all(got[i][0] + got[i][1] == got[i + 1][0] for i in range(world - 1))
    assert sharding.shard_heads(8, 32, 4, 1) == (2, 2, 8, 8)
    assert sharding.shard_heads(10, 40, 2, 1) == (5, 5, 20, 20)
    with pytest.raises(ValueError):
        sharding.shard_heads(10, 40, 4, 0)
    with pytest.raises(ValueError):
        sharding.split_even(4, 2, 2)


def _gloo_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        L, B, Hq = 3, 2, 8
        full = torch.arange(L * B * Hq * 128, dtype=torch.float32).reshape(L, B, Hq, 128)
        _, _, qs, qc = sharding.shard_heads(4, Hq, world, rank)
        out = sharding.gather_head_outputs(full[:, :, qs:qs + qc].contiguous(), world)
        ok = torch.equal(out, full)
        ms = sharding.max_over_ranks([1.0 + rank, 5.0 - rank], "cpu")
        bs, bc = sharding.shard_batch(5, world, rank)
        # the compression-time exchanges of head sharding: unit extremes (min / max) and code histograms (sum)
        g = torch.Generator().manual_seed(3)
        x = torch.randn(6, 2, 4, 128, generator=g).half()                 # [T, B, H, D], heads split over the ranks
        mine = x[:, :, 2 * rank:2 * rank + 2]
        mn, mx = mine.amin(dim=(2, 3)).reshape(-1), mine.amax(dim=(2, 3)).reshape(-1)
        sharding.reduce_extremes(mn, mx)
        ok = ok and torch.equal(mn, x.amin(dim=(2, 3)).reshape(-1)) and torch.equal(mx, x.amax(dim=(2, 3)).reshape(-1))
        hist = torch.bincount(torch.arange(10 * (rank + 1)) % 7, minlength=256)
        sharding.reduce_histogram(hist)
        ok = ok and torch.equal(hist, torch.bincount(torch.arange(10) % 7, minlength=256) + torch.bincount(torch.arange(20) % 7, minlength=256))
        q.put((rank, ok, ms, bs, bc))
    finally:
        dist.destroy_process_group()


def test_two_rank_gather_and_timing_reduce():
    world, port = 2, 29000 + os.getpid() % 2000
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_gloo_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(r[1] for r in res)
    assert res[0][2] == [2.0, 5.0] and res[1][2] == [2.0, 5.0]
    assert (res[0][3], res[0][4]) == (0, 3) and (res[1][3], res[1][4]) == (3, 2)


def test_synth_is_seeded_and_shaped():
    from kvcomp_b200.synth import make_kv
    k, v, q = make_kv(64, 2, 4, 128, seed=0, Hq=8)
    k2, v2, q2 = make_kv(64, 2, 4, 128, seed=0, Hq=8)
    assert torch.equal(k, k2) and torch.equal(v, v2) and torch.equal(q, q2)
    assert k.shape == (64, 2, 4, 128) and q.shape == (2, 8, 128) and k.dtype == torch.float16
    k3, _, _ = make_kv(64, 2, 4, 128, seed=0, layer=1)
    assert not torch.equal(k, k3)
    # per-channel outliers in K, per-token scale in V
    ks = k.float().std(dim=(0, 1))
    assert ks.max() / ks.median() > 3
    assert abs(q.float().std().item() - 1 / np.sqrt(128)) < 0.02


def test_bench_accounting_helpers():
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import bench
    assert list(bench._chunks(1)) == [1] and list(bench._chunks(4)) == [4] and list(bench._chunks(6)) == [4, 2]
    assert list(bench._chunks(5)) == [4, 1]
    cfg = bench.WORKLOADS["c1"]
    acct = {"k": dict(encoded=100, block_info=8, thread_info=128, quant_meta=3),
            "v": dict(encoded=50, block_info=8, thread_info=128, quant_meta=3)}
    assert bench.algorithmic_bytes(acct, cfg) == 100 + 50 + 2 * (8 + 128 + 3) + 2 * cfg["B"] * cfg["Hq"] * 128 * 2
    peak, kind = bench.peaks()
    assert peak > 1000 and kind in ("measured", "fallback")


def test_attention_run_plan_without_a_gpu():
    """kvc_attn_splits / kvc_attn_workspace are host arithmetic (given the SM count): how many partial
    results per head the library's own cut of the columns produces, and the bytes to hold them."""
    from kvcomp_b200 import _lib
    lib = _lib.load()
    sms = 148
    for (T, B, Hkv) in [(128, 1, 1), (1024, 1, 32), (4096, 8, 32), (32768, 16, 8), (16384, 32, 10), (131072, 1, 8)]:
        n_tiles = (T + 255) // 256
        parts = lib.kvc_attn_splits(T, B, Hkv, sms)
        assert 1 <= parts <= n_tiles
        # enough items for the CTAs the device holds, unless the cache has fewer tiles than that
        assert parts * B * Hkv >= min(n_tiles * B * Hkv, 3 * sms) or parts == n_tiles
        assert lib.kvc_attn_workspace(B, Hkv, parts) == 256 + B * Hkv * parts * 260 * 4     # one run still leaves a partial result when a tail follows
    assert lib.kvc_attn_splits(4096, 8, 32, sms) == 8          # runs of 2 tiles
    assert lib.kvc_attn_splits(32768, 16, 8, sms) == 20        # 10 runs of 9 tiles, then 10 of (at most) 4
    assert lib.kvc_attn_splits(0, 8, 32, sms) == 1


def test_recent_rows_buffer_against_a_list_model():
    """The in-place buffer of the cache's rows behind the stream ([kept dequantised rows | recent window]) does
    what a plain list of rows would: appends of every size, rows produced in place, fronts consumed into the kept
    part, kept rows given up, moves to the front and growth of the buffer, rebuilds."""
    import torch
    from kvcomp_b200.cache.kvcomp_encode import _RecentRows
    rng = np.random.default_rng(3)
    rr, kept, recent, nxt = _RecentRows(), [], [], 0
    shape = (2, 1, 4)

    def rows(n):
        nonlocal nxt
        t = torch.arange(nxt, nxt + n, dtype=torch.float32).view(n, 1, 1, 1).expand(n, *shape).contiguous()
        nxt += n
        return t

    def check():
        assert len(rr) == len(recent) and rr.kept == len(kept)
        got = rr.rows_from_kept(len(kept))
        want = kept + recent
        if not want:
            assert got is None
        else:
            assert got.is_contiguous() and [int(v) for v in got[:, 0, 0, 0]] == want
            assert [int(v) for v in rr.view()[:, 0, 0, 0]] == recent
    moves = 0
    for step in range(3000):
        op = rng.integers(0, 6)
        before = None if rr.buf is None else rr.buf.data_ptr()
        if op <= 1:                                   # append
            n = int(rng.choice([1, 1, 1, 2, 5, 40]))
            r = rows(n)
            rr.append(r, room=8)
            recent += [int(v) for v in r[:, 0, 0, 0]]
        elif op == 2:                                 # rows produced in place
            n = int(rng.integers(1, 4))
            place = rr.reserve(n, 8, shape, torch.float32, torch.device("cpu"))
            r = rows(n)
            place.copy_(r)
            rr.commit(n)
            recent += [int(v) for v in r[:, 0, 0, 0]]
        elif op == 3 and recent:                      # the window's front is compressed and kept as dequantised rows
            n = int(rng.integers(1, len(recent) + 1))
            rr.view()[:n] += 100000                   # "dequantised in place"
            rr.consume(n)
            kept += [v + 100000 for v in recent[:n]]
            recent = recent[n:]
        elif op == 4 and kept:                        # a reader has moved on
            k = int(rng.integers(0, len(kept) + 1))
            rr.rows_from_kept(k)
            kept = kept[len(kept) - k:]
        elif op == 5 and step % 7 == 0:               # start over (a prefill, a read from a file)
            k, r = rows(int(rng.integers(0, 4))), rows(int(rng.integers(0, 6)))
            rr.rebuild(k if k.shape[0] else None, r if r.shape[0] else None, room=8)
            kept, recent = [int(v) for v in k[:, 0, 0, 0]], [int(v) for v in r[:, 0, 0, 0]]
        moves += before is not None and rr.buf is not None and rr.buf.data_ptr() != before
        check()
    assert nxt > 3000 and moves < 400                 # the buffer is replaced now and then, not at every step
