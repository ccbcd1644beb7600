"""Throughput of the KIVI-style decode path (kv_attn of libflagrot_kivi.so) on one B200.

    python -m flagrot_releaser_b200.bench_kivi [--batch 32 --ctx 16384 --hq 64 --hkv 8 --steps 20]

Default workload: the Qwen-32B-shaped case of the baseline: 64 q / 8 kv heads (GQA 8), head 128, batch 32, context 16 384,
page 16, 4 BF16 sink + 128 BF16 window rows; pages written by the library's own value writer and key-group encoder
(K with outlier channels, V ~ N(0, 1)).  Prints one JSON line: quantised-page + BF16-row bytes read per second (CUDA events,
pools larger than L2 cycled) against the measured copy bandwidth (MEASURED_PEAKS.json beside the package's parent, else
the fallback 6 650 GB/s), and the writers' times for the cache build.
"""
from __future__ import annotations

import argparse
import json
import math
from pathlib import Path

import torch

from . import kivi as KV

PAGE, GRP, D = 16, 32, 128


def build(B, L, Hq, Hkv, dev, S, W, seed=0, ncopy=2):
    g = torch.Generator().manual_seed(seed)
    cb = KV.chunk_bytes(D)
    npg = L // PAGE
    NQ = 64
    qs = (torch.randn(Hkv, NQ, D, generator=g) * 0.5).float().contiguous().to(dev)
    lz = torch.full((Hkv, NQ), 3.0, dtype=torch.float32, device=dev)
    co = torch.ones(Hkv, D, device=dev)
    out_ch = torch.randperm(D, generator=g)[:6]
    pools, bts = [], []
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    wv = wk = 0.0
    for _ in range(ncopy):
        nb = B * npg + 3
        pool = torch.zeros(nb, Hkv, cb, dtype=torch.uint8, device=dev)
        bt = torch.randperm(nb - 3, generator=g).view(B, npg).int()
        for b in range(B):
            kv = torch.randn(L, 2 * Hkv, D, generator=g)
            kv[:, :Hkv, out_ch] *= 10
            kv = kv.bfloat16().to(dev)
            pos = torch.arange(L)
            slots = (bt[b].long()[pos // PAGE] * PAGE + pos % PAGE).to(dev)
            gp = torch.arange(L).view(L // GRP, GRP)
            sidx = torch.where(gp < S, torch.full_like(gp, -1), gp).contiguous().to(dev)
            dslot = (bt[b].long()[gp // PAGE] * PAGE + gp % PAGE).contiguous().to(dev)
            ev[0].record()
            KV.v_write(kv, slots, co, None, pool, Hkv, D)
            ev[1].record()
            KV.k_encode(kv, sidx, dslot, qs, lz, 1 / math.sqrt(D), pool, Hkv, D)
            ev[2].record()
            torch.cuda.synchronize()
            wv += ev[0].elapsed_time(ev[1])
            wk += ev[1].elapsed_time(ev[2])
        pools.append(pool)
        bts.append(bt.to(dev))
    n = ncopy * B * L
    return pools, bts, wv * 1e3 / n, wk * 1e3 / n            # writer microseconds per token (all kv heads)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--ctx", type=int, default=16384)
    ap.add_argument("--hq", type=int, default=64)
    ap.add_argument("--hkv", type=int, default=8)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    S, W = 4, 128
    G = a.hq // a.hkv
    pools, bts, us_v, us_k = build(a.batch, a.ctx, a.hq, a.hkv, dev, S, W)
    T = S + W
    ring = torch.randn(a.batch + 1, T, 2 * a.hkv, D).bfloat16().to(dev)
    q = torch.randn(a.batch, a.hq, D).bfloat16().to(dev)
    out = torch.zeros(a.batch, a.hq * D, dtype=torch.bfloat16, device=dev)
    cached = torch.full((a.batch,), a.ctx - W, dtype=torch.int32, device=dev)
    tl = torch.full((a.batch,), T, dtype=torch.int32, device=dev)
    ti = torch.arange(a.batch, dtype=torch.int32, device=dev)
    ns, chunk = KV.plan(a.batch, a.ctx, a.hkv)
    ws = KV.Workspace(a.batch * a.hkv * (ns + 1), G, D, dev)

    def run(i):
        c = i % len(pools)
        KV.attn(q, pools[c], bts[c], cached, out, ns, chunk, ws, 1.4426950408889634 / math.sqrt(D), S, G,
                ring=ring.view(-1, 2 * a.hkv, D), tail_len=tl, tail_idx=ti, T=T)

    for i in range(max(a.warmup, 3)):
        run(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(a.steps):
        run(i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / a.steps
    cell = KV.cell_bytes(D)
    nbytes = a.batch * a.hkv * cell * (a.ctx - W - S) + a.batch * T * 2 * a.hkv * D * 2 + a.batch * a.hq * D * 4
    peak_file = Path(__file__).resolve().parents[1] / "MEASURED_PEAKS.json"
    peak, which = (float(json.loads(peak_file.read_text())["hbm_gbs"]), "measured") if peak_file.exists() else (6650.0, "fallback")
    ach = nbytes / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "kivi_decode_attention_kv_gbps", "value": ach, "unit": "GB/s", "ms_per_step": ms, "steps": a.steps,
        "config": {"workload": f"kivi2:32 decode, batch {a.batch} x ctx {a.ctx}, {a.hq} q / {a.hkv} kv heads, page 16, s4w128",
                   "nsplit": ns, "chunk": chunk, "l2": f"{len(pools)} distinct {pools[0].numel() >> 20} MiB pools cycled"},
        "roofline": {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "peak_source": which,
                     "kernel": "k_kv_attn_mma2 (page splits + BF16 window split) + k_kv_merge", "us_per_launch": ms * 1e3, "algorithmic_bytes": nbytes},
        "writers": {"kv_v_write_us_per_token": us_v, "kv_k_encode_us_per_token": us_k},
        "gpu_launches": 3 * a.steps, "data": "synthetic"}))


if __name__ == "__main__":
    main()
