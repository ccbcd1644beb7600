"""Throughput of the prefix-cached multi-query prefill path (prep_q + attn + merge of libflagrot_mq.so) on one B200.

    python -m flagrot_releaser_b200.bench_mq [--batch 4 --new 512 --cached 32768 --kind konlya --kernel 3 --steps 20]

Default workload: batch 4, a 512-token query chunk per request over 32768 cached tokens, 32 q / 8 kv heads, head 128,
page 16, INT4 pages written by the library's own writer (synthetic K with outlier channels, V ~ N(0, 1)).  Prints one JSON
line: useful attention TFLOP/s (4 * 128 * q heads * visible (query, key) pairs / time; the causal triangle is counted
exactly), per-launch times from CUDA events, and the fraction of the measured dense bf16 peak (MEASURED_PEAKS.json beside
the package's parent, else the fallback 1590 TFLOP/s).  The pool (> 126 MB) is larger than L2.
"""
from __future__ import annotations

import argparse
import json
import math
from pathlib import Path

import torch

from . import kernels as K
from . import prefill_mq as MQ

PAGE = 16


def build(batch, new, cached, Hq, Hkv, kind, dev, seed=0):
    g = torch.Generator().manual_seed(seed)
    L = cached + new
    npg = -(-L // PAGE)
    total = batch * npg + 3
    nb = 2 if kind in ("int2a", "konlya2") else 4
    pool = torch.zeros(total, Hkv, (80 if nb == 2 else 144) * PAGE, dtype=torch.uint8, device=dev)
    perm = torch.randperm(batch * npg, generator=g).int()
    bt = perm.view(batch, npg).contiguous()
    A = torch.randn(Hkv, 128, 128, generator=g) / math.sqrt(128)
    CT = (A @ A.transpose(1, 2) + 0.1 * torch.eye(128)).contiguous().to(dev)
    co = torch.ones(Hkv, 128, device=dev)
    zeros = torch.zeros(2 * Hkv, 4, dtype=torch.uint8, device=dev)
    out_ch = torch.randperm(128, generator=g)[:6]
    for r in range(batch):
        for t0 in range(0, L, 8192):
            n = min(8192, L - t0)
            kv = torch.randn(n, 2 * Hkv, 128, generator=g)
            kv[:, :Hkv, out_ch] *= 10
            pos = torch.arange(t0, t0 + n)
            sl = (bt[r].long()[pos // PAGE] * PAGE + pos % PAGE).to(dev)
            if kind.startswith("konlya"):
                K.cb_write(kv.bfloat16().to(dev), sl, CT, co, kind, pool, PAGE)
            else:
                K.v2_write(kv.bfloat16().to(dev), sl, zeros, 32, pool, PAGE, fmt=kind)
    q = torch.randn(batch * new, Hq, 128, generator=g).bfloat16().to(dev)
    reqs = [(r, r * new, (r + 1) * new, L, cached) for r in range(batch)]
    return pool, bt.to(dev), q, reqs, nb


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--new", type=int, default=512)
    ap.add_argument("--cached", type=int, default=32768)
    ap.add_argument("--hq", type=int, default=32)
    ap.add_argument("--hkv", type=int, default=8)
    ap.add_argument("--kind", default="konlya")
    ap.add_argument("--kernel", type=int, default=None)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    G = a.hq // a.hkv
    pool, bt, q, reqs, nb = build(a.batch, a.new, a.cached, a.hq, a.hkv, a.kind, dev)
    plan = MQ.build_plan(reqs, G, a.hkv, 0, dev, kernel=a.kernel)
    out = torch.zeros(q.shape[0], a.hq * 128, dtype=torch.bfloat16, device=dev)
    scale = 1 / math.sqrt(128)
    konly = a.kind.startswith("konlya")

    def run():
        q16 = MQ.prep_q(q, scale * MQ.LOG2E, G, idx=plan.idx)
        opart, ml = MQ.attn(q16, pool, bt, plan, G, 0, konly=konly, int2=nb == 2)
        MQ.merge(plan, opart, ml, G, out=out)
        return q16, opart, ml

    for _ in range(max(a.warmup, 3)):
        q16, opart, ml = run()
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    tot = att = 0.0
    for _ in range(a.steps):
        ev[0].record()
        q16 = MQ.prep_q(q, scale * MQ.LOG2E, G, idx=plan.idx)
        ev[1].record()
        opart, ml = MQ.attn(q16, pool, bt, plan, G, 0, konly=konly, int2=nb == 2)
        ev[2].record()
        MQ.merge(plan, opart, ml, G, out=out)
        ev[3].record()
        torch.cuda.synchronize()
        tot += ev[0].elapsed_time(ev[3])
        att += ev[1].elapsed_time(ev[2])
    tot, att = tot / a.steps, att / a.steps
    pairs = a.batch * a.new * (a.cached + (a.new + 1) / 2)
    flops = 4.0 * 128 * a.hq * pairs
    peak_file = Path(__file__).resolve().parents[1] / "MEASURED_PEAKS.json"
    peak, which = (float(json.loads(peak_file.read_text())["bf16_tflops"]), "measured") if peak_file.exists() else (1590.0, "fallback")
    cell = 80 if nb == 2 else 144
    print(json.dumps({
        "metric": "mq_prefill_attention_tflops", "value": flops / (tot * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": tot,
        "config": {"workload": f"prefix-cached prefill, batch {a.batch} x {a.new} new over {a.cached} cached, {a.hq} q / {a.hkv} kv "
                               f"heads, {a.kind} pages", "kernel": plan.kernel, "rows": plan.rows, "tiles": plan.ntiles,
                   "items": plan.nitems},
        "roofline": {"bound": "tensor", "achieved": flops / (att * 1e-3) / 1e12, "peak": peak, "unit": "TFLOP/s",
                     "frac": flops / (att * 1e-3) / 1e12 / peak, "peak_source": which, "kernel": "k_mq", "us_per_launch": att * 1e3,
                     "useful_flops": flops, "page_bytes_read_once": a.batch * (a.cached + a.new) * a.hkv * cell},
        "steps": a.steps, "gpu_launches": 3 * a.steps, "data": "synthetic"}))


if __name__ == "__main__":
    main()
