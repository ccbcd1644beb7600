"""Benchmarks of the FlagRot KV-cache hot path on B200.  Headline (default): paged decode over INT4 (konlya) pages on the
Llama-3.1-8B-shaped batch-64 x 4K workload.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg2|cfg3|cfg4|cfg5a|cfg5b|writers]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workloads (the configurations of the baseline; all inputs seeded synthetic, caches written by the library's own writers):
  cfg2   INT4 konlya decode, 32 q / 8 kv heads, batch 64 x ctx 4096, s4w128.  N GPUs: every rank runs the full batch on its
         own pool (weak scaling, no data-path collective).
  cfg3   INT2 konlya2 decode with centred keys, batch 256 x ctx 8192.  N GPUs: rows [r B / N, (r + 1) B / N) per rank (strong).
  cfg4   KIVI-style INT2 decode, 64 q / 8 kv heads, batch 32 x ctx 16384.  N GPUs: kv heads [r Hkv / N, ...) and their q heads
         per rank (tensor parallel by kv head, strong); calibration rows sliced the same way.
  cfg5a  prefix-cached prefill, 4 requests x 512 new tokens over 32768 cached, INT4 konlya pages (tensor-bound; requests
         are dealt over the ranks).
  cfg5b  one sequence of 131072 tokens, INT4 konlya: the KV sequence is split over the ranks, every rank emits (o, m, l)
         rows (fr_attn_partial), an NCCL all-gather of 130 floats per (row, head) and fr_merge_partials finish the step.
  writers  the cache writers against the reference's own sm_100a-capable kernels (oracle/_ref), T = 64 and T = 65536 (scattered and consecutive slots).

A step = one pass of the hot path over one batch: the writer appends one token per sequence and the decode attention reads
every sequence's cache (prefill: q staging + attention + item merge).  `value` has every input resident in HBM (the
resident step is replayed as one CUDA graph per pool copy); `e2e` measures the same step through the C-ABI front end with
this step's inputs copied from pinned host memory and the output copied back inside the timed region (the KV cache is the
path's state and lives in HBM, as in the plugin).  Pools larger than L2 are cycled.  Before the K timed steps the same step
runs untimed for --sustain-s seconds, so that clocks and power are those of a loaded GPU; the roofline figure comes from a
kernel-only loop of at least --sustain-s seconds with the SM clock sampled over that loop.
The reference arm (--impl reference) times the reference's own CPU implementation of the path on the host cores: its
PyTorch page parser (kernels.py dequant_cb_pages / kivi.py dequant_groups, byte code under oracle/_ref/pyref) + fp32
attention with all host threads; when that byte code is absent, the numpy restatement under oracle/.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
LOG2E = 1.4426950408889634
P = 16
SCALE = 1 / math.sqrt(128)

WORKLOADS = {
    "cfg2": dict(path="decode", kind="konlya", nb=4, B=64, L=4096, Hq=32, Hkv=8, S=4, W=128, center=False, shard="replica",
                 name="llama-3.1-8b-shaped int4 konlya decode, batch 64 x ctx 4096, page 16, s4w128"),
    "cfg3": dict(path="decode", kind="konlya2", nb=2, B=256, L=8192, Hq=32, Hkv=8, S=4, W=128, center=True, shard="batch",
                 name="qwen3-8b-shaped int2 konlya2 decode, batch 256 x ctx 8192, page 16, s4w128, centred keys"),
    "cfg4": dict(path="kivi", B=32, L=16384, Hq=64, Hkv=8, S=4, W=128, shard="kvhead",
                 name="qwen-32b-shaped kivi2:32 decode, batch 32 x ctx 16384, 64 q / 8 kv heads, page 16, s4w128"),
    "cfg4p8": dict(path="kivi", B=32, L=16384, Hq=64, Hkv=8, S=4, W=128, shard="kvhead", f8=True,
                   name="qwen-32b-shaped kivi2p8 (FP8 scale / min, 2.5 bits) decode, batch 32 x ctx 16384, 64 q / 8 kv heads, page 16, s4w128"),
    "cfg5a": dict(path="prefill", kind="konlya", nb=4, B=4, new=512, L=32768, Hq=32, Hkv=8, shard="request",
                  name="prefix-cached prefill, 4 requests x 512 new tokens over 32768 cached, 32 q / 8 kv heads, int4 konlya pages"),
    "cfg5b": dict(path="decode", kind="konlya", nb=4, B=1, L=131072, Hq=32, Hkv=8, S=4, W=128, center=False, shard="kvseq",
                  name="int4 konlya decode, batch 1 x ctx 131072, page 16, s4w128, KV-sequence sharded"),
    "writers": dict(path="writers", name="cache writers against the reference's own kernels, T = 64 and T = 65536, 8 kv heads"),
}


def peaks():
    """(hbm GB/s, dense bf16 TFLOP/s burst, sustained, source)"""
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        d = json.loads(f.read_text())
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
    return 6650.0, 1590.0, 1400.0, "fallback"


class ClockSampler:
    """samples SM clock and throttle reasons with nvidia-smi while a timed region runs (query only)."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                                          "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.1)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, pw, reasons = [], [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
                pw.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------------- timing
def max_over_ranks(ms, dist, device="cuda"):
    """the slowest rank's time (all-reduce MAX), identical on every rank"""
    if dist is None:
        return ms
    t = torch.tensor([ms], dtype=torch.float32, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def timed(fn, steps, warmup, dist=None, sustain_s=0.0):
    """W warm-up steps (+ the same step repeated untimed for sustain_s seconds), then exactly `steps` steps between two
    CUDA events on the launch stream, bracketed by barrier + synchronize; max over ranks.  Returns ms per step."""
    if dist is not None:
        dist.barrier()                                   # ranks enter a leg together (a step may wait for its peers)
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    n = warmup
    if sustain_s > 0:
        # the untimed load: a step count fixed from a short probe and agreed over the ranks (a step may hold a collective,
        # so every rank has to run the same number of them)
        t0 = time.perf_counter()
        for _ in range(8):
            fn(n)
            n += 1
        torch.cuda.synchronize()
        est = max_over_ranks((time.perf_counter() - t0) * 1e3 / 8, dist)
        for _ in range(min(200000, int(math.ceil(sustain_s * 1e3 / max(est, 1e-3))))):
            fn(n)
            n += 1
        torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn(n + i)
    e1.record()
    torch.cuda.synchronize()
    ms = max_over_ranks(e0.elapsed_time(e1), dist)
    if dist is not None:
        dist.barrier()
    return ms / steps


def sustained(fn, est_ms, seconds, gpu_index):
    """a loop of at least `seconds` of back-to-back launches (count fixed beforehand from est_ms) timed by CUDA events, with
    the SM clock sampled over the loop.  Returns (ms per launch, launches, clocks)."""
    n = max(20, int(math.ceil(seconds * 1e3 / max(est_ms, 1e-3))))
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    smp = ClockSampler(gpu_index).start()
    time.sleep(0.15)                                     # the sampler's first line takes a moment
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(n):
        fn(3 + i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / n
    return ms, n, smp.stop()


def graph_of(fn):
    """fn() captured as one CUDA graph (fn has run before: kernel attributes are set)"""
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    return g


# ---------------------------------------------------------------------------------------------- FlagRot INT4 / INT2 decode
def kvseq_local_len(L, W, world):
    """context length of one rank when the page tokens [0, L - W) of a sequence are split evenly over `world` ranks (every
    rank keeps the W window rows in its count, as the single-GPU convention does)."""
    return (L - W) // world + W


class DecodeWorkload:
    """cfg2 / cfg3 / cfg5b: fr_cb_write (T = batch) + fr_cb_attn over konlya / konlya2 pages with BF16 sink + window rows."""

    metric, unit, bound = "decode_attention_kv_gbps", "GB/s", "hbm"

    def __init__(self, w, rank, world, dev, a):
        from flagrot_releaser_b200 import kernels as K
        self.K, self.w, self.rank, self.world, self.dev, self.a = K, w, rank, world, dev, a
        self.kvseq = w["shard"] == "kvseq"
        self.B = w["B"] // world if w["shard"] == "batch" else w["B"]
        assert self.B >= 1 and (w["shard"] != "batch" or w["B"] % world == 0), "the batch must divide over the ranks"
        self.cell = 144 if w["nb"] == 4 else 80
        self.Lloc = kvseq_local_len(w["L"], w["W"], world) if self.kvseq else w["L"]
        per_copy = self.B * self.Lloc * w["Hkv"] * self.cell
        # pool copies cycled: an explicit --ncopy, else enough distinct memory that no page survives in L2 between steps
        self.ncopy = a.ncopy if a.ncopy > 0 else min(64, max(1 if per_copy > (600 << 20) else 3, -(-(400 << 20) // per_copy)))
        self.build(seed=1234 + rank)
        ns, ch = K.plan_cb(self.B, self.Lloc - w["W"], w["Hkv"], P, w["kind"], a.nsplit or None, tail=True)
        self.plan = (ns, ch)
        self.ws = K.Workspace(self.B, w["Hkv"], self.B * w["Hkv"] * (ns + 1), dev)
        self.dist = None
        self.xchg = None

    def build(self, seed):
        """synthetic inputs of the named shape and the quantised caches (written by the library's own dynamic writer, which
        the parity tests hold bit-exact).  ncopy distinct pools (distinct random page tables over distinct memory) are cycled
        so that no page is L2-resident between steps."""
        K, w, dev, B, L = self.K, self.w, self.dev, self.B, self.Lloc
        g = torch.Generator().manual_seed(seed)
        Hkv, Hq = w["Hkv"], w["Hq"]
        npages_seq = L // P
        npool = B * npages_seq + 7
        qs = torch.randn(Hkv, 512, 128, generator=g) * (torch.rand(Hkv, 1, 128, generator=g) + 0.5).sqrt()
        Cq = (torch.einsum("hnd,hne->hde", qs, qs) / 512).contiguous()
        self.CT = Cq.transpose(1, 2).contiguous().to(dev)
        self.co = (torch.rand(Hkv, 128, generator=g) + 0.5).to(dev)
        out_ch = torch.stack([torch.randperm(128, generator=g)[:6] for _ in range(Hkv)])          # 5 % of channels x10
        self.kmu = offs = None
        if w["center"]:
            offs = torch.randn(Hkv, 128, generator=g) * math.sqrt(2.0)
            self.kmu = offs.float().contiguous().to(dev)
        chunk_b = K.cb_chunk_bytes(w["kind"], P)
        self.pools, self.bts = [], []
        rows_per = 64 * 1024
        for _ in range(self.ncopy):
            pool = torch.randint(0, 256, (npool, Hkv, chunk_b), dtype=torch.uint8, generator=g).to(dev)
            bt = torch.randperm(npool, generator=g)[:B * npages_seq].reshape(B, npages_seq).int()
            pos = torch.arange(L)
            slots = (bt.long()[:, pos // P] * P + pos % P).reshape(-1)
            for r0 in range(0, B * L, rows_per):
                n = min(rows_per, B * L - r0)
                kv = torch.randn(n, 2 * Hkv, 128, generator=g)
                for h in range(Hkv):
                    kv[:, h, out_ch[h]] *= 10
                if offs is not None:
                    kv[:, :Hkv] += offs
                K.cb_write(kv.bfloat16().to(dev), slots[r0:r0 + n].to(dev), self.CT, self.co, w["kind"], pool, P, kmu=self.kmu)
            torch.cuda.synchronize()
            self.pools.append(pool)
            self.bts.append(bt.to(dev))
        T = w["S"] + w["W"]
        self.ring = torch.randn(B, T, 2 * Hkv, 128, generator=g).bfloat16().to(dev)
        self.tail_len = torch.full((B,), T, dtype=torch.int32, device=dev)
        self.seq = torch.full((B,), L - w["W"], dtype=torch.int32, device=dev)
        self.q_host = torch.randn(B, Hq, 128, generator=g).bfloat16().pin_memory()
        self.kv_host = torch.randn(B, 2 * Hkv, 128, generator=g).bfloat16().pin_memory()
        self.out_host = torch.empty(B, Hq * 128, dtype=torch.bfloat16).pin_memory()
        self.out = torch.empty(B, Hq * 128, dtype=torch.bfloat16, device=dev)
        self.q, self.kv = self.q_host.to(dev), self.kv_host.to(dev)
        if self.kvseq:
            self.part = torch.zeros(B, Hq, 130, dtype=torch.float32, device=dev)
            self.parts = torch.zeros(self.world, B, Hq, 130, dtype=torch.float32, device=dev)
        # the appended token of every sequence goes to position L - W - 1 of its row (a scattered slot per sequence)
        self.slots = [(bt.long()[:, (L - w["W"] - 1) // P] * P + (L - w["W"] - 1) % P).contiguous() for bt in self.bts]
        self.slots_host = [s.cpu().pin_memory() for s in self.slots]

    # ---- the step
    def _attn_args(self, c):
        w, ring = self.w, self.ring
        return dict(tail=ring, tail_len=self.tail_len, tail_idx=None, tail_bs=ring.stride(0), tail_ts=ring.stride(1))

    def resident(self, c):
        K, w = self.K, self.w
        ns, ch = self.plan
        if self.kvseq:
            return self.resident_kvseq(c)
        K.cb_write(self.kv, self.slots[c], self.CT, self.co, w["kind"], self.pools[c], P, kmu=self.kmu)
        K.cb_attn(self.q, self.pools[c], self.bts[c], self.seq, self.out, ns, ch, self.ws, LOG2E * SCALE, w["kind"], page=P,
                  kv_start=w["S"], **self._attn_args(c))

    def resident_kvseq(self, c):
        """the last rank appends the new token, every rank attends over its slice (rank 0 also over the BF16 sink / window
        rows), partial rows are all-gathered (NCCL) and merged"""
        K, w = self.K, self.w
        ns, ch = self.plan
        first, last = self.rank == 0, self.rank == self.world - 1
        if last:
            K.cb_write(self.kv, self.slots[c], self.CT, self.co, w["kind"], self.pools[c], P, kmu=self.kmu)
        tkw = self._attn_args(c) if first else {}
        K.attn_partial(self.q, self.pools[c], self.bts[c], self.seq, self.part, ns, ch, self.ws, LOG2E * SCALE, w["kind"], page=P,
                       kv_start=w["S"] if first else 0, **tkw)
        if self.dist is not None and self.a.kvseq_exchange == "p2p":
            if self.xchg is None:                          # set-up on the first (uncaptured) step: buffers + IPC handles
                self.xchg = K.ShardExchange(self.rank, self.world, self.part.shape[0] * self.part.shape[1], self.dist)
            self.xchg.merge(self.part, self.out)           # one kernel: push to the peers, wait, merge
        elif self.dist is not None:
            self.dist.all_gather_into_tensor(self.parts.view(-1, *self.part.shape[1:]), self.part)
            K.merge_partials_into(self.parts, self.out)
        else:
            K.merge_partials_into(self.part[None], self.out)

    def kernel(self, c):
        K, w = self.K, self.w
        ns, ch = self.plan
        K.cb_attn(self.q, self.pools[c], self.bts[c], self.seq, self.out, ns, ch, self.ws, LOG2E * SCALE, w["kind"], page=P,
                  kv_start=w["S"], **self._attn_args(c))

    def e2e(self, c):
        if self.a.e2e_launch == "graph" and not (self.kvseq and self.world > 1):
            # the whole step - copies in, append, decode, copy back - as ONE graph launch (graphs.HostStep)
            hs = self.__dict__.setdefault("hsteps", {})
            if c not in hs:
                from flagrot_releaser_b200.graphs import HostStep
                hs[c] = HostStep([(self.q, self.q_host), (self.kv, self.kv_host), (self.slots[c], self.slots_host[c])],
                                 lambda: self.resident(c), [(self.out_host, self.out)])
            hs[c].run()
            return
        self.q.copy_(self.q_host, non_blocking=True)
        if not self.kvseq or self.rank == self.world - 1:
            self.kv.copy_(self.kv_host, non_blocking=True)
            self.slots[c].copy_(self.slots_host[c], non_blocking=True)
        g = getattr(self, "graphs", None)
        if g is not None:
            g[c].replay()
        else:
            self.resident(c)
        self.out_host.copy_(self.out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    # ---- accounting
    def job_units(self):
        """algorithmic bytes of the decode read of the whole job (all ranks)"""
        w = self.w
        n = self.world if w["shard"] == "replica" else 1
        return n * self._bytes(w["B"], w["L"])

    def _bytes(self, B, L):
        w = self.w
        return (B * w["Hkv"] * self.cell * (L - w["W"] - w["S"]) + B * (w["S"] + w["W"]) * 2 * w["Hkv"] * 128 * 2
                + B * w["Hq"] * 128 * 2 * 2)

    def launch_units(self):
        """algorithmic bytes of this rank's decode launch (kvseq: rank 0 carries the BF16 rows)"""
        w = self.w
        if self.kvseq:
            return self._bytes(self.B, w["L"]) - self.B * w["Hkv"] * self.cell * (w["L"] - self.Lloc)
        return self._bytes(self.B, w["L"])

    def copies(self):
        return int(self.q_host.numel() * 2 + self.kv_host.numel() * 2 + self.B * 8), int(self.out_host.numel() * 2)

    launches = property(lambda self: 3 if self.kvseq else 2)    # append (keys + value rows, one launch), decode [, merge]
    kernel_name = property(lambda self: f"k_decode<{self.w['nb']}, key-only>")

    def config(self):
        w, world = self.w, self.world
        par = {"replica": f"batch replicas x{world}, no collective", "batch": f"batch-sharded x{world} ({self.B} rows per rank), no collective",
               "kvseq": (f"kv-sequence sharded x{world}, (o, m, l) rows pushed to the peers and merged by one kernel over peer memory"
                         if self.a.kvseq_exchange == "p2p" else
                         f"kv-sequence sharded x{world}, NCCL all-gather of (o, m, l) rows + LSE merge")}[w["shard"]]
        return {"batch_per_gpu": self.B, "nsplit": self.plan[0], "chunk": self.plan[1],
                "l2": f"{self.ncopy} distinct {self.pools[0].numel() >> 20} MiB pools cycled "
                      f"({self.ncopy * self.pools[0].numel() >> 20} MiB in all, more than the 126 MB L2)",
                "parallelism": par if world > 1 else "single gpu",
                "step": (("fr_cb_write (last rank) + fr_attn_partial + fr_xchg_merge" if self.a.kvseq_exchange == "p2p" and self.world > 1
                          else "fr_cb_write (last rank) + fr_attn_partial + all-gather + fr_merge_partials") if self.kvseq
                         else "fr_cb_write (T = batch) + fr_cb_attn")}

    def status(self):
        return self.K.device_status()


# ---------------------------------------------------------------------------------------------- KIVI decode
class KiviWorkload:
    """cfg4: kv_v_write (T = batch) + kv_attn over kivi2:32 pages; tensor parallel by kv head."""

    metric, unit, bound = "decode_attention_kv_gbps", "GB/s", "hbm"
    GRP, D = 32, 128

    def __init__(self, w, rank, world, dev, a):
        from flagrot_releaser_b200 import kivi as KV
        self.KV, self.w, self.rank, self.world, self.dev, self.a = KV, w, rank, world, dev, a
        assert w["Hkv"] % world == 0, "kv heads must divide over the ranks"
        self.Hkv = w["Hkv"] // world                       # this rank's kv heads [rank Hkv, (rank + 1) Hkv) and their q heads
        self.G = w["Hq"] // w["Hkv"]
        self.B, self.L, self.S, self.W = w["B"], w["L"], w["S"], w["W"]
        self.f8 = bool(w.get("f8", False))                 # kivi2p8 pages
        per_copy = self.B * (self.L // P) * self.Hkv * KV.chunk_bytes(self.D, self.f8)
        self.ncopy = a.ncopy if a.ncopy > 0 else min(64, max(2, -(-(400 << 20) // per_copy)))
        self.build(seed=4321)
        self.plan = KV.plan(self.B, self.L, self.Hkv) if not a.nsplit else (a.nsplit, max(256, -(-self.L // a.nsplit // 128) * 128))
        self.ws = KV.Workspace(self.B * self.Hkv * (self.plan[0] + 1), self.G, self.D, dev)

    def build(self, seed):
        KV, dev, B, L, D, GRP, S = self.KV, self.dev, self.B, self.L, self.D, self.GRP, self.S
        g = torch.Generator().manual_seed(seed)            # the same stream on every rank: the job's tensors, then sliced
        Hall, h0, Hkv, G = self.w["Hkv"], self.rank * self.Hkv, self.Hkv, self.G
        NQ = 64                                            # calibration queries per kv head (N(0, 0.3^2), log-normaliser 5.0)
        sl = slice(h0, h0 + Hkv)
        self.qs = (torch.randn(Hall, NQ, D, generator=g) * 0.3)[sl].contiguous().to(dev)
        self.lz = torch.full((Hkv, NQ), 5.0, dtype=torch.float32, device=dev)
        self.co = (torch.rand(Hall, D, generator=g) + 0.5)[sl].contiguous().to(dev)
        out_ch = torch.stack([torch.randperm(D, generator=g)[:6] for _ in range(Hall)])[sl]
        npg = L // P
        self.pools, self.bts = [], []
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        self.us_v = self.us_k = 0.0
        for _ in range(self.ncopy):
            nb = B * npg + 3
            pool = torch.zeros(nb, Hkv, KV.chunk_bytes(D, self.f8), dtype=torch.uint8, device=dev)
            bt = torch.randperm(nb - 3, generator=g).view(B, npg).int()
            for b in range(B):
                kv = torch.randn(L, 2 * Hkv, D, generator=g)
                for h in range(Hkv):
                    kv[:, h, out_ch[h]] *= 10
                kv = kv.bfloat16().to(dev)
                pos = torch.arange(L)
                slots = (bt[b].long()[pos // P] * P + pos % P).to(dev)
                gp = torch.arange(L).view(L // GRP, GRP)
                sidx = torch.where(gp < S, torch.full_like(gp, -1), gp).contiguous().to(dev)
                dslot = (bt[b].long()[gp // P] * P + gp % P).contiguous().to(dev)
                ev[0].record()
                KV.v_write(kv, slots, self.co, None, pool, Hkv, D, f8=self.f8)
                ev[1].record()
                KV.k_encode(kv, sidx, dslot, self.qs, self.lz, SCALE, pool, Hkv, D, f8=self.f8)
                ev[2].record()
                torch.cuda.synchronize()
                self.us_v += ev[0].elapsed_time(ev[1]) * 1e3
                self.us_k += ev[1].elapsed_time(ev[2]) * 1e3
            self.pools.append(pool)
            self.bts.append(bt.to(dev))
        ntok = self.ncopy * B * L
        self.us_v, self.us_k = self.us_v / ntok, self.us_k / ntok
        T = self.S + self.W
        Hq = Hkv * G
        self.T = T
        self.ring = torch.randn(B + 1, T, 2 * Hkv, D, generator=g).bfloat16().to(dev)
        self.q_host = torch.randn(B, Hq, D, generator=g).bfloat16().pin_memory()
        self.kv_host = torch.randn(B, 2 * Hkv, D, generator=g).bfloat16().pin_memory()
        self.out_host = torch.empty(B, Hq * D, dtype=torch.bfloat16).pin_memory()
        self.q, self.kv = self.q_host.to(dev), self.kv_host.to(dev)
        self.out = torch.zeros(B, Hq * D, dtype=torch.bfloat16, device=dev)
        self.cached = torch.full((B,), L - self.W, dtype=torch.int32, device=dev)
        self.tl = torch.full((B,), T, dtype=torch.int32, device=dev)
        self.ti = torch.arange(B, dtype=torch.int32, device=dev)
        # the appended value row of every sequence lands at position L - W - 1 (keys are encoded per completed group)
        self.slots = [(bt.long()[:, (L - self.W - 1) // P] * P + (L - self.W - 1) % P).contiguous() for bt in self.bts]
        self.slots_host = [s.cpu().pin_memory() for s in self.slots]

    def kernel(self, c):
        ns, chunk = self.plan
        self.KV.attn(self.q, self.pools[c], self.bts[c], self.cached, self.out, ns, chunk, self.ws, LOG2E * SCALE, self.S, self.G,
                     ring=self.ring.view(-1, 2 * self.Hkv, self.D), tail_len=self.tl, tail_idx=self.ti, T=self.T, f8=self.f8)

    def resident(self, c):
        self.KV.v_write(self.kv, self.slots[c], self.co, None, self.pools[c], self.Hkv, self.D, f8=self.f8)
        self.kernel(c)

    def e2e(self, c):
        self.q.copy_(self.q_host, non_blocking=True)
        self.kv.copy_(self.kv_host, non_blocking=True)
        self.slots[c].copy_(self.slots_host[c], non_blocking=True)
        g = getattr(self, "graphs", None)
        if g is not None:
            g[c].replay()
        else:
            self.resident(c)
        self.out_host.copy_(self.out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def _bytes(self, Hkv):
        cell = self.KV.cell_bytes(self.D, self.f8)
        return (self.B * Hkv * cell * (self.L - self.W - self.S) + self.B * self.T * 2 * Hkv * self.D * 2
                + self.B * Hkv * self.G * self.D * 2 * 2)

    def job_units(self):
        return self._bytes(self.w["Hkv"])

    def launch_units(self):
        return self._bytes(self.Hkv)

    def copies(self):
        return int(self.q_host.numel() * 2 + self.kv_host.numel() * 2 + self.B * 8), int(self.out_host.numel() * 2)

    launches = 3                                           # value append, page + window splits (one launch), split merge
    kernel_name = "k_kv_attn_mma2 (page splits + BF16 window split) + k_kv_merge"

    def config(self):
        return {"batch_per_gpu": self.B, "kv_heads_per_gpu": self.Hkv, "nsplit": self.plan[0], "chunk": self.plan[1],
                "l2": f"{self.ncopy} distinct {self.pools[0].numel() >> 20} MiB pools cycled",
                "parallelism": (f"tensor parallel by kv head x{self.world} ({self.Hkv} kv heads + {self.Hkv * self.G} q heads per rank, "
                                f"calibration rows sliced alike), no collective in the path") if self.world > 1 else "single gpu",
                "step": "kv_v_write (T = batch) + kv_attn",
                "writers_us_per_token": {"kv_v_write": self.us_v, "kv_k_encode": self.us_k}}

    def status(self):
        return 0

    def race_reference(self):
        """the reference's own kv_attn (kivi.cu built unmodified for sm_100a, oracle/_ref) on the same pools and plan: a bench
        leg only, never the product path"""
        p = ROOT / "oracle" / "_ref" / "libflagrot_kivi_ref.so"
        if not p.exists():
            return None
        L = ctypes.CDLL(str(p))
        PP, I, LL, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
        L.kv_attn.argtypes = [PP, LL, PP, PP, LL, PP, I, I, I, I, I, I, I, F, PP, PP, PP, I, PP, PP, PP, LL, I, PP]
        L.kv_attn.restype = I
        ns, chunk = self.plan
        out2 = torch.zeros_like(self.out)
        ring = self.ring.view(-1, 2 * self.Hkv, self.D)

        f8 = 0

        def run(c):
            rc = L.kv_attn(self.q.data_ptr(), self.q.stride(0), self.pools[c].data_ptr(), self.bts[c].data_ptr(), self.bts[c].stride(0),
                           self.cached.data_ptr(), self.S, self.B, self.Hkv, self.G, self.D, ns, chunk, LOG2E * SCALE, ring.data_ptr(),
                           self.tl.data_ptr(), self.ti.data_ptr(), self.T, self.ws.opart.data_ptr(), self.ws.ml.data_ptr(),
                           out2.data_ptr(), out2.stride(0), f8, torch.cuda.current_stream().cuda_stream)
            assert rc == 0, rc
        res = {}
        for name, f8 in (("plain", int(self.f8)),) + ((("fast", 3),) if self.f8 else ()):    # kivi2p8 also has the reference's "fast" variant
            ms = timed(lambda i: run(i % self.ncopy), 10, 3)
            self.kernel(0)
            run(0)
            torch.cuda.synchronize()
            diff = float((self.out.float() - out2.float()).abs().max())
            res[name] = {"kernel": "reference kv_attn (k_attn3 + k_merge, mma.sync) at sm_100a" + (", fast variant" if f8 & 2 else ""),
                         "us_per_launch": ms * 1e3, "GB/s": self.launch_units() / (ms * 1e-3) / 1e9, "max_abs_diff_vs_ours": diff}
        return res["plain"] if len(res) == 1 else res


# ---------------------------------------------------------------------------------------------- prefix-cached prefill
class PrefillWorkload:
    """cfg5a: frmq_prep_q + frmq_attn + frmq_merge over INT4 konlya pages; requests dealt over the ranks."""

    metric, unit, bound = "mq_prefill_attention_tflops", "TFLOP/s", "tensor"

    def __init__(self, w, rank, world, dev, a):
        from flagrot_releaser_b200 import kernels as K
        from flagrot_releaser_b200 import prefill_mq as MQ
        self.K, self.MQ, self.w, self.rank, self.world, self.dev, self.a = K, MQ, w, rank, world, dev, a
        assert w["B"] % world == 0, "the requests must divide over the ranks"
        self.B, self.new, self.cached, self.Hq, self.Hkv = w["B"] // world, w["new"], w["L"], w["Hq"], w["Hkv"]
        self.G = self.Hq // self.Hkv
        self.konly = w["kind"].startswith("konlya")
        self.build(seed=99 + rank)
        self.plan = MQ.build_plan(self.reqs, self.G, self.Hkv, 0, dev)
        self.out = torch.zeros(self.q.shape[0], self.Hq * 128, dtype=torch.bfloat16, device=dev)

    def build(self, seed):
        K, dev, w = self.K, self.dev, self.w
        g = torch.Generator().manual_seed(seed)
        L = self.cached + self.new
        npg = -(-L // P)
        total = self.B * npg + 3
        pool = torch.zeros(total, self.Hkv, (80 if w["nb"] == 2 else 144) * P, dtype=torch.uint8, device=dev)
        bt = torch.randperm(self.B * npg, generator=g).int().view(self.B, npg).contiguous()
        A = torch.randn(self.Hkv, 128, 128, generator=g) / math.sqrt(128)
        CT = (A @ A.transpose(1, 2) + 0.1 * torch.eye(128)).contiguous().to(dev)
        co = torch.ones(self.Hkv, 128, device=dev)
        out_ch = torch.randperm(128, generator=g)[:6]
        for r in range(self.B):
            for t0 in range(0, L, 8192):
                n = min(8192, L - t0)
                kv = torch.randn(n, 2 * self.Hkv, 128, generator=g)
                kv[:, :self.Hkv, out_ch] *= 10
                pos = torch.arange(t0, t0 + n)
                sl = (bt[r].long()[pos // P] * P + pos % P).to(dev)
                K.cb_write(kv.bfloat16().to(dev), sl, CT, co, w["kind"], pool, P)
        self.pool, self.bt = pool, bt.to(dev)
        self.q_host = torch.randn(self.B * self.new, self.Hq, 128, generator=g).bfloat16().pin_memory()
        self.q = self.q_host.to(dev)
        self.out_host = torch.empty(self.B * self.new, self.Hq * 128, dtype=torch.bfloat16).pin_memory()
        self.reqs = [(r, r * self.new, (r + 1) * self.new, L, self.cached) for r in range(self.B)]

    def resident(self, c):
        MQ = self.MQ
        self.q16 = MQ.prep_q(self.q, SCALE * MQ.LOG2E, self.G, idx=self.plan.idx)
        self.opart, self.ml = MQ.attn(self.q16, self.pool, self.bt, self.plan, self.G, 0, konly=self.konly, int2=self.w["nb"] == 2)
        MQ.merge(self.plan, self.opart, self.ml, self.G, out=self.out)

    def kernel(self, c):
        self.MQ.attn(self.q16, self.pool, self.bt, self.plan, self.G, 0, konly=self.konly, int2=self.w["nb"] == 2)

    def e2e(self, c):
        self.q.copy_(self.q_host, non_blocking=True)
        self.resident(c)
        self.out_host.copy_(self.out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def _flops(self, B):
        pairs = B * self.new * (self.cached + (self.new + 1) / 2)     # the causal triangle is counted exactly
        return 4.0 * 128 * self.Hq * pairs

    def job_units(self):
        return self._flops(self.w["B"])

    def launch_units(self):
        return self._flops(self.B)

    def copies(self):
        return int(self.q_host.numel() * 2), int(self.out_host.numel() * 2)

    launches = 3
    kernel_name = "k_mq_tc<4, key-only> (tcgen05)"
    ncopy = 1

    def config(self):
        return {"requests_per_gpu": self.B, "kernel": self.plan.kernel, "rows": self.plan.rows, "tiles": self.plan.ntiles,
                "items": self.plan.nitems, "l2": f"one {self.pool.numel() >> 20} MiB pool (more than the 126 MB L2), read once per step",
                "parallelism": f"requests dealt over {self.world} ranks, no collective" if self.world > 1 else "single gpu",
                "step": "frmq_prep_q + frmq_attn + frmq_merge"}

    def status(self):
        return self.MQ.device_status()


# ---------------------------------------------------------------------------------------------- writers vs the reference's kernels
def writers_race(dev):
    """our writers against the reference's own kernels built for sm_100a (oracle/_ref): a bench leg only.  Per entry and
    T: microseconds per call (CUDA events, 10 calls after 3 warm-up calls), identical arguments and pools, both libraries
    called through their C entries directly (the same host cost per call on both sides)."""
    from flagrot_releaser_b200 import kernels as K
    from flagrot_releaser_b200 import kivi as KV
    res = {}
    PP, I, LL, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    w3 = ROOT / "oracle" / "_ref" / "libflagrot_w3ref.so"
    kr = ROOT / "oracle" / "_ref" / "libflagrot_kivi_ref.so"
    Hkv = 8
    g = torch.Generator().manual_seed(7)
    qs = torch.randn(Hkv, 512, 128, generator=g)
    Cq = (torch.einsum("hnd,hne->hde", qs, qs) / 512).contiguous()
    CT, co = Cq.transpose(1, 2).contiguous().to(dev), (torch.rand(Hkv, 128, generator=g) + 0.5).to(dev)
    mask = (torch.rand(2 * Hkv, 4, generator=g) < 0.5).to(torch.uint8).to(dev)
    hfull = (torch.rand(2 * Hkv, generator=g) < 0.4).to(torch.uint8).to(dev)
    st = lambda: torch.cuda.current_stream().cuda_stream  # noqa: E731
    # slots: a random permutation (every token on its own, the worst case for the value codes, whose words are shared by
    # 8 tokens) and, for the bulk size, the consecutive slots a prefill actually writes (whole pages of one sequence)
    for T, contiguous in ((64, False), (65536, False), (65536, True)):
        kv = torch.randn(T, 2 * Hkv, 128, generator=g)
        kv[:, :Hkv, :6] *= 10
        kv = kv.bfloat16().to(dev)
        npg = T // P + 64
        slots = (torch.arange(T) + 3 * P if contiguous else torch.randperm(npg * P, generator=g)[:T]).to(torch.int64).to(dev)
        pool = torch.zeros(npg, Hkv, 144 * P, dtype=torch.uint8, device=dev)
        row = {"ours": {}, "reference": {}}
        L, sg0 = K.lib(), K.sign_words()
        row["ours"]["fr_cb_write3 konlya"] = timed(lambda i: L.fr_cb_write3(
            kv.data_ptr(), kv.stride(0), slots.data_ptr(), 0, T, Hkv, P, CT.data_ptr(), co.data_ptr(), None, None, sg0, 10,
            pool.data_ptr(), 1, 1, st(), None), 10, 3) * 1e3
        row["ours"]["fr_w3_static_write int4a"] = timed(lambda i: L.fr_w3_static_write(
            kv.data_ptr(), kv.stride(0), slots.data_ptr(), T, Hkv, P, mask.data_ptr(), hfull.data_ptr(), 1, pool.data_ptr(), 0,
            st(), None), 10, 3) * 1e3
        rf = reference_front()
        if w3.exists():
            R = ctypes.CDLL(str(w3))
            R.fr_cb_write3.argtypes = [PP, LL, PP, I, I, I, I, PP, PP, PP, PP, PP, I, PP, I, I, PP, PP]
            R.fr_w3_static_write.argtypes = [PP, LL, PP, I, I, I, PP, PP, I, PP, I, PP, PP]
            sg = K.sign_words()
            if rf is not None:
                # the reference's kernel reads its ranking tables (C1, beta) unconditionally: they come from the reference's own
                # host routine w3_calib(C_q), the persistent-grid sizes from its w3_nchunk, exactly as its cb_write3 wrapper does
                RK = rf[0]
                C1, beta = RK.w3_calib(Cq)
                C1, beta = C1.to(dev), beta.to(dev)
                nk, nv = RK.w3_nchunk(Hkv, RK.W3_CTAS_PER_SM), RK.w3_nchunk(Hkv, RK.W3_VCTAS_PER_SM)
                row["reference"]["fr_cb_write3 konlya"] = timed(lambda i: R.fr_cb_write3(
                    kv.data_ptr(), kv.stride(0), slots.data_ptr(), 0, T, Hkv, P, CT.data_ptr(), co.data_ptr(), C1.data_ptr(),
                    beta.data_ptr(), sg, 10, pool.data_ptr(), nk, nv, st(), None), 10, 3) * 1e3
            row["reference"]["fr_w3_static_write int4a"] = timed(lambda i: R.fr_w3_static_write(
                kv.data_ptr(), kv.stride(0), slots.data_ptr(), T, Hkv, P, mask.data_ptr(), hfull.data_ptr(), 1, pool.data_ptr(), 0,
                st(), None), 10, 3) * 1e3
        # KIVI writers
        D, GRP = 128, 32
        kpool = torch.zeros(npg, Hkv, KV.chunk_bytes(D), dtype=torch.uint8, device=dev)
        cqs = (torch.randn(Hkv, 64, D, generator=g) * 0.3).to(dev)
        lz = torch.full((Hkv, 64), 5.0, device=dev)
        ng = max(T // GRP, 1)
        gp = torch.arange(ng * GRP).view(ng, GRP) % T
        sidx = gp.contiguous().to(dev)
        dslot = slots[gp.reshape(-1)].view(ng, GRP).contiguous()
        LK = KV.lib()
        row["ours"]["kv_v_write"] = timed(lambda i: LK.kv_v_write(kv.data_ptr(), kv.stride(0), T, Hkv, D, slots.data_ptr(),
                                                                  co.data_ptr(), None, kpool.data_ptr(), 0, None, 0, st()), 10, 3) * 1e3
        row["ours"]["kv_k_encode"] = timed(lambda i: LK.kv_k_encode(kv.data_ptr(), kv.stride(0), None, 0, sidx.data_ptr(),
                                                                    dslot.data_ptr(), ng, Hkv, D, cqs.data_ptr(), lz.data_ptr(), 64,
                                                                    SCALE, kpool.data_ptr(), 0, None, 0, st()), 10, 3) * 1e3
        if kr.exists():
            R = ctypes.CDLL(str(kr))
            R.kv_v_write.argtypes = [PP, LL, I, I, I, PP, PP, PP, PP, I, PP, I, PP]
            R.kv_k_encode.argtypes = [PP, LL, PP, LL, PP, PP, I, I, I, PP, PP, I, F, PP, I, PP, I, PP]
            row["reference"]["kv_v_write"] = timed(lambda i: R.kv_v_write(kv.data_ptr(), kv.stride(0), T, Hkv, D, slots.data_ptr(),
                                                                         co.data_ptr(), None, kpool.data_ptr(), 0, None, 0, st()), 10, 3) * 1e3
            row["reference"]["kv_k_encode"] = timed(lambda i: R.kv_k_encode(kv.data_ptr(), kv.stride(0), None, 0, sidx.data_ptr(),
                                                                           dslot.data_ptr(), ng, Hkv, D, cqs.data_ptr(), lz.data_ptr(), 64,
                                                                           SCALE, kpool.data_ptr(), 0, None, 0, st()), 10, 3) * 1e3
        res[f"T={T}" + (" consecutive slots" if contiguous else "")] = row
    return res


# ---------------------------------------------------------------------------------------------- the reference's CPU path
def reference_front():
    """the reference's own Python front ends kernels.py and kivi.py (byte code built by oracle/build_ref.sh), or None"""
    try:
        from oracle import pyref
        if not pyref.available():
            return None
        return pyref.load("kernels"), pyref.load("kivi")
    except Exception:
        return None


def _scale_words(rs, shape):
    """sane scale words (positive fp16 around 2^-8 .. 2^-4) with random flag bits and zero points"""
    return rs.randint(0x1C00, 0x2C00, shape).astype(np.uint16) | (rs.randint(0, 2, shape) << 15).astype(np.uint16)


def cpu_arm(wname, w, steps, warmup):
    """the reference's CPU implementation of the workload's attention on a bounded sample, all host threads.  Returns
    (metric value scaled to the sample's work, seconds per step, cpu_baseline object)."""
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    rs = np.random.RandomState(0)
    ref = reference_front()
    if w["path"] == "decode":
        from oracle import flagrot_oracle as O
        Hkv, Hq, L, nb = w["Hkv"], w["Hq"], min(w["L"], 16384), w["nb"]
        nseq = 2 if w["L"] <= 16384 else 1
        npool = nseq * (L // P)
        pool = rs.randint(0, 256, (npool, Hkv, O.chunk_bytes(nb, P)), dtype=np.uint8)
        off = (128 * P, 144 * P) if nb == 4 else (64 * P, 80 * P)
        pool[:, :, off[0]:off[1]] = _scale_words(rs, (npool, Hkv, 8 * P)).view(np.uint8).reshape(npool, Hkv, 16 * P)
        bt = rs.permutation(npool).reshape(nseq, L // P).astype(np.int32)
        T = w["S"] + w["W"]
        G = Hq // Hkv
        unit_bytes = (nseq * Hkv * (144 if nb == 4 else 80) * (L - w["W"] - w["S"]) + nseq * T * 2 * Hkv * 128 * 2 + nseq * Hq * 128 * 4)
        sample = f"{nseq} of {w['B']} batch rows, all {Hkv} kv heads, context {L}" + ("" if L == w["L"] else f" of {w['L']}")
        if ref is not None:
            RK = ref[0]
            poolt, btt = torch.from_numpy(pool), torch.from_numpy(bt).long()
            q = torch.randn(nseq, Hq, 128).bfloat16().float()
            ring = torch.randn(nseq, T, 2 * Hkv, 128).bfloat16().float()

            def step():
                # kernels.py dequant_cb_pages (the plugin's PyTorch page parser) + fp32 attention over pages [S, L - W) and the BF16 rows
                Kp, Vp = RK.dequant_cb_pages(poolt, P, w["kind"], torch.float32)
                o = torch.empty(nseq, Hq, 128)
                for b in range(nseq):
                    k = torch.cat([Kp[btt[b]].reshape(L, Hkv, 128)[w["S"]:L - w["W"]], ring[b, :, :Hkv]])
                    v = torch.cat([Vp[btt[b]].reshape(L, Hkv, 128)[w["S"]:L - w["W"]], ring[b, :, Hkv:]])
                    s = torch.einsum("hgd,thd->hgt", q[b].view(Hkv, G, 128), k) * SCALE
                    o[b] = torch.einsum("hgt,thd->hgd", torch.softmax(s, -1), v).reshape(Hq, 128)
                return o
            kind, how = "reference", "the reference's PyTorch page parser (kernels.py dequant_cb_pages) + fp32 einsum / softmax attention"
        else:
            from oracle import cpu_decode as C
            qb = (rs.randn(nseq, Hq, 128).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
            ringb = (rs.randn(nseq, T, 2 * Hkv, 128).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
            lens, tl = np.full(nseq, L - w["W"], np.int32), np.full(nseq, T, np.int32)

            def step():
                return C.decode_rows_fp32(qb, pool, bt, lens, SCALE, nb, P, True, list(range(nseq)), tail=ringb, tail_len=tl, kv_start=w["S"])
            kind, how = "port", "fp32 numpy restatement of the reference's page parser + attention (oracle/cpu_decode.py)"
        to_metric = lambda sec: unit_bytes / sec / 1e9  # noqa: E731
    elif w["path"] == "kivi":
        from oracle import kivi_oracle as KO
        Hkv, Hq, L, D = w["Hkv"], w["Hq"], w["L"], 128
        G = Hq // Hkv
        nseq = 1
        npool = nseq * (L // P)
        f8 = bool(w.get("f8", False))
        pool = rs.randint(0, 256, (npool, Hkv, KO.CB8 if f8 else KO.CB), dtype=np.uint8)
        if f8:                                                                 # finite FP8 (scale | flag, min) pairs
            for lo, hi in ((KO.OFF_KM8, KO.OFF_VC8), (KO.OFF_VM8, KO.CB8)):
                m = pool[:, :, lo:hi]
                m[(m & 0x7F) > 0x50] &= 0xCF
        else:
            for lo, hi in ((KO.OFF_KM, KO.OFF_VC), (KO.OFF_VM, KO.OFF_VF)):   # finite fp16 (scale | flag, min) pairs
                pool[:, :, lo:hi] = _scale_words(rs, (npool, Hkv, (hi - lo) // 2)).view(np.uint8).reshape(npool, Hkv, hi - lo)
        bt = rs.permutation(npool).reshape(nseq, L // P).astype(np.int32)
        T = w["S"] + w["W"]
        unit_bytes = nseq * Hkv * (80 if f8 else 97) * (L - w["W"] - w["S"]) + nseq * T * 2 * Hkv * D * 2 + nseq * Hq * D * 4
        sample = f"{nseq} of {w['B']} batch rows, all {Hkv} kv heads, context {L}"
        if ref is not None:
            RKV = ref[1]
            poolt, btt = torch.from_numpy(pool), torch.from_numpy(bt).long()
            q = torch.randn(nseq, Hq, D).bfloat16().float()
            ring = torch.randn(nseq, T, 2 * Hkv, D).bfloat16().float()

            def step():
                o = torch.empty(nseq, Hq, D)
                for b in range(nseq):
                    k, v = RKV.dequant_groups(poolt[btt[b]], D, f8=f8)        # [L, Hkv, D] in the original basis
                    k = torch.cat([k.float()[w["S"]:L - w["W"]], ring[b, :, :Hkv]])
                    v = torch.cat([v.float()[w["S"]:L - w["W"]], ring[b, :, Hkv:]])
                    s = torch.einsum("hgd,thd->hgt", q[b].view(Hkv, G, D), k) * SCALE
                    o[b] = torch.einsum("hgt,thd->hgd", torch.softmax(s, -1), v).reshape(Hq, D)
                return o
            kind, how = "reference", "the reference's PyTorch page parser (kivi.py dequant_groups) + fp32 einsum / softmax attention"
        else:
            qb = (rs.randn(nseq, Hq, D).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
            ringb = (rs.randn(nseq, T, 2 * Hkv, D).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)

            def step():
                return KO.decode_reference(qb, pool, bt, np.full(nseq, L - w["W"], np.int32), SCALE, w["S"], G, ring=ringb,
                                           tail_len=np.full(nseq, T, np.int32), tail_idx=np.arange(nseq), f8=f8)
            kind, how = "port", "float64 numpy restatement of the reference's page parser + attention (oracle/kivi_oracle.py)"
        to_metric = lambda sec: unit_bytes / sec / 1e9  # noqa: E731
    else:   # prefill: one request, 64 of its 512 new tokens, all heads, over the cached keys
        from oracle import flagrot_oracle as O
        Hkv, Hq, L, nq = w["Hkv"], w["Hq"], w["L"], 64
        G = Hq // Hkv
        npool = (L + w["new"]) // P
        pool = rs.randint(0, 256, (npool, Hkv, O.chunk_bytes(4, P)), dtype=np.uint8)
        pool[:, :, 128 * P:144 * P] = _scale_words(rs, (npool, Hkv, 8 * P)).view(np.uint8).reshape(npool, Hkv, 16 * P)
        flops = 4.0 * 128 * Hq * nq * (L + (nq + 1) / 2)
        sample = f"1 of {w['B']} requests, {nq} of {w['new']} new tokens, all {Hq} q heads, {L} cached keys"
        q = torch.randn(nq, Hq, 128).bfloat16().float()
        if ref is not None:
            RK = ref[0]
            poolt = torch.from_numpy(pool)

            def step():
                Kp, Vp = RK.dequant_cb_pages(poolt, P, "konlya", torch.float32)
                k, v = Kp.reshape(-1, Hkv, 128)[:L + nq], Vp.reshape(-1, Hkv, 128)[:L + nq]
                s = torch.einsum("qhgd,thd->hgqt", q.view(nq, Hkv, G, 128), k) * SCALE
                vis = torch.arange(L + nq)[None, :] <= (L + torch.arange(nq))[:, None]
                s = s.masked_fill(~vis[None, None], float("-inf"))
                return torch.einsum("hgqt,thd->qhgd", torch.softmax(s, -1), v)
            kind, how = "reference", "the reference's PyTorch page parser (kernels.py dequant_cb_pages) + masked fp32 attention"
        else:
            from oracle import mq_oracle as MO
            bt_row = np.arange(npool, dtype=np.int32)

            def step():
                kk, vv = MO.request_cache(pool, bt_row, L + nq, 4, True)
                return MO.attention(q.numpy(), kk, vv, L + np.arange(nq), 0, SCALE)
            kind, how = "port", "float64 numpy restatement (oracle/mq_oracle.py)"
        to_metric = lambda sec: flops / sec / 1e12  # noqa: E731
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        step()
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    if not times:
        return None, None, None
    sec = float(np.mean(times))
    val = to_metric(sec)
    unit = "TFLOP/s" if w["path"] == "prefill" else "GB/s"
    return val, sec, dict(value=val, unit=unit, cores=cores, kind=kind, sample=f"{sample}; {how}, {cores} threads")


# ---------------------------------------------------------------------------------------------- main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS))
    ap.add_argument("--nsplit", type=int, default=0, help="force the split count (0: the planner's choice)")
    ap.add_argument("--ncopy", type=int, default=0, help="pool copies cycled (0: enough to exceed L2 several times)")
    ap.add_argument("--cpu-steps", type=int, default=3, help="steps of the cpu_baseline leg (0: skip it)")
    ap.add_argument("--sustain-s", type=float, default=0.5, help="seconds of untimed load before the timed steps, and the least "
                                                                  "length of the kernel-only loop behind the roofline figure")
    ap.add_argument("--no-step-graph", action="store_true", help="resident step: separate launches from Python instead of a CUDA graph")
    ap.add_argument("--batch", type=int, default=0, help="override the workload's batch (requests for cfg5a): smaller cases for "
                                                         "profiler captures; the line's config names the batch actually run")
    ap.add_argument("--kvseq-exchange", default="p2p", choices=["p2p", "nccl"],
                    help="kv-sequence shard: partial rows exchanged and merged by one kernel over peer memory (fr_xchg_merge) or "
                         "by an NCCL all-gather + fr_merge_partials")
    ap.add_argument("--e2e-launch", default="calls", choices=["calls", "graph"],
                    help="e2e leg of the decode workloads: copies issued from Python around the step graph, or copies + step as one "
                         "graph launch (graphs.HostStep)")
    ap.add_argument("--race", action="store_true", help="also time the reference's own sm_100a-capable kernel on the same pools (cfg4)")
    a = ap.parse_args()
    w = dict(WORKLOADS[a.workload])
    if a.batch > 0 and "B" in w:
        w["name"] += f" [batch overridden: {a.batch} instead of {w['B']}]"
        w["B"] = a.batch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    metric = "mq_prefill_attention_tflops" if w["path"] == "prefill" else "decode_attention_kv_gbps"
    unit = "TFLOP/s" if w["path"] == "prefill" else "GB/s"

    if a.impl == "reference":
        if rank != 0:
            return
        if w["path"] == "writers":
            print(json.dumps({"impl": "reference", "unavailable": "the writers workload races GPU kernels; it has no CPU arm"}))
            return
        steps, warm = max(1, a.steps), max(0, a.warmup)
        val, sec, cb = cpu_arm(a.workload, w, steps, warm)
        print(json.dumps({"impl": "reference", "metric": metric, "value": val, "unit": unit, "n_gpus": a.gpus, "steps": steps,
                          "warmup": warm, "ms_per_step": sec * 1e3, "higher_is_better": True,
                          "scaling": "weak" if w["shard"] == "replica" else "strong", "vs_baseline": None,
                          "dtype": "f32", "data": "synthetic", "config": {"workload": w["name"]}, "cpu_baseline": cb, "gpu_launches": 0,
                          "e2e": {"value": val, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return

    a.warmup = max(a.warmup, 3)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        torch.cuda.set_device(local)
        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local))
        dist = dist_mod
    else:
        local = 0
        torch.cuda.set_device(0)
    dev = torch.device("cuda", local)

    if w["path"] == "writers":
        res = writers_race(dev)
        if rank == 0:
            print(json.dumps({"metric": "writer_us_per_call", "unit": "us", "config": {"workload": w["name"]}, "data": "synthetic",
                              "writers": res}))
        return

    wl = {"decode": DecodeWorkload, "kivi": KiviWorkload, "prefill": PrefillWorkload}[w["path"]](w, rank, world, dev, a)
    if getattr(wl, "kvseq", False):
        wl.dist = dist
    nc = wl.ncopy
    # the resident step replayed as one CUDA graph per pool copy: the same launches, one call from Python, so that the figure
    # does not depend on how fast the host thread of a rank issues launches (prefill allocates its partials per step: eager)
    graphs = None
    if not a.no_step_graph and w["path"] != "prefill":
        try:
            for c in range(nc):
                wl.resident(c)
            graphs = [graph_of(lambda c=c: wl.resident(c)) for c in range(nc)]
        except Exception as e:                              # e.g. a collective that cannot be captured here
            if rank == 0:
                print(f"bench: step graph unavailable ({type(e).__name__}: {e}); separate launches", file=sys.stderr)
            graphs = None
            torch.cuda.synchronize()
    wl.graphs = graphs
    run_res = (lambda i: wl.graphs[i % nc].replay()) if graphs is not None else (lambda i: wl.resident(i % nc))
    use_graph = graphs is not None
    del graphs
    sampler = ClockSampler(local).start() if rank == 0 else None
    ms = timed(run_res, a.steps, a.warmup, dist, a.sustain_s)
    clocks = sampler.stop() if rank == 0 else None
    ms_e2e = timed(lambda i: wl.e2e(i % nc), a.steps, a.warmup, dist, min(a.sustain_s, 0.2))
    if dist is not None:
        dist.barrier()
    wl.resident(0)                                          # (prefill: the kernel-only loop reuses the staged q)
    ms_burst = timed(lambda i: wl.kernel(i % nc), a.steps, a.warmup, None)
    ms_k, n_k, clk_k = sustained(lambda i: wl.kernel(i % nc), ms_burst, a.sustain_s, local)
    ms_long, n_long, _ = sustained(run_res, ms, a.sustain_s, local) if dist is None else (None, 0, None)
    status = wl.status()
    race = wl.race_reference() if (a.race and hasattr(wl, "race_reference")) else None

    def leave():
        """captured graphs that hold collectives go before the process group does; a rank that still cannot tear its
        communicator down must not keep the job (and the GPUs) waiting: the results are out, so it exits at once"""
        if dist is None:
            return
        wl.graphs = None
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)
    if rank != 0:
        leave()
        return
    hbm, tf_burst, tf_sus, which = peaks()
    scale = 1e12 if wl.bound == "tensor" else 1e9
    peak = tf_sus if wl.bound == "tensor" else hbm
    ach = wl.launch_units() / (ms_k * 1e-3) / scale
    traffic = None
    tf = ROOT / "profiles" / "traffic.json"
    if tf.exists():
        traffic = json.loads(tf.read_text()).get(a.workload)
    h2d, d2h = wl.copies()
    cfg = {"workload": w["name"], **wl.config(), "device_status": status,
           "timing": f"{a.warmup} warm-up steps + {a.sustain_s} s of the same step untimed, then {a.steps} timed steps (CUDA events)"}
    line = {
        "metric": metric, "value": wl.job_units() / (ms * 1e-3) / scale, "unit": unit, "n_gpus": world, "steps": a.steps,
        "warmup": a.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak" if w["shard"] == "replica" else "strong",
        "vs_baseline": None, "dtype": "f16" if wl.bound == "tensor" else "u8", "data": "synthetic", "config": cfg,
        "e2e": {"value": wl.job_units() / (ms_e2e * 1e-3) / scale, "unit": unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": ms_e2e, "launch": ("copies in, step and copy back as one CUDA graph" if getattr(wl, "hsteps", None)
                                                   else "copies from Python, the step as one CUDA graph" if use_graph
                                                   else "separate launches from Python")},
        "gpu_launches": wl.launches * a.steps,
        "roofline": {"bound": wl.bound, "achieved": ach, "peak": peak, "unit": unit, "frac": ach / peak, "traffic": traffic,
                     "kernel": wl.kernel_name, "peak_source": which + (" (sustained dense bf16)" if wl.bound == "tensor" else " (copy)"),
                     "us_per_launch": ms_k * 1e3, "launches_timed": n_k, "algorithmic_units": wl.launch_units(),
                     "us_per_launch_burst": ms_burst * 1e3, "clocks": clk_k,
                     "us_x_sm_mhz": (ms_k * 1e3 * clk_k["sm_mhz"]) if clk_k and clk_k.get("sm_mhz") else None,
                     **({"frac_of_8000": ach / 8000.0} if wl.bound == "hbm" else {"frac_of_burst_peak": ach / tf_burst})},
        "clocks": clocks,
    }
    if ms_long is not None:
        line["sustained"] = {"ms_per_step": ms_long, "steps": n_long, "value": wl.job_units() / (ms_long * 1e-3) / scale}
    if race is not None:
        line["reference_kernel"] = race
    if world == 1 and a.cpu_steps > 0:
        _, _, cb = cpu_arm(a.workload, w, a.cpu_steps, 1)
        line["cpu_baseline"] = cb
    print(json.dumps(line))
    leave()


if __name__ == "__main__":
    main()
