"""Headline benchmark: FlagRot paged decode over INT4 (konlya) pages on the Llama-3.1-8B-shaped batch-64 x 4K workload.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg2|cfg3]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A step = one pass of the hot path over one batch: the dynamic writer appends one token per sequence (fr_cb_write, T = B)
and the paged decode attention reads every sequence's cache (fr_cb_attn), with the 4 sink + 128 window tokens in BF16.
The resident step is captured once per pool copy and replayed as a CUDA graph (--no-step-graph: two launches from Python).
metric: decode-attention KV GB/s = algorithmic bytes of the decode read (pages [S, L - W) * 144 B per (token, kv head) +
BF16 window rows + q / out) divided by the step time.  `value` has every input resident in HBM; `e2e` measures the same
step through the C-ABI front end with this step's q / new kv / slots copied from pinned host memory and the output
copied back, inside the timed region (the KV cache itself is the path's state and lives in HBM, as in the plugin).
Multi-GPU: the batch shards across ranks with no data-path collective (weak scaling: every rank runs the same per-GPU
batch on its own pool); time = max over ranks.
The reference arm (--impl reference) times the reference's CPU path for this workload (fp32 dequantise + attention over
the same pages, oracle/cpu_decode.py, numpy with all host threads) on a bounded sample of the batch.
"""
from __future__ import annotations

import argparse
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

WORKLOADS = {
    # Llama-3.1-8B-shaped INT4 FlagRot decode: 32 q / 8 kv heads, d 128, batch 64, context 4096, 4 sinks + 128 window BF16
    "cfg2": dict(kind="konlya", nb=4, B=64, L=4096, Hq=32, Hkv=8, S=4, W=128, center=False,
                 name="llama-3.1-8b-shaped int4 konlya decode, batch 64 x ctx 4096, page 16, s4w128"),
    # Qwen3-8B-shaped INT2 FlagRot decode, batch 256 x 8192 (per-GPU batch = 256 / n when sharded)
    "cfg3": dict(kind="konlya2", nb=2, B=256, L=8192, Hq=32, Hkv=8, S=4, W=128, center=True,
                 name="qwen3-8b-shaped int2 konlya2 decode, batch 256 x ctx 8192, page 16, s4w128, centred keys"),
    # one very long sequence, INT4 konlya, context 131072: the KV sequence is sharded over the ranks, every rank emits
    # (o, m, l) rows (fr_attn_partial), an NCCL all-gather of 130 floats per (row, head) and the LSE merge finish the step
    "cfg5b": dict(kind="konlya", nb=4, B=1, L=131072, Hq=32, Hkv=8, S=4, W=128, center=False, shard="kvseq",
                  name="int4 konlya decode, batch 1 x ctx 131072, page 16, s4w128, KV-sequence sharded"),
}


def algorithmic_bytes(w, B=None):
    B = w["B"] if B is None else B
    cell = 144 if w["nb"] == 4 else 80
    pages = B * w["Hkv"] * cell * (w["L"] - w["W"] - w["S"])
    tail = B * (w["S"] + w["W"]) * 2 * w["Hkv"] * 128 * 2
    qo = B * w["Hq"] * 128 * 2 * 2
    return pages + tail + qo


def peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        return float(json.loads(f.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True).start()
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------------- workload state
def make_state(w, B, dev, seed, ncopy, rank=0, world=1):
    """synthetic inputs of the named shape and the quantised caches (written by the library's own dynamic writer, which
    the parity tests hold bit-exact).  ncopy distinct pools (distinct random page tables over distinct memory) are cycled
    so that no page is L2-resident between steps."""
    from flagrot_releaser_b200 import kernels as K
    g = torch.Generator().manual_seed(seed)
    Hkv, Hq, L = w["Hkv"], w["Hq"], w["L"]
    kvseq = w.get("shard") == "kvseq"
    if kvseq:                                   # this rank's slice of the page tokens [0, L - W); window rows stay BF16
        L = kvseq_local_len(w["L"], w["W"], world)
    npages_seq = L // P
    npool = B * npages_seq + 7
    qs = torch.randn(Hkv, 512, 128, generator=g) * (torch.rand(Hkv, 1, 128, generator=g) + 0.5).sqrt()
    Cq = (torch.einsum("hnd,hne->hde", qs, qs) / 512).contiguous()
    co = torch.rand(Hkv, 128, generator=g) + 0.5
    CT = Cq.transpose(1, 2).contiguous().to(dev)
    cod = co.to(dev)
    out_ch = torch.stack([torch.randperm(128, generator=g)[:6] for _ in range(Hkv)])          # 5 % of channels x10
    kmu = None
    offs = None
    if w["center"]:
        offs = torch.randn(Hkv, 128, generator=g) * math.sqrt(2.0)
        kmu = offs.float().contiguous().to(dev)
    chunk_b = K.cb_chunk_bytes(w["kind"], P)
    pools, bts = [], []
    rows_per = 64 * 1024
    for c in range(ncopy):
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
            K.cb_write(kv.bfloat16().to(dev), slots[r0:r0 + n].to(dev), CT, cod, w["kind"], pool, P, kmu=kmu)
        torch.cuda.synchronize()
        pools.append(pool)
        bts.append(bt.to(dev))
    T = w["S"] + w["W"]
    ring = torch.randn(B, T, 2 * Hkv, 128, generator=g).bfloat16().to(dev)
    st = dict(K=K, w=w, B=B, CT=CT, co=cod, kmu=kmu, pools=pools, bts=bts, ring=ring,
              tail_len=torch.full((B,), T, dtype=torch.int32, device=dev),
              seq=torch.full((B,), L - w["W"], dtype=torch.int32, device=dev),
              q_host=torch.randn(B, Hq, 128, generator=g).bfloat16().pin_memory(),
              kv_host=torch.randn(B, 2 * Hkv, 128, generator=g).bfloat16().pin_memory(),
              out_host=torch.empty(B, Hq * 128, dtype=torch.bfloat16).pin_memory(),
              out=torch.empty(B, Hq * 128, dtype=torch.bfloat16, device=dev))
    st["q"] = st["q_host"].to(dev)
    st["kv"] = st["kv_host"].to(dev)
    st["Lloc"], st["rank"], st["world"] = L, rank, world
    if kvseq:
        st["part"] = torch.zeros(B, Hq, 130, dtype=torch.float32, device=dev)
        st["parts"] = torch.zeros(world, B, Hq, 130, dtype=torch.float32, device=dev)
    # the appended token of every sequence goes to position L - W - 1 of its row (a scattered slot per sequence)
    st["slots"] = [(bt.long()[:, (L - w["W"] - 1) // P] * P + (L - w["W"] - 1) % P).contiguous() for bt in bts]
    st["slots_host"] = [s.cpu().pin_memory() for s in st["slots"]]
    return st


def plan(st, nsplit):
    K, w = st["K"], st["w"]
    ns, ch = K.plan_cb(st["B"], st["Lloc"] - w["W"], w["Hkv"], P, w["kind"], nsplit)
    st["plan"] = (ns, ch)
    st["ws"] = K.Workspace(st["B"], w["Hkv"], st["B"] * w["Hkv"] * (ns + 1), st["pools"][0].device)


def step(st, i, e2e=False):
    """one pass of the hot path on pool copy i; returns nothing (asynchronous unless e2e reads the result back).
    e2e: the step from pinned host buffers and back, replayed as one CUDA graph per pool copy (captured at first use)."""
    K, w = st["K"], st["w"]
    c = i % len(st["pools"])
    if e2e and st.get("graphs", False):
        gs = st.setdefault("_graphs", {})
        if c not in gs:
            from flagrot_releaser_b200.graphs import HostStep
            step(st, c, e2e=False)                                      # first calls set kernel attributes
            gs[c] = HostStep([(st["q"], st["q_host"]), (st["kv"], st["kv_host"]), (st["slots"][c], st["slots_host"][c])],
                             lambda: step(st, c, e2e=False), [(st["out_host"], st["out"])])
        gs[c].run()
        return
    pool, bt = st["pools"][c], st["bts"][c]
    ns, ch = st["plan"]
    if e2e:
        st["q"].copy_(st["q_host"], non_blocking=True)
        st["kv"].copy_(st["kv_host"], non_blocking=True)
        st["slots"][c].copy_(st["slots_host"][c], non_blocking=True)
    K.cb_write(st["kv"], st["slots"][c], st["CT"], st["co"], w["kind"], pool, P, kmu=st["kmu"])
    ring = st["ring"]
    K.cb_attn(st["q"], pool, bt, st["seq"], st["out"], ns, ch, st["ws"], LOG2E / math.sqrt(128), w["kind"], tail=ring,
              tail_len=st["tail_len"], tail_idx=None, tail_bs=ring.stride(0), tail_ts=ring.stride(1), page=P, kv_start=w["S"])
    if e2e:
        st["out_host"].copy_(st["out"], non_blocking=True)
        torch.cuda.current_stream().synchronize()


def step_kvseq(st, i, e2e=False, dist=None):
    """KV-sequence sharded step: the last rank appends the new token, every rank attends over its slice (rank 0 also over
    the BF16 sink / window rows), partial rows are all-gathered (NCCL) and merged."""
    K, w = st["K"], st["w"]
    c = i % len(st["pools"])
    pool, bt = st["pools"][c], st["bts"][c]
    ns, ch = st["plan"]
    first, last = st["rank"] == 0, st["rank"] == st["world"] - 1
    if e2e:
        st["q"].copy_(st["q_host"], non_blocking=True)
        if last:
            st["kv"].copy_(st["kv_host"], non_blocking=True)
            st["slots"][c].copy_(st["slots_host"][c], non_blocking=True)
    if last:
        K.cb_write(st["kv"], st["slots"][c], st["CT"], st["co"], w["kind"], pool, P, kmu=st["kmu"])
    ring = st["ring"]
    tkw = dict(tail=ring, tail_len=st["tail_len"], tail_idx=None, tail_bs=ring.stride(0), tail_ts=ring.stride(1)) if first else {}
    K.attn_partial(st["q"], pool, bt, st["seq"], st["part"], ns, ch, st["ws"], LOG2E / math.sqrt(128), w["kind"], page=P,
                   kv_start=w["S"] if first else 0, **tkw)
    if dist is not None:
        dist.all_gather_into_tensor(st["parts"].view(-1, *st["part"].shape[1:]), st["part"])   # concatenated along dim 0
        K.merge_partials_into(st["parts"], st["out"])
    else:
        K.merge_partials_into(st["part"][None], st["out"])
    if e2e:
        st["out_host"].copy_(st["out"], non_blocking=True)
        torch.cuda.current_stream().synchronize()


def decode_only(st, i):
    K, w = st["K"], st["w"]
    c = i % len(st["pools"])
    ns, ch = st["plan"]
    ring = st["ring"]
    K.cb_attn(st["q"], st["pools"][c], st["bts"][c], st["seq"], st["out"], ns, ch, st["ws"], LOG2E / math.sqrt(128), w["kind"],
              tail=ring, tail_len=st["tail_len"], tail_idx=None, tail_bs=ring.stride(0), tail_ts=ring.stride(1), page=P,
              kv_start=w["S"])


def kvseq_local_len(L, W, world):
    """context length of one rank when the page tokens [0, L - W) of a sequence are split evenly over `world` ranks (every
    rank keeps the W window rows in its count, as the single-GPU convention does)."""
    return (L - W) // world + W


def max_over_ranks(ms, dist, device):
    """the slowest rank's time (all-reduce MAX), identical on every rank"""
    if dist is None:
        return ms
    t = torch.tensor([ms], dtype=torch.float32, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def timed(fn, steps, warmup, dist=None):
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn(warmup + i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if dist is not None:
        ms = max_over_ranks(ms, dist, "cuda")
        dist.barrier()
    return ms / steps


# ---------------------------------------------------------------------------------------------- CPU arm
def cpu_arm(w, steps, warmup, sample_rows=2):
    """the reference's CPU path on a bounded sample: `sample_rows` rows of the batch, all kv heads, full context."""
    from oracle import cpu_decode as C
    from oracle import flagrot_oracle as O
    rs = np.random.RandomState(0)
    Hkv, Hq, L = w["Hkv"], w["Hq"], w["L"]
    nseq = sample_rows
    npool = nseq * (L // P)
    pool = rs.randint(0, 256, (npool, Hkv, O.chunk_bytes(w["nb"], P)), dtype=np.uint8)
    # sane scale words (positive fp16 around 2^-8 .. 2^-4) with random flag bits and zero points, random codes
    for off in ((128 * P, 144 * P) if w["nb"] == 4 else (64 * P, 80 * P)),:
        words = (rs.randint(0x1C00, 0x2C00, (npool, Hkv, 8 * P)).astype(np.uint16) | (rs.randint(0, 2, (npool, Hkv, 8 * P)) << 15).astype(np.uint16))
        pool[:, :, off[0]:off[1]] = words.view(np.uint8).reshape(npool, Hkv, 16 * P)
    bt = rs.permutation(npool).reshape(nseq, L // P).astype(np.int32)
    q = (rs.randn(nseq, Hq, 128).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
    T = w["S"] + w["W"]
    ring = (rs.randn(nseq, T, 2 * Hkv, 128).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
    lens = np.full(nseq, L - w["W"], np.int32)
    tl = np.full(nseq, T, np.int32)
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        C.decode_rows_fp32(q, pool, bt, lens, 1 / math.sqrt(128), w["nb"], P, True, list(range(nseq)), tail=ring, tail_len=tl,
                           kv_start=w["S"])
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    if not times:                                  # --cpu-steps 0: no CPU leg
        return None, None, None
    sec = float(np.mean(times))
    gbs = algorithmic_bytes(w, nseq) / sec / 1e9
    cores = os.cpu_count() or 1
    return gbs, sec, dict(value=gbs, unit="GB/s", cores=cores, kind="port",
                          sample=f"{nseq} of {w['B']} batch rows, all {Hkv} kv heads, full context {L}; fp32 numpy "
                                 f"dequantise + attention, {cores} threads")


# ---------------------------------------------------------------------------------------------- main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--workload", default="cfg2")
    ap.add_argument("--nsplit", type=int, default=0, help="force the split count (0: the planner's choice)")
    ap.add_argument("--ncopy", type=int, default=3)
    ap.add_argument("--cpu-steps", type=int, default=3)
    ap.add_argument("--no-step-graph", action="store_true", help="resident step: separate launches from Python instead of a CUDA graph")
    ap.add_argument("--graph", action="store_true", help="e2e: one CUDA graph per step (flagrot_releaser_b200.graphs.HostStep) "
                                                         "instead of separate launches from Python; measured equal within noise")
    a = ap.parse_args()
    a.warmup = max(a.warmup, 3) if a.impl == "ours" else a.warmup
    w = WORKLOADS[a.workload]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if a.impl == "reference":
        if rank != 0:
            return
        gbs, sec, cb = cpu_arm(w, max(1, min(a.steps, 5)), min(a.warmup, 1))
        print(json.dumps({"impl": "reference", "metric": "decode_attention_kv_gbps", "value": gbs, "unit": "GB/s",
                          "n_gpus": a.gpus, "steps": max(1, min(a.steps, 5)), "warmup": min(a.warmup, 1),
                          "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                          "dtype": "u8", "data": "synthetic", "config": {"workload": w["name"]},
                          "cpu_baseline": cb, "gpu_launches": 0,
                          "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return

    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        torch.cuda.set_device(local)
        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local))
        dist = dist_mod
    else:
        torch.cuda.set_device(0)
    dev = torch.device("cuda", local if world > 1 else 0)
    B = w["B"]                                          # weak scaling: every rank runs the full per-GPU batch
    kvseq = w.get("shard") == "kvseq"
    if kvseq:                                           # strong scaling: the pools shrink with the rank count; keep the cycled set > L2
        local = B * kvseq_local_len(w["L"], w["W"], world) * w["Hkv"] * (144 if w["nb"] == 4 else 80)
        a.ncopy = max(a.ncopy, -(-(192 << 20) // local))
    st = make_state(w, B, dev, seed=1234 + rank, ncopy=a.ncopy, rank=rank, world=world)
    plan(st, a.nsplit or None)
    st["graphs"] = a.graph
    sampler = ClockSampler(local if world > 1 else 0)
    if rank == 0:
        sampler.start()
    if kvseq:
        ms = timed(lambda i: step_kvseq(st, i, dist=dist), a.steps, a.warmup, dist)
        ms_e2e = timed(lambda i: step_kvseq(st, i, e2e=True, dist=dist), a.steps, a.warmup, dist)
    else:
        if a.no_step_graph:
            ms = timed(lambda i: step(st, i), a.steps, a.warmup, dist)
        else:
            # the resident step (append + decode) is replayed as one CUDA graph per pool copy: the same two kernels, one launch
            # from Python, so that the figure does not depend on how fast the host thread of a rank issues launches
            vg = []
            for c in range(len(st["pools"])):
                step(st, c)                                             # first calls set kernel attributes
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    step(st, c)
                vg.append(g)
            ms = timed(lambda i: vg[i % len(vg)].replay(), a.steps, a.warmup, dist)
        ms_e2e = timed(lambda i: step(st, i, e2e=True), a.steps, a.warmup, dist)
    ms_dec = timed(lambda i: decode_only(st, i), a.steps, a.warmup, None)
    clocks = sampler.stop() if rank == 0 else None
    status = st["K"].device_status()
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return
    nbytes = algorithmic_bytes(w)
    peak, which = peaks()
    nloc = nbytes
    if kvseq:                                           # bytes of this rank's decode launch (rank 0 carries the BF16 rows)
        cell = 144 if w["nb"] == 4 else 80
        nloc = nbytes - B * w["Hkv"] * cell * (w["L"] - w["W"] - w["S"]) + B * w["Hkv"] * cell * (st["Lloc"] - w["W"] - w["S"])
    ach = nloc / (ms_dec * 1e-3) / 1e9
    nwork = nbytes if kvseq else world * nbytes          # strong scaling: the job is one sequence
    traffic = None
    tf = ROOT / "profiles" / "traffic.json"
    if tf.exists():
        traffic = json.loads(tf.read_text()).get(a.workload)
    line = {
        "metric": "decode_attention_kv_gbps", "value": nwork / (ms * 1e-3) / 1e9, "unit": "GB/s", "n_gpus": world,
        "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong" if kvseq else "weak",
        "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": {"workload": w["name"], "batch_per_gpu": B, "nsplit": st["plan"][0], "chunk": st["plan"][1],
                   "l2": f"{a.ncopy} distinct {st['pools'][0].numel() >> 20} MiB pools cycled "
                         f"({a.ncopy * st['pools'][0].numel() >> 20} MiB in all, more than the 126 MB L2)",
                   "parallelism": ((f"kv-sequence sharded x{world}, NCCL all-gather of (o, m, l) rows + LSE merge" if kvseq
                                    else f"batch-sharded x{world}") if world > 1 else "single gpu"),
                   "step": ("fr_cb_write (last rank) + fr_attn_partial + all-gather + merge" if kvseq
                            else "fr_cb_write (T = batch) + fr_cb_attn" + ("" if a.no_step_graph else ", replayed as one CUDA graph")),
                   "device_status": status},
        "e2e": {"value": nwork / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s",
                "h2d_bytes_per_step": int(st["q_host"].numel() * 2 + st["kv_host"].numel() * 2 + B * 8),
                "d2h_bytes_per_step": int(st["out_host"].numel() * 2), "ms_per_step": ms_e2e,
                "launch": ("separate launches from Python" if (not a.graph or kvseq) else
                           "one CUDA graph per step: 3 host-to-device copies, writer, decode, copy back")},
        "gpu_launches": (3 if kvseq else 2) * a.steps,   # append (keys + value rows, one launch), decode [, merge]
        "roofline": {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "traffic": traffic,
                     "kernel": "k_decode<4, key-only>" if w["nb"] == 4 else "k_decode<2, key-only>", "peak_source": which,
                     "us_per_launch": ms_dec * 1e3, "algorithmic_bytes": nloc, "frac_of_8000": ach / 8000.0},
        "clocks": clocks,
    }
    if world == 1:
        _, _, cb = cpu_arm(w, a.cpu_steps, 1)
        line["cpu_baseline"] = cb
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
