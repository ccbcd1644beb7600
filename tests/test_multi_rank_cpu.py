"""Host logic of the multi-GPU paths, run as gloo ranks on the CPU (world sizes 2 and 4): the max-over-ranks timing
reduction of bench.py; the KV-sequence shard -> all-gather -> LSE merge step (kernels.merge_partials on rows each rank
computed for its own slice of the sequence); the KV-head (tensor-parallel) shard, where every rank owns Hkv / n kv heads,
their q heads and the matching calibration rows and no exchange is needed (an all-gather of the head slices only verifies
it); and the batch shard (rows [r B / n, (r + 1) B / n) per rank) - each against attention computed on the whole problem."""
from __future__ import annotations

import math
import os
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _partial(q, k, v, scale):
    """normalised rows + (m in log2 units, l) of attention over one slice: [B, Hq, 130]; k / v [B, T, Hkv, 128], GQA"""
    G = q.shape[1] // k.shape[2]
    kk, vv = k.repeat_interleave(G, 2), v.repeat_interleave(G, 2)
    s = torch.einsum("bhd,bkhd->bhk", q, kk) * scale * 1.4426950408889634
    m = s.amax(-1)
    p = torch.exp2(s - m[..., None])
    l = p.sum(-1)
    o = torch.einsum("bhk,bkhd->bhd", p, vv) / l[..., None]
    return torch.cat([o, m[..., None], l[..., None]], -1)


def _worker(rank, world, port, out):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import bench
    from flagrot_releaser_b200 import kernels as K
    # 1. timing reduction
    slow = bench.max_over_ranks(float(rank + 1), dist, "cpu")
    # 2. KV-sequence shard of one long sequence
    g = torch.Generator().manual_seed(7)
    B, Hq, Hkv, L, W = 4, 8, 4, 4096 + 128, 128
    scale = 1 / math.sqrt(128)
    q = torch.randn(B, Hq, 128, generator=g)
    k = torch.randn(B, L - W, Hkv, 128, generator=g)
    v = torch.randn(B, L - W, Hkv, 128, generator=g)
    full = _partial(q, k, v, scale)[..., :128]
    n = bench.kvseq_local_len(L, W, world) - W
    part = _partial(q, k[:, rank * n:(rank + 1) * n], v[:, rank * n:(rank + 1) * n], scale).contiguous()
    parts = torch.empty(world, B, Hq, 130)
    dist.all_gather_into_tensor(parts.view(world * B, Hq, 130), part)      # concatenation along dim 0
    err_seq = float((K.merge_partials(parts) - full).abs().max())
    # 3. KV-head shard: this rank's kv heads [rank Hkv / n, ...), the q heads of those kv heads (contiguous: q head = kv
    #    head * G + g) and, for a writer, the calibration rows of the same kv heads
    hk = Hkv // world
    G = Hq // Hkv
    hs = slice(rank * hk, (rank + 1) * hk)
    qs_ = slice(rank * hk * G, (rank + 1) * hk * G)
    mine = _partial(q[:, qs_], k[:, :, hs], v[:, :, hs], scale)[..., :128].contiguous()        # [B, Hq / n, 128]
    heads = torch.empty(world, B, hk * G, 128)
    dist.all_gather_into_tensor(heads.view(world * B, hk * G, 128), mine)
    err_head = float((heads.permute(1, 0, 2, 3).reshape(B, Hq, 128) - full).abs().max())
    calib = torch.arange(Hkv * 3.0).view(Hkv, 3)                            # stands for C_q^T / c_o / kmu rows [Hkv, ...]
    calib_ok = bool((calib[hs][:, 0] == torch.arange(rank * hk, (rank + 1) * hk) * 3.0).all())
    # 4. batch shard
    bs = slice(rank * B // world, (rank + 1) * B // world)
    rows = _partial(q[bs], k[bs], v[bs], scale)[..., :128].contiguous()
    allrows = torch.empty(B, Hq, 128)
    dist.all_gather_into_tensor(allrows, rows)
    err_batch = float((allrows - full).abs().max())
    out[rank] = (slow, err_seq, n, err_head, calib_ok, err_batch)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_ranks_gloo(world):
    with mp.Manager() as mgr:
        out = mgr.dict()
        port = 29500 + (os.getpid() + 7 * world) % 2000
        mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
        res = dict(out)
    assert sorted(res) == list(range(world))
    for r in range(world):
        slow, err_seq, n, err_head, calib_ok, err_batch = res[r]
        assert slow == float(world)             # every rank reports the slowest rank's time
        assert n == 4096 // world
        assert err_seq < 1e-5, err_seq
        assert err_head < 1e-5 and calib_ok, err_head
        assert err_batch < 1e-5, err_batch
