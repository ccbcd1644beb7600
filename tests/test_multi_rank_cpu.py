"""Host logic of the multi-GPU paths, run as two gloo ranks on the CPU: the max-over-ranks timing reduction of bench.py and
the KV-sequence shard -> all-gather -> LSE merge step (kernels.merge_partials on rows each rank computed for its own
slice of the sequence) against attention over the whole sequence."""
from __future__ import annotations

import math
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _partial(q, k, v, scale):
    """normalised rows + (m in log2 units, l) of attention over one slice: [B, Hq, 130]"""
    s = torch.einsum("bhd,bkhd->bhk", q, k) * scale * 1.4426950408889634
    m = s.amax(-1)
    p = torch.exp2(s - m[..., None])
    l = p.sum(-1)
    o = torch.einsum("bhk,bkhd->bhd", p, v) / l[..., None]
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
    B, Hq, L, W = 2, 4, 4096 + 128, 128
    q = torch.randn(B, Hq, 128, generator=g)
    k = torch.randn(B, L - W, Hq, 128, generator=g)
    v = torch.randn(B, L - W, Hq, 128, generator=g)
    n = bench.kvseq_local_len(L, W, world) - W
    part = _partial(q, k[:, rank * n:(rank + 1) * n], v[:, rank * n:(rank + 1) * n], 1 / math.sqrt(128)).contiguous()
    parts = torch.empty(world, B, Hq, 130)
    dist.all_gather_into_tensor(parts.view(world * B, Hq, 130), part)      # concatenation along dim 0
    merged = K.merge_partials(parts)
    full = _partial(q, k, v, 1 / math.sqrt(128))[..., :128]
    out[rank] = (slow, float((merged - full).abs().max()), n)
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_gloo():
    world = 2
    with mp.Manager() as mgr:
        out = mgr.dict()
        port = 29500 + os.getpid() % 2000
        mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
        res = dict(out)
    assert sorted(res) == [0, 1]
    for r in range(world):
        slow, err, n = res[r]
        assert slow == 2.0                      # every rank reports the slowest rank's time
        assert n == 2048
        assert err < 1e-5, err
