"""Seeded multi-query prefill cases shared by the golden generator, the CPU oracle tests and the GPU parity tests.  The request
mixes follow the categories the reference checks (integrations/vllm_flagrot/scripts/bench_mq_prefill.py:99-118): one or
several requests per launch, partial pages and 64-key blocks, a window shift, sink tokens, G 1 / 4 / 5 / 8."""
from __future__ import annotations

import numpy as np
import torch

from oracle import flagrot_oracle as O
from _util import bits, calib

NO_EXT = -(1 << 30)

# (requests [(bt row, q0, q1, L, s)], G, Hkv, shift, sink, ext)
PLAN_CASES = [
    ([(0, 0, 1000, 1000, 0)], 4, 8, 0, 0, None),
    ([(0, 0, 300, 777, 477)], 4, 8, 0, 0, None),
    ([(0, 0, 145, 10145, 10000)], 4, 8, 0, 0, None),
    ([(0, 0, 1, 3000, 2999)], 4, 8, 0, 0, None),
    ([(0, 0, 17, 17, 0)], 4, 8, 0, 0, None),
    ([(0, 0, 5, 16, 11)], 4, 8, 0, 0, None),
    ([(0, 0, 145, 9000, 8855), (1, 145, 445, 12000, 11700), (2, 445, 462, 5003, 4986), (3, 462, 1162, 700, 0),
      (4, 1162, 1226, 20000, 19936)], 4, 8, 0, 0, None),
    ([(0, 0, 2048, 2048, 0)], 4, 8, 128, 0, None),
    ([(0, 0, 70, 130, 60)], 4, 8, 64, 0, None),
    ([(0, 0, 300, 8191, 7891), (1, 300, 3300, 3000, 0)], 4, 8, 128, 4, None),
    ([(0, 0, 1200, 33000, 31800)], 4, 8, 0, 0, None),
    ([(0, 0, 200, 6000, 5800), (1, 200, 500, 300, 0)], 5, 8, 0, 0, None),
    ([(0, 0, 200, 6000, 5800), (1, 200, 500, 300, 0)], 8, 4, 0, 0, None),
    ([(0, 0, 200, 6000, 5800)], 1, 8, 0, 0, None),
    ([(0, 0, 64, 4000, 3936), (1, 64, 164, 900, 800)], 4, 8, 128, 4, {0: 3900, 1: 500}),
]

# one request per case: pages hold positions [0, L - W); queries are the last nq positions of the L
ATTN_CASES = [
    dict(kind="konlya", bits=4, key_only=True, Hkv=2, G=4, L=150, nq=24, W=0, S=0, seed=1),
    dict(kind="konlya", bits=4, key_only=True, Hkv=2, G=4, L=200, nq=20, W=32, S=4, seed=2),
    dict(kind="konlya2", bits=2, key_only=True, Hkv=2, G=2, L=40, nq=40, W=0, S=0, seed=3),
    dict(kind="int4a", bits=4, key_only=False, Hkv=2, G=4, L=130, nq=17, W=16, S=0, seed=4),
    dict(kind="int2a", bits=2, key_only=False, Hkv=1, G=5, L=81, nq=12, W=0, S=4, seed=5),
]


def rand_kv(n, Hkv, g):
    """rows [n, 2 Hkv, 128] fp32, K heads first, with outlier key channels and a value offset."""
    k = torch.randn(n, Hkv, 128, generator=g)
    v = torch.randn(n, Hkv, 128, generator=g)
    k[..., 5] *= 8
    k[..., 70] += 4
    v[..., 3] += 2
    return torch.cat([k, v], 1)


def rand_q(nq, Hq, g):
    q = torch.randn(nq, Hq, 128, generator=g) * 2
    q[..., 5] *= 4
    return q.bfloat16()


def block_table(lens, g, spare=7, pad=3):
    """shuffled block table [R, max pages + pad]; unused entries point at in-range canary pages (the last `spare` pages,
    never written), so an over-read changes results instead of faulting."""
    npg = [-(-max(n, 1) // 16) for n in lens]
    total = sum(npg) + spare
    perm = torch.randperm(total - spare, generator=g)
    bt = torch.full((len(lens), max(npg) + pad), total - 1, dtype=torch.int32)
    o = 0
    for i, n in enumerate(npg):
        bt[i, :n] = perm[o:o + n].to(torch.int32)
        bt[i, n:] = total - 1 - (i % spare)
        o += n
    return bt, total


def make_request_pool(case):
    """numpy pool / block-table row / q bits of one ATTN_CASES entry, packed by the oracle (static: no flags)."""
    g = torch.Generator().manual_seed(1000 + case["seed"])
    Hkv, L, W, bitsn = case["Hkv"], case["L"], case["W"], case["bits"]
    n = L - W
    bt, total = block_table([n], g)
    rs = np.random.RandomState(case["seed"])
    pool = rs.randint(0, 256, (total, Hkv, O.chunk_bytes(bitsn, 16)), dtype=np.uint8)
    kv = rand_kv(n, Hkv, g).bfloat16()
    if case["key_only"]:
        Cq, _ = calib(Hkv, g)
        codes, words, _ = O.dynamic_rows(bits(kv), Cq.numpy(), bitsn, None, recip=True)
    else:
        codes, words = O.static_rows(bits(kv), None, None, bitsn, None, recip=True)
    pos = np.arange(n)
    slots = bt[0].numpy().astype(np.int64)[pos // 16] * 16 + pos % 16
    O.write_pool(pool, slots, codes, words, bitsn, 16)
    q = rand_q(case["nq"], Hkv * case["G"], g)
    return pool, bt[0].numpy(), bits(q)
