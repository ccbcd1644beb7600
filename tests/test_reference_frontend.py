"""Drop-in boundary: this repository's three libraries loaded through the reference's OWN, unmodified ctypes front ends
(integrations/vllm_flagrot/vllm_flagrot/kernels.py:140-177, kivi.py:49-77, prefill_mq.py:57-86).  Those modules honour
FLAGROT_LIB / FLAGROT_KIVI_LIB / FLAGROT_MQ_LIB / FLAGROT_NO_REBUILD; their lib() checks the ABI version and sets every
argtypes / restype line, so a missing or renamed symbol fails here before any kernel runs.

The front ends are used as byte code compiled by oracle/build_ref.sh into oracle/_ref/pyref (git-ignored build output, like
the reference libraries beside it) and loaded by oracle/pyref.py; the tests skip when it was not built.  The CPU test loads the libraries only.  The GPU
tests run one writer + decode step, one KIVI step and one prefill step through the reference's modules and through this
package's front end and compare the results byte for byte (same library, same launches: any difference is a marshalling
difference)."""
from __future__ import annotations

import math
from pathlib import Path

import pytest
import torch

from oracle import pyref

ROOT = Path(__file__).resolve().parents[1]
LIBDIR = ROOT / "flagrot_releaser_b200" / "lib"
ENV = {"FLAGROT_LIB": LIBDIR / "libflagrot_kernels.so", "FLAGROT_KIVI_LIB": LIBDIR / "libflagrot_kivi.so",
       "FLAGROT_MQ_LIB": LIBDIR / "libflagrot_mq.so"}


@pytest.fixture(scope="module")
def ref_front():
    """(kernels, kivi, prefill_mq) of the reference, pointed at this repository's libraries"""
    if not pyref.available():
        pytest.skip("oracle/_ref/pyref not built (oracle/build_ref.sh needs the reference checkout)")
    for v in ENV.values():
        assert v.exists(), f"{v} missing: run python -m flagrot_releaser_b200._build"
    mods = tuple(pyref.load(m, ENV) for m in ("kernels", "kivi", "prefill_mq"))
    return mods


def test_reference_loaders_accept_the_libraries(ref_front):
    RK, RKV, RMQ = ref_front
    assert RK.lib().fr_abi_version() == 9 and RKV.lib().kv_abi_version() == 9 and RMQ.lib().frmq_abi_version() == 7
    assert Path(RK.lib()._name).resolve() == ENV["FLAGROT_LIB"].resolve()
    assert Path(RKV.lib()._name).resolve() == ENV["FLAGROT_KIVI_LIB"].resolve()
    assert Path(RMQ.lib()._name).resolve() == ENV["FLAGROT_MQ_LIB"].resolve()
    # helpers the plugin calls on the host side agree with this package's mirror
    from flagrot_releaser_b200 import kernels as K
    for kind in ("konlya", "konlya2"):
        assert RK.cb_chunk_bytes(kind, 16) == K.cb_chunk_bytes(kind, 16) == RK.lib().fr_cb_chunk_bytes(RK.CB_KINDS[kind], 16)
    for fmt in ("int4a", "int2a"):
        assert RK.v2_chunk_bytes(16, 128, fmt) == K.v2_chunk_bytes(16, 128, fmt)
    assert RK.lib().fr_cb_nsg() == 15


DEV = "cuda"
LOG2E = 1.4426950408889634


def _kv(T, Hkv, g):
    kv = torch.randn(T, 2 * Hkv, 128, generator=g)
    kv[:, :Hkv, :4] *= 6
    return kv.bfloat16()


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["konlya", "konlya2"])
def test_writer_and_decode_through_reference_front_end(ref_front, kind):
    RK = ref_front[0]
    from flagrot_releaser_b200 import kernels as K
    g = torch.Generator().manual_seed(3)
    B, Hkv, G, L, P, S, W = 3, 8, 4, 1500, 16, 4, 128
    T = S + W
    npg = B * (-(-L // P)) + 5
    chunk_b = RK.cb_chunk_bytes(kind, P)
    pool0 = torch.randint(0, 256, (npg, Hkv, chunk_b), dtype=torch.uint8, generator=g)
    bt = torch.randperm(npg, generator=g)[:B * (-(-L // P))].view(B, -1).int()
    qs = torch.randn(Hkv, 256, 128, generator=g)
    Cq = (torch.einsum("hnd,hne->hde", qs, qs) / 256).contiguous()
    CT = Cq.transpose(1, 2).contiguous().to(DEV)
    co = (torch.rand(Hkv, 128, generator=g) + 0.5).to(DEV)
    kv = _kv(B * L, Hkv, g).to(DEV)
    pos = torch.arange(L)
    slots = (bt.long()[:, pos // P] * P + pos % P).reshape(-1).to(DEV)
    q = torch.randn(B, G * Hkv, 128, generator=g).bfloat16().to(DEV)
    ring = torch.randn(B, T, 2 * Hkv, 128, generator=g).bfloat16().to(DEV)
    tl = torch.tensor([T, 17, 0], dtype=torch.int32, device=DEV)
    lens = torch.tensor([L - W, L - W - 100, 33], dtype=torch.int32, device=DEV)
    res = []
    for F in (RK, K):
        pool = pool0.clone().to(DEV)
        F.cb_write(kv, slots, CT, co, kind, pool, P)
        ns, ch = F.plan_cb(B, L, Hkv, P, kind)          # the reference's planner is driven by this library's occupancy answer
        ws = F.Workspace(B, Hkv, B * Hkv * (ns + 1), DEV)
        out = torch.zeros(B, G * Hkv * 128, dtype=torch.bfloat16, device=DEV)
        F.cb_attn(q, pool, bt.to(DEV), lens, out, ns, ch, ws, LOG2E / math.sqrt(128), kind, tail=ring, tail_len=tl,
                  tail_idx=None, tail_bs=ring.stride(0), tail_ts=ring.stride(1), page=P, kv_start=S)
        torch.cuda.synchronize()
        assert int(ws.counter.abs().sum()) == 0
        res.append((pool.cpu(), out.cpu(), (ns, ch)))
    assert torch.equal(res[0][0], res[1][0]), "pool bytes differ between the two front ends"
    if res[0][2] == res[1][2]:
        assert torch.equal(res[0][1], res[1][1]), "outputs differ between the two front ends on the same plan"
    else:                                                # different planners, same attention within rounding of the merge order
        assert (res[0][1].float() - res[1][1].float()).abs().max() <= 2e-2, res[0][2:] + res[1][2:]
    assert not torch.isnan(res[0][1].float()).any()


@pytest.mark.gpu
def test_static_writer_through_reference_front_end(ref_front):
    RK = ref_front[0]
    from flagrot_releaser_b200 import kernels as K
    g = torch.Generator().manual_seed(4)
    Hkv, T, P = 8, 700, 16
    kv = _kv(T, Hkv, g).to(DEV)
    npg = T // P + 9
    mask = (torch.rand(2 * Hkv, 4, generator=g) < 0.5).to(torch.uint8).to(DEV)
    hfull = (torch.rand(2 * Hkv, generator=g) < 0.4).to(torch.uint8).to(DEV)
    slots = torch.randperm(npg * P, generator=g)[:T].to(torch.int64).to(DEV)
    for fmt in ("int4a", "int2a"):
        pool0 = torch.randint(0, 256, (npg, Hkv, RK.v2_chunk_bytes(P, 128, fmt)), dtype=torch.uint8, generator=g)
        a, b = pool0.clone().to(DEV), pool0.clone().to(DEV)
        RK.w3_static_write(kv, slots, mask, hfull, a, P, fmt=fmt)
        K.w3_static_write(kv, slots, mask, hfull, b, P, fmt=fmt)
        torch.cuda.synchronize()
        assert torch.equal(a, b), fmt


@pytest.mark.gpu
def test_kivi_step_through_reference_front_end(ref_front):
    RKV = ref_front[1]
    from flagrot_releaser_b200 import kivi as KV
    g = torch.Generator().manual_seed(5)
    B, Hkv, G, D, L, S, W, PAGE, GRP = 2, 4, 8, 128, 1200, 4, 128, 16, 32
    T = S + W
    npgr = (-(-L // GRP)) * 2
    nb = B * npgr + 3
    pool0 = torch.randint(0, 256, (nb, Hkv, RKV.chunk_bytes(D)), dtype=torch.uint8, generator=g)
    bt = torch.randperm(nb, generator=g)[:B * npgr].view(B, npgr).int()
    qs = (torch.randn(Hkv, 64, D, generator=g) * 0.3).to(DEV)
    lz = torch.full((Hkv, 64), 5.0, device=DEV)
    co = (torch.rand(Hkv, D, generator=g) + 0.5).to(DEV)
    q = (torch.randn(B, Hkv * G, D, generator=g) * 0.5).bfloat16().to(DEV)
    ring = torch.randn(B + 1, T, 2 * Hkv, D, generator=g).bfloat16().to(DEV)
    cached = torch.full((B,), L - W, dtype=torch.int32, device=DEV)
    tl = torch.full((B,), T, dtype=torch.int32, device=DEV)
    ti = torch.arange(B, dtype=torch.int32, device=DEV)
    rows = [_kv(L, Hkv, g).to(DEV) for _ in range(B)]
    res = []
    for F in (RKV, KV):
        pool = pool0.clone().to(DEV)
        for b in range(B):
            pos = torch.arange(L)
            F.v_write(rows[b], (bt[b].long()[pos // PAGE] * PAGE + pos % PAGE).to(DEV), co, None, pool, Hkv, D)
            gp = torch.arange((L // GRP) * GRP).view(-1, GRP)
            sidx = torch.where(gp < S, torch.full_like(gp, -1), gp).contiguous().to(DEV)
            dslot = (bt[b].long()[gp // PAGE] * PAGE + gp % PAGE).contiguous().to(DEV)
            F.k_encode(rows[b], sidx, dslot, qs, lz, 1 / math.sqrt(D), pool, Hkv, D)
        ns, chunk = RKV.plan(B, L, Hkv)                  # the reference's own plan: chunks are multiples of 32, not of 128
        ws = F.Workspace(B * Hkv * (ns + 1), G, D, DEV)
        out = torch.zeros(B, Hkv * G * D, dtype=torch.bfloat16, device=DEV)
        F.attn(q, pool, bt.to(DEV), cached, out, ns, chunk, ws, LOG2E / math.sqrt(D), S, G, ring=ring.view(-1, 2 * Hkv, D),
               tail_len=tl, tail_idx=ti, T=T)
        torch.cuda.synchronize()
        res.append((pool.cpu(), out.cpu()))
    assert torch.equal(res[0][0], res[1][0]) and torch.equal(res[0][1], res[1][1])
    assert not torch.isnan(res[0][1].float()).any()


@pytest.mark.gpu
@pytest.mark.parametrize("kernel", [1, 2, 3])
def test_prefill_step_through_reference_front_end(ref_front, kernel):
    RK, _, RMQ = ref_front
    from flagrot_releaser_b200 import prefill_mq as MQ
    g = torch.Generator().manual_seed(6)
    Hkv, G, P, L, nq = 2, 4, 16, 2100, 300
    npg = -(-L // P) + 4
    pool = torch.randint(0, 256, (npg, Hkv, 144 * P), dtype=torch.uint8, generator=g).to(DEV)
    bt = torch.randperm(npg, generator=g)[:-(-L // P)].view(1, -1).int().to(DEV)
    kv = _kv(L, Hkv, g).to(DEV)
    pos = torch.arange(L)
    RK.v2_write(kv, (bt[0].cpu().long()[pos // P] * P + pos % P).to(DEV), torch.zeros(2 * Hkv, 4, dtype=torch.uint8, device=DEV), 32,
                pool, P, fmt="int4a")
    q = torch.randn(nq, Hkv * G, 128, generator=g).bfloat16().to(DEV)
    reqs = [(0, 0, nq, L, L - nq)]
    res = []
    for F in (RMQ, MQ):
        plan = F.build_plan(reqs, G, Hkv, 0, DEV, kernel=kernel)
        q16 = F.prep_q(q, LOG2E / math.sqrt(128), G, idx=plan.idx)
        opart, ml = F.attn(q16, pool, bt, plan, G, 0, konly=False)
        o, lse = F.merge(plan, opart, ml, G, fp32=True, want_lse=True)
        torch.cuda.synchronize()
        res.append((q16.cpu(), o.cpu(), lse.cpu(), (plan.ntiles, plan.nitems, plan.rows)))
    assert torch.equal(res[0][0], res[1][0]), "staged q differs"
    assert res[0][3][2] == res[1][3][2] == (64 if kernel == 1 else 128)
    if res[0][3] == res[1][3]:
        assert torch.equal(res[0][1], res[1][1]) and torch.equal(res[0][2], res[1][2])
    else:                                                # this package's planner may balance the item split differently
        assert (res[0][1] - res[1][1]).abs().max() <= 2e-3
    assert not torch.isnan(res[0][1]).any()
