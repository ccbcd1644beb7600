"""The allocation-free decode entry (fr_cb_attn_noalloc): for hosts that cannot hand the library a workspace because
they cannot allocate device memory (a serving worker with a frozen memory pool, a C host that only forwards pointers).
Its split partials live in an array inside the library, so this test checks what a user relies on: the same bytes as
fr_cb_attn with a caller workspace, on two calls in a row (the second call finds the first call's leftovers in the
array), no growth of allocated device memory across the calls, and a clean refusal of a request that does not fit.
Collected last on purpose: a run that stops at the first failure has then already covered every other test."""
import math

import pytest
import torch

from tests._util import P, calib

pytestmark = pytest.mark.gpu
DEV = "cuda"
LOG2E = 1.4426950408889634


def _case(K, kind, seed):
    g = torch.Generator().manual_seed(seed)
    Hkv, lens = 8, [300, 4101, 17, 0]
    B = len(lens)
    need = [(n + P - 1) // P for n in lens]
    npg = sum(need) + 5
    ids = torch.randperm(npg, generator=g)[:sum(need)]
    bt = torch.zeros(B, max(need), dtype=torch.int32)
    o = 0
    for b, n in enumerate(need):
        bt[b, :n] = ids[o:o + n].int()
        o += n
    pool = torch.randint(0, 256, (npg, Hkv, K.cb_chunk_bytes(kind, P)), dtype=torch.uint8, generator=g).to(DEV)
    Cq, co = calib(Hkv, g)
    CT = Cq.transpose(1, 2).contiguous().to(DEV)
    for b, n in enumerate(lens):
        if n == 0:
            continue
        kv = torch.randn(n, 2 * Hkv, 128, generator=g)
        kv[:, :Hkv, :4] *= 6
        pos = torch.arange(n)
        sl = (bt[b].long()[pos // P] * P + pos % P).to(DEV)
        K.cb_write(kv.bfloat16().to(DEV), sl, CT, co.to(DEV), kind, pool, P)
    q = torch.randn(B, 4 * Hkv, 128, generator=g).bfloat16().to(DEV)
    ring = torch.randn(6, 132, 2 * Hkv, 128, generator=g).bfloat16().to(DEV)
    tail_idx = torch.tensor([4, 1, 3, 0], dtype=torch.int32, device=DEV)
    tail_len = torch.tensor([132, 7, 0, 40], dtype=torch.int32, device=DEV)
    seq = torch.tensor(lens, dtype=torch.int32, device=DEV)
    tkw = dict(tail=ring, tail_len=tail_len, tail_idx=tail_idx, tail_bs=ring.stride(0), tail_ts=ring.stride(1), kv_start=4)
    return q, pool, bt.to(DEV), seq, tkw, B, Hkv


@pytest.mark.parametrize("kind", ["konlya", "konlya2"])
def test_noalloc_entry_matches_workspace_entry_twice(kind):
    from flagrot_releaser_b200 import kernels as K
    K.lib()
    qscale = LOG2E / math.sqrt(128)
    results = []
    for call, (seed, ns, ch) in enumerate(((11, 3, 1408), (12, 1, 4160))):
        q, pool, bt, seq, tkw, B, Hkv = _case(K, kind, seed)
        ws = K.Workspace(B, Hkv, B * Hkv * (ns + 1), DEV)
        ref = torch.zeros(B, 4 * Hkv * 128, dtype=torch.bfloat16, device=DEV)
        K.cb_attn(q, pool, bt, seq, ref, ns, ch, ws, qscale, kind, **tkw)
        out = torch.zeros_like(ref)
        # a first call, so that the one-time work per device (the module that holds the array is loaded, its address looked
        # up) lies behind us; the measured call must then leave the device's free memory alone.  The driver's own figure is
        # used: torch's counter would not see a cudaMalloc made inside the library.
        assert K.cb_attn_noalloc(q, pool, bt, seq, out, ns, ch, qscale, kind, **tkw) == 0
        torch.cuda.synchronize()
        out.zero_()
        before, free_before = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
        rc = K.cb_attn_noalloc(q, pool, bt, seq, out, ns, ch, qscale, kind, **tkw)
        torch.cuda.synchronize()
        assert rc == 0
        assert torch.cuda.memory_allocated() == before
        assert torch.cuda.mem_get_info()[0] >= free_before - (1 << 20), "the call took device memory"
        assert K.device_status() == 0
        err = (out.float() - ref.float()).abs().max().item()
        assert err <= 2e-2, (call, err)          # the tolerance of the decode parity tests ...
        results.append(torch.equal(out, ref))
    assert all(results), "... and in fact the same bytes: both entries run one kernel over the same partial layout"


def test_noalloc_entry_rejects_what_does_not_fit():
    from flagrot_releaser_b200 import kernels as K
    K.lib()
    q, pool, bt, seq, tkw, B, Hkv = _case(K, "konlya", 13)
    out = torch.zeros(B, 4 * Hkv * 128, dtype=torch.bfloat16, device=DEV)
    # 512 splits of a 4-row batch fit (about 34 MB would not): ask for far more rows than the array can serve
    big_B = 4096
    qb = q[:1].expand(big_B, -1, -1)
    rc = K.lib().fr_cb_attn_noalloc(qb.data_ptr(), 0, pool.data_ptr(), bt.data_ptr(), 0, seq.data_ptr(), big_B, Hkv, P, 8, 1024,
                                    1.0, 10, out.data_ptr(), 0, None, None, None, 0, 0, None, 0)
    assert rc == -9
    assert K.lib().fr_cb_attn_noalloc(q.data_ptr(), q.stride(0), pool.data_ptr(), bt.data_ptr(), bt.stride(0), seq.data_ptr(),
                                      B, Hkv, P, 1, 4160, 1.0, 3, out.data_ptr(), out.stride(0), None, None, None, 0, 0, None,
                                      0) == -4
