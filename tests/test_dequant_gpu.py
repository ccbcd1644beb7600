"""fr_dequant_pages (the CUDA form of the "fa" prefill path's page dequantisation, reference
vllm_flagrot/attention/backend.py:1744-1789) against the oracle's float64 parser: key-only pages come back in the original
basis by their per-token flags, static pages by the layer's block masks and whole-head flags; fp32 output within fp32
rounding of the butterflies, bf16 output equal to the rounded fp32 output; ranges that start and end inside a page; pages
of 16 and 32 tokens."""
import numpy as np
import pytest
import torch

from oracle import flagrot_oracle as O
from tests._util import bits, calib, edge_rows

pytestmark = pytest.mark.gpu
DEV = "cuda"
FMT = {"int4a": (4, False), "int2a": (2, False), "konlya": (4, True), "konlya2": (2, True), "int4": (4, False)}


@pytest.mark.parametrize("fmt", sorted(FMT))
@pytest.mark.parametrize("P", [16, 32])
def test_dequant_pages_vs_oracle(fmt, P):
    from flagrot_releaser_b200 import kernels as K
    nb, key_only = FMT[fmt]
    g = torch.Generator().manual_seed(17 + P + nb)
    Hkv, L = 4, 333
    npg = (L + P - 1) // P
    total = npg + 6
    kvb = edge_rows(L, Hkv, g, scale_k=4.0)
    kv = kvb.to(DEV)
    pool = torch.randint(0, 256, (total, Hkv, K.v2_chunk_bytes(P, 128, fmt)), dtype=torch.uint8, generator=g).to(DEV)
    bt = torch.randperm(total, generator=g)[:npg].int()
    pos = torch.arange(L)
    slots = (bt.long()[pos // P] * P + pos % P).to(DEV)
    mask = (torch.rand(2 * Hkv, 4, generator=g) < 0.5).to(torch.uint8)
    hfull = (torch.rand(2 * Hkv, generator=g) < 0.5).to(torch.uint8)
    hfull[0], hfull[Hkv] = 1, 1
    if key_only:
        Cq, co = calib(Hkv, g)
        K.cb_write(kv, slots, Cq.transpose(1, 2).contiguous().to(DEV), co.to(DEV), fmt, pool, P)
    else:
        K.w3_static_write(kv, slots, mask.to(DEV), hfull.to(DEV), pool, P, fmt=fmt)
    torch.cuda.synchronize()
    with np.errstate(invalid="ignore", over="ignore"):
        pages = pool.cpu().numpy()[bt.numpy().astype(np.int64)]
        Kp, Vp = O.dequant_pool_sym(pages, P, False) if fmt == "int4" else O.dequant_pool(pages, nb, P, key_only)   # [npg, P, Hkv, 128]
    kr, vr = Kp.reshape(npg * P, Hkv, 128)[:L], Vp.reshape(npg * P, Hkv, 128)[:L]
    kw = {}
    if not key_only:       # stored basis -> original: block flags (orthonormal H32), then the whole head (x = H128 y / 8)
        km, vm = mask[:Hkv].numpy().astype(bool), mask[Hkv:].numpy().astype(bool)
        H128 = O.hadamard(128) * np.sqrt(128.0) / 8.0
        kr, vr = O.sel_rot64(kr, km), O.sel_rot64(vr, vm)
        kr = np.where(hfull[:Hkv].numpy().astype(bool)[None, :, None], kr @ H128, kr)
        vr = np.where(hfull[Hkv:].numpy().astype(bool)[None, :, None], vr @ H128, vr)
        kw = dict(kmask=mask[:Hkv].contiguous().to(DEV), vmask=mask[Hkv:].contiguous().to(DEV),
                  kfull=hfull[:Hkv].contiguous().to(DEV), vfull=hfull[Hkv:].contiguous().to(DEV))
    btd = bt.to(DEV)
    for a, n in ((0, L), (5, 300), (P, 2 * P), (37, 38), (L - 1, L)):
        k32, v32 = K.dequant_pages(pool, btd, a, n, fmt, page=P, dtype=torch.float32, **kw)
        k16, v16 = K.dequant_pages(pool, btd, a, n, fmt, page=P, dtype=torch.bfloat16, **kw)
        torch.cuda.synchronize()
        for got, ref, what in ((k32, kr[a:n], "K"), (v32, vr[a:n], "V")):
            err = np.abs(got.double().cpu().numpy() - ref).max()
            assert err <= 2e-5 * max(np.abs(ref).max(), 1.0), (fmt, P, a, n, what, err)
        assert torch.equal(k16, k32.to(torch.bfloat16)) and torch.equal(v16, v32.to(torch.bfloat16))
    # the recovered keys / values are the written rows up to the quantisation error (a sanity check of the whole chain)
    x = O.bf16_bits_to_f32(bits(kvb)).astype(np.float64)
    rel = np.abs(kr - x[:, :Hkv]).mean() / np.abs(x[:, :Hkv]).mean()
    assert rel < (0.2 if nb == 4 else 0.6), rel


def test_dequant_pages_refusals():
    from flagrot_releaser_b200 import kernels as K
    L = K.lib()
    assert L.fr_dequant_pages(3, None, None, 0, 16, 2, 16, None, None, None, None, None, None, 0, None) == -4     # not a page format
    assert L.fr_dequant_pages(4, None, None, 0, 16, 2, 16, None, None, None, None, None, None, 0, None) == -3     # null pool / table / outputs
    assert L.fr_dequant_pages(5, None, None, 0, 16, 2, 8, None, None, None, None, None, None, 0, None) == -5
    assert L.fr_dequant_pages(5, None, None, 7, 7, 2, 16, None, None, None, None, None, None, 0, None) == 0
