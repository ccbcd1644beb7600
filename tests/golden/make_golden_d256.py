"""Generates tests/golden/static_d256.npz: the static writer path for head dim 256 as the reference's own PyTorch code
computes it on CPU.

    python tests/golden/make_golden_d256.py [/path/to/reference]   (the reference checkout; else $FLAGROT_REFERENCE, else ./reference)

Recorded (inputs as bf16 bit patterns):
  kv / mask / hfull / kmu   rows [T, 2 Hkv, 256], block flags [2 Hkv, 8], whole-head flags [2 Hkv], key centre [Hkv, 256]
  hf                        kernels/test_w3_static.py head_fwht_ref on the 256-d heads (the emulation of fr_head_fwht)
  {plain,both}_q4/_w4/_q2/_w2   kernels/ref.sel_fwht_rb + kernels/ref.int4a_quant, blockflag.formats.quant_asym_dep(bits 2)
                            + scale_word on the 256-d rows (after hf and the centre for "both")
  {int4a,int2a}_pool / _codes / _sbits / _K / _V   a pool packed by the oracle's packer as two half chunks per (page, head)
                            and READ BACK BY THE REFERENCE'S PARSERS with Dh = 256 (vllm_flagrot/kernels.py parse_pages /
                            dequant_v2_pages): pins the half-chunk layout
The reference tree is needed only to regenerate the file, never to run the tests.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))

import make_golden as MG  # noqa: E402  (sets the reference's paths from argv / the environment)

K, R, FM, O = MG.K, MG.R, MG.FM, MG.O
P = 16


def main():
    g = torch.Generator().manual_seed(256)
    Hkv, T, npg = 2, 45, 3
    kv = torch.cat([MG.edge_rows(T, Hkv, g), MG.edge_rows(T, Hkv, g)], -1)                  # [T, 2 Hkv, 256]
    mask = (torch.rand(2 * Hkv, 8, generator=g) < 0.5).to(torch.uint8)
    hfull = torch.tensor([0, 1, 1, 0], dtype=torch.uint8)
    kmu = (torch.randn(Hkv, 256, generator=g) * 0.5).float()
    slots = torch.randperm(npg * P, generator=g)[:T].long()
    slots[torch.rand(T, generator=g) < 0.1] = -1
    out = dict(kv=MG.bits_of(kv), mask=mask.numpy(), hfull=hfull.numpy(), kmu=kmu.numpy(), slots=slots.numpy())
    hf = MG.head_fwht_ref(kv, hfull)
    out["hf"] = MG.bits_of(hf)
    for tag, x, km in (("plain", kv, None), ("both", hf, kmu)):
        xf = x.float().clone()
        if km is not None:
            xf[:, :Hkv] = xf[:, :Hkv] - km
        y = R.sel_fwht_rb(xf.reshape(T, 2 * Hkv * 256), mask, 32).reshape(T, 2 * Hkv, 256)
        q4, w4 = R.int4a_quant(y)
        q2, z2, s2, _ = FM.quant_asym_dep(y, 32, False, 2)
        w2 = FM.scale_word(s2, z2, 2).squeeze(-1)
        out[f"{tag}_q4"] = q4.numpy().astype(np.uint8)
        out[f"{tag}_w4"] = w4.numpy().astype(np.int32)
        out[f"{tag}_q2"] = q2.reshape(y.shape).numpy().astype(np.uint8)
        out[f"{tag}_w2"] = (w2.numpy().astype(np.int32) & 0xFFFF)
    for fmt, bits in (("int4a", 4), ("int2a", 2)):
        rs = np.random.RandomState(256 + bits)
        pool = rs.randint(0, 256, (npg, Hkv, 2 * O.chunk_bytes(bits, P)), dtype=np.uint8)
        out[f"{fmt}_pool0"] = pool.copy()
        codes, words = O.static_rows_256(out["kv"], mask.numpy(), hfull.numpy(), bits, kmu.numpy(), recip=False)
        O.write_pool(pool.reshape(npg, 2 * Hkv, -1), slots.numpy(), codes, words, bits, P)
        tp = torch.from_numpy(pool)
        c, m, sb = K.parse_pages(tp, P, fmt, Dh=256)
        Kp, Vp = K.dequant_v2_pages(tp, P, torch.float64, fmt=fmt, Dh=256)
        out[f"{fmt}_pool"] = pool
        out[f"{fmt}_codes"] = c.numpy().astype(np.int8)
        out[f"{fmt}_sbits"] = sb.numpy()
        out[f"{fmt}_K"] = Kp.numpy().astype(np.float32)
        out[f"{fmt}_V"] = Vp.numpy().astype(np.float32)
        assert np.array_equal(out[f"{fmt}_codes"], c.numpy())
        assert np.array_equal(out[f"{fmt}_K"].astype(np.float64), Kp.numpy(), equal_nan=True)
        assert np.array_equal(out[f"{fmt}_V"].astype(np.float64), Vp.numpy(), equal_nan=True)
    np.savez_compressed(HERE / "static_d256.npz", **out)
    print({n: a.shape for n, a in out.items()})


if __name__ == "__main__":
    torch.manual_seed(0)
    main()
