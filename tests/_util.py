"""helpers shared by the GPU parity tests: bf16 bit views, seeded inputs in the shapes the reference's tests use."""
from __future__ import annotations

import ctypes
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[1]
P = 16


def bits(t: torch.Tensor) -> np.ndarray:
    """bf16 tensor -> uint16 bit patterns (numpy, CPU)."""
    return t.detach().contiguous().cpu().view(torch.int16).numpy().view(np.uint16).copy()


def edge_rows(T, Hkv, g, scale_k=6.0):
    """Gaussian rows with outlier key channels and boundary groups: all positive / all negative / zero / FP16-subnormal
    scale / x300 / constant / single non-zero element (the cases of the reference's
    integrations/vllm_flagrot/tests/test_kernels.py:239-256)."""
    kv = torch.randn(T, 2 * Hkv, 128, generator=g)
    kv[:, :Hkv, :4] *= scale_k
    grp = kv.view(T, 2 * Hkv, 4, 32)
    sel = torch.rand(T, 2 * Hkv, 4, generator=g)
    grp[sel < 0.04] = grp[sel < 0.04].abs() + 0.5
    m = (sel >= 0.04) & (sel < 0.08)
    grp[m] = -grp[m].abs() - 0.5
    grp[(sel >= 0.08) & (sel < 0.10)] = 0.0
    grp[(sel >= 0.10) & (sel < 0.12)] *= 1e-5
    grp[(sel >= 0.12) & (sel < 0.14)] *= 300
    grp[(sel >= 0.14) & (sel < 0.15)] = 1.25
    one = (sel >= 0.15) & (sel < 0.16)
    grp[one] = 0.0
    grp[..., 5][one] = 3.0
    return kv.bfloat16()


def calib(Hkv, g, nq=256):
    """C_q = second moment of nq calibration queries with 8 outlier channels, c_o ~ U(0.1, 1.1)."""
    qs = torch.randn(Hkv, nq, 128, generator=g)
    qs[:, :, :8] *= 4
    Cq = torch.einsum("hnd,hne->hde", qs, qs) / nq
    co = torch.rand(Hkv, 128, generator=g) + 0.1
    return Cq.contiguous(), co


def slot_patterns(T, npg, g):
    out = {"rand": torch.randperm(npg * P, generator=g)[:T], "contig": torch.arange(T) + 3 * P}
    holes = torch.arange(T) + 3
    holes[torch.rand(T, generator=g) < 0.1] = -1
    out["holes"] = holes
    return {k: v.to(torch.int64) for k, v in out.items()}


def strided_kv(kvb: torch.Tensor, dev):
    """kv as a slice of a wider [T, 2 Hkv + 8, 128] buffer (token stride != row count), like a fused qkv output."""
    T, H2, Dh = kvb.shape
    base = torch.zeros(T, H2 + 8, Dh, dtype=torch.bfloat16, device=dev)
    base[:, 4:4 + H2] = kvb.to(dev)
    return base[:, 4:4 + H2]


def ref_lib(name: str):
    """a reference library built by oracle/build_ref.sh, or None."""
    p = ROOT / "oracle" / "_ref" / name
    return ctypes.CDLL(str(p)) if p.exists() else None
