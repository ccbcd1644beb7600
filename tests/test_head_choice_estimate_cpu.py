"""The error bar of the bulk key writer's head-choice estimate, checked on CPU.

The CUDA kernel (k_dyn_keys_bulk) takes the choice base / H128 from E_c = sum_i e_i (C~ e~)_i with TF32 operands when the
bars E_c +- DELTA * B_c, B_c = sum_i |e_i| (|C~| |e~|)_i, do not overlap, and evaluates the criterion's fixed-order fp32 sums
otherwise.  Its derivation claims |herr_c - E_c| <= 0.0020 * B_c for operands within 2^-10 of their values.  Here the
operands are truncated to TF32 (the worst case the derivation allows, every error in the same direction), E and B are
evaluated in float64, and herr is the oracle's fixed-order value (pinned to the reference by the golden tests)."""
import numpy as np
import torch

from oracle import flagrot_oracle as O
from tests._util import bits, calib, edge_rows

DELTA = 0.003          # DYN_DELTA of csrc/fr_writer.cu


def tf32_trunc(x):
    return (np.ascontiguousarray(x, dtype=np.float32).view(np.uint32) & np.uint32(0xFFFFE000)).view(np.float32)


def candidates(x, C, nb):
    """errors of the two head candidates exactly as encode_keys forms them"""
    y1 = O.fwht(x, O.RB)
    rec0 = O.quant_asym_err(x, nb, True)
    rec1 = O.fwht(O.quant_asym_err(y1, nb, True), O.RB)
    ch = O.local_err_k(rec1 - x, C) < O.local_err_k(rec0 - x, C)
    recb = np.where(np.repeat(ch, O.RB, -1), rec1, rec0)
    recF = O.fwht(O.quant_asym_err(O.fwht(x, O.D), nb, True), O.D)
    return recb - x, recF - x


def test_estimate_error_bar_holds_and_decides_most_choices():
    g = torch.Generator().manual_seed(31)
    Hkv, T = 4, 600
    Cq, _ = calib(Hkv, g)
    C = Cq.numpy().astype(np.float32)
    rows = {"edge": edge_rows(T, Hkv, g), "normal": torch.randn(T, 2 * Hkv, 128, generator=g).bfloat16(),
            "offset": (torch.randn(T, 2 * Hkv, 128, generator=g) + 3 * torch.randn(1, 2 * Hkv, 128, generator=g)).bfloat16()}
    for nb in (4, 2):
        for name, kv in rows.items():
            x = O.bf16_bits_to_f32(bits(kv))[:, :Hkv]
            es = candidates(x, C, nb)
            E, B, herr = [], [], []
            for e in es:
                et, Ct = tf32_trunc(e).astype(np.float64), tf32_trunc(C).astype(np.float64)
                E.append(np.einsum("thi,hik,thk->th", e.astype(np.float64), Ct, et))
                B.append(np.einsum("thi,hik,thk->th", np.abs(e).astype(np.float64), np.abs(Ct), np.abs(et)))
                herr.append(O.head_err_k(e, C).astype(np.float64))
            for c in range(2):
                live = B[c] > 1e-20
                assert np.all(np.abs(herr[c] - E[c])[live] <= 0.0020 * B[c][live]), (nb, name, c)
            surely_f = E[1] + DELTA * B[1] < E[0] - DELTA * B[0]
            surely_b = E[1] - DELTA * B[1] > E[0] + DELTA * B[0]
            exact = herr[1] < herr[0]
            assert np.all(exact[surely_f]) and not np.any(exact[surely_b]), (nb, name)
            decided = (surely_f | surely_b).mean()
            assert decided > 0.6, (nb, name, decided)
