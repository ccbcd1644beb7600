"""fp32 CPU decode step over FlagRot pages, for timing only: the reference's CPU path for this workload is "parse the
pages with the PyTorch layout parser, dequantise, inverse-rotate, fp32 attention" (integrations/vllm_flagrot/vllm_flagrot/
kernels.py:694-743 followed by the attention of integrations/vllm_flagrot/tests/test_kernels.py:37-56).  This module restates
that path with numpy in fp32 (BLAS matmuls use every host thread numpy was given).  TEST / BENCH INFRASTRUCTURE ONLY:
used by the cpu_baseline and reference legs of bench.py, never by the package."""
from __future__ import annotations

import numpy as np

from . import flagrot_oracle as O

F32 = np.float32


def decode_rows_fp32(q_bits, pool, bt, lens, scale, bits, P, key_only, rows, tail=None, tail_len=None, tail_idx=None,
                     kv_start=0):
    """decode attention of the batch rows `rows` (a bounded sample of the batch) in fp32.  Returns fp32 [len(rows), Hq, 128]."""
    q = O.bf16_bits_to_f32(q_bits)
    Hq = q.shape[1]
    Hkv = pool.shape[1]
    G = Hq // Hkv
    kb, ks, vb, vs, ksw, vsw = O._maps(bits, P)
    fm = (1 << bits) - 1
    H32 = O.hadamard(32).astype(F32)
    H128 = O.hadamard(128).astype(F32)
    out = np.zeros((len(rows), Hq, 128), F32)
    for n, b in enumerate(rows):
        L = int(lens[b])
        a = min(kv_start, L)
        npg = (L + P - 1) // P
        pg = pool[np.asarray(bt[b, :npg], dtype=np.int64)]                           # [npg, Hkv, chunk]
        kc = ((pg[:, :, kb] >> ks.astype(np.uint8)) & fm).astype(F32)                 # [npg, Hkv, P, 128]
        vc = ((pg[:, :, vb] >> vs.astype(np.uint8)) & fm).astype(F32)
        kw = pg[:, :, ksw].astype(np.uint16) | (pg[:, :, ksw + 1].astype(np.uint16) << 8)   # [npg, Hkv, P, 4]
        vw = pg[:, :, vsw].astype(np.uint16) | (pg[:, :, vsw + 1].astype(np.uint16) << 8)
        with np.errstate(invalid="ignore", over="ignore"):
            k = (kc.reshape(npg, Hkv, P, 4, 32) - (kw & fm).astype(F32)[..., None]) * O.word_value(kw)[..., None]
            v = (vc.reshape(npg, Hkv, P, 4, 32) - (vw & fm).astype(F32)[..., None]) * O.word_value(vw)[..., None]
            if key_only:
                lk = ((kw >> 15) & 1).astype(bool)
                fk = ((vw[..., 0] >> 15) & 1).astype(bool)
                kl = np.where(lk[..., None], k @ H32, k).reshape(npg, Hkv, P, 128)
                k = np.where(fk[..., None], k.reshape(npg, Hkv, P, 128) @ H128, kl)
        k = k.reshape(npg, Hkv, P, 128).transpose(1, 0, 2, 3).reshape(Hkv, npg * P, 128)[:, a:L]
        v = v.reshape(npg, Hkv, P, 128).transpose(1, 0, 2, 3).reshape(Hkv, npg * P, 128)[:, a:L]
        if tail is not None:
            r = int(tail_idx[b]) if tail_idx is not None else b
            tn = min(int(tail_len[b]), 256)
            tf = O.bf16_bits_to_f32(tail[r, :tn])                                    # [tn, 2 Hkv, 128]
            k = np.concatenate([k, tf[:, :Hkv].transpose(1, 0, 2)], 1)
            v = np.concatenate([v, tf[:, Hkv:].transpose(1, 0, 2)], 1)
        if k.shape[1] == 0:
            continue
        qh = q[b].reshape(Hkv, G, 128)
        s = np.matmul(qh, k.transpose(0, 2, 1)) * F32(scale)                         # [Hkv, G, L]
        p = np.exp(s - s.max(-1, keepdims=True))
        p /= p.sum(-1, keepdims=True)
        out[n] = np.matmul(p, v).reshape(Hq, 128)
    return out
