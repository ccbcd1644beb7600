"""Generates tests/golden/sym_int4.npz: the symmetric INT4 page format (`int4`) as the reference's own PyTorch code computes
and reads it on CPU, on the rows of tests/golden/writer_static.npz.

    python tests/golden/make_golden_sym.py [/path/to/reference]   (the reference checkout; else $FLAGROT_REFERENCE, else ./reference)

Recorded:
  {plain,hfull,kmu,both}_q / _s   kernels/ref.py int4_quant (codes q + 8 unpacked, FP16 scale bit patterns) of the rows after
                                  the whole-head step, key centering and kernels/ref.py sel_fwht_rb, as in writer_static.npz
  pool / pool_codes / pool_mag    a pool of random bytes with sane scale words and what vllm_flagrot/kernels.py
                                  parse_int4_pages(asym=False) reads out of it: pins the sign-magnitude bit layout
  pool_K / pool_V                 kernels.py dequant_v2_pages(fmt "int4") of that pool in float64
  {a,b}_qk / _qv / _wk / _wv / _mode / _local / _herr   kernels/codebook_ref.py encode(cfg "konly", qk "cache") on the inputs of
                                  tests/golden/writer_dynamic.npz (codes q + 8, words assembled as
                                  integrations/vllm_flagrot/tests/test_int2.py:141-152 does)
The reference tree is needed only to regenerate the file, never to run the tests.
"""
from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REF = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("FLAGROT_REFERENCE", "reference"))
sys.path.insert(0, str(REF))
sys.path.insert(0, str(REF / "kernels"))
sys.path.insert(0, str(REF / "integrations" / "vllm_flagrot"))

import codebook_ref as CR  # noqa: E402
import ref as R  # noqa: E402
from vllm_flagrot import kernels as K  # noqa: E402


def bf16_of(bits):
    return torch.from_numpy(bits.astype(np.int16)).view(torch.bfloat16)


def main():
    g = np.load(HERE / "writer_static.npz")
    kv = bf16_of(g["kv"])
    T, H2, _ = kv.shape
    Hkv = H2 // 2
    mask, kmu = torch.from_numpy(g["mask"]), torch.from_numpy(g["kmu"])
    out = {}
    for tag, hf, km in (("plain", False, False), ("hfull", True, False), ("kmu", False, True), ("both", True, True)):
        x = bf16_of(g[f"{tag}_hf"]) if hf else kv
        xf = x.float().clone()
        if km:
            xf[:, :Hkv] = xf[:, :Hkv] - kmu
        y = R.sel_fwht_rb(xf.reshape(T, H2 * 128), mask, 32).reshape(T, H2, 128)
        qp, s = R.int4_quant(y)
        out[f"{tag}_q"] = R.unpack_nibbles(qp).numpy().astype(np.uint8)                 # q + 8
        out[f"{tag}_s"] = s.view(torch.int16).numpy().astype(np.int32) & 0xFFFF
    gen = torch.Generator().manual_seed(909)
    P, Np, Hp = 16, 5, 2
    pool = torch.randint(0, 256, (Np, Hp, 144 * P), generator=gen, dtype=torch.uint8)
    words = torch.randint(0x1C00, 0x2C00, (Np, Hp, 8 * P), generator=gen).to(torch.int16)
    pool[:, :, 128 * P:144 * P] = words.view(torch.uint8).reshape(Np, Hp, 16 * P)
    codes, mag, _ = K.parse_int4_pages(pool, P, asym=False)
    Kp, Vp = K.dequant_v2_pages(pool, P, torch.float64, fmt="int4")
    out.update(pool=pool.numpy(), pool_codes=codes.numpy().astype(np.int8), pool_mag=mag.numpy(),
               pool_K=Kp.numpy(), pool_V=Vp.numpy())
    d = np.load(HERE / "writer_dynamic.npz")
    for name in ("a", "b"):
        kvd = bf16_of(d[f"{name}_kv"])
        Hd = kvd.shape[1] // 2
        Cq, co = torch.from_numpy(d[f"{name}_Cq"]), torch.from_numpy(d[f"{name}_co"])
        k = kvd[:, :Hd].float()
        if f"{name}_kmu" in d.files:
            k = k - torch.from_numpy(d[f"{name}_kmu"])
        ek = CR.encode(k, Cq, co, "k", cfg="konly", qk="cache")
        ev = CR.encode(kvd[:, Hd:].float(), Cq, co, "v", cfg="konly", qk="cache")
        wk = ek["s"].half().view(torch.int16).to(torch.int32) & 0xFFFF
        wk = wk | (((ek["mode"] == 0)[..., None] & (ek["local"] == 1)).to(torch.int32) << 15)
        wv = ev["s"].half().view(torch.int16).to(torch.int32) & 0xFFFF
        wv[..., 0] |= (ek["mode"] == 2).to(torch.int32) << 15
        out[f"{name}_qk"] = ek["q"].numpy().astype(np.int8)
        out[f"{name}_qv"] = ev["q"].numpy().astype(np.int8)
        out[f"{name}_wk"], out[f"{name}_wv"] = wk.numpy().astype(np.int32), wv.numpy().astype(np.int32)
        out[f"{name}_mode"] = ek["mode"].numpy().astype(np.int8)
        out[f"{name}_local"] = ek["local"].numpy().astype(np.int8)
        out[f"{name}_herr"] = ek["head_errs"].numpy()
    np.savez_compressed(HERE / "sym_int4.npz", **out)
    print({n: a.shape for n, a in out.items()})


if __name__ == "__main__":
    main()
