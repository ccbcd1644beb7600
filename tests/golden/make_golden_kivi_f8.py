"""Generates tests/golden/kivi_f8.npz: the kivi2p8 pages (INT2 codes, FP8 E4M3 scale and minimum) as the reference's own
PyTorch code computes them on CPU, on the inputs of tests/golden/kivi.npz.

    python tests/golden/make_golden_kivi_f8.py [/path/to/reference]   (the reference checkout; else $FLAGROT_REFERENCE, else ./reference)

Recorded:
  e4m3_in / e4m3_out        blockflag.formats._e4m3 (clamp to +-448, round to nearest even) on fp32 values over 40 binades
  k_rec_ident / v_rec_ident plain KIVI reconstructions with spec kivi2f8:32 (keys along the token axis per 32-token group,
                            values along the head dim), blockflag.formats.fake_kivi_f8
  k_local / k_head / k_rec_dyn / v_rec_dyn   the simulator's dynamic choices and reconstructions with that spec (the
                            functions integrations/vllm_flagrot/tests/test_kivi.py:72-88 uses)
  pool / pool_K / pool_V    a random kivi2p8 pool [2 ng, Hkv, 1280] and what vllm_flagrot/kivi.py dequant_groups(f8=True)
                            reads out of it in the original basis: pins the byte layout and the flag positions
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
sys.path.insert(0, str(REF / "integrations" / "vllm_flagrot"))

from blockflag import formats as FM  # noqa: E402
from blockflag import qattention as QA  # noqa: E402
from blockflag.hadamard import fwht  # noqa: E402
from vllm_flagrot import kivi as KV  # noqa: E402

SPEC = "kivi2f8:32"


def bf16_of(bits):
    return torch.from_numpy(bits.astype(np.int16)).view(torch.bfloat16)


def main():
    g = np.load(HERE / "kivi.npz")
    k, v = bf16_of(g["k"]), bf16_of(g["v"])
    qs, lz, co = torch.from_numpy(g["qs"]), torch.from_numpy(g["lz"]), torch.from_numpy(g["co"])
    S, qscale = int(g["S"]), float(g["qscale"])
    T, H, _ = k.shape
    ng = T // 32
    out = {}
    gen = torch.Generator().manual_seed(808)
    x = torch.randn(8192, generator=gen) * torch.exp2(torch.randint(-14, 12, (8192,), generator=gen).float())
    x[:8] = torch.tensor([0.0, -0.0, 448.0, 449.0, -1000.0, 2.0 ** -9, 2.0 ** -10, 3 * 2.0 ** -10])
    out["e4m3_in"], out["e4m3_out"] = x.numpy(), FM._e4m3(x).numpy()

    QA.KV.update(dyn=dict(rule="att", local=["H"], head=["F"], group=1, only=None), sink=0, qs={0: qs}, lz={0: lz},
                 qscale=qscale, co={0: co}, xf=None, dynstat={})
    xf = k.float().permute(1, 0, 2)[None]
    vf = v.float().permute(1, 0, 2)[None]
    rec_id, rec_dyn = torch.empty_like(xf), torch.empty_like(xf)
    lbs, fbs = [], []
    for a, b_ in [(S, 32)] + [(32 * i, 32 * i + 32) for i in range(1, ng)]:
        seg = xf[:, :, a:b_]
        rec_id[:, :, a:b_] = QA._fake_tok_(seg, SPEC)
        rec_dyn[:, :, a:b_] = QA.dyn_quant(seg, SPEC, 32, "k", 0, "token")
        W = QA._weights("k", 0, seg)
        Q = lambda y: QA._fake_tok(y, SPEC)  # noqa: E731
        recs = [Q(seg), fwht(Q(fwht(seg, 32)), 32)]
        errs = QA._pool_tokens(torch.stack([QA._vec_err(r - seg, W, 32) for r in recs]), 32, 3)
        ch = errs.argmin(0)
        sel = ch[..., None].expand(*ch.shape, 32).reshape(seg.shape)
        r = torch.where(sel == 1, recs[1], recs[0])
        F = fwht(Q(fwht(seg, 128)), 128)
        he = QA._pool_tokens(torch.stack([QA._head_err(h - seg, W) for h in (r, F)]), 32, 3)
        lbs.append(ch[0][:, 0].numpy())
        fbs.append(he.argmin(0)[0][:, 0].numpy())
    rec_id[:, :, :S] = xf[:, :, :S]
    rec_dyn[:, :, :S] = xf[:, :, :S]
    out.update(k_rec_ident=rec_id[0].permute(1, 0, 2).numpy(), k_rec_dyn=rec_dyn[0].permute(1, 0, 2).numpy(),
               k_local=np.stack(lbs).astype(np.int8), k_head=np.stack(fbs).astype(np.int8))
    out["v_rec_ident"] = FM.fake(vf, SPEC)[0].permute(1, 0, 2).numpy()
    out["v_rec_dyn"] = QA.dyn_quant(vf, SPEC, 32, "v", 0)[0].permute(1, 0, 2).numpy()

    # a random pool read by the reference's parser (NaN bytes 0x7F / 0xFF of the metadata replaced)
    npg, Hp = 6, 2
    pool = torch.randint(0, 256, (npg, Hp, KV.chunk_bytes(128, True)), generator=gen, dtype=torch.uint8)
    meta = torch.cat([pool[..., 4 * 128:5 * 128], pool[..., 9 * 128:10 * 128]], -1)
    meta[(meta & 0x7F) == 0x7F] = 0x3A
    pool[..., 4 * 128:5 * 128], pool[..., 9 * 128:10 * 128] = meta[..., :128], meta[..., 128:]
    Kp, Vp = KV.dequant_groups(pool, 128, "orig", f8=True)
    out.update(pool=pool.numpy(), pool_K=Kp.numpy(), pool_V=Vp.numpy())
    np.savez_compressed(HERE / "kivi_f8.npz", **out)
    print({n: a.shape for n, a in out.items()})


if __name__ == "__main__":
    torch.manual_seed(0)
    main()
