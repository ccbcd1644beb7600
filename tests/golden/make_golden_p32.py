"""Generates tests/golden/pages_p32.npz: pools of 32-token pages packed by the oracle's packer on the rows of
tests/golden/pages.npz and READ BACK BY THE REFERENCE'S PARSERS (vllm_flagrot/kernels.py parse_pages / dequant_cb_pages /
dequant_v2_pages with P = 32), for konlya, konlya2, static int4a and static int2a.  Pins the 32-token page layout (code
planes, scale-word planes, flag bits) the same way pages.npz pins the 16-token one.

    python tests/golden/make_golden_p32.py [/path/to/reference]   (the reference checkout; else $FLAGROT_REFERENCE, else ./reference)

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
sys.path.insert(0, str(HERE.parents[1]))
sys.path.insert(0, str(REF))
sys.path.insert(0, str(REF / "integrations" / "vllm_flagrot"))

from vllm_flagrot import kernels as K  # noqa: E402

from oracle import flagrot_oracle as O  # noqa: E402

P = 32


def main():
    g = np.load(HERE / "pages.npz")
    kv, Cq, mask = g["kv"], g["Cq"], g["mask"]
    T, Hkv, npg = kv.shape[0], kv.shape[1] // 2, 3
    gen = torch.Generator().manual_seed(3232)
    slots = torch.randperm(npg * P, generator=gen)[:T].long()
    slots[torch.rand(T, generator=gen) < 0.1] = -1
    out = dict(slots=slots.numpy())
    for kind, bits, key_only in (("konlya", 4, True), ("konlya2", 2, True), ("int4a", 4, False), ("int2a", 2, False)):
        rs = np.random.RandomState(32)
        pool = rs.randint(0, 256, (npg, Hkv, O.chunk_bytes(bits, P)), dtype=np.uint8)
        out[f"{kind}_pool0"] = pool.copy()
        if key_only:
            codes, words, _ = O.dynamic_rows(kv, Cq, bits, None, recip=False)
        else:
            codes, words = O.static_rows(kv, mask, None, bits, None, recip=False)
        O.write_pool(pool, slots.numpy(), codes, words, bits, P)
        tp = torch.from_numpy(pool)
        c, m, sb = K.parse_pages(tp, P, kind)
        out[f"{kind}_pool"] = pool
        out[f"{kind}_codes"] = c.numpy().astype(np.int8)
        assert np.array_equal(out[f"{kind}_codes"], c.numpy())
        out[f"{kind}_sbits"] = sb.numpy()
        if key_only:
            Kp, Vp = K.dequant_cb_pages(tp, P, kind, torch.float64)
        else:
            Kp, Vp = K.dequant_v2_pages(tp, P, torch.float64, fmt=kind)
        # (computed by the reference in fp32 and widened: fp32 holds them exactly)
        out[f"{kind}_K"] = Kp.numpy().astype(np.float32)
        out[f"{kind}_V"] = Vp.numpy().astype(np.float32)
        assert np.array_equal(out[f"{kind}_K"].astype(np.float64), Kp.numpy(), equal_nan=True)
        assert np.array_equal(out[f"{kind}_V"].astype(np.float64), Vp.numpy(), equal_nan=True)
    np.savez_compressed(HERE / "pages_p32.npz", **out)
    print({n: a.shape for n, a in out.items()})


if __name__ == "__main__":
    torch.manual_seed(0)
    main()
