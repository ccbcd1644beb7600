"""Head dim 256, static writer path: the oracle against outputs of the reference's own PyTorch code
(tests/golden/static_d256.npz, written by tests/golden/make_golden_d256.py)."""
import numpy as np
import pytest

from oracle import flagrot_oracle as O

P = 16


def test_head_transform_matches_reference_emulation(golden_dir):
    g = np.load(golden_dir / "static_d256.npz")
    assert np.array_equal(O.head_fwht(g["kv"], g["hfull"], 1.0 / 16.0), g["hf"])


@pytest.mark.parametrize("tag", ["plain", "both"])
@pytest.mark.parametrize("bits", [4, 2])
def test_static_rows_match_reference_quantizers(golden_dir, tag, bits):
    g = np.load(golden_dir / "static_d256.npz")
    hf, km = (g["hfull"], g["kmu"]) if tag == "both" else (None, None)
    codes, words = O.static_rows_256(g["kv"], g["mask"], hf, bits, km, recip=False)
    T, H2 = g["kv"].shape[:2]
    Hkv = H2 // 2
    # half heads h' = 2 h + half back to rows [T, 2 Hkv, 256], K rows first
    q = np.concatenate([codes[:, :, 0].reshape(T, Hkv, 256), codes[:, :, 1].reshape(T, Hkv, 256)], 1)
    w = np.concatenate([words[:, :, 0].reshape(T, Hkv, 8), words[:, :, 1].reshape(T, Hkv, 8)], 1)
    assert np.array_equal(q, g[f"{tag}_q{bits}"])
    assert np.array_equal(w, g[f"{tag}_w{bits}"])


@pytest.mark.parametrize("fmt,bits", [("int4a", 4), ("int2a", 2)])
def test_half_chunk_layout_matches_reference_parsers(golden_dir, fmt, bits):
    g = np.load(golden_dir / "static_d256.npz")
    npg, Hkv = g[f"{fmt}_pool0"].shape[:2]
    codes, words = O.static_rows_256(g["kv"], g["mask"], g["hfull"], bits, g["kmu"], recip=False)
    pool = g[f"{fmt}_pool0"].copy()
    O.write_pool(pool.reshape(npg, 2 * Hkv, -1), g["slots"], codes, words, bits, P)
    assert np.array_equal(pool, g[f"{fmt}_pool"])
    raw, wd = O.parse_pool(pool.reshape(npg, 2 * Hkv, -1), bits, P)            # [npg, 2 Hkv, P, 2, 128], [.., 4]
    z = (wd & ((1 << bits) - 1)).astype(np.int16)
    c = raw.astype(np.int16) - np.repeat(z, 32, -1)

    def cat(x):                                                                 # two half heads -> one 256-d head
        return x.reshape(npg, Hkv, 2, P, 2, x.shape[-1]).transpose(0, 1, 3, 4, 2, 5).reshape(npg, Hkv, P, 2, -1)

    assert np.array_equal(cat(c), g[f"{fmt}_codes"])
    assert np.array_equal(cat(wd.view(np.int16) if wd.dtype == np.uint16 else wd.astype(np.uint16).view(np.int16)), g[f"{fmt}_sbits"])
    # stored-basis values: codes x scale, exact products
    with np.errstate(invalid="ignore", over="ignore"):
        mag = (wd.astype(np.uint16) & 0x7FFF).view(np.float16).astype(np.float64)
        val = cat(c.astype(np.float64) * np.repeat(mag, 32, -1))              # [npg, Hkv, P, 2, 256]
    for i, name in enumerate(("K", "V")):
        ref = g[f"{fmt}_{name}"].astype(np.float64)                             # [npg, P, Hkv, 256]
        mine = val[:, :, :, i].transpose(0, 2, 1, 3)
        ok = np.isfinite(ref) & np.isfinite(mine)
        assert np.array_equal(mine[ok], ref[ok])
