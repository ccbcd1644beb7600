"""Pins the symmetric INT4 (`int4`) part of oracle/flagrot_oracle.py to the reference's own PyTorch code
(tests/golden/sym_int4.npz, written by tests/golden/make_golden_sym.py): quantiser codes and FP16 scale words bit for bit,
the sign-magnitude page layout against the reference's parser."""
import numpy as np
import pytest

from oracle import flagrot_oracle as O


@pytest.fixture(scope="module")
def g(golden_dir):
    return np.load(golden_dir / "sym_int4.npz"), np.load(golden_dir / "writer_static.npz")


@pytest.mark.parametrize("tag,hf,km", [("plain", False, False), ("hfull", True, False), ("kmu", False, True), ("both", True, True)])
def test_static_rows_bit_exact(g, tag, hf, km):
    s, w = g
    q, words = O.static_rows_sym(w["kv"], w["mask"], w["hfull"] if hf else None, w["kmu"] if km else None)
    Hkv = w["kv"].shape[1] // 2
    qref = s[f"{tag}_q"].astype(np.int16) - 8                                        # [T, 2 Hkv, 128]
    sref = s[f"{tag}_s"]
    assert np.array_equal(q[:, :, 0], qref[:, :Hkv]) and np.array_equal(q[:, :, 1], qref[:, Hkv:])
    assert np.array_equal(words[:, :, 0], sref[:, :Hkv]) and np.array_equal(words[:, :, 1], sref[:, Hkv:])
    assert (np.abs(q) == 7).any() and (q == 0).any()


def test_page_layout_matches_reference_parser(g):
    s, _ = g
    codes, words = O.parse_pool_sym(s["pool"], 16)                                   # [Np, H, P, 2, 128]
    assert np.array_equal(codes, s["pool_codes"])
    assert np.array_equal(O.word_value(words).astype(np.float32), s["pool_mag"])
    K, V = O.dequant_pool_sym(s["pool"], 16, key_only=False)                         # [Np, P, H, 128]
    np.testing.assert_allclose(K, s["pool_K"], rtol=0, atol=1e-12)
    np.testing.assert_allclose(V, s["pool_V"], rtol=0, atol=1e-12)


def test_pack_parse_round_trip():
    rs = np.random.RandomState(2)
    P, Hkv, T = 32, 3, 100
    q = rs.randint(-7, 8, (T, Hkv, 2, 128)).astype(np.int8)
    w = rs.randint(0x1C00, 0x2C00, (T, Hkv, 2, 4)).astype(np.int32)
    pool0 = rs.randint(0, 256, (5, Hkv, 144 * P), dtype=np.uint8)
    pool = pool0.copy()
    slots = rs.permutation(5 * P)[:T]
    slots[::9] = -1
    O.write_pool_sym(pool, slots, q, w, P)
    c, ww = O.parse_pool_sym(pool, P)
    ok = slots >= 0
    pg, pos = slots[ok] // P, slots[ok] % P
    assert np.array_equal(c[pg, :, pos], q[ok]) and np.array_equal(ww[pg, :, pos].astype(np.int32), w[ok])
    # cells that were not written keep their bytes: every unwritten (page, position) parses as before
    c0, w0 = O.parse_pool_sym(pool0, P)
    untouched = np.ones((5, P), bool)
    untouched[pg, pos] = False
    assert np.array_equal(c[untouched.nonzero()[0], :, untouched.nonzero()[1]], c0[untouched.nonzero()[0], :, untouched.nonzero()[1]])


@pytest.mark.parametrize("name", ["a", "b"])
def test_dynamic_konly_encoder_matches_reference(g, golden_dir, name):
    s, _ = g
    d = np.load(golden_dir / "writer_dynamic.npz")
    kmu = d[f"{name}_kmu"] if f"{name}_kmu" in d.files else None
    codes, words, ek = O.dynamic_rows_sym(d[f"{name}_kv"], d[f"{name}_Cq"], kmu)
    assert np.array_equal(codes[:, :, 0], s[f"{name}_qk"]) and np.array_equal(codes[:, :, 1], s[f"{name}_qv"])
    assert np.array_equal(words[:, :, 0], s[f"{name}_wk"]) and np.array_equal(words[:, :, 1], s[f"{name}_wv"])
    assert np.array_equal(ek["fflag"], s[f"{name}_mode"] == 2) and np.array_equal(ek["local"], s[f"{name}_local"] == 1)
    assert np.array_equal(ek["head_errs"].view(np.uint32), s[f"{name}_herr"].view(np.uint32))
    assert ek["fflag"].any() and ek["local"].any() and (~ek["fflag"]).any()
