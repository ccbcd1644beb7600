"""Pins the numpy oracle against outputs of the reference's own PyTorch code (tests/golden/*.npz, written by
tests/golden/make_golden.py): codes, scale / flag words and choices bit for bit; page layouts against the reference's
parsers; float64 decode attention against the reference-style expectation."""
import numpy as np
import pytest

from oracle import flagrot_oracle as O

P = 16


@pytest.fixture(scope="module")
def dyn(golden_dir):
    return np.load(golden_dir / "writer_dynamic.npz")


@pytest.mark.parametrize("name", ["a", "b"])
@pytest.mark.parametrize("bits", [4, 2])
def test_dynamic_encoder_matches_reference(dyn, name, bits):
    kv = dyn[f"{name}_kv"]
    kmu = dyn[f"{name}_kmu"] if f"{name}_kmu" in dyn.files else None
    codes, words, ek = O.dynamic_rows(kv, dyn[f"{name}_Cq"], bits, kmu, recip=False)
    assert np.array_equal(codes[:, :, 0], dyn[f"{name}_{bits}_qk"])
    assert np.array_equal(codes[:, :, 1], dyn[f"{name}_{bits}_qv"])
    assert np.array_equal(words[:, :, 0], dyn[f"{name}_{bits}_wk"])
    assert np.array_equal(words[:, :, 1], dyn[f"{name}_{bits}_wv"])
    assert np.array_equal(ek["fflag"], dyn[f"{name}_{bits}_mode"] == 2)
    assert np.array_equal(ek["local"], dyn[f"{name}_{bits}_local"] == 1)
    # the criterion itself: head errors in the reference's fixed fp32 order, bit for bit
    assert np.array_equal(ek["head_errs"].view(np.uint32), dyn[f"{name}_{bits}_herr"].view(np.uint32))
    # both rotation choices occur in the fixture (otherwise the flags would be pinned vacuously)
    assert ek["fflag"].any() and ek["local"].any() and (~ek["fflag"]).any()


def test_static_writer_matches_reference(golden_dir):
    g = np.load(golden_dir / "writer_static.npz")
    for tag, hf, km in (("plain", None, None), ("hfull", g["hfull"], None), ("kmu", None, g["kmu"]),
                        ("both", g["hfull"], g["kmu"])):
        if hf is not None:
            assert np.array_equal(O.head_fwht(g["kv"], hf, 1.0 / 16.0), g[f"{tag}_hf"])
        for bits in (4, 2):
            codes, words = O.static_rows(g["kv"], g["mask"], hf, bits, km, recip=False)
            Hkv = g["kv"].shape[1] // 2
            q = np.concatenate([codes[:, :, 0], codes[:, :, 1]], 1)
            w = np.concatenate([words[:, :, 0], words[:, :, 1]], 1)
            assert q.shape[1] == 2 * Hkv
            assert np.array_equal(q, g[f"{tag}_q{bits}"]), (tag, bits)
            assert np.array_equal(w, g[f"{tag}_w{bits}"]), (tag, bits)


@pytest.mark.parametrize("kind,bits,key_only", [("konlya", 4, True), ("konlya2", 2, True), ("int4a", 4, False),
                                                ("int2a", 2, False)])
@pytest.mark.parametrize("P", [16, 32])
def test_page_layout_matches_reference_parsers(golden_dir, kind, bits, key_only, P):
    src = np.load(golden_dir / "pages.npz")
    g = src if P == 16 else np.load(golden_dir / "pages_p32.npz")       # 32-token pages: same rows, other slots
    kv, slots = src["kv"], g["slots"]
    if key_only:
        codes, words, _ = O.dynamic_rows(kv, src["Cq"], bits, None, recip=False)
    else:
        codes, words = O.static_rows(kv, src["mask"], None, bits, None, recip=False)
    pool = g[f"{kind}_pool0"].copy()
    O.write_pool(pool, slots, codes, words, bits, P)
    assert np.array_equal(pool, g[f"{kind}_pool"])
    # the oracle's parser agrees with the reference's parser on every cell of the pool (garbage cells included)
    raw, wd = O.parse_pool(pool, bits, P)
    z = (wd & ((1 << bits) - 1)).astype(np.int16)
    assert np.array_equal(raw.astype(np.int16) - np.repeat(z, 32, -1), g[f"{kind}_codes"])
    assert np.array_equal(wd.view(np.int16), g[f"{kind}_sbits"])
    with np.errstate(invalid="ignore", over="ignore"):
        Kp, Vp = O.dequant_pool(pool, bits, P, key_only)
    # (the reference dequantises and applies the inverse Hadamard in fp32 before widening; the oracle works in float64:
    # agreement to fp32 rounding of a 128-term sum.  Values are exact products: no tolerance.)
    ok = np.isfinite(g[f"{kind}_K"]) & np.isfinite(Kp) & (np.abs(g[f"{kind}_K"]) < 1e30)
    np.testing.assert_allclose(Kp[ok], g[f"{kind}_K"][ok], rtol=1e-5, atol=1e-5 * np.abs(Kp[ok]).max())
    okv = np.isfinite(g[f"{kind}_V"]) & np.isfinite(Vp)
    assert np.array_equal(Vp[okv], g[f"{kind}_V"][okv])
    # the written cells read back as what was encoded
    live = slots >= 0
    cell = raw.transpose(0, 2, 1, 3, 4).reshape(-1, *raw.shape[1:2], 2, 128)[slots[live]]
    assert np.array_equal(cell, codes[live])
    # partial writes: K-only then V-only calls give the same bytes as one call
    pool2 = g[f"{kind}_pool0"].copy()
    O.write_pool(pool2, slots, codes, words, bits, P, which="v")
    O.write_pool(pool2, slots, codes, words, bits, P, which="k")
    assert np.array_equal(pool2, pool)


@pytest.mark.parametrize("kind,bits,key_only", [("konlya", 4, True), ("konlya2", 2, True), ("int4a", 4, False),
                                                ("int2a", 2, False)])
def test_decode_reference_matches(golden_dir, kind, bits, key_only):
    g = np.load(golden_dir / "decode.npz")
    kv = g["kv"]
    B, L = kv.shape[:2]
    Hkv = kv.shape[2] // 2
    bt = g["bt"]
    npg = B * (L // P) + 7
    rows = kv.reshape(B * L, 2 * Hkv, 128)
    slots = (bt.astype(np.int64)[:, np.arange(L) // P] * P + np.arange(L) % P).reshape(-1)
    pool = np.random.RandomState(7).randint(0, 256, (npg, Hkv, O.chunk_bytes(bits, P)), dtype=np.uint8)
    if key_only:
        codes, words, _ = O.dynamic_rows(rows, g["Cq"], bits, None, recip=False)
    else:
        codes, words = O.static_rows(rows, g["mask"], None, bits, None, recip=False)
    O.write_pool(pool, slots, codes, words, bits, P)
    km = None if key_only else g["mask"][:Hkv]
    vm = None if key_only else g["mask"][Hkv:]
    lens = g["lens"]
    o = O.decode_reference(g["q"], pool, bt, lens, float(g["scale"]), bits, P, key_only, km, vm)
    np.testing.assert_allclose(o, g[f"{kind}_plain"], rtol=0, atol=2e-5)
    o = O.decode_reference(g["q"], pool, bt, lens, float(g["scale"]), bits, P, key_only, km, vm, tail=g["ring"],
                           tail_len=g["tail_len"], tail_idx=g["tail_idx"], kv_start=int(g["kv_start"]))
    np.testing.assert_allclose(o, g[f"{kind}_tail"], rtol=0, atol=2e-5)


def test_recip_mode_differs_only_through_the_scale():
    """the GPU arithmetic (multiply by fp32(1 / lv)) changes the scale by at most one ulp; codes move by at most one step."""
    rs = np.random.RandomState(5)
    y = rs.randn(4096, 128).astype(np.float32)
    for bits in (4, 2):
        q0, w0 = O.quant_asym_store(y, bits, recip=False)
        q1, w1 = O.quant_asym_store(y, bits, recip=True)
        assert np.abs(q0.astype(int) - q1.astype(int)).max() <= 1
        assert (q0 != q1).mean() < 0.02
        assert np.abs((w0 >> bits) - (w1 >> bits)).max() <= 1


@pytest.mark.parametrize("D", [128, 256])
def test_head_fwht_is_the_sylvester_matrix(D):
    """small integers: every partial sum is exact in fp32, so the butterflies must equal the matrix product, and the
    bf16 rounding of scale * y is exact for |y| / 16 below 2^8"""
    rs = np.random.RandomState(D)
    x = rs.randint(-1, 2, (5, 3, D)).astype(np.float32)
    H = np.array([[1.0]])
    while H.shape[0] < D:
        H = np.block([[H, H], [H, -H]])
    assert np.array_equal(O.fwht_unnorm(x, D), x.astype(np.float64) @ H)
    xb = O.f32_to_bf16_bits(x)
    flags = np.array([1, 0, 1], np.uint8)
    y = O.bf16_bits_to_f32(O.head_fwht(xb, flags, 1.0 / 16.0))
    exp = O.bf16_bits_to_f32(O.f32_to_bf16_bits((x.astype(np.float64) @ H / 16).astype(np.float32)))
    assert np.array_equal(y[:, 0], exp[:, 0]) and np.array_equal(y[:, 2], exp[:, 2]) and np.array_equal(y[:, 1], x[:, 1])
