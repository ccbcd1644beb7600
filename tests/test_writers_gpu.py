"""GPU parity of the paged cache writers, through the C ABI (ctypes front end), against the numpy oracle in GPU
arithmetic (recip=True) and, where oracle/_ref holds the reference's own writer built for sm_100a, against that library
byte for byte.  Pools are pre-filled with random bytes and compared whole: bytes that a call must not touch stay put."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import flagrot_oracle as O
from tests._util import P, bits, calib, edge_rows, ref_lib, slot_patterns, strided_kv

pytestmark = pytest.mark.gpu
DEV = "cuda"
HKV = 8


@pytest.fixture(scope="module")
def K():
    from flagrot_releaser_b200 import kernels
    kernels.lib()
    return kernels


@pytest.mark.parametrize("D", [128, 256])
def test_head_fwht_bit_exact(K, D):
    g = torch.Generator().manual_seed(7)
    for T, H in ((1, 32), (5, 16), (300, 8)):
        base = torch.randn(T, H + 3, D, generator=g).bfloat16().to(DEV)
        x = base[:, 1:H + 1]
        flags = (torch.rand(H, generator=g) < 0.5).to(torch.uint8)
        y = K.head_fwht(x, flags.to(DEV), 1 / 16)                            # (1 / 16: the orthonormal scale of D = 256)
        exp = O.head_fwht(bits(x), flags.numpy(), 1 / 16)
        assert np.array_equal(bits(y), exp)
        xc = x.contiguous()
        K.head_fwht(xc, flags.to(DEV), 1 / 16, out=xc)                       # in place
        assert torch.equal(xc, y)
        assert torch.equal(y[:, ~flags.bool()], x[:, ~flags.bool()])


@pytest.mark.parametrize("fmt,nb", [("int4a", 4), ("int2a", 2), ("int4", 4)])
@pytest.mark.parametrize("T", [1, 7, 64, 129, 257, 1000])
def test_static_writer_vs_oracle(K, fmt, nb, T):
    g = torch.Generator().manual_seed(100 + T + nb)
    kvb = edge_rows(T, HKV, g)
    kv = strided_kv(kvb, DEV)
    npg = (T + P - 1) // P + 5
    kmu = (torch.randn(HKV, 128, generator=g) * 0.5).float()
    for smode, slots in slot_patterns(T, npg, g).items():
        for hmode in ("none", "rand"):
            for bmode in ("zero", "rand"):
                for cen in (False, True):
                    hfull = (torch.rand(2 * HKV, generator=g) < 0.5).to(torch.uint8) if hmode == "rand" else None
                    mask = ((torch.rand(2 * HKV, 4, generator=g) < 0.5) & (bmode == "rand")).to(torch.uint8)
                    pool0 = torch.randint(0, 256, (npg, HKV, K.v2_chunk_bytes(P, 128, fmt)), dtype=torch.uint8, generator=g)
                    exp = pool0.numpy().copy()
                    if fmt == "int4":       # symmetric: sign-magnitude codes, plain FP16 scale words
                        codes, words = O.static_rows_sym(bits(kvb), mask.numpy(), None if hfull is None else hfull.numpy(),
                                                         kmu.numpy() if cen else None)
                        O.write_pool_sym(exp, slots.numpy(), codes, words, P)
                    else:
                        codes, words = O.static_rows(bits(kvb), mask.numpy(), None if hfull is None else hfull.numpy(), nb,
                                                     kmu.numpy() if cen else None, recip=True)
                        O.write_pool(exp, slots.numpy(), codes, words, nb, P)
                    pool = pool0.clone().to(DEV)
                    K.w3_static_write(kv, slots.to(DEV), mask.to(DEV), None if hfull is None else hfull.to(DEV), pool, P,
                                      fmt=fmt, kmu=kmu.to(DEV) if cen else None)
                    torch.cuda.synchronize()
                    assert np.array_equal(pool.cpu().numpy(), exp), (smode, hmode, bmode, cen)
                    if hfull is None:   # the unfused entry gives the same bytes
                        pool = pool0.clone().to(DEV)
                        K.v2_write(kv, slots.to(DEV), mask.to(DEV), 32, pool, P, fmt=fmt, kmu=kmu.to(DEV) if cen else None)
                        torch.cuda.synchronize()
                        assert np.array_equal(pool.cpu().numpy(), exp), ("v2_write", smode, bmode, cen)
                    else:               # ... and so does head_fwht followed by the unfused entry
                        pool = pool0.clone().to(DEV)
                        x = K.head_fwht(kv, hfull.to(DEV), 1 / 16)
                        K.v2_write(x, slots.to(DEV), mask.to(DEV), 32, pool, P, fmt=fmt, kmu=kmu.to(DEV) if cen else None)
                        torch.cuda.synchronize()
                        assert np.array_equal(pool.cpu().numpy(), exp), ("fwht+v2_write", smode, bmode, cen)


@pytest.mark.parametrize("kind,nb", [("konlya", 4), ("konlya2", 2), ("konly", 4)])
@pytest.mark.parametrize("T", [1, 7, 64, 129, 300, 521])
def test_dynamic_writer_vs_oracle(K, kind, nb, T):
    g = torch.Generator().manual_seed(200 + T + nb)
    kvb = edge_rows(T, HKV, g)
    kv = strided_kv(kvb, DEV)
    Cq, co = calib(HKV, g)
    CT = Cq.transpose(1, 2).contiguous().to(DEV)
    npg = (T + P - 1) // P + 5
    kmu = (torch.randn(HKV, 128, generator=g) * 0.5).float()
    for cen in (False, True):
        if kind == "konly":     # symmetric INT4: one quantiser form, sign-magnitude pages
            codes, words, ek = O.dynamic_rows_sym(bits(kvb), Cq.numpy(), kmu.numpy() if cen else None)
        else:
            codes, words, ek = O.dynamic_rows(bits(kvb), Cq.numpy(), nb, kmu.numpy() if cen else None, recip=True)
        if T >= 64:
            assert ek["fflag"].any() and ek["local"].any()
        for smode, slots in slot_patterns(T, npg, g).items():
            pool0 = torch.randint(0, 256, (npg, HKV, K.cb_chunk_bytes(kind, P)), dtype=torch.uint8, generator=g)
            exp = pool0.numpy().copy()
            if kind == "konly":
                O.write_pool_sym(exp, slots.numpy(), codes, words, P)
            else:
                O.write_pool(exp, slots.numpy(), codes, words, nb, P)
            km = kmu.to(DEV) if cen else None
            for how in ("v1", "v3", "v3split"):
                pool = pool0.clone().to(DEV)
                if how == "v1":
                    K.cb_write(kv, slots.to(DEV), CT, co.to(DEV), kind, pool, P, kmu=km)
                else:
                    K.cb_write3(kv, slots.to(DEV), CT, co.to(DEV), None, None, kind, pool, P, split=how == "v3split", kmu=km)
                torch.cuda.synchronize()
                got = pool.cpu().numpy()
                assert np.array_equal(got, exp), (how, smode, cen, int((got != exp).sum()))


@pytest.mark.parametrize("T", [7, 257])
def test_writers_32_token_pages_vs_oracle(K, T):
    """pages of 32 tokens (the reference dispatches page 16 and 32: kernels/csrc/attn_decode_v2.cu:2018-2060): static and
    dynamic writers, whole pools byte for byte against the oracle packed with P = 32"""
    P32 = 32
    g = torch.Generator().manual_seed(700 + T)
    kvb = edge_rows(T, HKV, g)
    kv = kvb.to(DEV)
    npg = (T + P32 - 1) // P32 + 4
    slots = torch.randperm(npg * P32, generator=g)[:T].to(torch.int64)
    slots[::9] = -1
    mask = (torch.rand(2 * HKV, 4, generator=g) < 0.5).to(torch.uint8)
    hfull = (torch.rand(2 * HKV, generator=g) < 0.4).to(torch.uint8)
    Cq, co = calib(HKV, g)
    CT = Cq.transpose(1, 2).contiguous().to(DEV)
    for fmt, kind, nb in (("int4a", "konlya", 4), ("int2a", "konlya2", 2)):
        pool0 = torch.randint(0, 256, (npg, HKV, K.v2_chunk_bytes(P32, 128, fmt)), dtype=torch.uint8, generator=g)
        codes, words = O.static_rows(bits(kvb), mask.numpy(), hfull.numpy(), nb, None, recip=True)
        exp = pool0.numpy().copy()
        O.write_pool(exp, slots.numpy(), codes, words, nb, P32)
        pool = pool0.clone().to(DEV)
        K.w3_static_write(kv, slots.to(DEV), mask.to(DEV), hfull.to(DEV), pool, P32, fmt=fmt)
        torch.cuda.synchronize()
        assert np.array_equal(pool.cpu().numpy(), exp), (fmt, int((pool.cpu().numpy() != exp).sum()))
        codes, words, _ = O.dynamic_rows(bits(kvb), Cq.numpy(), nb, None, recip=True)
        exp = pool0.numpy().copy()
        O.write_pool(exp, slots.numpy(), codes, words, nb, P32)
        pool = pool0.clone().to(DEV)
        K.cb_write(kv, slots.to(DEV), CT, co.to(DEV), kind, pool, P32)
        torch.cuda.synchronize()
        assert np.array_equal(pool.cpu().numpy(), exp), (kind, int((pool.cpu().numpy() != exp).sum()))


def test_writer_two_calls_commute(K):
    """value half before key half gives the same bytes (bit 15 of the V group-0 word belongs to the key half)."""
    g = torch.Generator().manual_seed(5)
    T = 77
    kvb = edge_rows(T, HKV, g)
    kv = kvb.to(DEV)
    Cq, co = calib(HKV, g)
    CT = Cq.transpose(1, 2).contiguous().to(DEV)
    npg = 12
    slots = torch.randperm(npg * P, generator=g)[:T].to(torch.int64).to(DEV)
    L = K.lib()
    for kind, nb in (("konlya", 4), ("konlya2", 2)):
        pool0 = torch.randint(0, 256, (npg, HKV, K.cb_chunk_bytes(kind, P)), dtype=torch.uint8, generator=g).to(DEV)
        a, b = pool0.clone(), pool0.clone()
        K.cb_write(kv, slots, CT, co.to(DEV), kind, a, P)
        st = torch.cuda.current_stream().cuda_stream
        args = (kv.data_ptr(), kv.stride(0), slots.data_ptr(), 0, T, HKV, P, CT.data_ptr(), co.to(DEV).data_ptr(), None, None,
                K.sign_words(), K.CB_KINDS[kind], b.data_ptr())
        assert L.fr_cb_write3(*args, -1, 1, st, None) == 0
        assert L.fr_cb_write3(*args, 1, -1, st, None) == 0
        torch.cuda.synchronize()
        assert torch.equal(a, b)


def test_writer_error_codes(K):
    L = K.lib()
    z = torch.zeros(64, dtype=torch.uint8, device=DEV)
    assert L.fr_v2_write(6, z.data_ptr(), 0, z.data_ptr(), 1, 1, 16, None, 32, z.data_ptr(), None, 128, None) == -4
    assert L.fr_v2_write(5, z.data_ptr(), 0, z.data_ptr(), 1, 1, 8, None, 32, z.data_ptr(), None, 128, None) == -5
    assert L.fr_v2_write(5, z.data_ptr(), 0, z.data_ptr(), 1, 1, 16, None, 32, z.data_ptr(), None, 64, None) == -8    # head dims other than 128 and 256
    assert L.fr_v2_write(5, z.data_ptr(), 0, z.data_ptr(), 0, 1, 16, None, 32, z.data_ptr(), None, 128, None) == 0   # T = 0
    assert L.fr_cb_write(z.data_ptr(), 0, z.data_ptr(), 0, 1, 1, 16, 1, z.data_ptr(), z.data_ptr(), K.sign_words(), 3,
                         z.data_ptr(), None, 128, None) == -4
    assert L.fr_head_fwht(z.data_ptr(), 0, z.data_ptr(), 0, 1, 1, z.data_ptr(), 1.0, None, 64) == -8
    assert L.fr_w3_static_write(z.data_ptr(), 0, z.data_ptr(), 1, 1, 16, None, None, 3, z.data_ptr(), 0, None, None) == -4


def test_all_slots_skipped_leaves_pool_untouched(K):
    g = torch.Generator().manual_seed(9)
    kv = edge_rows(9, HKV, g).to(DEV)
    Cq, co = calib(HKV, g)
    slots = torch.full((9,), -1, dtype=torch.int64, device=DEV)
    pool0 = torch.randint(0, 256, (4, HKV, 2304), dtype=torch.uint8, generator=g).to(DEV)
    pool = pool0.clone()
    K.cb_write(kv, slots, Cq.transpose(1, 2).contiguous().to(DEV), co.to(DEV), "konlya", pool, P)
    K.w3_static_write(kv, slots, None, None, pool, P, fmt="int4a")
    torch.cuda.synchronize()
    assert torch.equal(pool, pool0)


# ------------------------------------------------------------------ against the reference's own CUDA writer
def _ref():
    L = ref_lib("libflagrot_w3ref.so")
    if L is None:
        pytest.skip("oracle/_ref/libflagrot_w3ref.so not built")
    Pp, I, LL = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    L.fr_cb_write3.argtypes = [Pp, LL, Pp, I, I, I, I, Pp, Pp, Pp, Pp, Pp, I, Pp, I, I, Pp, Pp]
    L.fr_w3_static_write.argtypes = [Pp, LL, Pp, I, I, I, Pp, Pp, I, Pp, I, Pp, Pp]
    L.fr_head_fwht.argtypes = [Pp, LL, Pp, LL, I, I, Pp, ctypes.c_float, Pp, I]
    return L


def ref_writer_tables(Cq):
    """host tables that the reference's fused writer takes besides C_q^T (layout: reference
    kernels/csrc/attn_codebook.cuh:96-100): an fp16 image C1 of the symmetrised C_q scaled by a power of two, and
    per-block bounds on what ranking candidates with C1 instead of C_q can get wrong.  The reference resolves every
    candidate pair its bound cannot separate with its exact fp32 path, so any valid bound yields the same bytes.  This
    test uses no correction rows (rows 128.. stay zero) and the correspondingly larger bound
    ||E||_2 (1 + 2^-10) + 2^-16 rho(|C|), E = scaled C_sym - C1, +1 %.  Only needed to drive the reference library."""
    C = Cq.double()
    H = C.shape[0]
    Cs = (C + C.transpose(1, 2)) / 2
    amax = Cs.abs().amax((1, 2)).clamp_min(1e-300)
    sc = (2.0 ** torch.floor(torch.log2(2.0 ** 14 / amax)))[:, None, None]
    C1 = (Cs * sc).float().half()
    E = Cs * sc - C1.double()
    M = (C.abs() + C.abs().transpose(1, 2)) / 2 * sc
    rho = lambda X: torch.linalg.eigvalsh(X).abs().amax(-1)  # noqa: E731
    tab = torch.zeros(H, 168, 128, dtype=torch.float16)
    tab[:, :128] = C1
    aux = torch.zeros(H, 48, dtype=torch.float64)
    for bi, (lo, hi) in enumerate([(0, 128)] + [(32 * j, 32 * j + 32) for j in range(4)]):
        aux[:, bi] = (rho(E[:, lo:hi, lo:hi]) * (1 + 2.0 ** -10) + 2.0 ** -16 * rho(M[:, lo:hi, lo:hi])) * 1.01
        aux[:, 8 + 8 * bi:16 + 8 * bi] = torch.arange(lo, lo + 8, dtype=torch.float64)
    aux[:, 5] = 2.0 ** -40 * rho(M)
    return tab.contiguous(), aux.float().contiguous()


@pytest.mark.parametrize("T", [1, 64, 257, 700, 1000, 4097])
def test_dynamic_writer_vs_reference_library(K, T):
    R = _ref()
    g = torch.Generator().manual_seed(300 + T)
    kv = edge_rows(T, HKV, g).to(DEV)
    Cq, co = calib(HKV, g)
    CT = Cq.transpose(1, 2).contiguous().to(DEV)
    C1, beta = ref_writer_tables(Cq)
    C1, beta, cod = C1.to(DEV), beta.to(DEV), co.to(DEV)
    npg = (T + P - 1) // P + 5
    kmu = (torch.randn(HKV, 128, generator=g) * 0.5).float().to(DEV)
    st = torch.cuda.current_stream().cuda_stream
    nk, nv = max(1, 2 * 148 // HKV), max(1, 3 * 148 // HKV)
    for kind in ("konlya", "konlya2", "konly"):
        for smode, slots in slot_patterns(T, npg, g).items():
            slots = slots.to(DEV)
            for km in (None, kmu):
                pool0 = torch.randint(0, 256, (npg, HKV, K.cb_chunk_bytes(kind, P)), dtype=torch.uint8, generator=g).to(DEV)
                a, b = pool0.clone(), pool0.clone()
                rc = R.fr_cb_write3(kv.data_ptr(), kv.stride(0), slots.data_ptr(), 0, T, HKV, P, CT.data_ptr(), cod.data_ptr(),
                                    C1.data_ptr(), beta.data_ptr(), K.sign_words(), K.CB_KINDS[kind], a.data_ptr(), nk, nv, st,
                                    None if km is None else km.data_ptr())
                assert rc == 0
                K.cb_write(kv, slots, CT, cod, kind, b, P, kmu=km)
                torch.cuda.synchronize()
                assert torch.equal(a, b), (kind, smode, km is not None, int((a != b).sum()))


@pytest.mark.parametrize("T", [1, 64, 257, 1000, 4097])
def test_static_writer_vs_reference_library(K, T):
    R = _ref()
    g = torch.Generator().manual_seed(400 + T)
    kv = edge_rows(T, HKV, g).to(DEV)
    npg = (T + P - 1) // P + 5
    kmu = (torch.randn(HKV, 128, generator=g) * 0.5).float().to(DEV)
    st = torch.cuda.current_stream().cuda_stream
    for fmt, asym in (("int4a", 1), ("int2a", 2), ("int4", 0)):
        for smode, slots in slot_patterns(T, npg, g).items():
            slots = slots.to(DEV)
            for hm in (False, True):
                hfull = (torch.rand(2 * HKV, generator=g) < 0.5).to(torch.uint8).to(DEV) if hm else None
                mask = (torch.rand(2 * HKV, 4, generator=g) < 0.5).to(torch.uint8).to(DEV)
                for km in (None, kmu):
                    pool0 = torch.randint(0, 256, (npg, HKV, K.v2_chunk_bytes(P, 128, fmt)), dtype=torch.uint8, generator=g).to(DEV)
                    a, b = pool0.clone(), pool0.clone()
                    rc = R.fr_w3_static_write(kv.data_ptr(), kv.stride(0), slots.data_ptr(), T, HKV, P, mask.data_ptr(),
                                              None if hfull is None else hfull.data_ptr(), asym, a.data_ptr(), 0, st,
                                              None if km is None else km.data_ptr())
                    assert rc == 0
                    K.w3_static_write(kv, slots, mask, hfull, b, P, fmt=fmt, kmu=km)
                    torch.cuda.synchronize()
                    assert torch.equal(a, b), (fmt, smode, hm, km is not None, int((a != b).sum()))


@pytest.mark.parametrize("D", [128, 256])
def test_head_fwht_vs_reference_library(K, D):
    """the whole-head Hadamard against the reference's own kernels (k_head_fwht / k_head_fwht256), strided rows included"""
    R = _ref()
    g = torch.Generator().manual_seed(500 + D)
    st = torch.cuda.current_stream().cuda_stream
    for T, H in ((1, 4), (33, 16), (1000, 8)):
        base = (torch.randn(T, H + 2, D, generator=g) * torch.exp2(torch.randint(-6, 7, (T, H + 2, 1), generator=g).float())).bfloat16().to(DEV)
        x = base[:, 1:H + 1]
        flags = (torch.rand(H, generator=g) < 0.6).to(torch.uint8).to(DEV)
        a = torch.empty(T, H, D, dtype=torch.bfloat16, device=DEV)
        assert R.fr_head_fwht(x.data_ptr(), x.stride(0), a.data_ptr(), a.stride(0), T, H, flags.data_ptr(), 1 / 16, st, D) == 0
        b = K.head_fwht(x, flags, 1 / 16)
        torch.cuda.synchronize()
        assert torch.equal(a.view(torch.int16), b.view(torch.int16)), (T, H)


@pytest.mark.parametrize("fmt,nb", [("int4a", 4), ("int2a", 2)])
@pytest.mark.parametrize("page", [16, 32])
def test_static_writer_head_dim_256(K, fmt, nb, page):
    """head dim 256: fr_head_fwht (H256 / 16 on flagged heads) + fr_v2_write(hd = 256), two 128-d half chunks per (page,
    kv head), against the oracle's bytes; untouched bytes stay untouched"""
    g = torch.Generator().manual_seed(2560 + nb + page)
    for T in (1, 45, 300):
        kv = torch.cat([edge_rows(T, HKV, g), edge_rows(T, HKV, g)], -1).to(DEV)            # [T, 2 Hkv, 256]
        npg = (T + page - 1) // page + 3
        mask = (torch.rand(2 * HKV, 8, generator=g) < 0.5).to(torch.uint8)
        hfull = (torch.rand(2 * HKV, generator=g) < 0.5).to(torch.uint8)
        kmu = (torch.randn(HKV, 256, generator=g) * 0.5).float()
        slots = torch.randperm(npg * page, generator=g)[:T].long()
        slots[torch.rand(T, generator=g) < 0.1] = -1
        pool0 = torch.randint(0, 256, (npg, HKV, K.v2_chunk_bytes(page, 256, fmt)), dtype=torch.uint8, generator=g)
        for km in (None, kmu):
            pool = pool0.clone().to(DEV)
            x = K.head_fwht(kv, hfull.to(DEV), 1 / 16)
            K.v2_write(x, slots.to(DEV), mask.to(DEV), 32, pool, page, fmt=fmt, kmu=None if km is None else km.to(DEV))
            torch.cuda.synchronize()
            codes, words = O.static_rows_256(bits(kv), mask.numpy(), hfull.numpy(), nb, None if km is None else km.numpy())
            exp = pool0.numpy().copy()
            O.write_pool(exp.reshape(npg, 2 * HKV, -1), slots.numpy(), codes, words, nb, page)
            got = pool.cpu().numpy()
            assert np.array_equal(got, exp), (T, km is not None, int((got != exp).sum()))


@pytest.mark.parametrize("kind", ["konlya", "konlya2", "konly"])
def test_bulk_key_writer_estimate_and_exact_sums_agree(K, kind):
    """the bulk key writer decides most head choices from a tensor-core estimate with an error bar and the rest from the
    exact fixed-order sums: both routes must give the same bytes, and the estimate must actually decide something"""
    g = torch.Generator().manual_seed(77)
    T = 3001
    Cq, co = calib(HKV, g)
    CT, cod = Cq.transpose(1, 2).contiguous().to(DEV), co.to(DEV)
    npg = (T + P - 1) // P + 3
    slots = torch.randperm(npg * P, generator=g)[:T].long().to(DEV)
    rows = {"edge": edge_rows(T, HKV, g), "normal": torch.randn(T, 2 * HKV, 128, generator=g).bfloat16(),
            "tiny": (torch.randn(T, 2 * HKV, 128, generator=g) * 1e-18).bfloat16(),
            "huge": (torch.randn(T, 2 * HKV, 128, generator=g) * 1e18).bfloat16()}
    try:
        for name, kv in rows.items():
            kv = kv.to(DEV)
            pool0 = torch.randint(0, 256, (npg, HKV, K.cb_chunk_bytes(kind, P)), dtype=torch.uint8, generator=g).to(DEV)
            a, b = pool0.clone(), pool0.clone()
            K.lib().fr_dyn_writer_exact_only(0)
            K.dyn_writer_stats(reset=True)
            K.cb_write(kv, slots, CT, cod, kind, a, P)
            pairs, exact = K.dyn_writer_stats()
            assert pairs == T * HKV, (name, pairs)
            if name in ("edge", "normal"):
                assert exact < pairs // 2, (name, pairs, exact)
            K.lib().fr_dyn_writer_exact_only(1)
            K.dyn_writer_stats(reset=True)
            K.cb_write(kv, slots, CT, cod, kind, b, P)
            assert K.dyn_writer_stats() == (T * HKV, T * HKV)
            assert torch.equal(a, b), (name, int((a != b).sum()))
    finally:
        K.lib().fr_dyn_writer_exact_only(0)
