"""CPU restatement (numpy) of the FlagRot KV-cache hot path: quantizers, selective rotation, the key-only 2x2 dynamic
encoder, the static writer, the paged byte layouts (packer + parser) and float64 decode attention over parsed pages.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this module; it is the checker used by tests/,
__graft_entry__.smoke() and the cpu_baseline / reference legs of bench.py.

Every function cites the reference file:line it restates (paths relative to the reference project root).  Parity is
pinned: tests/golden/*.npz hold outputs of the reference's own PyTorch code (kernels/ref.py, kernels/codebook_ref.py,
blockflag/formats.py, vllm_flagrot/kernels.py parsers) run on CPU on seeded inputs, produced by tests/golden/make_golden.py;
tests/test_oracle_golden.py checks this module against them bit for bit.

Arithmetic note (`recip`): the reference's scale is `(max - min) / lv` with a Python scalar `lv`.  torch on CPU performs a
true IEEE division; torch on CUDA and the reference's CUDA kernels multiply by fp32(1 / lv)
(kernels/csrc/attn_cb_common.cuh:55-58, kernels/csrc/attn_decode_v2.cu:1701-1711).  recip=False reproduces the CPU
reference (what the golden vectors pin), recip=True the GPU arithmetic (what the CUDA writers are compared with).
All other operations are single, separately rounded fp32 operations in the reference's order.
"""
from __future__ import annotations

import math

import numpy as np

F32 = np.float32
D, RB, NG = 128, 32, 4

# ------------------------------------------------------------------------------------------------ bf16 helpers


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    """uint16 bf16 bit patterns -> float32 values (exact)."""
    return (bits.astype(np.uint32) << np.uint32(16)).view(F32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit patterns, round to nearest even (finite inputs)."""
    u = np.ascontiguousarray(x, dtype=F32).view(np.uint32)
    r = ((u >> np.uint32(16)) & np.uint32(1)) + np.uint32(0x7FFF)
    return ((u + r) >> np.uint32(16)).astype(np.uint16)


def bf16_round(x: np.ndarray) -> np.ndarray:
    return bf16_bits_to_f32(f32_to_bf16_bits(x))


# ------------------------------------------------------------------------------------------------ Hadamard
def fwht_unnorm(x: np.ndarray, B: int) -> np.ndarray:
    """Sylvester butterflies (a + b, a - b), stages h = 1, 2, 4, ... in fp32, no scaling (kernels/ref.py:22-32)."""
    shp = x.shape
    K = shp[-1]
    y = np.asarray(x, dtype=F32).reshape(-1, K // B, B)
    h = 1
    while h < B:
        y = y.reshape(-1, K // B, B // (2 * h), 2, h)
        a, b = y[..., 0, :], y[..., 1, :]
        y = np.stack((a + b, a - b), axis=-2)
        h *= 2
    return y.reshape(shp)


def fwht(x: np.ndarray, B: int) -> np.ndarray:
    """block-diagonal orthonormal Hadamard along the last dim: butterflies then one multiply by fp32(1 / sqrt(B))
    (kernels/ref.py:22-33)."""
    return fwht_unnorm(x, B) * F32(1.0 / math.sqrt(B))


def sel_fwht_rb(x: np.ndarray, mask: np.ndarray, rb: int) -> np.ndarray:
    """element k rotated iff mask[k // rb] (kernels/ref.py:36-42); x [..., K], mask with K / rb elements."""
    m = np.asarray(mask).reshape(-1).astype(bool)
    if not m.any():
        return np.asarray(x, dtype=F32)
    y = fwht(x, rb)
    return np.where(np.repeat(m, rb), y, np.asarray(x, dtype=F32))


def head_fwht(x_bits: np.ndarray, flags: np.ndarray, scale: float) -> np.ndarray:
    """whole-head Hadamard of selected heads: out = flags[h] ? bf16(scale * H_D x) : x, with the unnormalised +-1
    Sylvester H_D in fp32 and one bf16 rounding (integrations/vllm_flagrot/csrc/flagrot_capi.cu:160-197).
    x_bits uint16 [T, H, D] -> uint16 [T, H, D]."""
    x = bf16_bits_to_f32(x_bits)
    y = fwht_unnorm(x, x.shape[-1]) * F32(scale)
    yb = f32_to_bf16_bits(y)
    f = np.asarray(flags).astype(bool)[None, :, None]
    return np.where(f, yb, x_bits)


# ------------------------------------------------------------------------------------------------ quantizers
def scale_word(s: np.ndarray, z: np.ndarray, bits: int = 4) -> np.ndarray:
    """FP16 bit pattern nearest (integer distance, ties up) to RN_fp16(s) whose `bits` low bits equal z, clamped to
    [0, 0x7C00 - 2^bits] (blockflag/formats.py:135-146,168-174; kernels/csrc/attn_cb_common.cuh:48-54)."""
    h = np.asarray(s, dtype=F32).astype(np.float16).view(np.uint16).astype(np.int32)
    zi = np.asarray(z).astype(np.int32)
    m = 1 << bits
    x = np.minimum(np.maximum(h - zi + m // 2, 0) & ~(m - 1), 0x7C00 - m)
    return (x + zi).astype(np.int32)


def word_value(wd: np.ndarray) -> np.ndarray:
    """scale word (sign bit masked) read as FP16 -> fp32 (blockflag/formats.py:148-149)."""
    return (np.asarray(wd).astype(np.uint16) & np.uint16(0x7FFF)).view(np.float16).astype(F32)


def _grp(v: np.ndarray, g: int = RB) -> np.ndarray:
    v = np.asarray(v, dtype=F32)
    return v.reshape(*v.shape[:-1], v.shape[-1] // g, g)


def _asym_params(mn, mx, bits, recip):
    lv = (1 << bits) - 1
    d = mx - mn
    s = d * (F32(1.0) / F32(lv)) if recip else d / F32(lv)
    s = np.maximum(s, F32(1e-12))
    z = np.rint(-mn / s)
    return s, z


def quant_asym_store(y: np.ndarray, bits: int = 4, recip: bool = True):
    """stored form of the asymmetric quantizer (int4ah:32 / int2ah:32), groups of 32 along the last dim: range widened
    to include 0, s = max((max' - min') / lv, 1e-12), z = rne(-min' / s), q = clamp(rne(y / s) + z, 0, lv)
    (blockflag/formats.py:153-165; kernels/csrc/attn_decode_v2.cu:1704-1715).
    Returns codes uint8 [..., D] and scale words int32 [..., D / 32] (z in the low bits, no flag)."""
    b = _grp(y)
    lv = (1 << bits) - 1
    mn = np.minimum(b.min(-1, keepdims=True), F32(0.0))
    mx = np.maximum(b.max(-1, keepdims=True), F32(0.0))
    with np.errstate(divide="ignore", invalid="ignore"):
        s, z = _asym_params(mn, mx, bits, recip)
        q = np.clip(np.rint(b / s) + z, 0, lv)
    wd = scale_word(s, z, bits)
    return q.astype(np.uint8).reshape(np.shape(y)), wd[..., 0]


def quant_asym_err(y: np.ndarray, bits: int = 4, recip: bool = True) -> np.ndarray:
    """error form (int4a:32 / int2a:32 of the simulator): FP32 scale from the unwidened range, unbounded zero point,
    deq = (q - z) * s (kernels/codebook_ref.py:99-108; kernels/csrc/attn_cb_common.cuh:64-69)."""
    b = _grp(y)
    lv = (1 << bits) - 1
    mn, mx = b.min(-1, keepdims=True), b.max(-1, keepdims=True)
    with np.errstate(divide="ignore", invalid="ignore"):
        s, z = _asym_params(mn, mx, bits, recip)
        qa = np.clip(np.rint(b / s) + z, 0, lv)
    return ((qa - z) * s).reshape(np.shape(y))


# ------------------------------------------------------------------------------------------------ selection criterion
def tree(p: np.ndarray) -> np.ndarray:
    """halving tree sum v[:n/2] + v[n/2:] (kernels/codebook_ref.py:119-123)."""
    while p.shape[-1] > 1:
        n = p.shape[-1] // 2
        p = p[..., :n] + p[..., n:]
    return p[..., 0]


def seq_matvec(M: np.ndarray, e: np.ndarray, k0: int, k1: int) -> np.ndarray:
    """u_i = sequential fp32 sum over k in [k0, k1) of M[h, i, k] * e[t, h, k], every product and sum rounded
    separately (kernels/codebook_ref.py:126-131).  M [H, n, K], e [T, H, K] -> [T, H, n]."""
    u = M[None, :, :, k0] * e[:, :, None, k0]
    for k in range(k0 + 1, k1):
        u = u + M[None, :, :, k] * e[:, :, None, k]
    return u


def local_err_k(e: np.ndarray, C: np.ndarray) -> np.ndarray:
    """per 32-vector key error under the diagonal blocks of C (kernels/codebook_ref.py:134-145)."""
    out = []
    for j in range(e.shape[-1] // RB):
        sl = slice(RB * j, RB * (j + 1))
        ej = e[..., sl]
        out.append(tree(ej * seq_matvec(C[:, sl, sl], ej, 0, RB)))
    return np.stack(out, -1)


def head_err_k(e: np.ndarray, C: np.ndarray) -> np.ndarray:
    """whole-head key error: u = ((U0 + U1) + U2) + U3 over the 32-column blocks, tree of e * u
    (kernels/codebook_ref.py:148-156)."""
    U = [seq_matvec(C, e, RB * b, RB * (b + 1)) for b in range(e.shape[-1] // RB)]
    u = U[0]
    for b in range(1, len(U)):
        u = u + U[b]
    return tree(e * u)


def encode_keys(x: np.ndarray, C: np.ndarray, bits: int = 4, recip: bool = True):
    """key-only 2x2 encoder of the kinds konlya (bits 4) / konlya2 (bits 2): per 32-vector {I, H32} by the C-weighted
    error of the error-form quantizer, per head {base, H128}; strict-< first argmin; stored codes / words from the
    stored-form quantizer of the chosen transformed vector (kernels/codebook_ref.py:166-236 with cfg konlya / konlya2).
    x fp32 [T, H, 128] (already centred), C fp32 [H, 128, 128].
    Returns dict: q uint8 [T, H, 128] (stored coordinates), word int32 [T, H, 4] (z in the low bits, bit 15 = H32 flag
    of the group when the head choice is base), fflag bool [T, H] (whole-head H128 chosen), local bool [T, H, 4]."""
    x = np.asarray(x, dtype=F32)
    C = np.asarray(C, dtype=F32)
    y0, y1 = x, fwht(x, RB)
    q0, w0 = quant_asym_store(y0, bits, recip)
    q1, w1 = quant_asym_store(y1, bits, recip)
    rec0 = quant_asym_err(y0, bits, recip)
    rec1 = fwht(quant_asym_err(y1, bits, recip), RB)
    err0 = local_err_k(rec0 - x, C)
    err1 = local_err_k(rec1 - x, C)
    ch = err1 < err0                                                      # [T, H, 4]
    sel = np.repeat(ch, RB, -1)
    qb = np.where(sel, q1, q0)
    wb = np.where(ch, w1, w0)
    recb = np.where(sel, rec1, rec0)
    yF = fwht(x, D)
    qF, wF = quant_asym_store(yF, bits, recip)
    recF = fwht(quant_asym_err(yF, bits, recip), D)
    eb = head_err_k(recb - x, C)
    eF = head_err_k(recF - x, C)
    fflag = eF < eb                                                       # [T, H]
    q = np.where(fflag[..., None], qF, qb)
    word = np.where(fflag[..., None], wF, wb | (ch.astype(np.int32) << 15))
    return dict(q=q.astype(np.uint8), word=word.astype(np.int32), fflag=fflag, local=ch & ~fflag[..., None],
                head_errs=np.stack([eb, eF]), local_errs=np.stack([err0, err1]))


def encode_values(x: np.ndarray, bits: int = 4, recip: bool = True):
    """values of the key-only kinds: no transform, stored-form quantizer (kernels/codebook_ref.py:72,199)."""
    q, w = quant_asym_store(np.asarray(x, dtype=F32), bits, recip)
    return dict(q=q, word=w)


def dynamic_rows(kv_bits: np.ndarray, C: np.ndarray, bits: int = 4, kmu: np.ndarray | None = None, recip: bool = True):
    """dynamic (konlya / konlya2) writer on bf16 rows kv [T, 2 Hkv, 128] (K rows first): codes uint8 [T, Hkv, 2, 128] and
    final 16-bit words int32 [T, Hkv, 2, 4] (K: z | H32 flag; V: z | the KEY's whole-head flag in group 0)
    (integrations/vllm_flagrot/tests/test_int2.py:141-152; kernels/csrc/attn_codebook.cu:97-104,286-289)."""
    kv = bf16_bits_to_f32(kv_bits)
    Hkv = kv.shape[1] // 2
    k = kv[:, :Hkv]
    if kmu is not None:
        k = k - np.asarray(kmu, dtype=F32)[None]
    ek = encode_keys(k, C, bits, recip)
    ev = encode_values(kv[:, Hkv:], bits, recip)
    vw = ev["word"].copy()
    vw[..., 0] |= ek["fflag"].astype(np.int32) << 15
    codes = np.stack([ek["q"], ev["q"]], 2)
    words = np.stack([ek["word"], vw], 2)
    return codes, words, ek


def static_rows(kv_bits: np.ndarray, mask: np.ndarray | None, hfull: np.ndarray | None, bits: int = 4,
                kmu: np.ndarray | None = None, recip: bool = True):
    """static writer on bf16 rows kv [T, 2 Hkv, 128]: [hfull rows -> bf16(H128 x / 16)] -> K rows minus kmu (stored basis)
    -> flagged 32-blocks rotated by H32 -> stored-form quantizer (kernels/csrc/attn_decode_v2.cu:1717-1760;
    kernels/csrc/attn_codebook.cuh:127-146; integrations/vllm_flagrot/tests/test_kernels.py:318-326).
    mask uint8 [2 Hkv, 4], hfull uint8 [2 Hkv].  Returns codes uint8 [T, Hkv, 2, 128], words int32 [T, Hkv, 2, 4]."""
    H2 = kv_bits.shape[1]
    Hkv = H2 // 2
    if hfull is not None:
        kv_bits = head_fwht(kv_bits, hfull, 1.0 / 16.0)
    x = bf16_bits_to_f32(kv_bits).copy()
    if kmu is not None:
        x[:, :Hkv] = x[:, :Hkv] - np.asarray(kmu, dtype=F32)[None]
    if mask is not None:
        T = x.shape[0]
        x = sel_fwht_rb(x.reshape(T, H2 * D), np.asarray(mask), RB).reshape(T, H2, D)
    q, w = quant_asym_store(x, bits, recip)
    codes = np.stack([q[:, :Hkv], q[:, Hkv:]], 2)
    words = np.stack([w[:, :Hkv], w[:, Hkv:]], 2)
    return codes, words


def static_rows_256(kv_bits: np.ndarray, mask: np.ndarray | None, hfull: np.ndarray | None, bits: int = 4,
                    kmu: np.ndarray | None = None, recip: bool = True):
    """static writer for head dim 256: the whole-head step is H256 / 16 over the full head
    (integrations/vllm_flagrot/csrc/flagrot_capi.cu:200-245); after it the two 128-d halves of a head are written as two
    half heads, kv [T, 2 Hkv, 256] = [T, 4 Hkv, 128], mask [2 Hkv, 8] = [4 Hkv, 4], kmu [Hkv, 256] = [2 Hkv, 128], pool
    [., Hkv, 2 chunk] = [., 2 Hkv, chunk] (kernels/csrc/attn_decode_v2.cu:2050-2055).  Returns codes [T, 2 Hkv, 2, 128] and
    words [T, 2 Hkv, 2, 4] over the half heads h' = 2 h + half."""
    T, H2, Dh = kv_bits.shape
    assert Dh == 256
    if hfull is not None:
        kv_bits = head_fwht(kv_bits, hfull, 1.0 / 16.0)
    return static_rows(kv_bits.reshape(T, 2 * H2, D), None if mask is None else np.asarray(mask).reshape(2 * H2, 4), None, bits,
                       None if kmu is None else np.asarray(kmu, dtype=F32).reshape(H2, D), recip)


# ------------------------------------------------------------------------------------------------ page layouts
def chunk_bytes(bits: int, page: int) -> int:
    """bytes per (page, kv head): 144 P (INT4) / 80 P (INT2) (kernels/csrc/attn_decode_v2.cuh:14-46)."""
    return page * (144 if bits == 4 else 80)


_MAPS: dict = {}


def _maps(bits: int, P: int):
    """byte offset and bit shift of every element of a (page, head) chunk, from the layout specification
    (kernels/csrc/attn_decode_v2.cuh:14-46; kernels/csrc/attn_cb_common.cuh:144-156).
    Returns kb, ks [P, 128] (K code byte / shift), vb, vs [P, 128], ksw [P, 4], vsw [P, 4] (scale word byte offsets)."""
    key = (bits, P)
    if key in _MAPS:
        return _MAPS[key]
    t = np.arange(P)[:, None]
    d = np.arange(D)[None, :]
    j, r = d // 32, d % 32
    isB = (r >= 16).astype(np.int64)
    rr = r - 16 * isB
    tg, i = rr // 4, rr % 4
    w, gid, r8, m = (d % 64) // 16, d % 8, (d % 16) // 8, d // 64
    c8, ii, b = t // 8, (t % 8) // 2, t % 2
    e = (w * 8 + gid) * (P // 8) + c8
    slot8 = np.where((t % 8) % 2 == 1, 4 + (t % 8) // 2, (t % 8) // 2)
    jj = np.arange(4)[None, :]
    if bits == 4:
        kb = 64 * t + 16 * tg + 4 * j + i
        ks = 4 * isB + 0 * t
        vb = 64 * P + 16 * e + 4 * (2 * m + r8) + ii
        vs = 4 * b + 0 * d
        ksw = 128 * P + 8 * t + 2 * jj
        vsw = 136 * P + 2 * (jj * P + 8 * c8 + slot8)
    else:
        kb = 32 * (t ^ ((t >> 1) & 2)) + 8 * tg + 4 * (j // 2) + i
        ks = 4 * (j % 2) + 2 * isB + 0 * t
        vb = 32 * P + 8 * e + 4 * m + ii
        vs = 4 * r8 + 2 * b
        ksw = 64 * P + 8 * t + 2 * jj
        vsw = 72 * P + 2 * (jj * P + 8 * c8 + slot8)
    out = tuple(np.broadcast_to(a, (P, a.shape[1] if a.shape[1] > 1 else D)).astype(np.int64)
                for a in (kb, ks, vb, vs)) + (ksw.astype(np.int64), vsw.astype(np.int64))
    _MAPS[key] = out
    return out


def write_pool(pool: np.ndarray, slots: np.ndarray, codes: np.ndarray, words: np.ndarray, bits: int, P: int,
               which: str = "kv") -> None:
    """scatter encoded rows into the paged pool in place, touching only the bits of the written (token, head) cells
    (read-modify-write of shared V^T words as in kernels/csrc/attn_decode_v2.cu:1860-1871).
    pool uint8 [Np, Hkv, chunk]; slots int64 [T] (< 0 skipped); codes uint8 [T, Hkv, 2, 128]; words [T, Hkv, 2, 4];
    which: "kv" both rows, "k" / "v" one side only.  A "k" call also writes bit 15 of the V group-0 word (the key's
    whole-head flag) and a "v" call only that word's low 15 bits: the two-call contract of the reference's two-stream
    writer (kernels/csrc/attn_cb_write3.cuh:656-664)."""
    kb, ks, vb, vs, ksw, vsw = _maps(bits, P)
    Np, Hkv, CH = pool.shape
    flat = pool.reshape(-1)
    slots = np.asarray(slots).astype(np.int64)
    ok = slots >= 0
    tt = np.nonzero(ok)[0]
    if tt.size == 0:
        return
    page, pos = slots[tt] // P, slots[tt] % P
    base = (page[:, None] * Hkv + np.arange(Hkv)[None, :]) * CH                      # [n, Hkv]
    fm = (1 << bits) - 1

    def put_codes(bmap, smap, c):                                                      # c [n, Hkv, 128]
        idx = base[:, :, None] + bmap[pos][:, None, :]
        sh = smap[pos][:, None, :].astype(np.uint8)
        np.bitwise_and.at(flat, idx, (~(np.uint8(fm) << sh)).astype(np.uint8))
        np.bitwise_or.at(flat, idx, (c.astype(np.uint8) << sh).astype(np.uint8))

    def put_words(wmap, wv, keep_mask=0):                                              # wv [n, Hkv, 4]
        idx = base[:, :, None] + wmap[pos][:, None, :]
        wv = wv.astype(np.int64) & 0xFFFF
        if keep_mask:
            old = flat[idx].astype(np.int64) | (flat[idx + 1].astype(np.int64) << 8)
            wv = (old & keep_mask) | (wv & ~keep_mask & 0xFFFF)
        flat[idx] = (wv & 0xFF).astype(np.uint8)
        flat[idx + 1] = (wv >> 8).astype(np.uint8)

    if which in ("kv", "k"):
        put_codes(kb, ks, codes[tt, :, 0])
        put_words(ksw, words[tt, :, 0])
    if which == "kv":
        put_codes(vb, vs, codes[tt, :, 1])
        put_words(vsw, words[tt, :, 1])
    elif which == "k":      # only the flag bit of V group 0
        idx = base + vsw[pos][:, 0:1]
        hi = flat[idx + 1]
        flat[idx + 1] = (hi & np.uint8(0x7F)) | ((words[tt, :, 1, 0] >> 8) & 0x80).astype(np.uint8)
    elif which == "v":
        put_codes(vb, vs, codes[tt, :, 1])
        w = words[tt, :, 1].astype(np.int64)
        idx = base[:, :, None] + vsw[pos][:, None, :]
        old = flat[idx].astype(np.int64) | (flat[idx + 1].astype(np.int64) << 8)
        keep = np.zeros((1, 1, 4), dtype=np.int64)
        keep[..., 0] = 0x8000
        nw = (old & keep) | (w & ~keep & 0xFFFF)
        flat[idx] = (nw & 0xFF).astype(np.uint8)
        flat[idx + 1] = (nw >> 8).astype(np.uint8)


def parse_pool(pool: np.ndarray, bits: int, P: int):
    """raw codes uint8 [Np, Hkv, P, 2, 128] and scale words uint16 [Np, Hkv, P, 2, 4] of every cell of the pool
    (independent restatement of integrations/vllm_flagrot/vllm_flagrot/kernels.py:591-684)."""
    kb, ks, vb, vs, ksw, vsw = _maps(bits, P)
    fm = (1 << bits) - 1
    K = (pool[:, :, kb] >> ks.astype(np.uint8)) & fm
    V = (pool[:, :, vb] >> vs.astype(np.uint8)) & fm
    kw = pool[:, :, ksw].astype(np.uint16) | (pool[:, :, ksw + 1].astype(np.uint16) << 8)
    vw = pool[:, :, vsw].astype(np.uint16) | (pool[:, :, vsw + 1].astype(np.uint16) << 8)
    return np.stack([K, V], 3).astype(np.uint8), np.stack([kw, vw], 3)


_HM: dict = {}


def hadamard(n: int) -> np.ndarray:
    """orthonormal Sylvester Hadamard matrix in float64 (integrations/vllm_flagrot/vllm_flagrot/kernels.py:700-709)."""
    if n not in _HM:
        h = np.ones((1, 1))
        while h.shape[0] < n:
            h = np.block([[h, h], [h, -h]])
        _HM[n] = h / math.sqrt(n)
    return _HM[n]


def dequant_pool(pool: np.ndarray, bits: int, P: int, key_only: bool):
    """K, V float64 [Np, P, Hkv, 128] of every page.  key_only (konlya / konlya2): K in the ORIGINAL basis (inverse H32 of
    flagged groups, inverse H128 of flagged tokens), V plain (kernels.py:724-743); static formats: K and V in the
    STORED basis (kernels.py:686-697).  x = (c - z) * fp16(word & 0x7FFF) with z the low bits of the word."""
    codes, words = parse_pool(pool, bits, P)
    z = (words & np.uint16((1 << bits) - 1)).astype(np.float64)
    mag = word_value(words).astype(np.float64)
    Np, H = pool.shape[:2]
    d = (codes.astype(np.float64).reshape(Np, H, P, 2, NG, RB) - z[..., None]) * mag[..., None]
    k, v = d[..., 0, :, :], d[..., 1, :, :]
    if key_only:
        lk = ((words[..., 0, :] >> 15) & 1).astype(bool)                            # [Np, H, P, 4]
        fk = ((words[..., 1, 0] >> 15) & 1).astype(bool)                            # [Np, H, P]
        kl = np.where(lk[..., None], k @ hadamard(RB), k).reshape(Np, H, P, D)
        kf = k.reshape(Np, H, P, D) @ hadamard(D)
        k = np.where(fk[..., None], kf, kl)
    else:
        k = k.reshape(Np, H, P, D)
    return k.transpose(0, 2, 1, 3), v.reshape(Np, H, P, D).transpose(0, 2, 1, 3)


# ------------------------------------------------------------------------------------------------ decode attention
def sel_rot64(x: np.ndarray, mask: np.ndarray, rb: int = RB) -> np.ndarray:
    """x [..., H, D] float64, mask [H, D / rb]: per (head, block) orthonormal Hadamard
    (integrations/vllm_flagrot/tests/test_kernels.py:29-34)."""
    xb = x.reshape(*x.shape[:-1], x.shape[-1] // rb, rb)
    y = np.where(np.asarray(mask).astype(bool)[..., None], xb @ hadamard(rb), xb)
    return y.reshape(x.shape)


def attention(q: np.ndarray, Kc: np.ndarray, Vc: np.ndarray, lens, scale: float, tails=None, kv_start: int = 0):
    """float64 decode attention (integrations/vllm_flagrot/tests/test_kernels.py:37-56).  q [B, Hq, D]; Kc / Vc
    [B, Lmax, Hkv, D] valid in [kv_start, lens[b]); tails: list of (k, v) [n, Hkv, D] or None per row.  Rows with no
    key at all return 0."""
    B, Hq, Dh = q.shape
    G = Hq // Kc.shape[2]
    out = np.zeros((B, Hq, Dh))
    for b in range(B):
        a = min(kv_start, int(lens[b]))
        ks, vs = [Kc[b, a:int(lens[b])]], [Vc[b, a:int(lens[b])]]
        if tails is not None and tails[b] is not None:
            ks.append(tails[b][0])
            vs.append(tails[b][1])
        k = np.repeat(np.concatenate(ks).astype(np.float64), G, 1)
        v = np.repeat(np.concatenate(vs).astype(np.float64), G, 1)
        if k.shape[0] == 0:
            continue
        s = np.einsum("hd,lhd->hl", q[b].astype(np.float64), k) * scale
        p = np.exp(s - s.max(-1, keepdims=True))
        p = p / p.sum(-1, keepdims=True)
        out[b] = np.einsum("hl,lhd->hd", p, v)
    return out


def gather_cache(Kp: np.ndarray, Vp: np.ndarray, bt: np.ndarray, Lmax: int, P: int):
    """pages [Np, P, Hkv, D] + block table [B, n] -> per-row caches [B, npg * P, Hkv, D]."""
    npg = (max(Lmax, 1) + P - 1) // P
    idx = np.asarray(bt)[:, :npg].astype(np.int64)
    B = idx.shape[0]
    return (Kp[idx].reshape(B, npg * P, *Kp.shape[2:]), Vp[idx].reshape(B, npg * P, *Vp.shape[2:]))


def decode_reference(q_bits, pool, bt, lens, scale, bits, P, key_only, kmask=None, vmask=None, tail=None, tail_len=None,
                     tail_idx=None, kv_start=0, bf16_operands=False, sym=False):
    """decode attention of one step over a quantised pool, the way the reference tests build their expectation
    (integrations/vllm_flagrot/tests/test_kernels.py:119-150): dequantise the pages, float64 attention, BF16 tail rows
    treated identically.  Static formats: q and the tail are rotated into the stored basis by the block masks and the
    output is rotated back.  q_bits uint16 [B, Hq, 128]; tail uint16 [R, W, 2 Hkv, 128].  Returns float64 [B, Hq, 128].
    bf16_operands: the same attention with q, K and V rounded to bf16 first, still in the stored basis (the yardstick of
    the reference's own tolerance, sdpa_err in integrations/vllm_flagrot/tests/test_kernels.py:59-63)."""
    q = bf16_bits_to_f32(q_bits).astype(np.float64)
    B, Hq, _ = q.shape
    Hkv = pool.shape[1]
    G = Hq // Hkv
    Kp, Vp = dequant_pool_sym(pool, P, key_only) if sym else dequant_pool(pool, bits, P, key_only)   # sym: int4 / konly pages
    Lmax = int(max(max(lens), 1))
    Kc, Vc = gather_cache(Kp, Vp, bt, Lmax, P)
    rnd = (lambda a: bf16_round(a.astype(np.float32)).astype(np.float64)) if bf16_operands else (lambda a: a)
    tails = None
    if tail is not None:
        tf = bf16_bits_to_f32(tail).astype(np.float64)
        tails = []
        for b in range(B):
            r = int(tail_idx[b]) if tail_idx is not None else b
            n = min(int(tail_len[b]), 256)
            tails.append((tf[r, :n, :Hkv], tf[r, :n, Hkv:]))
    if key_only or (kmask is None and vmask is None):
        with np.errstate(invalid="ignore", over="ignore"):
            return attention(q, rnd(Kc), rnd(Vc), lens, scale, tails, kv_start)
    km = np.zeros((Hkv, NG), bool) if kmask is None else np.asarray(kmask).astype(bool)
    vm = np.zeros((Hkv, NG), bool) if vmask is None else np.asarray(vmask).astype(bool)
    qr = sel_rot64(q.reshape(B, Hkv, G, D).transpose(0, 2, 1, 3), km).transpose(0, 2, 1, 3).reshape(B, Hq, D)
    tr = None if tails is None else [(sel_rot64(t[0], km), sel_rot64(t[1], vm)) for t in tails]
    if bf16_operands:
        qr = rnd(qr)
        tr = None if tr is None else [(rnd(a), rnd(b)) for a, b in tr]
    with np.errstate(invalid="ignore", over="ignore"):
        o = attention(qr, rnd(Kc), rnd(Vc), lens, scale, tr, kv_start)
    return sel_rot64(o.reshape(B, Hkv, G, D).transpose(0, 2, 1, 3), vm).transpose(0, 2, 1, 3).reshape(B, Hq, D)


# ------------------------------------------------------------------------------------------------ symmetric INT4 (int4 / konly)
def quant_sym_store(y: np.ndarray):
    """symmetric INT4 per 32 (the `int4` page format): s = fp16(amax * fp32(1 / 7)), q = clamp(rne(y / s), -7, 7), q = 0
    where s = 0 (kernels/ref.py:151-160; kernels/csrc/attn_decode_v2.cu:1769-1781).  Returns q int8 [..., D] and the scale
    words int32 [..., D / 32] (the FP16 bit pattern of s; bit 15 is free for a flag)."""
    b = _grp(y)
    s16 = (np.abs(b).max(-1, keepdims=True) * (F32(1.0) / F32(7.0))).astype(np.float16)
    s = s16.astype(F32)
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.where(s != 0, np.rint(b / np.where(s != 0, s, F32(1.0))), F32(0.0))
    q = np.clip(q, -7, 7)
    return q.astype(np.int8).reshape(np.shape(y)), s16.view(np.uint16).astype(np.int32)[..., 0]


def static_rows_sym(kv_bits: np.ndarray, mask: np.ndarray | None, hfull: np.ndarray | None, kmu: np.ndarray | None = None):
    """static_rows for the symmetric format: codes int8 [T, Hkv, 2, 128] in [-7, 7], words int32 [T, Hkv, 2, 4]."""
    H2 = kv_bits.shape[1]
    Hkv = H2 // 2
    if hfull is not None:
        kv_bits = head_fwht(kv_bits, hfull, 1.0 / 16.0)
    x = bf16_bits_to_f32(kv_bits).copy()
    if kmu is not None:
        x[:, :Hkv] = x[:, :Hkv] - np.asarray(kmu, dtype=F32)[None]
    if mask is not None:
        T = x.shape[0]
        x = sel_fwht_rb(x.reshape(T, H2 * D), np.asarray(mask), RB).reshape(T, H2, D)
    q, w = quant_sym_store(x)
    return np.stack([q[:, :Hkv], q[:, Hkv:]], 2), np.stack([w[:, :Hkv], w[:, Hkv:]], 2)


def _maps_sym(P: int):
    """bit positions of the sign-magnitude elements of the symmetric layout (kernels/csrc/attn_decode_v2.cuh:26-28): element
    A_i of a 32-bit word: sign -> bit 7 of byte i, |q| -> bits 0 - 2 of byte i; B_i: sign -> bit 3 of byte i, |q| -> bits
    4 - 6 of byte (i + 3) % 4.  Which element of which word a (token, dim) is follows the INT4A maps (A = low nibble there).
    Returns per K and V: (magnitude byte, magnitude shift, sign byte, sign shift), each [P, 128]."""
    kb, ks, vb, vs, ksw, vsw = _maps(4, P)

    def conv(bm, sm):
        i = bm % 4
        base = bm - i
        isB = sm == 4
        return (np.where(isB, base + (i + 3) % 4, bm), np.where(isB, 4, 0), bm, np.where(isB, 3, 7))
    return conv(kb, ks), conv(vb, vs), ksw, vsw


def write_pool_sym(pool: np.ndarray, slots: np.ndarray, q: np.ndarray, words: np.ndarray, P: int) -> None:
    """write_pool for the symmetric format: q int8 [T, Hkv, 2, 128] in [-7, 7] (sign of zero: plus), words [T, Hkv, 2, 4]."""
    (kmap, vmap, ksw, vsw) = _maps_sym(P)
    Np, Hkv, CH = pool.shape
    flat = pool.reshape(-1)
    slots = np.asarray(slots).astype(np.int64)
    tt = np.nonzero(slots >= 0)[0]
    if tt.size == 0:
        return
    page, pos = slots[tt] // P, slots[tt] % P
    base = (page[:, None] * Hkv + np.arange(Hkv)[None, :]) * CH
    for side, (mb, ms, sb, ss), wmap in ((0, kmap, ksw), (1, vmap, vsw)):
        c = q[tt, :, side].astype(np.int16)
        mag, sgn = np.abs(c).astype(np.uint8), (c < 0).astype(np.uint8)
        for bm, sh, val, width in ((mb, ms, mag, 7), (sb, ss, sgn, 1)):
            idx = base[:, :, None] + bm[pos][:, None, :]
            s8 = sh[pos][:, None, :].astype(np.uint8)
            np.bitwise_and.at(flat, idx, (~(np.uint8(width) << s8)).astype(np.uint8))
            np.bitwise_or.at(flat, idx, (val << s8).astype(np.uint8))
        idx = base[:, :, None] + wmap[pos][:, None, :]
        wv = words[tt, :, side].astype(np.int64) & 0xFFFF
        flat[idx] = (wv & 0xFF).astype(np.uint8)
        flat[idx + 1] = (wv >> 8).astype(np.uint8)


def parse_pool_sym(pool: np.ndarray, P: int):
    """signed codes int8 [Np, Hkv, P, 2, 128] and scale words uint16 [Np, Hkv, P, 2, 4] (independent restatement of
    integrations/vllm_flagrot/vllm_flagrot/kernels.py:580-626 with asym=False)."""
    (kmap, vmap, ksw, vsw) = _maps_sym(P)
    out = []
    for mb, ms, sb, ss in (kmap, vmap):
        mag = ((pool[:, :, mb] >> ms.astype(np.uint8)) & 7).astype(np.int8)
        neg = ((pool[:, :, sb] >> ss.astype(np.uint8)) & 1).astype(bool)
        out.append(np.where(neg, -mag, mag))
    kw = pool[:, :, ksw].astype(np.uint16) | (pool[:, :, ksw + 1].astype(np.uint16) << 8)
    vw = pool[:, :, vsw].astype(np.uint16) | (pool[:, :, vsw + 1].astype(np.uint16) << 8)
    return np.stack(out, 3).astype(np.int8), np.stack([kw, vw], 3)


def dequant_pool_sym(pool: np.ndarray, P: int, key_only: bool):
    """dequant_pool for the symmetric format: x = q * fp16(word & 0x7FFF); key_only (konly): flags as for konlya."""
    codes, words = parse_pool_sym(pool, P)
    mag = word_value(words).astype(np.float64)
    Np, H = pool.shape[:2]
    d = codes.astype(np.float64).reshape(Np, H, P, 2, NG, RB) * mag[..., None]
    k, v = d[..., 0, :, :], d[..., 1, :, :]
    if key_only:
        lk = ((words[..., 0, :] >> 15) & 1).astype(bool)
        fk = ((words[..., 1, 0] >> 15) & 1).astype(bool)
        kl = np.where(lk[..., None], k @ hadamard(RB), k).reshape(Np, H, P, D)
        k = np.where(fk[..., None], k.reshape(Np, H, P, D) @ hadamard(D), kl)
    else:
        k = k.reshape(Np, H, P, D)
    return k.transpose(0, 2, 1, 3), v.reshape(Np, H, P, D).transpose(0, 2, 1, 3)


def dynamic_rows_sym(kv_bits: np.ndarray, C: np.ndarray, kmu: np.ndarray | None = None):
    """dynamic writer of the symmetric key-only kind `konly`: the konlya criterion (encode_keys) with the symmetric quantiser,
    whose error form is its stored form: deq = q * s, s = fp16(amax / 7) (kernels/codebook_ref.py:94-116 kind "cache",
    166-236 with cfg konly).  Returns codes int8 [T, Hkv, 2, 128] in [-7, 7], words int32 [T, Hkv, 2, 4] (FP16 scale bits;
    K: bit 15 = H32 flag of the group when the head choice is base; V group 0: bit 15 = the key's whole-head flag), and the
    key encoder's details."""
    kv = bf16_bits_to_f32(kv_bits)
    Hkv = kv.shape[1] // 2
    x = kv[:, :Hkv]
    if kmu is not None:
        x = x - np.asarray(kmu, dtype=F32)[None]
    C = np.asarray(C, dtype=F32)

    def qd(y):
        q, w = quant_sym_store(y)
        s = w.astype(np.uint16).view(np.float16).astype(F32)
        return q, w, (q.astype(F32).reshape(*w.shape, RB) * s[..., None]).reshape(np.shape(y))
    y1 = fwht(x, RB)
    q0, w0, d0 = qd(x)
    q1, w1, d1 = qd(y1)
    rec1 = fwht(d1, RB)
    err0, err1 = local_err_k(d0 - x, C), local_err_k(rec1 - x, C)
    ch = err1 < err0
    sel = np.repeat(ch, RB, -1)
    qb, wb, recb = np.where(sel, q1, q0), np.where(ch, w1, w0), np.where(sel, rec1, d0)
    qF, wF, dF = qd(fwht(x, D))
    eb, eF = head_err_k(recb - x, C), head_err_k(fwht(dF, D) - x, C)
    fflag = eF < eb
    qk = np.where(fflag[..., None], qF, qb)
    wk = np.where(fflag[..., None], wF, wb | (ch.astype(np.int32) << 15))
    qv, wv = quant_sym_store(kv[:, Hkv:])
    wv = wv.copy()
    wv[..., 0] |= fflag.astype(np.int32) << 15
    ek = dict(fflag=fflag, local=ch & ~fflag[..., None], head_errs=np.stack([eb, eF]))
    return np.stack([qk, qv], 2).astype(np.int8), np.stack([wk, wv], 2).astype(np.int32), ek
