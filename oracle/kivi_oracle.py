"""CPU restatement (numpy) of the FlagRot-KIVI INT2 path: the KIVI group quantizer, the per-token value encoder, the
per-(32-token group, kv head) key encoder with the attention-weighted selection rule, the page layout (packer + parser)
and float64 decode attention over parsed pages.

TEST INFRASTRUCTURE ONLY (used by tests/ and nothing else).  Restates integrations/vllm_flagrot/csrc/kivi.cu (semantics,
cited per function), blockflag/formats.py:103-116 (fake_kivi) and blockflag/qattention.py:105-145,147-188 (rule "att").
Pinned by tests/golden/kivi.npz (outputs of the reference's simulator run on CPU; tests/golden/make_golden.py):
plain-KIVI reconstructions bit for bit, dynamic choices statistically (the reference's own tests accept up to 2 %
mismatching choices for this encoder: integrations/vllm_flagrot/tests/test_kivi.py:140,175).
`recip`: s = (max - min) / 3 is a true division on the CPU reference and a multiply by fp32(1/3) on the GPU.
`f8=True` everywhere: the kivi2p8 pages (kivi.cu:28-35, 83-88): scale and minimum stored as FP8 E4M3 (round to nearest
even, saturating at +-448; formats.py:190-204 fake_kivi_f8), codes from the STORED values, chunk of 10 D bytes, flags in
the sign bits of the (non-negative) scales.  Pinned by tests/golden/kivi_f8.npz.
"""
from __future__ import annotations

import numpy as np

from .flagrot_oracle import F32, bf16_bits_to_f32, fwht, hadamard

D, NV, PAGE, GRP = 128, 4, 16, 32
CB = 12 * D + 16
OFF_KM, OFF_VC, OFF_VM, OFF_VF = 4 * D, 6 * D, 10 * D, 12 * D
KBIT = np.array([2 * (i >> 1) + 16 * (i & 1) for i in range(16)])
CB8 = 10 * D                                                     # kivi2p8: KC | KM [16][4][2] u8 | VC | VM [16][4][2] u8
OFF_KM8, OFF_VC8, OFF_VM8 = 4 * D, 5 * D, 9 * D


# ------------------------------------------------------------------------------------------------ FP8 E4M3 (kivi2p8)
def e4m3_round(x):
    """nearest E4M3 value (ties to even, 3 mantissa bits, exponents -6 .. 8, subnormal step 2^-9), saturating at +-448
    (kivi.cu:110-119; formats.py:190-192).  fp32 in, fp32 out; the sign of zero is kept."""
    x = np.clip(np.asarray(x, F32), F32(-448.0), F32(448.0)).astype(np.float64)
    a = np.abs(x)
    _, ex = np.frexp(a)                                          # a = m 2^ex, m in [0.5, 1)
    step = np.exp2(np.maximum(ex - 1, -6) - 3.0)
    return np.copysign(np.rint(a / step) * step, x).astype(F32)


def e4m3_bits(x):
    """the byte of e4m3_round(x): sign | 4-bit exponent (bias 7) | 3-bit mantissa."""
    v = e4m3_round(x).astype(np.float64)
    a = np.abs(v)
    _, ex = np.frexp(a)
    e = np.maximum(ex - 1, -6)
    sub = a < 2.0 ** -6
    mant = np.where(sub, a / 2.0 ** -9, a / np.exp2(e - 3.0) - 8)
    expo = np.where(sub, 0, e + 7)
    return ((np.signbit(v).astype(np.int64) << 7) | (expo.astype(np.int64) << 3) | mant.astype(np.int64)).astype(np.uint8)


E4M3_TABLE = np.array([(-1.0 if b & 0x80 else 1.0) * ((b & 7) * 2.0 ** -9 if ((b >> 3) & 15) == 0
                                                      else (8 + (b & 7)) * 2.0 ** (((b >> 3) & 15) - 10)) for b in range(256)])


def stored_params(mn, mx, recip=True, f8=False):
    """(scale, min) the quantizer works with: fp32 for kivi2 (their FP16 roundings are only what the page stores),
    the E4M3 values themselves for kivi2p8 (kivi.cu:120-125)."""
    s = kivi_params(mn, mx, recip)
    return (e4m3_round(s), e4m3_round(mn)) if f8 else (s, np.asarray(mn, F32))


def kivi_params(mn, mx, recip=True):
    """scale of a group with range [mn, mx] (kivi.cu:99-102; formats.py:108-110)."""
    d = (mx - mn).astype(F32)
    return d * (F32(1.0) / F32(3.0)) if recip else d / F32(3.0)


def kivi_quant(y, mn, s):
    """codes and reconstruction code * s + mn, every operation rounded separately (kivi.cu:103-109)."""
    d = np.where(s == 0, F32(1.0), s)
    q = np.rint(np.clip((y - mn) / d, 0, 3)).astype(F32)
    return q.astype(np.uint8), q * s + mn


def _f16(x):
    return np.asarray(x, F32).astype(np.float16)


# ------------------------------------------------------------------------------------------------ values (per token)
def encode_values(x, co, ident=False, vfix=None, recip=True, f8=False, M=None):
    """x fp32 [T, H, 128]; co fp32 [H, 128].  Candidates identity / H32 per 32-dim sub-vector / whole-head H128, groups of
    32 along the head dim; error sum d^2 co; H32 only if strictly better, whole head only if strictly better than the
    combination (kivi.cu:163-328).  Returns dict: codes uint8 [T, H, 128], meta float16 [T, H, 4, 2] (scale with the H32 flag
    in its sign, min), vf uint8 [T, H], cand int [T, H, 4] (0 I, 1 H32, 2 whole head), s / mn fp32 [T, H, 4] before storage.
    f8: meta is uint8 [T, H, 4, 2] (E4M3 scale | H32 flag << 7, E4M3 min).  M fp32 [H, 128, 128]: the error of a candidate is
    e^T M e instead of sum e^2 co (the diagonal 32 x 32 block for a sub-vector's I / H32 choice, the whole matrix for the
    whole-head candidate and for the chosen combination; kivi.cu:222-275)."""
    x = np.asarray(x, F32)
    T, H, _ = x.shape
    outs = []
    for c in range(3):
        y = x if c == 0 else fwht(x, 32 if c == 1 else D)
        b = y.reshape(T, H, NV, 32)
        mn, mx = b.min(-1, keepdims=True), b.max(-1, keepdims=True)
        s, mn = stored_params(mn, mx, recip, f8)
        q, r = kivi_quant(b, mn, s)
        r = r.reshape(T, H, D)
        rec = r if c == 0 else fwht(r, 32 if c == 1 else D)
        outs.append((q.reshape(T, H, D), s[..., 0], mn[..., 0], rec))
    if ident:
        cand = np.zeros((T, H, NV), int)
    elif vfix is not None:
        vfix = np.asarray(vfix)
        loc = ((vfix[:, None] >> np.arange(NV)[None]) & 1)
        cand = np.where(((vfix >> 16) & 1)[:, None] == 1, 2, loc)[None].repeat(T, 0)
    elif M is not None:
        Mm = np.asarray(M, F32)
        ev = [(o[3] - x).astype(F32) for o in outs]                                           # [T, H, 128]
        Mb = np.stack([Mm[:, 32 * j:32 * j + 32, 32 * j:32 * j + 32] for j in range(NV)], 1)     # [H, 4, 32, 32]
        blk = lambda e: np.einsum("thvi,hvik,thvk->thv", e.reshape(T, H, NV, 32), Mb, e.reshape(T, H, NV, 32))  # noqa: E731
        full = lambda e: np.einsum("thi,hik,thk->th", e, Mm, e)                               # noqa: E731
        useH = blk(ev[1]) < blk(ev[0])
        eb = np.where(np.repeat(useH, 32, -1), ev[1], ev[0])
        useF = full(ev[2]) < full(eb)
        cand = np.where(useF[..., None], 2, useH.astype(int))
    else:
        e = [((o[3] - x) ** 2 * np.asarray(co, F32)[None]).reshape(T, H, NV, 32).sum(-1) for o in outs]
        useH = e[1] < e[0]
        eB = np.where(useH, e[1], e[0]).sum(-1)
        useF = e[2].sum(-1) < eB
        cand = np.where(useF[..., None], 2, useH.astype(int))
    sel = np.repeat(cand, 32, -1)
    codes = np.choose(sel, [o[0] for o in outs])
    s = np.choose(cand, [o[1] for o in outs])
    mn = np.choose(cand, [o[2] for o in outs])
    if f8:
        meta = np.stack([(e4m3_bits(s) & 0x7F) | ((cand == 1).astype(np.uint8) << 7), e4m3_bits(mn)], -1)
    else:
        sh = _f16(s)
        sh = np.where(cand == 1, -np.abs(sh), sh)
        meta = np.stack([sh, _f16(mn)], -1)
    return dict(codes=codes.astype(np.uint8), meta=meta, vf=(cand[..., 0] == 2).astype(np.uint8), cand=cand, s=s, mn=mn)


# ------------------------------------------------------------------------------------------------ keys (per group)
def encode_key_group(x, valid, qs, lz, qsc, ident=False, kfix=None, recip=True, f8=False):
    """one 32-token group: x fp32 [32, H, 128], valid bool [32] (sinks excluded), calibration queries qs fp32 [H, NQ, 128],
    lz fp32 [H, NQ].  Per channel over the valid tokens: INT2 of the identity / per-token H32 / per-token H128 views; rule
    "att": w[t, q] = min(1, exp(qsc x_t . q - lz_q)), error of a candidate = sum_{t, q} w (q . e_t)^2 over the group (per
    sub-vector for I / H32); H32 only if strictly better, whole head only if strictly better than the combination
    (kivi.cu:343-663; qattention.py:127-145,166-188).  Returns codes uint8 [32, H, 128] (valid tokens), meta float16
    [H, 128, 2] (scale with flag signs: channel j < 4 -> sub-vector j is H32, channel 4 -> whole head; min), choices [H, 5],
    and the fp32 (scale, min) before storage.  f8: meta is uint8 [H, 128, 2] (E4M3 scale | flag << 7, E4M3 min) with the
    flags where kivi2p8 keeps them: sub-vector j -> channel 4 j (cell j, slot 0), whole head -> channel 16 (cell 4, slot 0);
    bit 7 of channels 4 i + 3 (cell i, slot 3) belongs to the value writer and is left 0 here."""
    x = np.asarray(x, F32)
    H = x.shape[1]
    vmask = np.asarray(valid, bool)
    views = [x, fwht(x, 32), fwht(x, D)]
    par, recs, codes = [], [], []
    for c, y in enumerate(views):
        yv = y[vmask]
        mn, mx = yv.min(0), yv.max(0)                                      # [H, 128]
        s, mn = stored_params(mn, mx, recip, f8)
        q, r = kivi_quant(y, mn[None], s[None])
        par.append((s, mn))
        codes.append(q)
        recs.append(r if c == 0 else fwht(r, 32 if c == 1 else D))
    choice = np.zeros((H, NV + 1), int)
    if kfix is not None and not ident:
        kfix = np.asarray(kfix)
        choice[:, :NV] = (kfix[:, None] >> np.arange(NV)[None]) & 1
        choice[:, NV] = (kfix >> 16) & 1
    elif not ident:
        e = [np.where(vmask[:, None, None], r - x, 0).astype(F32) for r in recs]          # [32, H, 128]
        lg = np.einsum("thd,hqd->thq", x, qs).astype(F32)
        with np.errstate(over="ignore"):
            w = np.minimum(np.exp(F32(qsc) * lg - lz[None]), F32(1.0)) * vmask[:, None, None]
        qb = qs.reshape(H, -1, NV, 32)
        aI = np.einsum("thvi,hqvi->thqv", e[0].reshape(32, H, NV, 32), qb)
        aH = np.einsum("thvi,hqvi->thqv", e[1].reshape(32, H, NV, 32), qb)
        aF = np.einsum("thd,hqd->thq", e[2], qs)
        EI = (w[..., None] * aI ** 2).sum((0, 2))                                        # [H, 4]
        EH = (w[..., None] * aH ** 2).sum((0, 2))
        ch = EH < EI
        aB = np.where(ch[None, :, None, :], aH, aI).sum(-1)
        EB = (w * aB ** 2).sum((0, 2))
        EF = (w * aF ** 2).sum((0, 2))
        choice[:, :NV] = ch
        choice[:, NV] = EF < EB
    useF = choice[:, NV] == 1
    cand = np.where(useF[:, None], 2, choice[:, :NV])                                     # [H, 4]
    sel = np.repeat(cand, 32, -1)                                                         # [H, 128]
    code = np.choose(sel[None], codes)
    s = np.choose(sel, [p[0] for p in par])
    mn = np.choose(sel, [p[1] for p in par])
    neg = np.zeros((H, D), bool)
    CHL = NV if f8 else 1                                                                 # channel of flag j: j CHL
    neg[:, 0:NV * CHL:CHL] = (~useF[:, None]) & (choice[:, :NV] == 1)
    neg[:, NV * CHL] = useF
    if f8:
        meta = np.stack([(e4m3_bits(s) & 0x7F) | (neg.astype(np.uint8) << 7), e4m3_bits(mn)], -1)
    else:
        sh = np.abs(_f16(s))
        meta = np.stack([np.where(neg, -sh, sh), _f16(mn)], -1)
    return dict(codes=code.astype(np.uint8), meta=meta, choice=choice, s=s, mn=mn)


# ------------------------------------------------------------------------------------------------ page layout
def write_values(pool, slots, codes, meta, vf, f8=False):
    """scatter per-token value fields (kivi.cu:294-327): VC byte lane = channels 4 lane .. + 3 at 2 bits each, VM pair per
    sub-vector, and the whole-head flag: the VF byte (kivi2, pool uint8 [Np, Hkv, 1552]) or bit 7 of the key scale byte of
    the token's cell, slot 3, whose other bits stay (kivi2p8, pool [Np, Hkv, 1280])."""
    Np, H, _ = pool.shape
    for t, slot in enumerate(np.asarray(slots)):
        if slot < 0:
            continue
        pg, off = int(slot) // PAGE, int(slot) % PAGE
        c = codes[t].reshape(H, 32, 4).astype(np.uint8)
        byte = c[..., 0] | (c[..., 1] << 2) | (c[..., 2] << 4) | (c[..., 3] << 6)
        if f8:
            pool[pg, :, OFF_VC8 + off * 32:OFF_VC8 + off * 32 + 32] = byte
            pool[pg, :, OFF_VM8 + off * 8:OFF_VM8 + off * 8 + 8] = np.asarray(meta[t], np.uint8).reshape(H, 8)
            kb = OFF_KM8 + off * 8 + 2 * (NV - 1)
            pool[pg, :, kb] = (pool[pg, :, kb] & 0x7F) | (np.asarray(vf[t], np.uint8) << 7)
            continue
        pool[pg, :, OFF_VC + off * 32:OFF_VC + off * 32 + 32] = byte
        pool[pg, :, OFF_VM + off * 16:OFF_VM + off * 16 + 16] = np.ascontiguousarray(meta[t]).view(np.uint8).reshape(H, 16)
        pool[pg, :, OFF_VF + off] = vf[t]


def write_key_group(pool, dslot, valid, codes, meta, f8=False):
    """one group's key fields (kivi.cu:600-662): code words of the valid tokens; the (scale, min) pairs of channels
    [4 i, 4 i + 4) go to the cell of the group's i-th position, for all 32 cells.  kivi2p8: bit 7 of the cell's slot-3
    scale byte is the value writer's and is kept (kivi.cu:633-648)."""
    H = pool.shape[1]
    sh = KBIT[np.arange(D) % 16]
    for i, slot in enumerate(np.asarray(dslot)):
        pg, off = int(slot) // PAGE, int(slot) % PAGE
        if valid[i]:
            w = (codes[i].astype(np.uint32) << sh[None].astype(np.uint32)).reshape(H, 8, 16)
            words = np.bitwise_or.reduce(w, -1).astype("<u4")
            pool[pg, :, off * 32:off * 32 + 32] = words.view(np.uint8).reshape(H, 32)
        if f8:
            cell = np.asarray(meta[:, 4 * i:4 * i + 4], np.uint8).reshape(H, 8).copy()
            kb = OFF_KM8 + off * 8
            cell[:, 6] = (cell[:, 6] & 0x7F) | (pool[pg, :, kb + 6] & 0x80)
            pool[pg, :, kb:kb + 8] = cell
            continue
        pool[pg, :, OFF_KM + off * 16:OFF_KM + off * 16 + 16] = np.ascontiguousarray(meta[:, 4 * i:4 * i + 4]).view(np.uint8).reshape(H, 16)


def _meta_fields(ch, f8):
    """raw page fields as float64: key (scale with flag sign, min) [npg, H, 16, 4, 2], value ditto, value whole-head flags
    [npg, H, 16], code bytes of keys [npg, H, 16, 32] and values."""
    npg, H, _ = ch.shape
    if f8:
        kmb = ch[..., OFF_KM8:OFF_VC8].reshape(npg, H, PAGE, NV, 2)
        vmb = ch[..., OFF_VM8:CB8].reshape(npg, H, PAGE, NV, 2)
        km, vm = E4M3_TABLE[kmb], E4M3_TABLE[vmb]
        # the sign of a stored scale is a flag even when the scale is zero: carry it as a sign the callers test with signbit
        km[..., 0] = np.copysign(np.abs(km[..., 0]), np.where(kmb[..., 0] & 0x80, -1.0, 1.0))
        vm[..., 0] = np.copysign(np.abs(vm[..., 0]), np.where(vmb[..., 0] & 0x80, -1.0, 1.0))
        vF = (kmb[..., NV - 1, 0] & 0x80) != 0
        km = km.copy()
        km[..., NV - 1, 0] = np.abs(km[..., NV - 1, 0])             # that sign bit is the value flag, not a key flag
        return km, vm, vF, ch[..., :4 * D].reshape(npg, H, PAGE, 32), ch[..., OFF_VC8:OFF_VM8].reshape(npg, H, PAGE, 32)
    km = np.ascontiguousarray(ch[..., OFF_KM:OFF_VC]).view(np.float16).reshape(npg, H, PAGE, NV, 2).astype(np.float64)
    vm = np.ascontiguousarray(ch[..., OFF_VM:OFF_VF]).view(np.float16).reshape(npg, H, PAGE, NV, 2).astype(np.float64)
    return (km, vm, ch[..., OFF_VF:OFF_VF + PAGE] != 0, ch[..., :4 * D].reshape(npg, H, PAGE, 32),
            ch[..., OFF_VC:OFF_VM].reshape(npg, H, PAGE, 32))


def dequant_groups(ch, f8=False):
    """chunks of whole groups [2 ng, Hkv, chunk] (pages 2 g, 2 g + 1 in order) -> K, V float64 [2 ng 16, Hkv, 128] in the
    original basis (independent restatement of integrations/vllm_flagrot/vllm_flagrot/kivi.py:208-265).  Key flags: sign
    of the scale of channel j CHL (sub-vector j is H32) and of channel NV CHL (whole head), CHL = 1 (kivi2) | NV (kivi2p8)."""
    npg, H, _ = ch.shape
    ng = npg // 2
    km, vm, vF, kcb, vcb = _meta_fields(ch, f8)
    kc = kcb.reshape(npg, H, PAGE, 8, 4)
    words = (kc[..., 0].astype(np.uint32) | (kc[..., 1].astype(np.uint32) << 8) | (kc[..., 2].astype(np.uint32) << 16)
             | (kc[..., 3].astype(np.uint32) << 24))
    codes = ((words[..., None] >> KBIT.astype(np.uint32)) & 3).reshape(npg, H, PAGE, D).astype(np.float64)
    kmg = km.reshape(ng, 2, H, PAGE, NV, 2).transpose(0, 2, 1, 3, 4, 5).reshape(ng, H, D, 2)
    s, mn = kmg[..., 0], kmg[..., 1]
    CHL = NV if f8 else 1
    lbits = np.signbit(s[..., 0:NV * CHL:CHL])
    fbit = np.signbit(s[..., NV * CHL])
    s = np.abs(s)
    codes = codes.reshape(ng, 2, H, PAGE, D).transpose(0, 2, 1, 3, 4).reshape(ng, H, 32, D)
    k = codes * s[:, :, None] + mn[:, :, None]
    kb = k.reshape(ng, H, 32, NV, 32)
    kh = np.where((lbits & ~fbit[..., None])[:, :, None, :, None], kb @ hadamard(32), kb).reshape(ng, H, 32, D)
    k = np.where(fbit[:, :, None, None], k @ hadamard(D), kh).transpose(0, 2, 1, 3).reshape(ng * 32, H, D)
    vcode = ((vcb[..., None] >> np.array([0, 2, 4, 6], np.uint8)) & 3).reshape(npg, H, PAGE, NV, 32).astype(np.float64)
    vs, vmn = vm[..., 0], vm[..., 1]
    vl = np.signbit(vs)
    v = vcode * np.abs(vs)[..., None] + vmn[..., None]
    vh = np.where(vl[..., None], v @ hadamard(32), v).reshape(npg, H, PAGE, D)
    v = np.where(vF[..., None], v.reshape(npg, H, PAGE, D) @ hadamard(D), vh).transpose(0, 2, 1, 3).reshape(npg * PAGE, H, D)
    return k, v


def decode_reference(q_bits, pool, bt, cached, scale, kv_start, G, ring=None, tail_len=None, tail_idx=None, f8=False):
    """float64 attention over page tokens [kv_start, cached[b]) + BF16 ring slots [0, tail_len[b]) of row tail_idx[b]
    (integrations/vllm_flagrot/tests/test_kivi.py:236-250).  ring uint16 [R, T, 2 Hkv, 128]."""
    q = bf16_bits_to_f32(q_bits).astype(np.float64)
    B, Hq, _ = q.shape
    H = Hq // G
    out = np.zeros((B, Hq, D))
    for b in range(B):
        c = int(cached[b])
        ks, vs = [], []
        if c > kv_start:
            ng = (c + GRP - 1) // GRP
            k, v = dequant_groups(pool[np.asarray(bt[b, :2 * ng], np.int64)], f8)
            ks.append(k[kv_start:c])
            vs.append(v[kv_start:c])
        if ring is not None and int(tail_len[b]) > 0:
            r = bf16_bits_to_f32(ring[int(tail_idx[b]) if tail_idx is not None else 0, :int(tail_len[b])]).astype(np.float64)
            ks.append(r[:, :H])
            vs.append(r[:, H:])
        if not ks:
            continue
        k, v = np.concatenate(ks), np.concatenate(vs)
        qb = q[b].reshape(H, G, D)
        s = np.einsum("hgd,thd->hgt", qb, k) * scale
        p = np.exp(s - s.max(-1, keepdims=True))
        p /= p.sum(-1, keepdims=True)
        out[b] = np.einsum("hgt,thd->hgd", p, v).reshape(Hq, D)
    return out
