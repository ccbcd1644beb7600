"""CPU restatement (numpy) of the FlagRot-KIVI INT2 path: the KIVI group quantizer, the per-token value encoder, the
per-(32-token group, kv head) key encoder with the attention-weighted selection rule, the page layout (packer + parser)
and float64 decode attention over parsed pages.

TEST INFRASTRUCTURE ONLY (used by tests/ and nothing else).  Restates integrations/vllm_flagrot/csrc/kivi.cu (semantics,
cited per function), blockflag/formats.py:103-116 (fake_kivi) and blockflag/qattention.py:105-145,147-188 (rule "att").
Pinned by tests/golden/kivi.npz (outputs of the reference's simulator run on CPU; tests/golden/make_golden.py):
plain-KIVI reconstructions bit for bit, dynamic choices statistically (the reference's own tests accept up to 2 %
mismatching choices for this encoder: integrations/vllm_flagrot/tests/test_kivi.py:140,175).
`recip`: s = (max - min) / 3 is a true division on the CPU reference and a multiply by fp32(1/3) on the GPU.
"""
from __future__ import annotations

import numpy as np

from .flagrot_oracle import F32, bf16_bits_to_f32, fwht, hadamard

D, NV, PAGE, GRP = 128, 4, 16, 32
CB = 12 * D + 16
OFF_KM, OFF_VC, OFF_VM, OFF_VF = 4 * D, 6 * D, 10 * D, 12 * D
KBIT = np.array([2 * (i >> 1) + 16 * (i & 1) for i in range(16)])


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
def encode_values(x, co, ident=False, vfix=None, recip=True):
    """x fp32 [T, H, 128]; co fp32 [H, 128].  Candidates identity / H32 per 32-dim sub-vector / whole-head H128, groups of
    32 along the head dim; error sum d^2 co; H32 only if strictly better, whole head only if strictly better than the
    combination (kivi.cu:163-328).  Returns dict: codes uint8 [T, H, 128], meta float16 [T, H, 4, 2] (scale with the H32 flag
    in its sign, min), vf uint8 [T, H], cand int [T, H, 4] (0 I, 1 H32, 2 whole head), s / mn fp32 [T, H, 4] before storage."""
    x = np.asarray(x, F32)
    T, H, _ = x.shape
    outs = []
    for c in range(3):
        y = x if c == 0 else fwht(x, 32 if c == 1 else D)
        b = y.reshape(T, H, NV, 32)
        mn, mx = b.min(-1, keepdims=True), b.max(-1, keepdims=True)
        s = kivi_params(mn, mx, recip)
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
    sh = _f16(s)
    sh = np.where(cand == 1, -np.abs(sh), sh)
    meta = np.stack([sh, _f16(mn)], -1)
    return dict(codes=codes.astype(np.uint8), meta=meta, vf=(cand[..., 0] == 2).astype(np.uint8), cand=cand, s=s, mn=mn)


# ------------------------------------------------------------------------------------------------ keys (per group)
def encode_key_group(x, valid, qs, lz, qsc, ident=False, kfix=None, recip=True):
    """one 32-token group: x fp32 [32, H, 128], valid bool [32] (sinks excluded), calibration queries qs fp32 [H, NQ, 128],
    lz fp32 [H, NQ].  Per channel over the valid tokens: INT2 of the identity / per-token H32 / per-token H128 views; rule
    "att": w[t, q] = min(1, exp(qsc x_t . q - lz_q)), error of a candidate = sum_{t, q} w (q . e_t)^2 over the group (per
    sub-vector for I / H32); H32 only if strictly better, whole head only if strictly better than the combination
    (kivi.cu:343-663; qattention.py:127-145,166-188).  Returns codes uint8 [32, H, 128] (valid tokens), meta float16
    [H, 128, 2] (scale with flag signs: channel j < 4 -> sub-vector j is H32, channel 4 -> whole head; min), choices [H, 5],
    and the fp32 (scale, min) before storage."""
    x = np.asarray(x, F32)
    H = x.shape[1]
    vmask = np.asarray(valid, bool)
    views = [x, fwht(x, 32), fwht(x, D)]
    par, recs, codes = [], [], []
    for c, y in enumerate(views):
        yv = y[vmask]
        mn, mx = yv.min(0), yv.max(0)                                      # [H, 128]
        s = kivi_params(mn, mx, recip)
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
    sh = np.abs(_f16(s))
    neg = np.zeros((H, D), bool)
    neg[:, :NV] = (~useF[:, None]) & (choice[:, :NV] == 1)
    neg[:, NV] = useF
    sh = np.where(neg, -sh, sh)
    return dict(codes=code.astype(np.uint8), meta=np.stack([sh, _f16(mn)], -1), choice=choice, s=s, mn=mn)


# ------------------------------------------------------------------------------------------------ page layout
def write_values(pool, slots, codes, meta, vf):
    """scatter per-token value fields (kivi.cu:305-327): VC byte lane = channels 4 lane .. + 3 at 2 bits each, VM half2 per
    sub-vector, VF byte.  pool uint8 [Np, Hkv, 1552]."""
    Np, H, _ = pool.shape
    for t, slot in enumerate(np.asarray(slots)):
        if slot < 0:
            continue
        pg, off = int(slot) // PAGE, int(slot) % PAGE
        c = codes[t].reshape(H, 32, 4).astype(np.uint8)
        pool[pg, :, OFF_VC + off * 32:OFF_VC + off * 32 + 32] = c[..., 0] | (c[..., 1] << 2) | (c[..., 2] << 4) | (c[..., 3] << 6)
        pool[pg, :, OFF_VM + off * 16:OFF_VM + off * 16 + 16] = np.ascontiguousarray(meta[t]).view(np.uint8).reshape(H, 16)
        pool[pg, :, OFF_VF + off] = vf[t]


def write_key_group(pool, dslot, valid, codes, meta):
    """one group's key fields (kivi.cu:600-662): code words of the valid tokens; the (scale, min) pairs of channels
    [4 i, 4 i + 4) go to the cell of the group's i-th position, for all 32 cells."""
    H = pool.shape[1]
    sh = KBIT[np.arange(D) % 16]
    for i, slot in enumerate(np.asarray(dslot)):
        pg, off = int(slot) // PAGE, int(slot) % PAGE
        if valid[i]:
            w = (codes[i].astype(np.uint32) << sh[None].astype(np.uint32)).reshape(H, 8, 16)
            words = np.bitwise_or.reduce(w, -1).astype("<u4")
            pool[pg, :, off * 32:off * 32 + 32] = words.view(np.uint8).reshape(H, 32)
        pool[pg, :, OFF_KM + off * 16:OFF_KM + off * 16 + 16] = np.ascontiguousarray(meta[:, 4 * i:4 * i + 4]).view(np.uint8).reshape(H, 16)


def dequant_groups(ch):
    """chunks of whole groups [2 ng, Hkv, 1552] (pages 2 g, 2 g + 1 in order) -> K, V float64 [2 ng 16, Hkv, 128] in the original
    basis (independent restatement of integrations/vllm_flagrot/vllm_flagrot/kivi.py:229-265)."""
    npg, H, _ = ch.shape
    ng = npg // 2
    kc = ch[..., :4 * D].reshape(npg, H, PAGE, 8, 4)
    words = (kc[..., 0].astype(np.uint32) | (kc[..., 1].astype(np.uint32) << 8) | (kc[..., 2].astype(np.uint32) << 16)
             | (kc[..., 3].astype(np.uint32) << 24))
    codes = ((words[..., None] >> KBIT.astype(np.uint32)) & 3).reshape(npg, H, PAGE, D).astype(np.float64)
    km = np.ascontiguousarray(ch[..., OFF_KM:OFF_VC]).view(np.float16).reshape(npg, H, PAGE, NV, 2)
    kmg = km.reshape(ng, 2, H, PAGE, NV, 2).transpose(0, 2, 1, 3, 4, 5).reshape(ng, H, D, 2).astype(np.float64)
    s, mn = kmg[..., 0], kmg[..., 1]
    lbits = np.signbit(s[..., :NV])
    fbit = np.signbit(s[..., NV])
    s = np.abs(s)
    codes = codes.reshape(ng, 2, H, PAGE, D).transpose(0, 2, 1, 3, 4).reshape(ng, H, 32, D)
    k = codes * s[:, :, None] + mn[:, :, None]
    kb = k.reshape(ng, H, 32, NV, 32)
    kh = np.where((lbits & ~fbit[..., None])[:, :, None, :, None], kb @ hadamard(32), kb).reshape(ng, H, 32, D)
    k = np.where(fbit[:, :, None, None], k @ hadamard(D), kh).transpose(0, 2, 1, 3).reshape(ng * 32, H, D)
    vc = ch[..., OFF_VC:OFF_VM].reshape(npg, H, PAGE, 32)
    vcode = ((vc[..., None] >> np.array([0, 2, 4, 6], np.uint8)) & 3).reshape(npg, H, PAGE, NV, 32).astype(np.float64)
    vm = np.ascontiguousarray(ch[..., OFF_VM:OFF_VF]).view(np.float16).reshape(npg, H, PAGE, NV, 2).astype(np.float64)
    vs, vmn = vm[..., 0], vm[..., 1]
    vl = np.signbit(vs)
    v = vcode * np.abs(vs)[..., None] + vmn[..., None]
    vF = ch[..., OFF_VF:OFF_VF + PAGE] != 0
    vh = np.where(vl[..., None], v @ hadamard(32), v).reshape(npg, H, PAGE, D)
    v = np.where(vF[..., None], v.reshape(npg, H, PAGE, D) @ hadamard(D), vh).transpose(0, 2, 1, 3).reshape(npg * PAGE, H, D)
    return k, v


def decode_reference(q_bits, pool, bt, cached, scale, kv_start, G, ring=None, tail_len=None, tail_idx=None):
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
            k, v = dequant_groups(pool[np.asarray(bt[b, :2 * ng], np.int64)])
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
