"""Generates tests/golden/*.npz by running the reference's own PyTorch code on CPU on seeded inputs.

    python tests/golden/make_golden.py [/path/to/reference]      (the reference checkout; else $FLAGROT_REFERENCE, else ./reference)

What is recorded (inputs as bf16 bit patterns, outputs exactly as the reference returned them):
  writer_dynamic.npz   kernels/codebook_ref.encode (cfg konlya / konlya2, qk asym / asym2) for keys and values, incl. the
                       edge rows of integrations/vllm_flagrot/tests/test_kernels.py:239-256 and a centred case
  writer_static.npz    kernels/ref.sel_fwht_rb + kernels/ref.int4a_quant, blockflag.formats.quant_asym_dep(bits 2) +
                       scale_word, and the whole-head fp32 butterfly + bf16 rounding step
  pages.npz            pools packed by the oracle's packer and READ BACK BY THE REFERENCE'S PARSERS
                       (vllm_flagrot/kernels.py parse_pages / dequant_cb_pages / dequant_v2_pages): pins both the packer and
                       the oracle's parser against the reference's layout code
  decode.npz           float64 attention over the reference-parsed pages (test_kernels.py ref_attn semantics) with BF16
                       tails, row indirection and kv_start, for the small configuration of the baseline (batch 2, 8 q / 2 kv
                       heads, context 512, page 16, 4 sinks + 32 window) in konlya, konlya2, static int4a and static int2a
The reference runs on CPU here, so its scale is a true division ((max - min) / lv); the oracle is pinned in that mode
(recip=False).  The reference tree is needed only to regenerate the files, never to run the tests.
"""
from __future__ import annotations

import math
import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REF = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("FLAGROT_REFERENCE", "reference"))   # checkout of the reference
sys.path.insert(0, str(HERE.parents[1]))
sys.path.insert(0, str(REF))
sys.path.insert(0, str(REF / "kernels"))
sys.path.insert(0, str(REF / "integrations" / "vllm_flagrot"))

import codebook_ref as CR  # noqa: E402
import ref as R  # noqa: E402
from blockflag import formats as FM  # noqa: E402
from vllm_flagrot import kernels as K  # noqa: E402

from oracle import flagrot_oracle as O  # noqa: E402

P = 16


def bits_of(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def edge_rows(T, Hkv, g, scale_k=6.0):
    """rows of integrations/vllm_flagrot/tests/test_kernels.py:239-256 (shape recipe re-stated, not the data)."""
    kv = torch.randn(T, 2 * Hkv, 128, generator=g)
    kv[:, :Hkv, :4] *= scale_k
    grp = kv.view(T, 2 * Hkv, 4, 32)
    sel = torch.rand(T, 2 * Hkv, 4, generator=g)
    grp[sel < 0.04] = grp[sel < 0.04].abs() + 0.5
    m = (sel >= 0.04) & (sel < 0.08)
    grp[m] = -grp[m].abs() - 0.5
    grp[(sel >= 0.08) & (sel < 0.10)] = 0.0
    grp[(sel >= 0.10) & (sel < 0.12)] *= 1e-5
    grp[(sel >= 0.12) & (sel < 0.14)] *= 300
    grp[(sel >= 0.14) & (sel < 0.15)] = 1.25
    one = (sel >= 0.15) & (sel < 0.16)
    grp[one] = 0.0
    grp[..., 5][one] = 3.0
    return kv.bfloat16()


def calib(Hkv, g, full=True):
    w = torch.rand(Hkv, 128, generator=g) + 0.5
    if full:
        qs = torch.randn(Hkv, 512, 128, generator=g) * w.sqrt()[:, None, :]
        Cq = torch.einsum("hnd,hne->hde", qs, qs) / 512
    else:
        Cq = torch.diag_embed(w)
    co = torch.rand(Hkv, 128, generator=g) + 0.5
    return Cq.contiguous(), co


def ref_words(ek, ev):
    """word assembly of integrations/vllm_flagrot/tests/test_int2.py:141-152."""
    wk = ek["s"].half().view(torch.int16).to(torch.int32) & 0xFFFF
    wk = wk | (((ek["mode"] == 0)[..., None] & (ek["local"] == 1)).to(torch.int32) << 15)
    wv = ev["s"].half().view(torch.int16).to(torch.int32) & 0xFFFF
    wv[..., 0] |= (ek["mode"] == 2).to(torch.int32) << 15
    return wk, wv


def gen_dynamic():
    out = {}
    g = torch.Generator().manual_seed(101)
    Hkv = 2
    for name, T, full, center in (("a", 96, True, False), ("b", 64, False, True)):
        kv = edge_rows(T, Hkv, g)
        Cq, co = calib(Hkv, g, full)
        kmu = None
        if center:
            kmu = (torch.randn(Hkv, 128, generator=g) * 0.5).float()
        out[f"{name}_kv"] = bits_of(kv)
        out[f"{name}_Cq"] = Cq.numpy()
        out[f"{name}_co"] = co.numpy()
        if kmu is not None:
            out[f"{name}_kmu"] = kmu.numpy()
        for cfg, qk, bits in (("konlya", "asym", 4), ("konlya2", "asym2", 2)):
            k = kv[:, :Hkv].float()
            if kmu is not None:
                k = k - kmu
            ek = CR.encode(k, Cq, co, "k", cfg=cfg, qk=qk)
            ev = CR.encode(kv[:, Hkv:].float(), Cq, co, "v", cfg=cfg, qk=qk)
            wk, wv = ref_words(ek, ev)
            out[f"{name}_{bits}_qk"] = ek["q"].numpy().astype(np.uint8)
            out[f"{name}_{bits}_qv"] = ev["q"].numpy().astype(np.uint8)
            out[f"{name}_{bits}_wk"] = wk.numpy().astype(np.int32)
            out[f"{name}_{bits}_wv"] = wv.numpy().astype(np.int32)
            out[f"{name}_{bits}_mode"] = ek["mode"].numpy().astype(np.int8)
            out[f"{name}_{bits}_local"] = ek["local"].numpy().astype(np.int8)
            out[f"{name}_{bits}_herr"] = ek["head_errs"].numpy()
            out[f"{name}_{bits}_rec"] = ek["rec"].numpy()
    np.savez_compressed(HERE / "writer_dynamic.npz", **out)
    return out


def _load_head_fwht_ref():
    """the reference's own torch emulation of fr_head_fwht (kernels/test_w3_static.py head_fwht_ref).  That script imports
    CUDA-only loaders at module level, so only this one function is taken from its source and executed."""
    import ast
    src = (REF / "kernels" / "test_w3_static.py").read_text()
    fn = next(n for n in ast.parse(src).body if isinstance(n, ast.FunctionDef) and n.name == "head_fwht_ref")
    ns = {"torch": torch}
    exec(compile(ast.Module(body=[fn], type_ignores=[]), "test_w3_static.py", "exec"), ns)
    return ns["head_fwht_ref"]


head_fwht_ref = _load_head_fwht_ref()


def gen_static():
    out = {}
    g = torch.Generator().manual_seed(202)
    Hkv, T = 2, 80
    kv = edge_rows(T, Hkv, g)
    mask = (torch.rand(2 * Hkv, 4, generator=g) < 0.5).to(torch.uint8)
    hfull = torch.tensor([1, 0, 0, 1], dtype=torch.uint8)
    kmu = (torch.randn(Hkv, 128, generator=g) * 0.5).float()
    out.update(kv=bits_of(kv), mask=mask.numpy(), hfull=hfull.numpy(), kmu=kmu.numpy())
    for tag, hf, km in (("plain", None, None), ("hfull", hfull, None), ("kmu", None, kmu), ("both", hfull, kmu)):
        x = kv if hf is None else head_fwht_ref(kv, hf)
        if hf is not None:
            out[f"{tag}_hf"] = bits_of(x)
        xf = x.float()
        if km is not None:
            xf = xf.clone()
            xf[:, :Hkv] = xf[:, :Hkv] - km
        y = R.sel_fwht_rb(xf.reshape(T, 2 * Hkv * 128), mask, 32).reshape(T, 2 * Hkv, 128)
        q4, w4 = R.int4a_quant(y)
        q2, z2, s2, _ = FM.quant_asym_dep(y, 32, False, 2)
        w2 = FM.scale_word(s2, z2, 2).squeeze(-1)
        out[f"{tag}_q4"] = q4.numpy().astype(np.uint8)
        out[f"{tag}_w4"] = w4.numpy().astype(np.int32)
        out[f"{tag}_q2"] = q2.reshape(y.shape).numpy().astype(np.uint8)
        out[f"{tag}_w2"] = (w2.numpy().astype(np.int32) & 0xFFFF)
    np.savez_compressed(HERE / "writer_static.npz", **out)
    return out


def ref_attn(q, Kc, Vc, lens, scale, tails=None, kv_start=0):
    """integrations/vllm_flagrot/tests/test_kernels.py:37-56 (float64 attention), restated for the generator."""
    B, Hq, Dh = q.shape
    G = Hq // Kc.shape[2]
    out = torch.zeros(B, Hq, Dh, dtype=torch.float64)
    for b in range(B):
        a = min(kv_start, lens[b])
        ks, vs = [Kc[b, a:lens[b]]], [Vc[b, a:lens[b]]]
        if tails is not None and tails[b] is not None:
            ks.append(tails[b][0])
            vs.append(tails[b][1])
        k = torch.cat(ks).double().repeat_interleave(G, 1)
        v = torch.cat(vs).double().repeat_interleave(G, 1)
        if k.shape[0] == 0:
            continue
        s = torch.einsum("hd,lhd->hl", q[b].double(), k) * scale
        p = torch.exp(s - s.amax(-1, keepdim=True))
        p = p / p.sum(-1, keepdim=True)
        out[b] = torch.einsum("hl,lhd->hd", p, v)
    return out


def sel_rot(x, mask, rb=32):
    H = K.hadamard(rb, x.device, x.dtype)
    xb = x.reshape(*x.shape[:-1], x.shape[-1] // rb, rb)
    return torch.where(mask[..., None].bool(), xb @ H, xb).reshape(x.shape)


def gen_pages_and_decode():
    """baseline configuration 0: batch 2, 8 q / 2 kv heads, d 128, context 512, page 16, 4 sinks + 32 window tokens in BF16;
    K ~ N(0,1) with 4 random channels per kv head x8, V, q ~ N(0,1), attention weights ~ U(0.5, 1.5)."""
    dec = {}
    g = torch.Generator().manual_seed(0)
    B, Hq, Hkv, L, S, W = 2, 8, 2, 512, 4, 32
    G = Hq // Hkv
    kv = torch.randn(B, L, 2 * Hkv, 128, generator=g)
    for h in range(Hkv):
        ch = torch.randperm(128, generator=g)[:4]
        kv[:, :, h, ch] *= 8
    kv = kv.bfloat16()
    q = torch.randn(B, Hq, 128, generator=g).bfloat16()
    Cq, co = calib(Hkv, g, True)
    npg = B * (L // P) + 7
    perm = torch.randperm(npg, generator=g)[:B * (L // P)].reshape(B, L // P).int()
    mask = (torch.rand(2 * Hkv, 4, generator=g) < 0.5).to(torch.uint8)
    lens = [L - W, L - W - 13]
    scale = 1 / math.sqrt(128)
    # BF16 ring rows: sinks then the newest W tokens of each sequence, 3 rows with indirection
    ring = torch.randn(3, S + W, 2 * Hkv, 128, generator=g).bfloat16()
    tail_idx = torch.tensor([2, 0], dtype=torch.int32)
    tail_len = torch.tensor([S + W, S + 20], dtype=torch.int32)
    for b in range(B):
        ring[int(tail_idx[b]), :S] = kv[b, :S]
        n = int(tail_len[b]) - S
        ring[int(tail_idx[b]), S:S + n] = kv[b, lens[b]:lens[b] + n]
    dec.update(q=bits_of(q), kv=bits_of(kv), Cq=Cq.numpy(), co=co.numpy(), bt=perm.numpy(), mask=mask.numpy(),
               lens=np.array(lens, np.int32), ring=bits_of(ring), tail_idx=tail_idx.numpy(), tail_len=tail_len.numpy(),
               scale=np.float64(scale), kv_start=np.int32(S))
    slots = (perm.long()[:, torch.arange(L) // P] * P + torch.arange(L) % P)          # [B, L]
    rows = kv.reshape(B * L, 2 * Hkv, 128)
    for kind, bits, key_only in (("konlya", 4, True), ("konlya2", 2, True), ("int4a", 4, False), ("int2a", 2, False)):
        rs = np.random.RandomState(7)
        pool = rs.randint(0, 256, (npg, Hkv, O.chunk_bytes(bits, P)), dtype=np.uint8)
        kvb = bits_of(rows)
        if key_only:
            codes, words, _ = O.dynamic_rows(kvb, Cq.numpy(), bits, None, recip=False)
        else:
            codes, words = O.static_rows(kvb, mask.numpy(), None, bits, None, recip=False)
        O.write_pool(pool, slots.reshape(-1).numpy(), codes, words, bits, P)
        tp = torch.from_numpy(pool)
        if key_only:
            Kp, Vp = K.dequant_cb_pages(tp, P, kind, torch.float64)
        else:
            Kp, Vp = K.dequant_v2_pages(tp, P, torch.float64, fmt=kind)
        Kc = Kp[perm.long()].reshape(B, L, Hkv, 128)
        Vc = Vp[perm.long()].reshape(B, L, Hkv, 128)
        tails = [(ring[int(tail_idx[b]), :int(tail_len[b]), :Hkv], ring[int(tail_idx[b]), :int(tail_len[b]), Hkv:])
                 for b in range(B)]
        for tag, tl, ks in (("plain", None, 0), ("tail", tails, S)):
            if key_only:
                o = ref_attn(q.double(), Kc, Vc, lens, scale, tl, ks)
            else:
                km, vm = mask[:Hkv].bool(), mask[Hkv:].bool()
                qr = sel_rot(q.double().view(B, Hkv, G, 128).transpose(1, 2), km).transpose(1, 2).reshape(B, Hq, 128)
                tr = None if tl is None else [(sel_rot(t[0].double(), km), sel_rot(t[1].double(), vm)) for t in tl]
                oo = ref_attn(qr, Kc, Vc, lens, scale, tr, ks)
                o = sel_rot(oo.view(B, Hkv, G, 128).transpose(1, 2), vm).transpose(1, 2).reshape(B, Hq, 128)
            dec[f"{kind}_{tag}"] = o.numpy()
    np.savez_compressed(HERE / "decode.npz", **dec)


def gen_pages():
    """small pools (6 pages, 2 kv heads) packed by the oracle at scattered slots with holes, read back by the
    reference's parsers."""
    pages = {}
    g = torch.Generator().manual_seed(303)
    Hkv, T, npg = 2, 61, 6
    kv = edge_rows(T, Hkv, g)
    Cq, co = calib(Hkv, g, True)
    mask = (torch.rand(2 * Hkv, 4, generator=g) < 0.5).to(torch.uint8)
    slots = torch.randperm(npg * P, generator=g)[:T].long()
    slots[torch.rand(T, generator=g) < 0.1] = -1
    pages.update(kv=bits_of(kv), Cq=Cq.numpy(), mask=mask.numpy(), slots=slots.numpy())
    for kind, bits, key_only in (("konlya", 4, True), ("konlya2", 2, True), ("int4a", 4, False), ("int2a", 2, False)):
        rs = np.random.RandomState(11)
        pool = rs.randint(0, 256, (npg, Hkv, O.chunk_bytes(bits, P)), dtype=np.uint8)
        pages[f"{kind}_pool0"] = pool.copy()
        if key_only:
            codes, words, _ = O.dynamic_rows(bits_of(kv), Cq.numpy(), bits, None, recip=False)
        else:
            codes, words = O.static_rows(bits_of(kv), mask.numpy(), None, bits, None, recip=False)
        O.write_pool(pool, slots.numpy(), codes, words, bits, P)
        tp = torch.from_numpy(pool)
        c, m, sb = K.parse_pages(tp, P, kind)                                        # reference parser
        pages[f"{kind}_pool"] = pool
        pages[f"{kind}_codes"] = c.numpy()
        pages[f"{kind}_sbits"] = sb.numpy()
        if key_only:
            Kp, Vp = K.dequant_cb_pages(tp, P, kind, torch.float64)
        else:
            Kp, Vp = K.dequant_v2_pages(tp, P, torch.float64, fmt=kind)
        pages[f"{kind}_K"] = Kp.numpy()
        pages[f"{kind}_V"] = Vp.numpy()
    np.savez_compressed(HERE / "pages.npz", **pages)


def gen_kivi():
    """FlagRot-KIVI (kivi2:32): plain KIVI reconstructions (blockflag.formats.fake via qattention._fake_tok_ for keys along the
    token axis, formats.fake for values) and the simulator's dynamic choices (the functions of
    integrations/vllm_flagrot/tests/test_kivi.py:72-88: qattention._weights / _vec_err / _head_err / _pool_tokens) and
    reconstructions (qattention.dyn_quant), each 32-token group on its own, group 0 without its 4 sink tokens."""
    from blockflag import qattention as QA
    from blockflag.hadamard import fwht
    g = torch.Generator().manual_seed(404)
    H, ng, S, NQ = 2, 6, 4, 192
    T = ng * 32
    mu = torch.randn(H, 128, generator=g) * 2.0
    mu[:, torch.randint(0, 128, (6,), generator=g)] *= 6
    k = (mu[None] + torch.randn(T, H, 128, generator=g) * (0.5 + torch.rand(H, 128, generator=g))).bfloat16()
    v = (torch.randn(T, H, 128, generator=g) * 0.3 + mu[None] * 0.05).bfloat16()
    qs = torch.randn(H, NQ, 128, generator=g) * 0.3
    lz = torch.full((H, NQ), 5.0)
    co = torch.rand(H, 128, generator=g) + 0.1
    qscale = 1 / math.sqrt(128)
    out = dict(k=bits_of(k), v=bits_of(v), qs=qs.numpy(), lz=lz.numpy(), co=co.numpy(), qscale=np.float64(qscale), S=np.int32(S))
    SPEC = "kivi2:32"
    QA.KV.update(dyn=dict(rule="att", local=["H"], head=["F"], group=1, only=None), sink=0, qs={0: qs}, lz={0: lz},
                 qscale=qscale, co={0: co}, xf=None, dynstat={})
    xf = k.float().permute(1, 0, 2)[None]                                    # [1, H, T, 128]
    vf = v.float().permute(1, 0, 2)[None]
    rec_id = torch.empty_like(xf)
    rec_dyn = torch.empty_like(xf)
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
        hs = he.argmin(0)
        lbs.append(ch[0][:, 0].numpy())                                      # [H, 4]
        fbs.append(hs[0][:, 0].numpy())                                      # [H]
    rec_id[:, :, :S] = xf[:, :, :S]
    rec_dyn[:, :, :S] = xf[:, :, :S]
    out.update(k_rec_ident=rec_id[0].permute(1, 0, 2).numpy(), k_rec_dyn=rec_dyn[0].permute(1, 0, 2).numpy(),
               k_local=np.stack(lbs).astype(np.int8), k_head=np.stack(fbs).astype(np.int8))
    out["v_rec_ident"] = FM.fake(vf, SPEC)[0].permute(1, 0, 2).numpy()
    out["v_rec_dyn"] = QA.dyn_quant(vf, SPEC, 32, "v", 0)[0].permute(1, 0, 2).numpy()
    np.savez_compressed(HERE / "kivi.npz", **out)


if __name__ == "__main__":
    torch.manual_seed(0)
    gen_dynamic()
    gen_static()
    gen_pages_and_decode()
    gen_pages()
    gen_kivi()
    for f in sorted(HERE.glob("*.npz")):
        print(f.name, f.stat().st_size)
