"""GPU parity of paged decode attention (static int4a / int2a, key-only konlya / konlya2) through the C ABI against the
oracle: float64 attention over the pages parsed by the oracle's independent layout parser, BF16 window rows treated
identically.  Case shapes follow the reference's integrations/vllm_flagrot/tests/test_kernels.py:82-175, 352-384:
lengths 1 .. 33000, windows with row indirection, shared / stride-0 block-table rows, kv_start, GQA groups 4 / 5 / 6 / 8 /
12, forced split counts, empty rows.

Tolerances (written here as the baseline states them): max-abs <= 2e-2 and relative RMS <= 1e-2 against the oracle on
the same quantised cache; in addition the reference's own, tighter criterion max|err| / max|ref| <= max(2 x the error of
attention on bf16-rounded operands, 4e-3)."""
import math

import numpy as np
import pytest
import torch

from oracle import flagrot_oracle as O
from tests._util import P, bits, calib

pytestmark = pytest.mark.gpu
DEV = "cuda"
LOG2E = 1.4426950408889634
FMT = {"int4a": (4, False), "int2a": (2, False), "konlya": (4, True), "konlya2": (2, True), "int4": (4, False), "konly": (4, True)}
SYM = ("int4", "konly")          # symmetric INT4 pages: sign-magnitude codes, plain FP16 scale words


@pytest.fixture(scope="module")
def K():
    from flagrot_releaser_b200 import kernels
    kernels.lib()
    return kernels


def alloc(lens, num_pages, g, P=P):
    need = [(n + P - 1) // P for n in lens]
    ids = torch.randperm(num_pages, generator=g)[:sum(need)]
    bt = torch.zeros(len(lens), max(max(need), 1), dtype=torch.int32)
    o = 0
    for b, n in enumerate(need):
        bt[b, :n] = ids[o:o + n].int()
        o += n
    return bt


def run_case(K, fmt, lens, win=None, bt_shared=False, seed=0, G=4, Hkv=8, kv_start=0, nsplit=None, partial=False, P=P):
    nb, key_only = FMT[fmt]
    g = torch.Generator().manual_seed(seed)
    B, Hq = len(lens), G * Hkv
    num_pages = (sum((n + P - 1) // P for n in lens) if not bt_shared else (max(lens) + P - 1) // P) + 7
    chunk_b = K.v2_chunk_bytes(P, 128, fmt)
    pool = torch.randint(0, 256, (num_pages, Hkv, chunk_b), dtype=torch.uint8, generator=g).to(DEV)   # garbage pool
    bt = alloc(lens if not bt_shared else [max(lens)], num_pages, g, P)
    mask = (torch.rand(2 * Hkv, 4, generator=g) < 0.5).to(torch.uint8)
    Cq, co = calib(Hkv, g)
    CT = Cq.transpose(1, 2).contiguous().to(DEV)
    for b in range(B if not bt_shared else 1):
        n = max(lens) if bt_shared else lens[b]
        if n == 0:
            continue
        kv = torch.randn(n, 2 * Hkv, 128, generator=g)
        kv[:, :Hkv, :4] *= 6
        kv = kv.bfloat16().to(DEV)
        pos = torch.arange(n)
        sl = (bt[b].long()[pos // P] * P + pos % P).to(DEV)
        if fmt == "konly":      # no dynamic writer for the symmetric key-only kind: rows packed by the oracle with random flags
            x = O.bf16_bits_to_f32(bits(kv.cpu()))
            qq, ww = O.quant_sym_store(x)
            codes = np.stack([qq[:, :Hkv], qq[:, Hkv:]], 2)
            words = np.stack([ww[:, :Hkv], ww[:, Hkv:]], 2)
            rs = np.random.RandomState(seed + b)
            words[:, :, 0] |= (rs.rand(n, Hkv, 4) < 0.3).astype(np.int32) << 15       # H32 flags of the key groups
            words[:, :, 1, 0] |= (rs.rand(n, Hkv) < 0.2).astype(np.int32) << 15       # whole-head flag of the key
            pn = pool.cpu().numpy()
            O.write_pool_sym(pn, sl.cpu().numpy(), codes, words, P)
            pool.copy_(torch.from_numpy(pn))
        elif key_only:
            K.cb_write(kv, sl, CT, co.to(DEV), fmt, pool, P)
        else:
            K.v2_write(kv, sl, mask.to(DEV), 32, pool, P, fmt=fmt)
    if bt_shared:
        bt = bt[:1].expand(B, -1)
        if bt_shared != "stride0":
            bt = bt.contiguous()
    btd = bt.to(DEV) if bt_shared != "stride0" else bt[:1].to(DEV).expand(B, -1)
    q = torch.randn(B, Hq, 128, generator=g).bfloat16()
    scale = 1 / math.sqrt(128)
    tail = tail_len = tail_idx = None
    if win is not None:
        W, R = win
        tail = torch.randn(R, W, 2 * Hkv, 128, generator=g).bfloat16()
        tail_idx = torch.randperm(R, generator=g)[:B].int()
        tail_len = torch.randint(0, W + 1, (B,), generator=g).int()
    torch.cuda.synchronize()
    pool_np = pool.cpu().numpy()
    km = None if key_only else mask[:Hkv].numpy()
    vm = None if key_only else mask[Hkv:].numpy()
    kw = dict(tail=None if tail is None else bits(tail), tail_len=None if tail is None else tail_len.numpy(),
              tail_idx=None if tail is None else tail_idx.numpy(), kv_start=kv_start)
    with np.errstate(invalid="ignore", over="ignore"):
        ref = O.decode_reference(bits(q), pool_np, bt.numpy(), lens, scale, nb, P, key_only, km, vm, sym=fmt in SYM, **kw)
        ref_bf = O.decode_reference(bits(q), pool_np, bt.numpy(), lens, scale, nb, P, key_only, km, vm, bf16_operands=True,
                                    sym=fmt in SYM, **kw)
    Lmax = max(max(lens), 1)
    ns, ch = (K.plan_cb(B, Lmax, Hkv, P, fmt, nsplit, G=G, tail=tail is not None) if key_only
              else K.plan_v2(B, Lmax, Hkv, P, nsplit, fmt=fmt, G=G, tail=tail is not None))
    NT = -(-G // 4)
    ws = K.Workspace(B, Hkv * NT, B * Hkv * NT * (ns + 1), DEV, 4, 128)
    qd = q.to(DEV)
    seq = torch.tensor(lens, dtype=torch.int32, device=DEV)
    tkw = {}
    if tail is not None:
        td = tail.to(DEV)
        tkw = dict(tail=td, tail_len=tail_len.to(DEV), tail_idx=tail_idx.to(DEV), tail_bs=td.stride(0), tail_ts=td.stride(1))
    if partial:
        part = torch.full((B, Hq, 130), float("nan"), dtype=torch.float32, device=DEV)
        K.attn_partial(qd, pool, btd, seq, part, ns, ch, ws, scale * LOG2E, fmt, None if key_only else mask[:Hkv].to(DEV),
                       None if key_only else mask[Hkv:].to(DEV), kv_start=kv_start, page=P, **tkw)
        got = part[..., :128].double().cpu().numpy()
    else:
        out = torch.full((B, Hq * 128), float("nan"), dtype=torch.bfloat16, device=DEV)
        if key_only and G == 4:
            K.cb_attn(qd, pool, btd, seq, out, ns, ch, ws, scale * LOG2E, fmt, kv_start=kv_start, page=P, **tkw)
        else:
            K.v2_attn(qd, pool, btd, seq, out, ns, ch, ws, scale * LOG2E, kmask=None if key_only else mask[:Hkv].to(DEV),
                      vmask=None if key_only else mask[Hkv:].to(DEV), fmt=fmt, kv_start=kv_start, page=P, **tkw)
        got = out.view(B, Hq, 128).double().cpu().numpy()
    torch.cuda.synchronize()
    assert K.device_status() == 0
    assert int(ws.counter.abs().sum()) == 0, "merge tickets must be left at zero"
    valid = np.array([lens[b] > min(kv_start, lens[b]) or (tail is not None and int(tail_len[b]) > 0) for b in range(B)])
    if not valid.any():
        return 0.0, 0.0, 0.0, 0.0
    err = np.abs(got[valid] - ref[valid])
    assert not np.isnan(got[valid]).any()
    mx = np.abs(ref[valid]).max()
    rel_rms = float(np.sqrt((err ** 2).mean()) / max(np.sqrt((ref[valid] ** 2).mean()), 1e-30))
    # error of the same attention with bf16-rounded operands (the reference's yardstick)
    sd = float(np.abs(ref_bf[valid] - ref[valid]).max())
    WORST[fmt] = max(WORST.get(fmt, 0.0), float(err.max()))
    return float(err.max()), rel_rms, float(err.max() / mx), sd / mx


WORST: dict = {}     # largest max-abs error seen per format in this session (printed by the last test of the file)


def check(res, what):
    """the baseline's bounds and the reference's own criterion (test_kernels.py:170-173):
    max|err| / max|ref| <= max(2 x the error of the same attention on bf16-rounded operands, 4e-3)"""
    e, rr, rel, sd_rel = res
    assert e <= 2e-2, (what, "max-abs", e)
    assert rr <= 1e-2, (what, "relative RMS", rr)
    assert rel <= max(2 * sd_rel, 4e-3), (what, "max|err| / max|ref|", rel, "limit", max(2 * sd_rel, 4e-3))


LENS = ([1], [77], [300, 4101, 17], [1000] * 5, [0, 513, 64])


@pytest.mark.parametrize("fmt", ["int4a", "int2a", "konlya", "konlya2", "int4", "konly"])
@pytest.mark.parametrize("win", [None, (32, 9), (256, 7)])
def test_decode_lengths_and_windows(K, fmt, win):
    for i, lens in enumerate(LENS):
        check(run_case(K, fmt, lens, win=win, seed=10 * i + (0 if win is None else win[0])), (fmt, lens, win))


@pytest.mark.parametrize("fmt", ["int4a", "int2a", "konlya", "konlya2"])
def test_decode_long_sequence(K, fmt):
    check(run_case(K, fmt, [33000], win=(256, 7), seed=3, Hkv=2), (fmt, 33000))
    check(run_case(K, fmt, [33000], seed=4, Hkv=2, nsplit=3), (fmt, 33000, "nsplit 3"))


@pytest.mark.parametrize("fmt", ["int4a", "konlya", "konlya2"])
@pytest.mark.parametrize("shared", ["copy", "stride0"])
def test_decode_shared_block_table_row(K, fmt, shared):
    check(run_case(K, fmt, list(range(1, 200, 7)), bt_shared=shared, win=(64, 40), seed=5), (fmt, shared))


@pytest.mark.parametrize("fmt", ["int4a", "int2a", "konlya", "konlya2", "int4", "konly"])
@pytest.mark.parametrize("ks", [4, 16, 37])
def test_decode_kv_start(K, fmt, ks):
    for i, lens in enumerate(([ks + 1], [77], [300, 4101, 17 + ks], [0, 513, 64 + ks])):
        for win in (None, (132, 9)):
            check(run_case(K, fmt, lens, win=win, kv_start=ks, seed=20 + i), (fmt, lens, win, ks))


@pytest.mark.parametrize("fmt", ["int4a", "konlya", "konlya2", "int4"])
@pytest.mark.parametrize("G,Hkv", [(5, 8), (8, 8), (12, 4), (6, 2)])
def test_decode_gqa_groups(K, fmt, G, Hkv):
    for i, lens in enumerate(([1], [300, 4101, 17], [0, 513, 64])):
        for win in (None, (64, 9)):
            check(run_case(K, fmt, lens, win=win, G=G, Hkv=Hkv, seed=30 + i), (fmt, G, Hkv, lens, win))


@pytest.mark.parametrize("fmt", ["int4a", "konlya"])
@pytest.mark.parametrize("nsplit", [1, 3])
def test_decode_forced_splits(K, fmt, nsplit):
    check(run_case(K, fmt, [300, 4101, 17], win=(32, 9), nsplit=nsplit, seed=40), (fmt, nsplit))


@pytest.mark.parametrize("fmt", ["int4a", "int2a", "konlya", "konlya2", "int4", "konly"])
def test_decode_32_token_pages(K, fmt):
    """pages of 32 tokens (one page per 32-token step of a warp; reference dispatch kernels/csrc/attn_decode_v2.cu:2018-2060)"""
    for i, (lens, win, ks) in enumerate((([1], None, 0), ([77, 300, 4101, 17], (32, 9), 0), ([0, 513, 64], (256, 7), 0),
                                          ([300, 4101, 54], (132, 9), 37))):
        check(run_case(K, fmt, lens, win=win, kv_start=ks, seed=60 + i, P=32), (fmt, lens, win, ks, "page 32"))
    check(run_case(K, fmt, [300, 4101, 17], win=(32, 9), nsplit=3, seed=64, P=32, G=8), (fmt, "page 32, G 8, 3 splits"))


def test_decode_partial_rows_merge(K):
    """the extension entry: rows of two KV-sequence shards merged on the host equal attention over the whole sequence."""
    check(run_case(K, "konlya", [300, 1000, 17], win=(32, 9), seed=50, partial=True), "partial")


def test_merge_partials_kernel(K):
    """fr_merge_partials against the torch merge: shards with no key (l = 0), -inf maxima, bf16 and fp32 outputs"""
    g = torch.Generator().manual_seed(5)
    R, B, Hq = 5, 3, 8
    parts = torch.randn(R, B, Hq, 130, generator=g)
    parts[..., 128] *= 6
    parts[..., 129] = torch.rand(R, B, Hq, generator=g) * 50
    parts[1, :, :, 129] = 0
    parts[1, :, :, 128] = float("-inf")
    parts[:, 2, 3, 129] = 0                      # a row nobody saw
    ref = K.merge_partials(parts)
    pd = parts.to(DEV).contiguous()
    o32 = K.merge_partials_into(pd, torch.empty(B, Hq, 128, dtype=torch.float32, device=DEV))
    o16 = K.merge_partials_into(pd, torch.empty(B, Hq * 128, dtype=torch.bfloat16, device=DEV))
    torch.cuda.synchronize()
    assert torch.allclose(o32.cpu(), ref, rtol=1e-5, atol=1e-5)
    assert torch.equal(o16.cpu().view(B, Hq, 128), o32.cpu().to(torch.bfloat16))
    assert float(o32[2, 3].abs().sum()) == 0.0


def test_decode_golden_baseline_config(K, golden_dir):
    """the reference-generated expectation of the small baseline configuration (batch 2, 8 q / 2 kv heads, context 512,
    4 sinks + 32 window): pools packed by the oracle in the CPU reference's arithmetic, outputs from the reference's
    parsers + float64 attention (tests/golden/decode.npz)."""
    g = np.load(golden_dir / "decode.npz")
    kv = g["kv"]
    B, L = kv.shape[:2]
    Hkv = kv.shape[2] // 2
    bt = g["bt"]
    npg = B * (L // P) + 7
    rows = kv.reshape(B * L, 2 * Hkv, 128)
    slots = (bt.astype(np.int64)[:, np.arange(L) // P] * P + np.arange(L) % P).reshape(-1)
    scale = float(g["scale"])
    q = torch.from_numpy(g["q"].view(np.int16)).view(torch.bfloat16).to(DEV)
    ring = torch.from_numpy(g["ring"].view(np.int16)).view(torch.bfloat16).to(DEV)
    lens = torch.from_numpy(g["lens"]).to(DEV)
    for fmt, (nb, key_only) in ((f, FMT[f]) for f in ("int4a", "int2a", "konlya", "konlya2")):      # the formats of the fixture
        pool = np.random.RandomState(7).randint(0, 256, (npg, Hkv, O.chunk_bytes(nb, P)), dtype=np.uint8)
        if key_only:
            codes, words, _ = O.dynamic_rows(rows, g["Cq"], nb, None, recip=False)
        else:
            codes, words = O.static_rows(rows, g["mask"], None, nb, None, recip=False)
        O.write_pool(pool, slots, codes, words, nb, P)
        pd = torch.from_numpy(pool).to(DEV)
        btd = torch.from_numpy(bt).to(DEV)
        ws = K.Workspace(B, Hkv, B * Hkv * 9, DEV)
        km = None if key_only else torch.from_numpy(g["mask"][:Hkv]).to(DEV)
        vm = None if key_only else torch.from_numpy(g["mask"][Hkv:]).to(DEV)
        for tag, tkw, ks in (("plain", {}, 0),
                             ("tail", dict(tail=ring, tail_len=torch.from_numpy(g["tail_len"]).to(DEV),
                                           tail_idx=torch.from_numpy(g["tail_idx"]).to(DEV), tail_bs=ring.stride(0),
                                           tail_ts=ring.stride(1)), int(g["kv_start"]))):
            for ns in (1, 2):
                out = torch.zeros(B, 8 * 128, dtype=torch.bfloat16, device=DEV)
                K.v2_attn(q, pd, btd, lens, out, ns, 512 // ns, ws, scale * LOG2E, kmask=km, vmask=vm, fmt=fmt, kv_start=ks,
                          **tkw)
                torch.cuda.synchronize()
                got = out.view(B, 8, 128).double().cpu().numpy()
                ref = g[f"{fmt}_{tag}"]
                err = np.abs(got - ref)
                assert err.max() <= 2e-2 and np.sqrt((err ** 2).mean() / (ref ** 2).mean()) <= 1e-2, (fmt, tag, ns, err.max())


def test_decode_error_codes(K):
    L = K.lib()
    z = torch.zeros(4096, dtype=torch.uint8, device=DEV)
    a = [z.data_ptr()] * 4
    common = lambda fmt, page, chunk, variant: L.fr_v2_attn(fmt, a[0], 512, a[1], a[2], 1, a[3], 1, 1, page, 1, chunk, 1.0,  # noqa: E731
                                                            None, None, 32, 0, 0, variant, 3, a[0], a[0], a[0], a[0], 512,
                                                            None, None, None, 0, 0, None, 4, 0)
    assert common(3, 16, 64, 264) == -4          # not a page format of this library
    assert common(5, 8, 64, 264) == -5           # pages of 16 or 32 tokens
    assert common(5, 16, 100, 264) == -3         # chunk must be a multiple of 64
    assert common(5, 16, 64, 264 | 4096) == -8   # head dim 256
    assert L.fr_cb_attn(a[0], 512, a[1], a[2], 1, a[3], 1, 1, 16, 1, 64, 1.0, K.sign_words(), 3, 0, 3, a[0], a[0], a[0], a[0],
                        512, None, None, None, 0, 0, None, 0) == -4
