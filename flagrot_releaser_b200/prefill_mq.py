"""Host side of libflagrot_mq.so for B200: prefix-cached multi-query prefill attention over the FlagRot INT4 / INT2 pages.
Mirrors the reference's integrations/vllm_flagrot/vllm_flagrot/prefill_mq.py (same names, arguments and errors):

  build_plan / Plan     host work list: query tiles x ranges of 64-key blocks   (reference prefill_mq.py:128-210)
  prep_q                q -> FP16 in the keys' stored basis, pre-scaled          (reference prefill_mq.py:213-225)
  attn                  partial attention of every (item, kv head)              (reference prefill_mq.py:228-243)
  merge                 combine the items of each tile                          (reference prefill_mq.py:246-264)
  win_gather / bf_merge BF16 window and sink parts                              (reference prefill_mq.py:283-308)

The library must exist (built by flagrot_releaser_b200/_build.py); FLAGROT_MQ_LIB overrides its location.  There is no
fallback.  Head size 128 only (a 256-wide head is refused with code -4).
"""
from __future__ import annotations

import ctypes
import math
import os
from dataclasses import dataclass
from pathlib import Path

import numpy as np
import torch

_PKG = Path(__file__).resolve().parent
D, PAGE, BN = 128, 16, 64
TILE_INTS, ITEM_INTS = 9, 4
LOG2E = 1.4426950408889634
ABI = 7
KERNEL = int(os.environ.get("FLAGROT_MQ_KERNEL", "3"))
KROWS = {1: 64, 2: 128, 3: 128}       # query rows per tile
KCTAS = {1: 1, 2: 1, 3: 1}            # resident CTAs per SM: every plan kernel runs the one tcgen05 kernel (shared / tensor memory)
WAVES = float(os.environ.get("FLAGROT_MQ_WAVES", "2"))
MIN_BLOCKS = int(os.environ.get("FLAGROT_MQ_MIN_BLOCKS", "4"))
NO_EXT = -(1 << 30)
_LIB = None
_NSM: dict = {}


def _lib_path() -> Path:
    return Path(os.environ.get("FLAGROT_MQ_LIB", _PKG / "lib" / "libflagrot_mq.so"))


def lib():
    global _LIB
    if _LIB is not None:
        return _LIB
    path = _lib_path()
    if not path.exists():
        raise RuntimeError(f"{path} not found: build it with `python -m flagrot_releaser_b200._build`; there is no fallback")
    L = ctypes.CDLL(str(path))
    P, I, LL, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    L.frmq_abi_version.restype = I
    if L.frmq_abi_version() != ABI:
        raise RuntimeError(f"libflagrot_mq ABI {L.frmq_abi_version()} != {ABI}: rebuild ({path})")
    L.frmq_last_error.restype = ctypes.c_char_p
    L.frmq_smem_bytes.restype = I
    L.frmq_device_status.restype = I
    L.frmq_prep_q.argtypes = [P, I, LL, P, I, I, I, P, P, F, P, I, P]
    L.frmq_attn.argtypes = [P, P, LL, P, LL, P, P, I, I, I, I, I, P, P, I, I, P, I]
    L.frmq_merge.argtypes = [P, I, P, P, I, I, I, P, LL, I, P, LL, I, P]
    L.frmq_win_gather.argtypes = [P, I, P, P, P, LL, P, LL, I, P, P, I, P]
    L.frmq_bf_merge.argtypes = [I, I, I, P, LL, P, P, P, P, P, P, P, P, P, I, I, F, P, LL, I, P]
    for n in ("frmq_prep_q", "frmq_attn", "frmq_merge", "frmq_win_gather", "frmq_bf_merge"):
        getattr(L, n).restype = I
    _LIB = L
    return L


def available() -> bool:
    try:
        lib()
        return True
    except (OSError, RuntimeError):
        return False


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(rc, what):
    if rc != 0:
        raise RuntimeError(f"{what}: failed (code {rc}, {lib().frmq_last_error().decode()})")


def device_status() -> int:
    """0, or the source line of a bounded device-side wait that gave up (sticky; synchronises the device)."""
    return int(lib().frmq_device_status())


def num_sms(device) -> int:
    key = str(device)
    if key not in _NSM:
        dev = torch.device(device)
        _NSM[key] = torch.cuda.get_device_properties(dev).multi_processor_count if dev.type == "cuda" else 148
    return _NSM[key]


@dataclass
class Plan:
    """Work list of one step, shared by all layers.  tiles [nt, 9] = (block-table row, compact row, output row, tokens,
    position of the first token, page keys, first item, items, ext); items [ni, 4] = (tile, first key block, end key
    block, 0); idx [m] = output row of each compact row.  buf holds the three, back to back, as one int32 tensor."""
    ntiles: int
    nitems: int
    m: int
    buf: torch.Tensor
    reqs: list
    kernel: int = 3
    rows: int = 128
    D: int = 128
    kmin: int = 0

    @property
    def tiles(self):
        return self.buf[:self.ntiles * TILE_INTS]

    @property
    def items(self):
        a = self.ntiles * TILE_INTS
        return self.buf[a:a + self.nitems * ITEM_INTS]

    @property
    def idx(self):
        a = self.ntiles * TILE_INTS + self.nitems * ITEM_INTS
        return self.buf[a:a + self.m]


def _balanced_split(blocks, Hkv: int, nsm: int, ctas_per_sm: int, min_blocks: int, start: int) -> int:
    """key blocks per item that minimise the estimated makespan: CTAs are dealt to nsm * ctas_per_sm slots in waves, an
    item costs its blocks plus a fixed start-up of about three blocks (q staging, pipeline fill, partial store)."""
    slots = nsm * ctas_per_sm
    top = int(blocks.max()) if blocks.size else 1
    best, best_cost = start, None
    for parts in range(1, 33):
        per = max(min_blocks, -(-top // parts))
        n = int(np.maximum(1, -(-blocks // per)).sum()) * Hkv
        cost = -(-n // slots) * (min(per, top) + 3)
        if best_cost is None or cost < best_cost:
            best, best_cost = per, cost
        if per == min_blocks:
            break
    return best


def plan_arrays(reqs, G: int, Hkv: int, shift: int, nsm: int, kernel: int, waves: float, min_blocks: int, ext=None,
                balance: bool = False):
    """The plan as host arrays (tiles [nt, 9], items [ni, 4], idx [m]); pure numpy, no device.  balance=False is the
    reference's split rule; balance=True picks the split that fills whole waves of CTAs."""
    rows = KROWS[kernel]
    tq = rows // G
    tile_rows, last_key, idx = [], [], []
    m = 0
    for (r, q0, q1, L, s) in reqs:
        e = ext.get(r, NO_EXT) if ext else NO_EXT
        nk = max(L - shift, e + 1, 0)                       # page keys any row of the request can see
        for t0 in range(0, q1 - q0, tq):
            nt = min(tq, q1 - q0 - t0)
            tile_rows.append((r, m + t0, q0 + t0, nt, s + t0, nk, 0, 0, e))
            last_key.append(max(0, min(nk, max(s + t0 + nt - shift, e + 1))))   # causal limit of the tile's last token
        idx.append(np.arange(q0, q1, dtype=np.int32))
        m += q1 - q0
    tiles = np.asarray(tile_rows, dtype=np.int32).reshape(-1, TILE_INTS)
    blocks = -(-np.asarray(last_key, dtype=np.int64) // BN)
    target = max(int(waves * KCTAS[kernel] * nsm), 1)
    per_item = max(min_blocks, -(-int(blocks.sum()) * Hkv // target))           # key blocks per work item
    if balance:
        per_item = _balanced_split(blocks, Hkv, nsm, KCTAS[kernel], min_blocks, per_item)
    nitem = np.maximum(1, -(-blocks // per_item)).astype(np.int64)
    first = np.cumsum(nitem) - nitem
    tiles[:, 6] = first
    tiles[:, 7] = nitem
    owner = np.repeat(np.arange(tiles.shape[0]), nitem)
    k = np.arange(int(nitem.sum())) - first[owner]
    kb0 = k * per_item
    kb1 = np.minimum(blocks[owner], kb0 + per_item)
    items = np.stack([owner, kb0, kb1, np.zeros_like(owner)], 1).astype(np.int32).reshape(-1, ITEM_INTS)
    return tiles, items, (np.concatenate(idx) if idx else np.zeros(0, np.int32)), m


def build_plan(reqs, G: int, Hkv: int, shift: int, device, sink: int = 0, kernel: int | None = None,
               waves: float | None = None, min_blocks: int | None = None, D: int = D, ext: dict | None = None,
               balance: bool | None = None) -> Plan:
    """reqs: list of (block-table row r, q0, q1, L, s): batch rows q0 .. q1 - 1 are positions s .. L - 1 of request r.
    The query at position i sees the page keys sink <= j <= max(i - shift, ext[r]).  The split size is chosen so that
    the grid has about waves x resident CTAs x SMs CTAs, with at least min_blocks 64-key blocks per item; balance
    (default: on unless waves is given) instead picks the split whose CTAs fill whole waves of the GPU."""
    if D != 128:
        raise RuntimeError(f"build_plan: head size {D} is not built for B200 (128 only)")
    kernel = KERNEL if kernel is None else kernel
    balance = (waves is None) if balance is None else balance
    tiles, items, idx, m = plan_arrays(reqs, G, Hkv, shift, num_sms(device), kernel,
                                       WAVES if waves is None else waves, MIN_BLOCKS if min_blocks is None else min_blocks, ext,
                                       balance)
    host = np.concatenate([tiles.reshape(-1), items.reshape(-1), idx]).astype(np.int32)
    return Plan(ntiles=tiles.shape[0], nitems=items.shape[0], m=m, buf=torch.from_numpy(host).to(device), reqs=list(reqs),
                kernel=kernel, rows=KROWS[kernel], D=D, kmin=int(sink))


def prep_q(q: torch.Tensor, qscale: float, G: int, idx: torch.Tensor | None = None, kfull=None, kmask=None):
    """q [n, Hq, 128] bf16 / fp32 (head rows contiguous) -> FP16 [m, Hq, 128] (rows idx of q, or all): rotated into the
    keys' stored basis (kfull[kv head]: H128 / 8; kmask[kv head, group]: orthonormal H32) and multiplied by qscale."""
    n, Hq, Dh = q.shape
    assert q.dtype in (torch.bfloat16, torch.float32) and q.stride(2) == 1 and q.stride(1) == Dh
    assert idx is None or idx.dtype == torch.int32
    m = idx.numel() if idx is not None else n
    q16 = torch.empty(m, Hq, Dh, dtype=torch.float16, device=q.device)
    _check(lib().frmq_prep_q(_ptr(q), int(q.dtype == torch.float32), q.stride(0), _ptr(idx), m, Hq, G, _ptr(kfull), _ptr(kmask),
                             float(qscale), _ptr(q16), Dh, _stream()), "frmq_prep_q")
    return q16


def attn(q16, pool, bt, plan: Plan, G: int, shift: int, konly: bool, int2: bool = False):
    """Partial attention of every (item, kv head): (opart [ni, Hkv, rows, 128] fp32, ml [ni, Hkv, rows, 2] fp32)."""
    Hkv, Dh = pool.shape[1], q16.shape[2]
    assert Dh == plan.D, (Dh, plan.D)
    assert pool.dtype == torch.uint8 and pool.stride(1) == (80 if int2 else 144) * PAGE and pool.stride(2) == 1
    assert bt.dtype == torch.int32 and bt.stride(1) == 1
    assert q16.dtype == torch.float16 and q16.is_contiguous() and q16.shape[1] == Hkv * G
    opart = torch.empty(plan.nitems, Hkv, plan.rows, Dh, dtype=torch.float32, device=q16.device)
    ml = torch.empty(plan.nitems, Hkv, plan.rows, 2, dtype=torch.float32, device=q16.device)
    _check(lib().frmq_attn(_ptr(q16), _ptr(pool), pool.stride(0), _ptr(bt), bt.stride(0), _ptr(plan.tiles), _ptr(plan.items),
                           plan.nitems, Hkv, G, shift, int(konly) | (2 if int2 else 0), _ptr(opart), _ptr(ml), plan.kernel, Dh,
                           _stream(), plan.kmin), "frmq_attn")
    return opart, ml


def merge(plan: Plan, opart, ml, G: int, out=None, fp32: bool = False, want_lse: bool = False):
    """Combines the items of each tile.  fp32=False: bf16 into `out` ([n, Hq * 128] view of the layer output, rows = the
    plan's output rows); fp32=True: o [m, Hq, 128] fp32 in compact rows.  want_lse: natural-log LSE [Hq, m]
    (-inf: no visible key).  Returns (o or out, lse or None)."""
    Hkv, Dh = opart.shape[1], opart.shape[3]
    Hq = Hkv * G
    lse = torch.empty(Hq, plan.m, dtype=torch.float32, device=opart.device) if want_lse else None
    if fp32:
        o = torch.empty(plan.m, Hq, Dh, dtype=torch.float32, device=opart.device)
        ots = Hq * Dh
    else:
        assert out is not None and out.dtype == torch.bfloat16 and out.stride(-1) == 1
        o, ots = out, out.stride(0)
    _check(lib().frmq_merge(_ptr(plan.tiles), plan.ntiles, _ptr(opart), _ptr(ml), Hkv, G, plan.rows, _ptr(o), ots, int(fp32),
                            _ptr(lse), plan.m if lse is not None else 0, Dh, _stream()), "frmq_merge")
    return o, lse


def ref_partial_lse_merge(parts):
    """LSE merge of [(o [n, H, D], lse [H, n] natural log; -inf / +inf = empty)]; fp32 result (torch, any device)."""
    ls = []
    for _, lse in parts:
        v = lse.float().transpose(0, 1).unsqueeze(-1)
        ls.append(torch.where(torch.isposinf(v), torch.full_like(v, -math.inf), v))
    top = torch.stack(ls).amax(0)
    num = sum(o.float() * torch.exp(v - top) for (o, _), v in zip(parts, ls))
    den = sum(torch.exp(v - top) for v in ls)
    return num / den


def win_gather(map_, nk, sinkb, preb, kch, vch, Hkv, D):
    """K / V [nk, Hkv, D] bf16 of the window call: row d from map_[d] = (kind << 32) | row; kind 0 = sinkb, 1 = preb
    (both [*, 2 Hkv, D], contiguous), 2 = the batch rows kch / vch ([n, Hkv * D] views, any row stride)."""
    kw = torch.empty(nk, Hkv, D, dtype=torch.bfloat16, device=kch.device)
    vw = torch.empty_like(kw)
    for t in (sinkb, preb):
        assert t is None or (t.is_contiguous() and t.dtype == torch.bfloat16)
    assert kch.stride(-1) == 1 and vch.stride(-1) == 1 and kch.dtype == torch.bfloat16
    _check(lib().frmq_win_gather(_ptr(map_), nk, _ptr(sinkb), _ptr(preb), _ptr(kch), kch.stride(0), _ptr(vch), vch.stride(0),
                                 Hkv, _ptr(kw), _ptr(vw), D, _stream()), "frmq_win_gather")
    return kw, vw


def bf_merge(q, idx, o_p, lse_p, o_w, lse_w, sk, row_req, row_pos, sk_len, S, W, scale, out, Hkv):
    """out[idx[c]] = LSE merge of the page part (o_p fp32 [m, Hq, D], lse_p [Hq, m]), the window part (o_w bf16
    [m, Hq, D], lse_w [Hq, m]; None when W = 0) and the sink part (sk bf16 [nreq, S, 2 Hkv, D], keys j < min(S, len) with
    j <= pos - W; None when S = 0) of compact row c; q = the batch's q rows [n, Hq, D]."""
    m, Hq, Dh = o_p.shape
    assert o_p.is_contiguous() and lse_p.is_contiguous() and idx.dtype == torch.int64
    assert q.stride(-1) == 1 and q.stride(-2) == Dh and out.stride(-1) == 1
    _check(lib().frmq_bf_merge(m, Hq, Hkv, _ptr(q), q.stride(0), _ptr(idx), _ptr(o_p), _ptr(lse_p), _ptr(o_w), _ptr(lse_w),
                               _ptr(sk), _ptr(row_req), _ptr(row_pos), _ptr(sk_len), S, W, float(scale), _ptr(out),
                               out.stride(0), Dh, _stream()), "frmq_bf_merge")
