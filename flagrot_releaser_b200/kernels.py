"""Host side of libflagrot_kernels.so for B200: ctypes loader, split planner, workspace and the launch wrappers.

Mirrors the interface of the reference's integrations/vllm_flagrot/vllm_flagrot/kernels.py (same function names,
argument meaning and error behaviour) so that code written against the reference front end runs unchanged:

  v2_write / w3_static_write / head_fwht      static writers            (reference kernels.py:330-345, 502-517, 538-552)
  cb_write / cb_write3                        dynamic key-only writer   (reference kernels.py:382-394, 472-499)
  v2_attn / cb_attn                           paged decode attention    (reference kernels.py:357-379, 519-535)
  plan_v2 / plan_cb / Workspace               split planner, workspace  (reference kernels.py:247-327)

The library is built in-tree by flagrot_releaser_b200/_build.py (nvcc, sm_100a) and must exist: there is no fallback
path.  FLAGROT_LIB overrides its location, as in the reference.  All launches go to torch's current CUDA stream and are
asynchronous; torch is used for device memory and streams only.
"""
from __future__ import annotations

import ctypes
import math
import os
from pathlib import Path

import torch

_PKG = Path(__file__).resolve().parent
ABI = 9
D, RB, NG = 128, 32, 4
V2_FMT = {"int4": 4, "int4a": 5, "konly": 6, "konlya": 7, "int2a": 8, "konlya2": 9}
CB_KINDS = {"konly": 6, "konlya": 10, "konlya2": 11}
INT2_FMTS = ("int2a", "konlya2")
K2 = ("konly", "konlya", "konlya2")
GEN, GT8, HD256 = 1024, 2048, 4096
STAGES = 3
MAX_CHUNK, MAX_SPLITS = 8192, 512
# split planner constants for B200 (tokens-equivalent fixed cost per CTA, per merged part)
PLAN_C0, PLAN_C1 = 640, 6
PLAN_CW = 900              # a BF16 window CTA in token equivalents


def _lib_path() -> Path:
    return Path(os.environ.get("FLAGROT_LIB", _PKG / "lib" / "libflagrot_kernels.so"))


_LIB = None


def lib():
    """the loaded library (ctypes).  Raises if it is missing or reports another ABI version."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = _lib_path()
    if not path.exists():
        raise RuntimeError(f"{path} not found: build it with `python -m flagrot_releaser_b200._build` (needs nvcc); "
                           "there is no fallback implementation")
    L = ctypes.CDLL(str(path))
    P, I, LL, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    L.fr_abi_version.restype = I
    if L.fr_abi_version() != ABI:
        raise RuntimeError(f"libflagrot_kernels ABI {L.fr_abi_version()} != {ABI}: rebuild ({path})")
    L.fr_v2_attn.argtypes = [I, P, LL, P, P, I, P, I, I, I, I, I, F, P, P, I, I, I, I, I, P, P, P, P, LL, P, P, P,
                             LL, LL, P, I, I]
    L.fr_v2_write.argtypes = [I, P, LL, P, I, I, I, P, I, P, P, I, P]
    L.fr_v2_occupancy.argtypes = [I, I, I, I]
    L.fr_v2_chunk_bytes.argtypes = [I, I]
    L.fr_cb_write.argtypes = [P, LL, P, I, I, I, I, I, P, P, P, I, P, P, I, P]
    L.fr_cb_attn.argtypes = [P, LL, P, P, I, P, I, I, I, I, I, F, P, I, I, I, P, P, P, P, LL, P, P, P, LL, LL, P, I]
    L.fr_cb_occupancy.argtypes = [I, I, I, I]
    L.fr_cb_chunk_bytes.argtypes = [I, I]
    L.fr_cb_write_smem.argtypes = [I, I, I]
    L.fr_last_error.restype = ctypes.c_char_p
    L.fr_head_fwht.argtypes = [P, LL, P, LL, I, I, P, F, P, I]
    L.fr_cb_write3.argtypes = [P, LL, P, I, I, I, I, P, P, P, P, P, I, P, I, I, P, P]
    L.fr_w3_static_write.argtypes = [P, LL, P, I, I, I, P, P, I, P, I, P, P]
    L.fr_cb_attn_noalloc.argtypes = [P, LL, P, P, I, P, I, I, I, I, I, F, I, P, LL, P, P, P, LL, LL, P, I]
    L.fr_attn_partial.argtypes = [I, P, LL, P, P, I, P, I, I, I, I, I, F, P, P, P, P, P, P, P, P, P, LL, LL, P, I, I]
    L.fr_merge_partials.argtypes = [P, I, I, P, I, P]
    L.fr_dequant_pages.argtypes = [I, P, P, I, I, I, I, P, P, P, P, P, P, I, P]
    L.fr_xchg_bytes.argtypes, L.fr_xchg_bytes.restype = [I], LL
    L.fr_xchg_alloc.argtypes = [I, ctypes.POINTER(P), ctypes.c_char_p]
    L.fr_xchg_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(P)]
    L.fr_xchg_close.argtypes = [P]
    L.fr_xchg_free.argtypes = [P]
    L.fr_xchg_merge.argtypes = [P, ctypes.POINTER(P), I, I, I, P, I, P]
    L.fr_xchg_selftest.argtypes = [ctypes.POINTER(P), ctypes.POINTER(P), I, I, ctypes.POINTER(P), I, P]
    L.fr_dyn_writer_stats.argtypes, L.fr_dyn_writer_stats.restype = [ctypes.POINTER(ctypes.c_ulonglong), I], I
    L.fr_dyn_writer_exact_only.argtypes, L.fr_dyn_writer_exact_only.restype = [I], None
    for n in ("fr_v2_attn", "fr_v2_write", "fr_v2_occupancy", "fr_v2_chunk_bytes", "fr_cb_write", "fr_cb_attn",
              "fr_cb_occupancy", "fr_cb_chunk_bytes", "fr_cb_nsg", "fr_head_fwht", "fr_cb_write3",
              "fr_w3_static_write", "fr_cb_write_smem", "fr_attn_partial", "fr_device_status", "fr_cb_attn_noalloc", "fr_merge_partials",
              "fr_xchg_alloc", "fr_xchg_open", "fr_xchg_close", "fr_xchg_free", "fr_xchg_merge", "fr_xchg_selftest",
              "fr_dequant_pages"):
        getattr(L, n).restype = I
    _LIB = L
    return L


def dyn_writer_stats(reset=False):
    """(pairs written, pairs whose head choice took the exact sums) of the bulk dynamic key writer since the last reset."""
    out = (ctypes.c_ulonglong * 2)()
    if lib().fr_dyn_writer_stats(out, int(reset)) != 0:
        raise RuntimeError("fr_dyn_writer_stats failed")
    return int(out[0]), int(out[1])


def _check(rc: int, what: str):
    if rc != 0:
        raise RuntimeError(f"{what}: launch failed (code {rc}, {lib().fr_last_error().decode()})")


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


_SG = None


def sign_words():
    """ctypes uint32[60]: the 15 sign vectors of the reference's codebooks (reference kernels.py:211-221).  The
    key-only kinds never read them; the argument exists for ABI compatibility."""
    global _SG
    if _SG is None:
        w = []
        for k in (0,) + tuple(range(2, 16)):
            g = torch.Generator().manual_seed(1234 + D + 7919 * k)
            b = (torch.randint(0, 2, (D,), generator=g) * 2 - 1 < 0).to(torch.int64)
            w += [int(sum(int(b[32 * j + i]) << i for i in range(32))) for j in range(4)]
        _SG = (ctypes.c_uint * len(w))(*w)
    return _SG


def v2_chunk_bytes(page: int, Dh: int = 128, fmt: str = "int4") -> int:
    return page * (80 if fmt in INT2_FMTS else 144) * Dh // 128


def cb_chunk_bytes(kind: str, page: int, Dh: int = 128) -> int:
    return page * (80 if kind in INT2_FMTS else 144) * Dh // 128


# ------------------------------------------------------------------ planner (host only)
def qtile(G: int, Dh: int = 128) -> int:
    """q heads per workspace slot as the reference sizes it (reference kernels.py:51-54)."""
    return 8 if Dh == 128 and 5 <= G <= 8 else 4


def v2_variant(fmt: str, G: int = 4, Dh: int = 128) -> int:
    if G == 4 and Dh == 128 and fmt in ("int4", "int4a", "int2a"):
        return 264
    return 264 | GEN | (GT8 if qtile(G, Dh) == 8 else 0) | (HD256 if Dh == 256 else 0)


def tile_of(variant: int) -> int:
    return 8 if (variant & GEN) and (variant & GT8) else 4


def vheads(Hkv: int, G: int, Dh: int = 128, fmt: str = "int4") -> int:
    return Hkv * -(-G // tile_of(v2_variant(fmt, G, Dh)))


_OCC: dict = {}
_NUM_SMS = None


def _slots_per_gpu(key, occ_fn) -> int:
    global _NUM_SMS
    if _NUM_SMS is None:
        _NUM_SMS = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    if key not in _OCC:
        _OCC[key] = max(1, occ_fn())
    return _OCC[key] * _NUM_SMS


def _dispatch_finish(classes, slots: int) -> int:
    """finish time of `slots` CTA slots that take CTAs in the given order, a freed slot always taking the next CTA:
    classes = [(count, cost), ...].  Slots with equal load are kept as groups, so the cost is per class, not per CTA."""
    groups = [[0, slots]]                                    # [load, number of slots], ascending load
    for n, c in classes:
        while n > 0:
            l0, k0 = groups[0]
            if len(groups) > 1:
                t = max(1, -(-(groups[1][0] - l0) // c))     # CTAs each slot of the lowest group takes before the next group is lower
            else:
                t = max(1, -(-n // k0))
            if n >= k0 * t:
                groups[0][0] = l0 + t * c
                n -= k0 * t
            else:
                q, rem = divmod(n, k0)
                groups[0] = [l0 + q * c, k0 - rem]
                if rem:
                    groups.append([l0 + (q + 1) * c, rem])
                n = 0
            groups.sort()
            merged = []
            for g in groups:                                 # equal loads become one group again
                if g[1] <= 0:
                    continue
                if merged and merged[-1][0] == g[0]:
                    merged[-1][1] += g[1]
                else:
                    merged.append(g)
            groups = merged
    return max(g[0] for g in groups)


def packed_cost(B: int, ctas_per_row: int, nse: int, chunk: int, slots: int, tail: bool = False, Lmax: int | None = None):
    """(finish time in token equivalents, rows_wide) of a launch with nse pieces of `chunk` tokens per row (rows of Lmax
    tokens: the last piece is shorter) when the library may cut the first rows_wide rows into nse - 1 wider pieces (what
    decode_launch does; csrc/fr_decode.cu pack_rows): wide CTAs first, then the narrow ones, the BF16 window CTAs last."""
    Lmax = nse * chunk if Lmax is None else Lmax

    def pieces(rows, n, size):
        last = Lmax - (n - 1) * size
        cl = [(rows * ctas_per_row * (n - 1), size + PLAN_C0)] if n > 1 else []
        return cl + [(rows * ctas_per_row, max(last, 1) + PLAN_C0)]

    def finish(r, cw):
        cl = (pieces(r, nse - 1, cw) if r else []) + (pieces(B - r, nse, chunk) if B - r else [])
        if tail:
            cl.append((B * ctas_per_row, PLAN_CW))
        return _dispatch_finish(cl, slots)
    best = (finish(0, 0), 0)
    if nse >= 2 and (nse * chunk) % (nse - 1) == 0:
        cw = nse * chunk // (nse - 1)
        if cw % 32 == 0 and cw <= MAX_CHUNK:
            step = max(1, B // 16)
            for r in sorted(set(list(range(step, B + 1, step)) + [B])):
                best = min(best, (finish(r, cw), r))
            for r in range(max(1, best[1] - step + 1), min(B, best[1] + step - 1) + 1):
                best = min(best, (finish(r, cw), r))
    return best


def plan_splits(B: int, Lmax: int, ctas_per_row: int, slots: int, nsplit=None, gran: int = 64, tail: bool = False):
    """(nsplit, chunk): chunk a multiple of 64 tokens, <= 8192, <= 512 splits.  Cost of a plan = the finish time of its CTAs
    dispatched over `slots` resident CTA slots (packed_cost: a CTA costs its tokens + C0, the library may widen the pieces
    of the first rows so that the last wave is full) plus C1 per merged part.  Pure host arithmetic (usable without a GPU)."""
    Lmax = max(1, int(Lmax))
    if nsplit is not None:
        chunk = min(MAX_CHUNK, math.ceil(Lmax / nsplit / gran) * gran)
        return math.ceil(Lmax / chunk), chunk
    best = None
    ns_hi = min(MAX_SPLITS, math.ceil(Lmax / gran))
    if B * ctas_per_row >= slots:                            # several CTAs per slot already: a handful of splits is all balance needs
        ns_hi = min(ns_hi, max(1, math.ceil(Lmax / MAX_CHUNK)) + 8)
    for ns in range(max(1, math.ceil(Lmax / MAX_CHUNK)), ns_hi + 1):
        for g in ((gran, gran * max(1, ns - 1)) if ns > 2 else (gran,)):         # also a chunk whose widened form is block-aligned
            chunk = math.ceil(Lmax / ns / g) * g
            if chunk > MAX_CHUNK:
                continue
            nse = math.ceil(Lmax / chunk)
            cost = packed_cost(B, ctas_per_row, nse, chunk, slots, tail, Lmax)[0] + (PLAN_C1 * nse if nse > 1 else 0)
            if best is None or cost < best[0] - 1e-9:
                best = (cost, nse, chunk)
    return best[1], best[2]


def plan_v2(B, Lmax, Hkv, page, nsplit=None, fmt="int4a", G=4, Dh=128, tail=False):
    """tail: the launch also carries one BF16 window CTA per (row, kv head, q tile) (they run last and fill the final wave)."""
    s = _slots_per_gpu(("v2", fmt), lambda: lib().fr_v2_occupancy(V2_FMT[fmt], v2_variant(fmt, G, Dh), STAGES, page))
    return plan_splits(B, Lmax, Hkv * -(-G // 4), s, nsplit, max(64, page), tail)


def plan_cb(B, Lmax, Hkv, page, kind, nsplit=None, G=4, Dh=128, tail=False):
    if G != 4 or Dh != 128:
        return plan_v2(B, Lmax, Hkv, page, nsplit, fmt=kind, G=G, Dh=Dh, tail=tail)
    s = _slots_per_gpu(("cb", kind), lambda: lib().fr_cb_occupancy(CB_KINDS[kind], 0, STAGES, page))
    return plan_splits(B, Lmax, Hkv, s, nsplit, max(64, page), tail)


class Workspace:
    """split partials for up to `parts` (row, kv head / q tile, split) slots of GT q heads x Dh dims, and the merge
    tickets (zeroed once, left zero by every call).  Allocate once before CUDA-graph capture
    (reference kernels.py:314-327)."""

    def __init__(self, rows: int, Hkv: int, parts: int, device, GT: int = 4, Dh: int = 128):
        self.rows, self.parts, self.HV, self.GT, self.Dh = rows, parts, Hkv, GT, Dh
        self.opart = torch.empty(parts * GT * Dh, device=device, dtype=torch.float32)
        self.mlpart = torch.empty(parts * GT * 2, device=device, dtype=torch.float32)
        self.counter = torch.zeros(rows * Hkv, device=device, dtype=torch.int32)

    def fits(self, B, Hkv, nsplit_total, GT=4, Dh=128):
        return (B <= self.rows and B * Hkv * nsplit_total <= self.parts and Hkv <= self.HV and GT * Dh <= self.GT * self.Dh
                and B * Hkv * nsplit_total * GT * Dh <= self.parts * self.GT * self.Dh)


# ------------------------------------------------------------------ launches
def _kmu(kmu, kv):
    if kmu is None:
        return None
    Hkv, Dh = kv.shape[1] // 2, kv.shape[2]
    assert kmu.dtype == torch.float32 and kmu.is_contiguous() and tuple(kmu.shape) == (Hkv, Dh) \
        and kmu.device == kv.device, (kmu.dtype, tuple(kmu.shape), (Hkv, Dh))
    return kmu.data_ptr()


def _rows_ok(kv):
    assert kv.dtype == torch.bfloat16 and kv.stride(2) == 1 and kv.stride(1) == kv.shape[2]
    assert kv.stride(0) % 4 == 0 and kv.data_ptr() % 8 == 0, "kv rows must be 8-byte aligned"


def v2_write(kv, slots, mask, rb, pool, page, fmt="int4a", kmu=None):
    """kv bf16 [T, 2*Hkv, Dh] (Dh 128 | 256) -> pool [num_pages, Hkv, chunk * Dh / 128] at slots int64 [T] (< 0 skipped);
    mask uint8 [2*Hkv, Dh / 32] (K rows first).  Dh 256: every head is stored as two 128-d half chunks."""
    T = kv.shape[0]
    if T == 0:
        return
    _rows_ok(kv)
    assert slots.dtype == torch.int64
    _check(lib().fr_v2_write(V2_FMT[fmt], kv.data_ptr(), kv.stride(0), slots.data_ptr(), T, kv.shape[1] // 2, page,
                             _ptr(mask), rb, pool.data_ptr(), _stream(), kv.shape[2], _kmu(kmu, kv)), "fr_v2_write")


def w3_static_write(kv, slots, mask, hfull, pool, page, fmt="int4a", path=0, kmu=None):
    """head_fwht(kv, hfull, 1/16) + v2_write fused (same pool bytes); kv in the ORIGINAL basis of the whole-head heads."""
    T = kv.shape[0]
    if T == 0:
        return
    _rows_ok(kv)
    assert slots.dtype == torch.int64
    slots = slots.contiguous()
    _check(lib().fr_w3_static_write(kv.data_ptr(), kv.stride(0), slots.data_ptr(), T, kv.shape[1] // 2, page,
                                    _ptr(mask), _ptr(hfull), {"int4": 0, "int4a": 1, "int2a": 2}[fmt], pool.data_ptr(),
                                    path, _stream(), _kmu(kmu, kv)), "fr_w3_static_write")


def cb_write(kv, slots, CT, co, kind, pool, page, tg=None, kmu=None):
    """kv bf16 [T, 2*Hkv, 128] -> pool at slots int64 [T]; CT [Hkv, 128, 128] = C_q^T, co [Hkv, 128] fp32."""
    T = kv.shape[0]
    if T == 0:
        return
    _rows_ok(kv)
    assert slots.dtype == torch.int64 and CT.dtype == torch.float32 and CT.is_contiguous()
    _check(lib().fr_cb_write(kv.data_ptr(), kv.stride(0), slots.data_ptr(), 0, T, kv.shape[1] // 2, page, tg or 1,
                             CT.data_ptr(), co.data_ptr(), sign_words(), CB_KINDS[kind], pool.data_ptr(), _stream(),
                             kv.shape[2], _kmu(kmu, kv)), "fr_cb_write")


_SIDE: dict = {}


def side_stream(device=None):
    """second stream of the split writer (one per device; create before CUDA-graph capture)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if dev not in _SIDE:
        _SIDE[dev] = torch.cuda.Stream(dev)
    return _SIDE[dev]


def cb_write3(kv, slots, CT, co, C1, beta, kind, pool, page, split=None, kmu=None):
    """same pool bytes as cb_write.  split (default T <= 256): key half on the current stream, value half on the side
    stream, joined by stream waits (CUDA-graph capturable).  C1 / beta (the reference's ranking tables) may be None."""
    T = kv.shape[0]
    if T == 0:
        return
    _rows_ok(kv)
    assert slots.dtype == torch.int64
    slots = slots.contiguous()
    Hkv = kv.shape[1] // 2
    L = lib()
    km = _kmu(kmu, kv)
    args = (kv.data_ptr(), kv.stride(0), slots.data_ptr(), 0, T, Hkv, page, CT.data_ptr(), co.data_ptr(), _ptr(C1),
            _ptr(beta), sign_words(), CB_KINDS[kind], pool.data_ptr())
    if split is None:
        split = T <= 256
    if not split:
        _check(L.fr_cb_write3(*args, 1, 1, _stream(), km), "fr_cb_write3")
        return
    cur = torch.cuda.current_stream()
    side = side_stream(kv.device)
    side.wait_stream(cur)
    _check(L.fr_cb_write3(*args, 1, -1, cur.cuda_stream, km), "fr_cb_write3 (keys)")
    _check(L.fr_cb_write3(*args, -1, 1, side.cuda_stream, None), "fr_cb_write3 (values)")
    cur.wait_stream(side)


def head_fwht(x, flags, scale, out=None):
    """x bf16 [T, H, D] (D = 128 or 256) -> out: scale * H_D x for the heads with flags[h] != 0, a copy otherwise; out may
    alias x."""
    T, H, Dh = x.shape
    assert x.dtype == torch.bfloat16 and x.stride(2) == 1 and x.stride(1) == Dh
    if out is None:
        out = torch.empty(T, H, Dh, dtype=x.dtype, device=x.device)
    assert out.stride(2) == 1 and out.stride(1) == Dh
    if T:
        _check(lib().fr_head_fwht(x.data_ptr(), x.stride(0), out.data_ptr(), out.stride(0), T, H, flags.data_ptr(),
                                  scale, _stream(), Dh), "fr_head_fwht")
    return out


def _bt_args(block_table):
    return block_table.data_ptr(), block_table.stride(0)


def _ws_ok(ws, B, Hkv, G, nparts):
    need = B * Hkv * -(-G // 4) * nparts * (4 * D)
    assert ws.opart.numel() >= need and ws.mlpart.numel() * 64 >= need and ws.counter.numel() >= B * Hkv, \
        "split-K workspace too small"


def v2_attn(q, pool, block_table, seq_lens, out, nsplit, chunk, ws, qscale, kmask=None, vmask=None, rb=32,
            tail=None, tail_len=None, tail_idx=None, tail_bs=None, tail_ts=None, page=16, fmt="int4a", kv_start=0):
    """q bf16 [B, G*Hkv, 128] -> out bf16 [B, G*Hkv*128]; qscale = softmax scale * log2(e); tail: BF16 rows (strides
    tail_bs / tail_ts elements) with tail_len int32 [B] (+ tail_idx int32 [B]); kv_start: leading tokens masked in the
    pages."""
    B, Hq, Dh = q.shape
    Hkv = pool.shape[1]
    G = Hq // Hkv
    assert Hq == G * Hkv and q.stride(2) == 1 and q.stride(1) == Dh and out.stride(1) == 1
    _ws_ok(ws, B, Hkv, G, nsplit + (tail is not None))
    bt, bts = _bt_args(block_table)
    _check(lib().fr_v2_attn(V2_FMT[fmt], q.data_ptr(), q.stride(0), pool.data_ptr(), bt, bts, seq_lens.data_ptr(), B,
                            Hkv, page, nsplit, chunk, qscale, _ptr(kmask), _ptr(vmask), rb, int(kmask is not None),
                            int(vmask is not None), v2_variant(fmt, G, Dh), STAGES, ws.opart.data_ptr(),
                            ws.mlpart.data_ptr(), ws.counter.data_ptr(), out.data_ptr(), out.stride(0), _ptr(tail),
                            _ptr(tail_len), _ptr(tail_idx), 0 if tail is None else tail_bs,
                            0 if tail is None else tail_ts, _stream(), G, int(kv_start)), "fr_v2_attn")


def cb_attn(q, pool, block_table, seq_lens, out, nsplit, chunk, ws, qscale, kind, tail=None, tail_len=None,
            tail_idx=None, tail_bs=None, tail_ts=None, page=16, kv_start=0):
    B, Hq, Dh = q.shape
    if Hq != 4 * pool.shape[1] or Dh != 128:
        return v2_attn(q, pool, block_table, seq_lens, out, nsplit, chunk, ws, qscale, tail=tail, tail_len=tail_len,
                       tail_idx=tail_idx, tail_bs=tail_bs, tail_ts=tail_ts, page=page, fmt=kind, kv_start=kv_start)
    Hkv = Hq // 4
    assert q.stride(2) == 1 and q.stride(1) == D and out.stride(1) == 1
    _ws_ok(ws, B, Hkv, 4, nsplit + (tail is not None))
    bt, bts = _bt_args(block_table)
    _check(lib().fr_cb_attn(q.data_ptr(), q.stride(0), pool.data_ptr(), bt, bts, seq_lens.data_ptr(), B, Hkv, page,
                            nsplit, chunk, qscale, sign_words(), CB_KINDS[kind], 0, STAGES, ws.opart.data_ptr(),
                            ws.mlpart.data_ptr(), ws.counter.data_ptr(), out.data_ptr(), out.stride(0), _ptr(tail),
                            _ptr(tail_len), _ptr(tail_idx), 0 if tail is None else tail_bs,
                            0 if tail is None else tail_ts, _stream(), int(kv_start)), "fr_cb_attn")


def cb_attn_noalloc(q, pool, block_table, seq_lens, out, nsplit, chunk, qscale, kind, tail=None, tail_len=None,
                    tail_idx=None, tail_bs=None, tail_ts=None, page=16, kv_start=0):
    """cb_attn for a caller that cannot allocate a Workspace: the partials live in a 16 MiB array inside the library.
    Returns the entry point's code (0 ok, -9: the request does not fit the built-in array) instead of raising on -9.
    Calls that overlap on the GPU share the array and must be serialised; make the first call on a device outside any
    stream capture."""
    B, Hq, Dh = q.shape
    Hkv = Hq // 4
    assert Hq == 4 * pool.shape[1] and Dh == D and q.stride(2) == 1 and q.stride(1) == D and out.stride(1) == 1
    bt, bts = _bt_args(block_table)
    rc = lib().fr_cb_attn_noalloc(q.data_ptr(), q.stride(0), pool.data_ptr(), bt, bts, seq_lens.data_ptr(), B, Hkv, page,
                                  nsplit, chunk, qscale, CB_KINDS[kind], out.data_ptr(), out.stride(0), _ptr(tail),
                                  _ptr(tail_len), _ptr(tail_idx), 0 if tail is None else tail_bs,
                                  0 if tail is None else tail_ts, _stream(), int(kv_start))
    if rc not in (0, -9):
        _check(rc, "fr_cb_attn_noalloc")
    return rc


def attn_partial(q, pool, block_table, seq_lens, part, nsplit, chunk, ws, qscale, fmt, kmask=None, vmask=None, tail=None,
                 tail_len=None, tail_idx=None, tail_bs=None, tail_ts=None, page=16, kv_start=0):
    """v2_attn that writes fp32 rows + (m, l) into part [B, Hq, 130] for a merge across KV-sequence shards."""
    B, Hq, Dh = q.shape
    Hkv = pool.shape[1]
    G = Hq // Hkv
    assert part.dtype == torch.float32 and part.is_contiguous() and tuple(part.shape) == (B, Hq, 130)
    _ws_ok(ws, B, Hkv, G, nsplit + (tail is not None))
    bt, bts = _bt_args(block_table)
    _check(lib().fr_attn_partial(V2_FMT[fmt], q.data_ptr(), q.stride(0), pool.data_ptr(), bt, bts, seq_lens.data_ptr(), B,
                                 Hkv, page, nsplit, chunk, qscale, _ptr(kmask), _ptr(vmask), ws.opart.data_ptr(),
                                 ws.mlpart.data_ptr(), ws.counter.data_ptr(), part.data_ptr(), _ptr(tail), _ptr(tail_len),
                                 _ptr(tail_idx), 0 if tail is None else tail_bs, 0 if tail is None else tail_ts,
                                 _stream(), G, int(kv_start)), "fr_attn_partial")


def merge_partials(parts: torch.Tensor) -> torch.Tensor:
    """parts fp32 [R, B, Hq, 130] (one per KV-sequence shard) -> merged rows fp32 [B, Hq, 128]
    (o = sum_r w_r l_r o_r / sum_r w_r l_r, w_r = 2^(m_r - max m); shards with no key have l = 0)."""
    o, m, l = parts[..., :128], parts[..., 128], parts[..., 129]
    M = m.amax(0, keepdim=True)
    w = torch.where(l > 0, torch.exp2(m - torch.where(torch.isinf(M), torch.zeros_like(M), M)), torch.zeros_like(l)) * l
    den = w.sum(0)
    return (w[..., None] * o).sum(0) / torch.where(den > 0, den, torch.ones_like(den))[..., None]


def merge_partials_into(parts: torch.Tensor, out: torch.Tensor):
    """merge_partials as one kernel launch (fr_merge_partials): parts fp32 [R, B, Hq, 130] contiguous on the device ->
    out [B, Hq * 128] (or [B, Hq, 128]) bf16 or fp32, contiguous."""
    R, B, Hq, _ = parts.shape
    assert parts.dtype == torch.float32 and parts.is_contiguous() and out.is_contiguous() and out.numel() == B * Hq * 128
    assert out.dtype in (torch.bfloat16, torch.float32)
    _check(lib().fr_merge_partials(parts.data_ptr(), R, B * Hq, out.data_ptr(), int(out.dtype == torch.float32), _stream()),
           "fr_merge_partials")
    return out


class ShardExchange:
    """Exchange + merge of KV-sequence shard partials over peer memory (fr_xchg_merge): every rank of the node owns one
    exchange buffer, maps the others' through CUDA IPC, and one kernel per rank pushes its partial rows [rows, 130] to every
    peer, waits (bounded) for theirs and merges.  Collective: all ranks call merge() the same number of times.  `dist` is
    torch.distributed (any backend: it only carries the 64-byte handles at set-up)."""

    def __init__(self, rank: int, world: int, rows: int, dist):
        assert 1 <= world <= 8 and 1 <= rows <= 1024
        self.rank, self.world, self.rows = rank, world, rows
        L = lib()
        own = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        _check(L.fr_xchg_alloc(rows, ctypes.byref(own), handle), "fr_xchg_alloc")
        self.own = own.value
        handles = [None] * world
        dist.all_gather_object(handles, handle.raw)
        self.ptrs = (ctypes.c_void_p * world)()
        self.opened = []
        for r in range(world):
            if r == rank:
                self.ptrs[r] = self.own
                continue
            p = ctypes.c_void_p()
            _check(L.fr_xchg_open(handles[r], ctypes.byref(p)), "fr_xchg_open")
            self.ptrs[r] = p.value
            self.opened.append(p.value)
        dist.barrier()

    def merge(self, part: torch.Tensor, out: torch.Tensor):
        """part fp32 [B, Hq, 130] of this rank -> out [B, Hq * 128] bf16 | fp32: the merge over all ranks' partials"""
        assert part.dtype == torch.float32 and part.is_contiguous() and part.numel() == self.rows * 130
        assert out.is_contiguous() and out.numel() == self.rows * 128 and out.dtype in (torch.bfloat16, torch.float32)
        _check(lib().fr_xchg_merge(part.data_ptr(), self.ptrs, self.rank, self.world, self.rows, out.data_ptr(),
                                   int(out.dtype == torch.float32), _stream()), "fr_xchg_merge")
        return out

    def close(self):
        L = lib()
        for p in self.opened:
            L.fr_xchg_close(p)
        self.opened = []
        if self.own:
            L.fr_xchg_free(self.own)
            self.own = None


def xchg_selftest(parts, outs):
    """R emulated ranks on ONE device as one cooperative launch: parts[r] fp32 [rows, 130] -> outs[r] [rows, 128]; every
    rank must end with the same merge.  Returns the exchange buffers (keep them to run further steps on the same buffers)."""
    L = lib()
    R, rows = len(parts), parts[0].shape[0]
    n = L.fr_xchg_bytes(rows)
    bufs = [torch.zeros(n, dtype=torch.uint8, device=parts[0].device) for _ in range(R)]
    return xchg_selftest_step(parts, outs, bufs), bufs


def xchg_selftest_step(parts, outs, bufs):
    L = lib()
    R, rows = len(parts), parts[0].shape[0]
    arr = lambda ts: (ctypes.c_void_p * R)(*[t.data_ptr() for t in ts])  # noqa: E731
    return L.fr_xchg_selftest(arr(parts), arr(bufs), R, rows, arr(outs), int(outs[0].dtype == torch.float32), _stream())


def dequant_pages(pool, bt_row, start, n, fmt, page=16, dtype=torch.bfloat16, kmask=None, vmask=None, kfull=None, vfull=None):
    """K, V [n - start, Hkv, 128] (bf16 | fp32) of positions [start, n) of the request with block-table row bt_row, in the
    original basis: the CUDA form of the "fa" prefill path's page dequantisation (reference backend.py:1744-1789).  Key-only
    kinds read the per-token flags from the pages; static formats take the layer's block masks [Hkv, 4] and whole-head flags
    [Hkv] (uint8)."""
    Hkv = pool.shape[1]
    assert bt_row.dtype == torch.int32 and bt_row.is_contiguous() and dtype in (torch.bfloat16, torch.float32)
    k = torch.empty(max(n - start, 0), Hkv, D, dtype=dtype, device=pool.device)
    v = torch.empty_like(k)
    if n > start:
        _check(lib().fr_dequant_pages(V2_FMT[fmt], pool.data_ptr(), bt_row.data_ptr(), int(start), int(n), Hkv, page, _ptr(kmask),
                                      _ptr(vmask), _ptr(kfull), _ptr(vfull), k.data_ptr(), v.data_ptr(),
                                      int(dtype == torch.float32), _stream()), "fr_dequant_pages")
    return k, v


def device_status() -> int:
    """0, or the source line of a bounded device-side wait that gave up (synchronises)."""
    return lib().fr_device_status()
