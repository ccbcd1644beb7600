// Prefix-cached multi-query prefill attention on the 5th-generation tensor cores: S = Q K^T and O += P V as tcgen05.mma
// with the accumulators, the Q operand and the P operand in tensor memory.  Included by mq_capi.cu inside its anonymous
// namespace (every plan kernel of frmq_attn runs it); work list, partial layout and numerics contract of the reference's kernels.
//
// CTA = (item, kv head): up to 128 query rows (the M tile; plans with 64-row tiles leave the upper half empty) x the item's
// 64-key blocks; 26 warps (72 registers each) with fixed roles:
//   warps 0-3, 20-23  softmax: two threads per query row r = tensor-memory lane r (warps w and 20 + w reach the same 32
//               lanes), each with 32 of the block's 64 score columns, read once and kept in registers: half-row maximum,
//               exchange with the partner through shared memory (a 64-thread named barrier), p = 2^(s - ref) into its half
//               of the P operand columns, and the row sum.  The reference is lazy: it only moves when the maximum grew by
//               more than 2^8 (p stays <= 256), so the O accumulator is rescaled a few times per item, not per block;
//   warps 4-19  conversion: raw page chunks -> FP16 operand tiles in shared memory (128-byte swizzle, K-major):
//               K [64 keys][128 dims] as (code - zero point) * scale, exact in FP16, one rounding (warps 4-11);
//               V^T [128 dims][64 keys] (warps 12-19); the two run side by side, each on its own hand-over barriers;
//   warp 24     issues the MMAs (lane 0; the whole warp waits) and owns the tensor-memory allocation;
//   warp 25     bulk-copies the four page chunks of a block into a 6-stage ring.
// Key-only pages (per-token rotation flags) are not rotated back per token: the kernel keeps Q in three bases (identity,
// per-group H32, whole-head H128) in tensor memory, the conversion drops each (key, group) into the operand tile of its
// base and zeros into the other two, and S accumulates the three products - three times the QK tensor work, which the
// tensor pipe has to spare, instead of a butterfly network per key on the CUDA cores.
// Pipelines: K / V tiles, S and P are double buffered; every hand-over is an mbarrier (bulk-copy bytes, thread arrivals
// or tcgen05.commit).  All waits are bounded; a wait that gives up sets a CTA-wide abort flag and the status word, after
// which every wait returns at once and the CTA runs to its end (results are garbage, the status says so).
#pragma once

constexpr int TQ_THREADS = 832;       // 26 warps
constexpr int TQ_SOFT = 128;          // query rows = softmax threads per column half
constexpr int TQ_CONV = 512;          // conversion threads (warps 4 .. 19)
constexpr int TQ_CONVH = 256;         // ... of which warps 4 .. 11 convert K tiles and warps 12 .. 19 V tiles
constexpr int TQ_WSOFTB = 20;         // warps 20 .. 23: the second softmax thread of every row (warps 0 .. 3: the first)
constexpr int TQ_WMMA = 24, TQ_WLOAD = 25;
constexpr int TQ_RAWST = 6;          // stages of the raw page ring: a block's chunks arrive about 1.5 us after they are asked for
__device__ int g_mq_status;

template <int NB, int NBASE> struct TQMap {
  static constexpr int CHUNK = MLay<NB>::CHUNK;
  static constexpr int KT = 0;                                   // [2 buffers][NBASE][2 dim halves][64 rows][128 B]
  static constexpr int KT_TILE = 16384;
  static constexpr int VT = KT + 2 * NBASE * KT_TILE;            // [2 buffers][128 rows][128 B]
  static constexpr int RAW = VT + 2 * 16384;                     // [TQ_RAWST][4 pages][CHUNK]
  static constexpr int RAW_STAGE = PPB * CHUNK;
  static constexpr int BAR = RAW + TQ_RAWST * RAW_STAGE;         // mbarriers
  static constexpr int NBAR = 2 * TQ_RAWST + 2 + 2 + 2 + 2 + 2 + 2 + 1 + 1 + 1;
  static constexpr int MISC = BAR + NBAR * 8;
  static constexpr int XCH = MISC + 16;                          // softmax pair exchange: float [2][2][128] maxima, [128] sums
  static constexpr int TOTAL = XCH + 5 * 128 * 4 + 1024;         // + slack for the 1024-byte alignment of the tiles
  static constexpr int QSTAGE_STRIDE = 272;                      // prologue: q rows staged over the K / V tiles
  static_assert(NBASE * 128 * QSTAGE_STRIDE <= RAW, "q staging fits in the tile region");
  static_assert(RAW % 16 == 0 && RAW_STAGE % 16 == 0 && BAR % 8 == 0, "alignment");
};
// tensor-memory columns
constexpr uint32_t TQ_O = 0, TQ_S = 128, TQ_P = 256, TQ_Q = 320;

FR_DEVI bool tq_wait_at(uint32_t bar, uint32_t parity, volatile uint32_t* abort, int line) {
  if (tc5::mbar_try(bar, parity)) return true;
  const bool was = *abort != 0;
  const bool ok = tc5::mbar_wait_abortable(bar, parity, abort);
  if (!ok && !was) atomicCAS(&g_mq_status, 0, line);     // the first wait that ran out names its line
  return ok;
}
#define tq_wait(bar, parity, abort) tq_wait_at(bar, parity, abort, __LINE__)
FR_DEVI bool tq_wait_relaxed_at(uint32_t bar, uint32_t parity, volatile uint32_t* abort, int line) {   // producers: sleeps between probes
  if (tc5::mbar_try(bar, parity)) return true;
  const bool was = *abort != 0;
  const bool ok = tc5::mbar_wait_relaxed(bar, parity, abort);
  if (!ok && !was) atomicCAS(&g_mq_status, 0, line);
  return ok;
}
#define tq_wait_relaxed(bar, parity, abort) tq_wait_relaxed_at(bar, parity, abort, __LINE__)

// K operand tiles of one 64-key block.  item = (key, tg pair, group j): the two code words (tg = 2 tgp, 2 tgp + 1) of group j
// carry dims 32 j + 8 tgp + {0..7} in the low fields and + 16 in the high fields of their bytes -> two 16-byte chunks.
// Key-only pages: the chunks go to the tile of the (key, group)'s base; the other two tiles must hold zeros there.  A
// thread meets the same slots of a buffer every second block, so it remembers the base it wrote last (prev, two bits per
// item and buffer) and only clears that tile when the base changed; the first use of a buffer clears both others.
template <int NB, bool KO>
FR_DEVI void tq_convert_k(uint32_t raw, uint32_t kt, int nvalid, int ctid, bool first, int buf, uint32_t& prev) {
  using L = MLay<NB>;
  constexpr uint32_t FM = NB == 4 ? 0x000F000Fu : 0x00030003u;
#pragma unroll
  for (int it = 0; it < (BN * 8) / TQ_CONVH; ++it) {
    const int item = ctid + TQ_CONVH * it, tok = item >> 3, tgp = (item >> 2) & 1, j = item & 3;
    const int pos = tok & 15;
    const uint32_t rc = raw + (tok >> 4) * L::CHUNK;
    const uint32_t dlo = (j >> 1) * 8192 + tc5::sw128_off(tok, 4 * (j & 1) + tgp);
    const uint32_t dhi = (j >> 1) * 8192 + tc5::sw128_off(tok, 4 * (j & 1) + tgp + 2);
    uint32_t o[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};     // lo: tg even dims 0 1 | 2 3 | tg odd 0 1 | 2 3; then hi alike
    int base = 0;
    if (tok < nvalid) {
      uint32_t w0, w1;
      if (NB == 4) {
        w0 = lds32(rc + 64 * pos + 32 * tgp + 4 * j);
        w1 = lds32(rc + 64 * pos + 32 * tgp + 16 + 4 * j);
      } else {
        const uint32_t a = rc + 32 * (pos ^ ((pos >> 1) & 2)) + 16 * tgp + 4 * (j >> 1);
        w0 = lds32(a) >> (4 * (j & 1));
        w1 = lds32(a + 8) >> (4 * (j & 1));
      }
      const uint32_t kw = lds16(rc + L::KS_OFF + 8 * pos + 2 * j);
      const uint32_t zz = ((kw & L::ZM) * 0x00010001u) | 0x64006400u;
      const uint32_t sc = (kw & 0x7FFFu) * 0x00010001u;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const uint32_t w = u ? w1 : w0;
        const uint32_t p01 = prmt(w, 0u, 0x4140u), p23 = prmt(w, 0u, 0x4342u);
        o[2 * u] = hmul2u(hsub2u((p01 & FM) | 0x64006400u, zz), sc);
        o[2 * u + 1] = hmul2u(hsub2u((p23 & FM) | 0x64006400u, zz), sc);
        o[4 + 2 * u] = hmul2u(hsub2u(((p01 >> NB) & FM) | 0x64006400u, zz), sc);
        o[5 + 2 * u] = hmul2u(hsub2u(((p23 >> NB) & FM) | 0x64006400u, zz), sc);
      }
      if constexpr (KO) {
        const bool ffl = (lds16(rc + L::VS_OFF + 2 * (8 * (pos >> 3) + fr::vslot8(pos))) & 0x8000u) != 0;
        base = ffl ? 2 : static_cast<int>(kw >> 15);
      }
    }
    if constexpr (KO) {
      const int sh = 2 * (2 * it + buf);
      const int old = static_cast<int>((prev >> sh) & 3u);
      prev = (prev & ~(3u << sh)) | (static_cast<uint32_t>(base) << sh);
      const uint32_t tb = kt + base * 16384;
      sts128(tb + dlo, o[0], o[1], o[2], o[3]);
      sts128(tb + dhi, o[4], o[5], o[6], o[7]);
      if (first) {
#pragma unroll
        for (int b = 1; b < 3; ++b) {
          const uint32_t tz = kt + ((base + b) % 3) * 16384;
          sts128(tz + dlo, 0u, 0u, 0u, 0u);
          sts128(tz + dhi, 0u, 0u, 0u, 0u);
        }
      } else if (old != base) {
        const uint32_t tz = kt + old * 16384;
        sts128(tz + dlo, 0u, 0u, 0u, 0u);
        sts128(tz + dhi, 0u, 0u, 0u, 0u);
      }
    } else {
      sts128(kt + dlo, o[0], o[1], o[2], o[3]);
      sts128(kt + dhi, o[4], o[5], o[6], o[7]);
    }
  }
}

// V^T operand tile [128 dims][64 keys]: item = (page, entry e, half m): the two code words (r8 = 0, 1) of dims
// 64 m + 16 w + gid + 8 r8 with the 8 tokens 8 c8 .. + 7 each -> two 16-byte chunks; they share the group's scale words.
template <int NB>
FR_DEVI void tq_convert_v(uint32_t raw, uint32_t vt, int nvalid, int ctid) {
  using L = MLay<NB>;
  constexpr uint32_t NM = NB == 4 ? 0x0F0F0F0Fu : 0x03030303u;
#pragma unroll
  for (int it = 0; it < (PPB * 64 * 2) / TQ_CONVH; ++it) {
    const int item = ctid + TQ_CONVH * it;
    const int pg = item >> 7, e = (item >> 1) & 63, m = item & 1;
    const int c8 = e & 1, gid = (e >> 1) & 7, w = e >> 4;
    const int d0 = 64 * m + 16 * w + gid, j = 2 * m + (w >> 1);
    const uint32_t rc = raw + pg * L::CHUNK;
    const int t0 = 16 * pg + 8 * c8;
    uint32_t o[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
    if (t0 < nvalid) {
      uint32_t wd[2];
      if (NB == 4) {
        const uint2 ww = lds64(rc + L::V_OFF + 16 * e + 8 * m);
        wd[0] = ww.x; wd[1] = ww.y;
      } else {
        const uint32_t ww = lds32(rc + L::V_OFF + 8 * e + 4 * m);
        wd[0] = ww; wd[1] = ww >> 4;
      }
      const uint4 sw = lds128(rc + L::VS_OFF + 2 * (j * PAGE + 8 * c8));     // scale words of tokens 0 2 4 6 | 1 3 5 7
      const uint32_t sp[4] = {prmt(sw.x, sw.z, 0x5410u), prmt(sw.x, sw.z, 0x7632u), prmt(sw.y, sw.w, 0x5410u), prmt(sw.y, sw.w, 0x7632u)};
      uint32_t zz[4], sc[4];
#pragma unroll
      for (int ii = 0; ii < 4; ++ii) {
        zz[ii] = (sp[ii] & (L::ZM | (L::ZM << 16))) | 0x64006400u;
        sc[ii] = sp[ii] & 0x7FFF7FFFu;
      }
#pragma unroll
      for (int r8 = 0; r8 < 2; ++r8) {
        const uint32_t ve = wd[r8] & NM, vo = (wd[r8] >> NB) & NM;     // even tokens | odd tokens, one byte each
#pragma unroll
        for (int ii = 0; ii < 4; ++ii) {
          const uint32_t u = (prmt(ve, vo, 0x0400u + 0x101u * ii) & 0x00FF00FFu) | 0x64006400u;
          o[4 * r8 + ii] = hmul2u(hsub2u(u, zz[ii]), sc[ii]);
        }
      }
      if (t0 + 8 > nvalid) {      // ragged end of the last block: tokens >= nvalid are zeros
#pragma unroll
        for (int q8 = 0; q8 < 8; ++q8) {
          const int ii = q8 & 3;
          if (t0 + 2 * ii >= nvalid) o[q8] &= 0xFFFF0000u;
          if (t0 + 2 * ii + 1 >= nvalid) o[q8] &= 0x0000FFFFu;
        }
      }
    }
    sts128(vt + tc5::sw128_off(d0, 2 * pg + c8), o[0], o[1], o[2], o[3]);
    sts128(vt + tc5::sw128_off(d0 + 8, 2 * pg + c8), o[4], o[5], o[6], o[7]);
  }
}

FR_DEVI uint32_t pack_h2_rn(float a, float b) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;\n" : "=r"(r) : "f"(b), "f"(a));
  return r;
}

template <int NB, bool KO>
__global__ void __launch_bounds__(TQ_THREADS, 1) k_mq_tc(const MqParams p) {
  using L = MLay<NB>;
  constexpr int NBASE = KO ? 3 : 1;
  using S = TQMap<NB, NBASE>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t sb = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (sb - smem_u32(smem_raw));
  const int tid = threadIdx.x, warp = __shfl_sync(FULLMASK, tid >> 5, 0), lane = tid & 31;   // warp: provably uniform
  const int item = blockIdx.x, h = blockIdx.y;
  const int* itp = p.items + ITEM_INTS * item;
  const int* tl = p.tiles + TILE_INTS * itp[0];
  const int req = tl[0], crow0 = tl[1], ntok = tl[3], pos0 = tl[4], nk = tl[5], ext = tl[8];
  const int G = p.G, Hq = p.Hkv * G, TQr = p.rows / G;     // rows = 128 or 64 query rows per tile (the plan's choice)
  const int kend = min(min(nk, itp[2] * BN), max(pos0 + ntok - p.shift, ext + 1));
  const int kb0 = itp[1];
  const int nblk = kend > kb0 * BN ? (kend + BN - 1) / BN - kb0 : 0;
  const long long pbase = (static_cast<long long>(item) * p.Hkv + h) * p.rows;

  if (nblk == 0) {          // nothing visible: empty partials
    if (tid < 128) {
      const int t = tid / G;
      if (tid < TQr * G && t < ntok) {
        float4* op = reinterpret_cast<float4*>(p.opart + (pbase + tid) * D);
#pragma unroll 4
        for (int i = 0; i < 32; ++i) op[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        *reinterpret_cast<float2*>(p.ml + (pbase + tid) * 2) = make_float2(MQ_NEG_INF, 0.f);
      }
    }
    return;
  }

  // ---- barriers, tensor memory
  const uint32_t bar = sb + S::BAR;
  const uint32_t b_rawf = bar, b_rawe = bar + 8 * TQ_RAWST, bb = bar + 16 * TQ_RAWST;
  const uint32_t b_kf = bb, b_ke = bb + 16, b_vf = bb + 32, b_ve = bb + 48;
  const uint32_t b_sf = bb + 64, b_pf = bb + 80, b_od = bb + 96, b_q = bb + 104, b_fin = bb + 112;
  volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(smem + S::MISC);
  volatile uint32_t* abortf = misc + 1;
  if (tid == 0) {
    for (int i = 0; i < TQ_RAWST; ++i) { tc5::mbar_init(b_rawf + 8 * i, 1); tc5::mbar_init(b_rawe + 8 * i, TQ_CONV); }
    for (int i = 0; i < 2; ++i) {
      tc5::mbar_init(b_kf + 8 * i, TQ_CONVH); tc5::mbar_init(b_ke + 8 * i, 1);
      tc5::mbar_init(b_vf + 8 * i, TQ_CONVH); tc5::mbar_init(b_ve + 8 * i, 1);
      tc5::mbar_init(b_sf + 8 * i, 1); tc5::mbar_init(b_pf + 8 * i, 2 * TQ_SOFT);
    }
    tc5::mbar_init(b_od, 1);
    tc5::mbar_init(b_fin, 1);
    tc5::mbar_init(b_q, 2 * TQ_SOFT);
    misc[1] = 0;
    tc5::mbar_init_fence();
  }
  if (warp == TQ_WMMA) {
    tc5::tmem_alloc(sb + S::MISC, 512);
    tc5::tmem_relinquish();
  }
  // ---- q rows of the tile -> shared memory staging [base][128 rows][272 B] (over the operand tiles, free for now)
  for (int c = tid; c < 128 * 16; c += TQ_THREADS) {
    const int r = c >> 4, c16 = c & 15, t = r / G;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r < TQr * G && t < ntok)
      v = *reinterpret_cast<const uint4*>(p.q + (static_cast<long long>(crow0 + t) * Hq + h * G + r % G) * D + 8 * c16);
    sts128(sb + r * S::QSTAGE_STRIDE + c16 * 16, v.x, v.y, v.z, v.w);
  }
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tbase = __shfl_sync(FULLMASK, misc[0], 0);
  if constexpr (KO) {       // the two rotated bases: warp per row, lane = 4 dims (fp32 butterflies, one rounding)
    for (int r = warp; r < 128; r += TQ_THREADS / 32) {
      const uint32_t src = sb + r * S::QSTAGE_STRIDE + lane * 8;
      uint32_t a, b;
      asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];\n" : "=r"(a), "=r"(b) : "r"(src));
      const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&a)), f1 = __half22float2(*reinterpret_cast<const __half2*>(&b));
      float x[4] = {f0.x, f0.y, f1.x, f1.y}, y[4] = {f0.x, f0.y, f1.x, f1.y};
      fr::fwht_row_stages(x, lane, 32);
      fr::fwht_row_stages(y, lane, 128);
      sts64(src + 128 * S::QSTAGE_STRIDE, pack_h2_rn(x[0] * fr::C32, x[1] * fr::C32), pack_h2_rn(x[2] * fr::C32, x[3] * fr::C32));
      sts64(src + 256 * S::QSTAGE_STRIDE, pack_h2_rn(y[0] * fr::C128, y[1] * fr::C128), pack_h2_rn(y[2] * fr::C128, y[3] * fr::C128));
    }
    __syncthreads();
  }

  const int kblk0 = kb0;
  const uint8_t* poolh = p.pool + static_cast<long long>(h) * L::CHUNK;
  const int* bt = p.bt + static_cast<long long>(req) * p.bt_stride;

  if (warp < 4 || (warp >= TQ_WSOFTB && warp < TQ_WSOFTB + 4)) {
    // =========================================================================== softmax warps
    // Two threads per query row: warps w and TQ_WSOFTB + w own the same 32 tensor-memory lanes (a warp reaches lanes
    // 32 (warp % 4) ..) and split the 64 key columns of a block (hf = 0 | 1).  Per block each reads its 32 scores once
    // (they stay in registers for both passes), the pair exchanges its two half-row maxima through shared memory
    // across a 64-thread named barrier, and each writes its half of the P operand; row sums stay per thread until the end.
    const int hf = warp >= TQ_WSOFTB ? 1 : 0;
    const int r = (warp & 3) * 32 + lane, t = r / G;
    const uint32_t lanebase = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int pairbar = 1 + (warp & 3);
    volatile float* xmax = reinterpret_cast<volatile float*>(smem + S::XCH);          // [parity][half][128 rows]
    volatile float* xsum = xmax + 4 * 128;                                             // [128 rows]
    const bool rval = r < TQr * G && t < ntok;
    const int lim = min(kend - 1, max(pos0 + t - p.shift, ext));
    // Q operand: this thread's half row of every base -> tensor memory (64 packed columns per base)
#pragma unroll
    for (int b = 0; b < NBASE; ++b) {
      uint32_t v[32];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint4 x = lds128(sb + (b * 128 + r) * S::QSTAGE_STRIDE + (32 * hf + 4 * i) * 4);
        v[4 * i] = x.x; v[4 * i + 1] = x.y; v[4 * i + 2] = x.z; v[4 * i + 3] = x.w;
      }
      tc5::tmem_st32(tbase + TQ_Q + b * 64 + 32 * hf + lanebase, v);
    }
    tc5::tmem_st_wait();
    tc5::fence_before_sync();
    tc5::mbar_arrive(b_q);

    float mref = MQ_NEG_INF, lsum = 0.f;
    for (int j = 0; j < nblk; ++j) {
      const int sbuf = j & 1, j0 = (kblk0 + j) * BN + 32 * hf;
      tq_wait(b_sf + 8 * sbuf, (j >> 1) & 1, abortf);
      tc5::fence_after_sync();
      const bool full = rval && j0 >= p.kmin && j0 + 31 <= lim;
      uint32_t sv[32];
      tc5::tmem_ld32(tbase + TQ_S + sbuf * 64 + 32 * hf + lanebase, sv);
      tc5::tmem_ld_wait();
      if (!full) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int key = j0 + i;
          if (!(rval && key >= p.kmin && key <= lim)) sv[i] = __float_as_uint(MQ_NEG_INF);
        }
      }
      // pass 1: maximum of the half row (four independent chains), then of the row
      float m4[4] = {MQ_NEG_INF, MQ_NEG_INF, MQ_NEG_INF, MQ_NEG_INF};
#pragma unroll
      for (int i = 0; i < 32; i += 8)
#pragma unroll
        for (int c = 0; c < 4; ++c) m4[c] = fmaxf(m4[c], fmaxf(__uint_as_float(sv[i + 2 * c]), __uint_as_float(sv[i + 2 * c + 1])));
      const float mxh = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
      xmax[((j & 1) * 2 + hf) * 128 + r] = mxh;
      asm volatile("bar.sync %0, 64;\n" ::"r"(pairbar) : "memory");
      const float mx = fmaxf(mxh, xmax[((j & 1) * 2 + (hf ^ 1)) * 128 + r]);
      float alpha = 1.f;
      const bool moved = mx > mref + 8.f || (mref == MQ_NEG_INF && mx > MQ_NEG_INF);
      if (moved) {
        alpha = mref == MQ_NEG_INF ? 0.f : ex2(mref - mx);
        mref = mx;
      }
      const float base = mref == MQ_NEG_INF ? 0.f : mref;
      // pass 2: p = 2^(s - ref) as packed FP16 straight into this half of the P operand; sum of the values in fp32
      float s4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t pk[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float p0 = ex2(__uint_as_float(sv[2 * i]) - base), p1 = ex2(__uint_as_float(sv[2 * i + 1]) - base);
        s4[i & 3] += p0 + p1;
        pk[i] = pack_h2_rn(p0, p1);
      }
      tc5::tmem_st16(tbase + TQ_P + sbuf * 32 + 16 * hf + lanebase, pk);
      lsum = lsum * alpha + ((s4[0] + s4[1]) + (s4[2] + s4[3]));
      // rescale of O (warp-collective; each thread of the pair takes 64 of the 128 columns) before P is released: the PV
      // of the previous block must have landed.  Both warps of a pair see the same `moved` for their rows.
      if (j > 0 && __any_sync(FULLMASK, moved)) {
        tq_wait(b_od, (j - 1) & 1, abortf);
        tc5::fence_after_sync();
#pragma unroll
        for (int c0 = 64 * hf; c0 < 64 * hf + 64; c0 += 32) {
          uint32_t o[32];
          tc5::tmem_ld32(tbase + TQ_O + c0 + lanebase, o);
          tc5::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tc5::tmem_st32(tbase + TQ_O + c0 + lanebase, o);
        }
      }
      tc5::tmem_st_wait();
      tc5::fence_before_sync();
      tc5::mbar_arrive(b_pf + 8 * sbuf);
    }
    // ---- partials: unnormalised O (relative to the reference), the reference (log2 units), the row sum
    // the last PV completes a barrier of its own: a parity wait on b_od can only tell the phase in flight from the one
    // before it, and here two of its phases (PV(nblk - 2), PV(nblk - 1)) may or may not have completed already
    tq_wait(b_fin, 0, abortf);
    tc5::fence_after_sync();
    if (hf == 1) xsum[r] = lsum;
    asm volatile("bar.sync %0, 64;\n" ::"r"(pairbar) : "memory");
    {
      float* op = p.opart + (pbase + r) * D;
#pragma unroll
      for (int c0 = 64 * hf; c0 < 64 * hf + 64; c0 += 32) {    // the loads are warp-collective: rows without a query take part, only the stores are predicated
        uint32_t o[32];
        tc5::tmem_ld32(tbase + TQ_O + c0 + lanebase, o);
        tc5::tmem_ld_wait();
        if (rval) {
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            *reinterpret_cast<float4*>(op + c0 + i) = make_float4(__uint_as_float(o[i]), __uint_as_float(o[i + 1]),
                                                                  __uint_as_float(o[i + 2]), __uint_as_float(o[i + 3]));
        }
      }
      if (rval && hf == 0) *reinterpret_cast<float2*>(p.ml + (pbase + r) * 2) = make_float2(mref, lsum + xsum[r]);
    }
    tc5::fence_before_sync();
  } else if (warp >= 4 && warp < 4 + TQ_CONVH / 32) {
    // =========================================================================== K conversion warps (two items per thread)
    const int ctid = tid - TQ_SOFT;
    tq_wait_relaxed(b_q, 0, abortf);          // the q staging (which lies over the operand tiles) has been read
    uint32_t prev = 0;
    for (int j = 0; j < nblk; ++j) {
      const int buf = j & 1, rs = j % TQ_RAWST;
      tq_wait_relaxed(b_rawf + 8 * rs, (j / TQ_RAWST) & 1, abortf);
      if (j >= 2) tq_wait_relaxed(b_ke + 8 * buf, ((j >> 1) - 1) & 1, abortf);     // QK(j - 2) has read this tile buffer
      tq_convert_k<NB, KO>(sb + S::RAW + rs * S::RAW_STAGE, sb + S::KT + buf * NBASE * S::KT_TILE, kend - (kblk0 + j) * BN, ctid,
                           j < 2, buf, prev);
      tc5::fence_async_smem();
      tc5::mbar_arrive(b_kf + 8 * buf);
      tc5::mbar_arrive(b_rawe + 8 * rs);
    }
  } else if (warp >= 4 + TQ_CONVH / 32 && warp < 4 + TQ_CONV / 32) {
    // =========================================================================== V conversion warps (two items per thread)
    // K and V tiles of a block are produced side by side: a block costs the longer of the two conversions, not their sum
    const int ctid = tid - TQ_SOFT - TQ_CONVH;
    tq_wait_relaxed(b_q, 0, abortf);
    for (int j = 0; j < nblk; ++j) {
      const int buf = j & 1, rs = j % TQ_RAWST;
      tq_wait_relaxed(b_rawf + 8 * rs, (j / TQ_RAWST) & 1, abortf);
      if (j >= 2) tq_wait_relaxed(b_ve + 8 * buf, ((j >> 1) - 1) & 1, abortf);     // PV(j - 2) has read this tile buffer
      tq_convert_v<NB>(sb + S::RAW + rs * S::RAW_STAGE, sb + S::VT + buf * 16384, kend - (kblk0 + j) * BN, ctid);
      tc5::fence_async_smem();
      tc5::mbar_arrive(b_vf + 8 * buf);
      tc5::mbar_arrive(b_rawe + 8 * rs);
    }
  } else if (warp == TQ_WMMA) {
    // =========================================================================== MMA issue (the warp waits, lane 0 issues)
    constexpr uint32_t id_qk = tc5::idesc(1, 0, 0, 128, BN), id_pv = tc5::idesc(1, 0, 0, 128, 128);
    tq_wait(b_q, 0, abortf);
    tc5::fence_after_sync();
    auto pv = [&](int i) {      // O (+)= P(i) V(i)
      const int buf = i & 1;
      tq_wait(b_pf + 8 * buf, (i >> 1) & 1, abortf);
      tq_wait(b_vf + 8 * buf, (i >> 1) & 1, abortf);
      tc5::fence_after_sync();
      if (tc5::elect_one()) {
        const uint32_t vt = sb + S::VT + buf * 16384;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          tc5::mma_f16_ts(tbase + TQ_O, tbase + TQ_P + buf * 32 + kk * 8, tc5::desc_sw128(vt + kk * 32, 1024), id_pv, (i | kk) > 0);
        tc5::mma_commit(b_ve + 8 * buf);
        tc5::mma_commit(b_od);
        if (i == nblk - 1) tc5::mma_commit(b_fin);
      }
      __syncwarp();
    };
    for (int j = 0; j < nblk; ++j) {
      const int buf = j & 1;
      tq_wait(b_kf + 8 * buf, (j >> 1) & 1, abortf);
      tc5::fence_after_sync();
      if (tc5::elect_one()) {
        const uint32_t kt = sb + S::KT + buf * NBASE * S::KT_TILE;
#pragma unroll
        for (int b = 0; b < NBASE; ++b)
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            tc5::mma_f16_ts(tbase + TQ_S + buf * 64, tbase + TQ_Q + b * 64 + kk * 8,
                            tc5::desc_sw128(kt + b * S::KT_TILE + (kk >> 2) * 8192 + (kk & 3) * 32, 1024), id_qk, (b | kk) > 0);
        tc5::mma_commit(b_sf + 8 * buf);
        tc5::mma_commit(b_ke + 8 * buf);
      }
      __syncwarp();
      if (j > 0) pv(j - 1);
    }
    pv(nblk - 1);
  } else if (warp == TQ_WLOAD) {
    // =========================================================================== page loader (the warp waits, lane 0 copies)
    for (int j = 0; j < nblk; ++j) {
      const int rs = j % TQ_RAWST, kb = kblk0 + j;
      if (j >= TQ_RAWST) tq_wait_relaxed(b_rawe + 8 * rs, ((j / TQ_RAWST) - 1) & 1, abortf);
      if (lane == 0) {
        const int npg = min(PPB, (kend - kb * BN + PAGE - 1) / PAGE);
        tc5::mbar_expect(b_rawf + 8 * rs, npg * L::CHUNK);
        for (int i = 0; i < npg; ++i)
          tc5::bulk_g2s(sb + S::RAW + rs * S::RAW_STAGE + i * L::CHUNK,
                        poolh + static_cast<long long>(bt[kb * PPB + i]) * p.page_stride, L::CHUNK, b_rawf + 8 * rs);
      }
      __syncwarp();
    }
  }
  tc5::fence_before_sync();
  __syncthreads();
  if (warp == TQ_WMMA) tc5::tmem_dealloc(tbase, 512);
}

template <int NB, bool KO>
int launch_mq_tc(const MqParams& p, int nitems, cudaStream_t st) {
  constexpr int smem = TQMap<NB, KO ? 3 : 1>::TOTAL;
  static unsigned long long ready = 0;
  if (!fr::smem_limit_ready(k_mq_tc<NB, KO>, smem, ready)) return -2;
  k_mq_tc<NB, KO><<<dim3(nitems, p.Hkv), TQ_THREADS, smem, st>>>(p);
  return cudaPeekAtLastError() == cudaSuccess ? 0 : -1;
}
