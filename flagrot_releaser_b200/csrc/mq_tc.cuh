// Prefix-cached multi-query prefill attention on the 5th-generation tensor cores: S = Q K^T and O += P V as tcgen05.mma
// with the accumulators, the Q operand and the P operand in tensor memory.  Included by mq_capi.cu inside its anonymous
// namespace (kernel 3 of frmq_attn); same work list, partial layout and numerics contract as the mma.sync kernel above.
//
// CTA = (item, kv head): 128 query rows x the item's 64-key blocks; 14 warps with fixed roles:
//   warps 0-3   softmax: thread r owns query row r = tensor-memory lane r.  Per block: load the 64 scores, (mask,) running
//               maximum with a lazy reference (the reference only moves when the maximum grew by more than 2^8, so the
//               O accumulator is rescaled a few times per item, not per block), p = 2^(s - ref) to FP16 into the P
//               operand columns, row sum in fp32;
//   warps 4-11  conversion: raw page chunks -> FP16 operand tiles in shared memory (128-byte swizzle, K-major):
//               K [64 keys][128 dims] as (code - zero point) * scale, exact in FP16, one rounding; V^T [128 dims][64 keys];
//   warp 12     issues the MMAs (lane 0; the whole warp waits) and owns the tensor-memory allocation;
//   warp 13     bulk-copies the four page chunks of a block into a 3-stage ring.
// Key-only pages (per-token rotation flags) are not rotated back per token: the kernel keeps Q in three bases (identity,
// per-group H32, whole-head H128) in tensor memory, the conversion drops each (key, group) into the operand tile of its
// base and zeros into the other two, and S accumulates the three products - three times the QK tensor work, which the
// tensor pipe has to spare, instead of a butterfly network per key on the CUDA cores.
// Pipelines: K / V tiles, S and P are double buffered; every hand-over is an mbarrier (bulk-copy bytes, thread arrivals
// or tcgen05.commit).  All waits are bounded; a wait that gives up sets a CTA-wide abort flag and the status word, after
// which every wait returns at once and the CTA runs to its end (results are garbage, the status says so).
#pragma once

constexpr int TQ_THREADS = 448;
constexpr int TQ_CONV = 256;          // conversion threads
constexpr int TQ_RAWST = 3;
__device__ int g_mq_status;

template <int NB, int NBASE> struct TQMap {
  static constexpr int CHUNK = MLay<NB>::CHUNK;
  static constexpr int KT = 0;                                   // [2 buffers][NBASE][2 dim halves][64 rows][128 B]
  static constexpr int KT_TILE = 16384;
  static constexpr int VT = KT + 2 * NBASE * KT_TILE;            // [2 buffers][128 rows][128 B]
  static constexpr int RAW = VT + 2 * 16384;                     // [3][4 pages][CHUNK]
  static constexpr int RAW_STAGE = PPB * CHUNK;
  static constexpr int BAR = RAW + TQ_RAWST * RAW_STAGE;         // mbarriers
  static constexpr int NBAR = 3 + 3 + 2 + 2 + 2 + 2 + 2 + 2 + 1 + 1;
  static constexpr int MISC = BAR + NBAR * 8;
  static constexpr int TOTAL = MISC + 16 + 1024;                 // + slack for the 1024-byte alignment of the tiles
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

// K operand tiles of one 64-key block.  item = (key, word): word (tg, j) of the key's 16 code words carries dims
// 32 j + 4 tg + {0..3} in the low fields and + 16 in the high fields of its four bytes.
template <int NB, bool KO>
FR_DEVI void tq_convert_k(uint32_t raw, uint32_t kt, int nvalid, int ctid) {
  using L = MLay<NB>;
  constexpr int NBASE = KO ? 3 : 1;
  constexpr uint32_t FM = NB == 4 ? 0x000F000Fu : 0x00030003u;
#pragma unroll
  for (int it = 0; it < (BN * 16) / TQ_CONV; ++it) {
    const int item = ctid + TQ_CONV * it, tok = item >> 4, tg = (item >> 2) & 3, j = item & 3;
    const int pos = tok & 15;
    const uint32_t rc = raw + (tok >> 4) * L::CHUNK;
    // destination inside a tile: dim half j >> 1, 16-byte chunk 4 (j & 1) + (tg >> 1) (+ 2 for the high fields), 8 (tg & 1)
    const uint32_t dlo = (j >> 1) * 8192 + tc5::sw128_off(tok, 4 * (j & 1) + (tg >> 1)) + 8 * (tg & 1);
    const uint32_t dhi = (j >> 1) * 8192 + tc5::sw128_off(tok, 4 * (j & 1) + (tg >> 1) + 2) + 8 * (tg & 1);
    uint32_t o[4] = {0u, 0u, 0u, 0u};     // lo dims 0 1 | lo dims 2 3 | hi dims 0 1 | hi dims 2 3
    int base = 0;
    if (tok < nvalid) {
      uint32_t w;
      if (NB == 4) w = lds32(rc + 64 * pos + 16 * tg + 4 * j);
      else w = lds32(rc + 32 * (pos ^ ((pos >> 1) & 2)) + 8 * tg + 4 * (j >> 1)) >> (4 * (j & 1));
      const uint32_t kw = lds16(rc + L::KS_OFF + 8 * pos + 2 * j);
      const uint32_t zz = ((kw & L::ZM) * 0x00010001u) | 0x64006400u;
      const uint32_t sc = (kw & 0x7FFFu) * 0x00010001u;
      const uint32_t p01 = prmt(w, 0u, 0x4140u), p23 = prmt(w, 0u, 0x4342u);
      o[0] = hmul2u(hsub2u((p01 & FM) | 0x64006400u, zz), sc);
      o[1] = hmul2u(hsub2u((p23 & FM) | 0x64006400u, zz), sc);
      o[2] = hmul2u(hsub2u(((p01 >> NB) & FM) | 0x64006400u, zz), sc);
      o[3] = hmul2u(hsub2u(((p23 >> NB) & FM) | 0x64006400u, zz), sc);
      if constexpr (KO) {
        const bool ffl = (lds16(rc + L::VS_OFF + 2 * (8 * (pos >> 3) + fr::vslot8(pos))) & 0x8000u) != 0;
        base = ffl ? 2 : static_cast<int>(kw >> 15);
      }
    }
#pragma unroll
    for (int b = 0; b < NBASE; ++b) {
      const bool on = b == base;
      sts64(kt + b * 16384 + dlo, on ? o[0] : 0u, on ? o[1] : 0u);
      sts64(kt + b * 16384 + dhi, on ? o[2] : 0u, on ? o[3] : 0u);
    }
  }
}

// V^T operand tile [128 dims][64 keys]: item = the 8 tokens of one (page, dim) code word -> one 16-byte chunk
template <int NB>
FR_DEVI void tq_convert_v(uint32_t raw, uint32_t vt, int nvalid, int ctid) {
  using L = MLay<NB>;
#pragma unroll
  for (int it = 0; it < (PPB * 64 * 4) / TQ_CONV; ++it) {
    const int item = ctid + TQ_CONV * it;
    const int pg = item >> 8, e = (item >> 2) & 63, s = item & 3;
    const int c8 = e & 1, gid = (e >> 1) & 7, w = e >> 4;
    const int m = s >> 1, r8 = s & 1;
    const int d = 64 * m + 16 * w + gid + 8 * r8, j = 2 * m + (w >> 1);
    const uint32_t rc = raw + pg * L::CHUNK;
    const int t0 = 16 * pg + 8 * c8;
    uint32_t o[4] = {0u, 0u, 0u, 0u};
    if (t0 < nvalid) {
      uint32_t word;
      if (NB == 4) word = lds32(rc + L::V_OFF + 16 * e + 4 * s);
      else word = lds32(rc + L::V_OFF + 8 * e + 4 * m) >> (4 * r8);
      const uint4 sw = lds128(rc + L::VS_OFF + 2 * (j * PAGE + 8 * c8));     // scale words of tokens 0 2 4 6 | 1 3 5 7
      const uint32_t sp[4] = {prmt(sw.x, sw.z, 0x5410u), prmt(sw.x, sw.z, 0x7632u), prmt(sw.y, sw.w, 0x5410u), prmt(sw.y, sw.w, 0x7632u)};
#pragma unroll
      for (int ii = 0; ii < 4; ++ii) {
        const uint32_t b = (word >> (8 * ii)) & 0xFFu;
        uint32_t u;
        if (NB == 4) u = (b & 15u) | ((b >> 4) << 16);
        else u = (b & 3u) | (((b >> 2) & 3u) << 16);
        const uint32_t zz = (sp[ii] & (L::ZM | (L::ZM << 16))) | 0x64006400u;
        uint32_t v = hmul2u(hsub2u(u | 0x64006400u, zz), sp[ii] & 0x7FFF7FFFu);
        if (t0 + 2 * ii >= nvalid) v &= 0xFFFF0000u;
        if (t0 + 2 * ii + 1 >= nvalid) v &= 0x0000FFFFu;
        o[ii] = v;
      }
    }
    sts128(vt + tc5::sw128_off(d, 2 * pg + c8), o[0], o[1], o[2], o[3]);
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
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int item = blockIdx.x, h = blockIdx.y;
  const int* itp = p.items + ITEM_INTS * item;
  const int* tl = p.tiles + TILE_INTS * itp[0];
  const int req = tl[0], crow0 = tl[1], ntok = tl[3], pos0 = tl[4], nk = tl[5], ext = tl[8];
  const int G = p.G, Hq = p.Hkv * G, TQr = 128 / G;
  const int kend = min(min(nk, itp[2] * BN), max(pos0 + ntok - p.shift, ext + 1));
  const int kb0 = itp[1];
  const int nblk = kend > kb0 * BN ? (kend + BN - 1) / BN - kb0 : 0;
  const long long pbase = (static_cast<long long>(item) * p.Hkv + h) * 128;

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
  const uint32_t b_rawf = bar, b_rawe = bar + 24, b_kf = bar + 48, b_ke = bar + 64, b_vf = bar + 80, b_ve = bar + 96;
  const uint32_t b_sf = bar + 112, b_pf = bar + 128, b_od = bar + 144, b_q = bar + 152;
  volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(smem + S::MISC);
  volatile uint32_t* abortf = misc + 1;
  if (tid == 0) {
    for (int i = 0; i < 3; ++i) { tc5::mbar_init(b_rawf + 8 * i, 1); tc5::mbar_init(b_rawe + 8 * i, TQ_CONV); }
    for (int i = 0; i < 2; ++i) {
      tc5::mbar_init(b_kf + 8 * i, TQ_CONV); tc5::mbar_init(b_ke + 8 * i, 1);
      tc5::mbar_init(b_vf + 8 * i, TQ_CONV); tc5::mbar_init(b_ve + 8 * i, 1);
      tc5::mbar_init(b_sf + 8 * i, 1); tc5::mbar_init(b_pf + 8 * i, 128);
    }
    tc5::mbar_init(b_od, 1);
    tc5::mbar_init(b_q, 128);
    misc[1] = 0;
    tc5::mbar_init_fence();
  }
  if (warp == 12) {
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
  const uint32_t tbase = misc[0];
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

  if (warp < 4) {
    // =========================================================================== softmax warps (thread = query row)
    const uint32_t lanebase = static_cast<uint32_t>(warp * 32) << 16;
    const int r = tid, t = r / G;
    const bool rval = r < TQr * G && t < ntok;
    const int lim = min(kend - 1, max(pos0 + t - p.shift, ext));
    // Q operand: this thread's row of every base -> tensor memory (64 packed columns per base)
#pragma unroll
    for (int b = 0; b < NBASE; ++b)
#pragma unroll
      for (int c0 = 0; c0 < 64; c0 += 32) {
        uint32_t v[32];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint4 x = lds128(sb + (b * 128 + r) * S::QSTAGE_STRIDE + (c0 + 4 * i) * 4);
          v[4 * i] = x.x; v[4 * i + 1] = x.y; v[4 * i + 2] = x.z; v[4 * i + 3] = x.w;
        }
        tc5::tmem_st32(tbase + TQ_Q + b * 64 + c0 + lanebase, v);
      }
    tc5::tmem_st_wait();
    tc5::fence_before_sync();
    tc5::mbar_arrive(b_q);

    float mref = MQ_NEG_INF, lsum = 0.f;
    for (int j = 0; j < nblk; ++j) {
      const int sbuf = j & 1, j0 = (kblk0 + j) * BN;
      tq_wait(b_sf + 8 * sbuf, (j >> 1) & 1, abortf);
      tc5::fence_after_sync();
      uint32_t sv[64];
      {
        uint32_t a[32], b2[32];
        tc5::tmem_ld32(tbase + TQ_S + sbuf * 64 + lanebase, a);
        tc5::tmem_ld32(tbase + TQ_S + sbuf * 64 + 32 + lanebase, b2);
        tc5::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) { sv[i] = a[i]; sv[32 + i] = b2[i]; }
      }
      const bool full = rval && j0 >= p.kmin && j0 + BN - 1 <= lim;
      float mx = MQ_NEG_INF;
      if (full) {
#pragma unroll
        for (int i = 0; i < 64; ++i) mx = fmaxf(mx, __uint_as_float(sv[i]));
      } else {
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const int key = j0 + i;
          const float x = (rval && key >= p.kmin && key <= lim) ? __uint_as_float(sv[i]) : MQ_NEG_INF;
          sv[i] = __float_as_uint(x);
          mx = fmaxf(mx, x);
        }
      }
      // lazy reference: move it only when the maximum outgrew it by 2^8 (p stays <= 256, far inside FP16)
      float alpha = 1.f;
      const bool moved = mx > mref + 8.f || (mref == MQ_NEG_INF && mx > MQ_NEG_INF);
      if (moved) {
        alpha = mref == MQ_NEG_INF ? 0.f : ex2(mref - mx);
        mref = mx;
      }
      const float base = mref == MQ_NEG_INF ? 0.f : mref;
      uint32_t pk[32];
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float p0 = ex2(__uint_as_float(sv[2 * i]) - base), p1 = ex2(__uint_as_float(sv[2 * i + 1]) - base);
        sum += p0 + p1;
        pk[i] = pack_h2_rn(p0, p1);
      }
      lsum = lsum * alpha + sum;
      // rescale of O (warp-collective) before P is released: the PV of the previous block must have landed
      if (j > 0 && __any_sync(FULLMASK, moved)) {
        tq_wait(b_od, (j - 1) & 1, abortf);
        tc5::fence_after_sync();
#pragma unroll
        for (int c0 = 0; c0 < 128; c0 += 32) {
          uint32_t o[32];
          tc5::tmem_ld32(tbase + TQ_O + c0 + lanebase, o);
          tc5::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tc5::tmem_st32(tbase + TQ_O + c0 + lanebase, o);
        }
      }
      tc5::tmem_st32(tbase + TQ_P + sbuf * 32 + lanebase, pk);
      tc5::tmem_st_wait();
      tc5::fence_before_sync();
      tc5::mbar_arrive(b_pf + 8 * sbuf);
    }
    // ---- partials: unnormalised O (relative to the reference), the reference (log2 units), the row sum
    // a parity wait can only tell the phase in flight from the one before it: at this point PV(nblk - 2) may still be
    // pending, so its phase is waited for first, then the last one
    if (nblk > 1) tq_wait(b_od, (nblk - 2) & 1, abortf);
    tq_wait(b_od, (nblk - 1) & 1, abortf);
    tc5::fence_after_sync();
    {
      float* op = p.opart + (pbase + r) * D;
#pragma unroll
      for (int c0 = 0; c0 < 128; c0 += 32) {    // the loads are warp-collective: rows without a query take part, only the stores are predicated
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
      if (rval) *reinterpret_cast<float2*>(p.ml + (pbase + r) * 2) = make_float2(mref, lsum);
    }
    tc5::fence_before_sync();
  } else if (warp < 12) {
    // =========================================================================== conversion warps
    const int ctid = tid - 128;
    tq_wait(b_q, 0, abortf);          // the q staging (which lies over the operand tiles) has been read
    for (int j = 0; j < nblk; ++j) {
      const int buf = j & 1, rs = j % TQ_RAWST;
      const uint32_t raw = sb + S::RAW + rs * S::RAW_STAGE;
      const int nvalid = kend - (kblk0 + j) * BN;
      tq_wait(b_rawf + 8 * rs, (j / TQ_RAWST) & 1, abortf);
      if (j >= 2) tq_wait(b_ke + 8 * buf, ((j >> 1) - 1) & 1, abortf);
      tq_convert_k<NB, KO>(raw, sb + S::KT + buf * NBASE * S::KT_TILE, nvalid, ctid);
      tc5::fence_async_smem();
      tc5::mbar_arrive(b_kf + 8 * buf);
      if (j >= 2) tq_wait(b_ve + 8 * buf, ((j >> 1) - 1) & 1, abortf);
      tq_convert_v<NB>(raw, sb + S::VT + buf * 16384, nvalid, ctid);
      tc5::fence_async_smem();
      tc5::mbar_arrive(b_vf + 8 * buf);
      tc5::mbar_arrive(b_rawe + 8 * rs);
    }
  } else if (warp == 12) {
    // =========================================================================== MMA issue (the warp waits, lane 0 issues)
    constexpr uint32_t id_qk = tc5::idesc(1, 0, 0, 128, BN), id_pv = tc5::idesc(1, 0, 0, 128, 128);
    tq_wait(b_q, 0, abortf);
    tc5::fence_after_sync();
    auto pv = [&](int i) {      // O (+)= P(i) V(i)
      const int buf = i & 1;
      tq_wait(b_pf + 8 * buf, (i >> 1) & 1, abortf);
      tq_wait(b_vf + 8 * buf, (i >> 1) & 1, abortf);
      tc5::fence_after_sync();
      if (lane == 0) {
        const uint32_t vt = sb + S::VT + buf * 16384;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          tc5::mma_f16_ts(tbase + TQ_O, tbase + TQ_P + buf * 32 + kk * 8, tc5::desc_sw128(vt + kk * 32, 1024), id_pv, (i | kk) > 0);
        tc5::mma_commit(b_ve + 8 * buf);
        tc5::mma_commit(b_od);
      }
      __syncwarp();
    };
    for (int j = 0; j < nblk; ++j) {
      const int buf = j & 1;
      tq_wait(b_kf + 8 * buf, (j >> 1) & 1, abortf);
      tc5::fence_after_sync();
      if (lane == 0) {
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
  } else {
    // =========================================================================== page loader (the warp waits, lane 0 copies)
    for (int j = 0; j < nblk; ++j) {
      const int rs = j % TQ_RAWST, kb = kblk0 + j;
      if (j >= TQ_RAWST) tq_wait(b_rawe + 8 * rs, ((j / TQ_RAWST) - 1) & 1, abortf);
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
  if (warp == 12) tc5::tmem_dealloc(tbase, 512);
}

template <int NB, bool KO>
int launch_mq_tc(const MqParams& p, int nitems, cudaStream_t st) {
  constexpr int smem = TQMap<NB, KO ? 3 : 1>::TOTAL;
  static bool set = false;
  if (!set) {
    if (cudaFuncSetAttribute(k_mq_tc<NB, KO>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -2;
    set = true;
  }
  k_mq_tc<NB, KO><<<dim3(nitems, p.Hkv), TQ_THREADS, smem, st>>>(p);
  return cudaPeekAtLastError() == cudaSuccess ? 0 : -1;
}
