// INT4 paged decode attention on the 5th-generation tensor cores (tcgen05, accumulators in tensor memory).  Included by
// fr_decode.cu inside namespace fr::(anonymous); shares the q prologue, the BF16 window CTA and the split merge with the
// mma.sync kernel and replaces the same reference kernels.
//
// Tokens sit on the M dimension of the MMA, so every accumulator row (= tensor-memory lane = thread) is one token and
// everything that depends on a token's scale words and flags is thread-local:
//   * a step = 128 tokens = 8 pages of one kv head, bulk-copied page by page into a 3-stage ring (thread 64);
//   * mask pass (the CTA's 128 threads): the packed nibbles are split into one code per byte and laid out as K-major u8
//     operands: K codes [4 groups][128 tokens][32 dims], V codes [128 dims][128 tokens];
//   * QK: per group one tcgen05.mma (M 128 tokens, N 16 | 32, K 32, u8 x s8 -> s32) against q in 14-bit fixed point split
//     hi / lo, for key-only pages in three bases (identity, per-group H32, whole-head H128); the token's thread picks the
//     base by its flags, removes the zero point with the matching sum of q and applies the group scale in fp32;
//   * softmax: running maximum per head over the CTA (warp redux + one 128-thread barrier per step);
//   * PV: P' = p * V-scale as an unsigned 14-bit integer relative to the step's largest term, two 7-bit digits, written by
//     the token's thread as the u8 operand [head, group, part][128 tokens]; four tcgen05.mma (M 128 dims, N 32, K 32 tokens)
//     accumulate the step; the thread of dim d folds its columns into fp32 every step (no integer carry-over); the V
//     zero-point term is accumulated per thread in fp32 and reduced once at the end;
//   * inside a step the MMA latencies hide behind CUDA-core work: QK is issued after the K mask pass and runs under the
//     fold of the previous step and the V mask pass; PV is issued at the end of the step and runs under the next K pass.
// Every mbarrier wait is bounded; a wait that gives up sets the sticky status word and a CTA-wide abort flag that makes
// the remaining waits return at once, so the CTA still reaches its barriers, frees its tensor memory and exits.
#pragma once

constexpr int TC_STEP = 128;   // tokens per step
constexpr int TC_ST = 3;       // raw page stages
constexpr int TC_THREADS = 128;

template <int NB, int NV> struct TMap {
  using L = DLay<NB>;
  static constexpr int NS = NV == 3 ? 32 : 16;                 // S columns per group: n = base * 8 + head * 2 + part
  static constexpr int RAW_STAGE = 8 * L::CHUNK;
  static constexpr int RAW = 0;
  static constexpr int KA = RAW + TC_ST * RAW_STAGE;            // [4 groups][16][2][8][16] u8
  static constexpr int VA = KA + 4 * 4096;                      // [4 slices][16][2][8][16] u8
  static constexpr int PB = VA + 4 * 4096;                      // [4 slices][4][2][8][16] s8
  static constexpr int QB = PB + 4096;                          // [4 groups][NS / 8][2][8][16] s8
  static constexpr int QT = QB + 4 * NS * 32;                   // int16 [NV][4][128]
  static constexpr int SQ = QT + NV * 4 * 128 * 2;              // int [NV][4][4]
  static constexpr int SF = SQ + NV * 16 * 4;                   // float [4]
  static constexpr int RED = SF + 16;                           // float [2][4][8]
  static constexpr int PIDX = RED + 2 * 4 * 8 * 4;              // int [MAXPG]
  static constexpr int MBAR = PIDX + MAXPG * 4;                 // u64: full[TC_ST], qk_done, pv_done
  static constexpr int MISC = MBAR + (TC_ST + 2) * 8;           // u32 tensor-memory base, u32 abort flag
  static constexpr int TOTAL = MISC + 16;
  static constexpr int TCOLS = NV == 3 ? 256 : 128;             // S 4 * NS + O 32 columns, rounded to a power of two
  static_assert(TC_ST * RAW_STAGE >= NWARP * (4 * 128 + 8) * 4, "merge scratch aliases the raw ring");
  static_assert(KA % 128 == 0 && QB % 128 == 0, "operand tiles are 128-byte aligned");
};

FR_DEVI uint32_t lds32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(a));
  return v;
}
FR_DEVI uint32_t lds16(uint32_t a) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];\n" : "=h"(v) : "r"(a));
  return v;
}
FR_DEVI void sts32(uint32_t a, uint32_t v) { asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(a), "r"(v) : "memory"); }
FR_DEVI void sts8(uint32_t a, int v) { asm volatile("st.shared.u8 [%0], %1;\n" ::"r"(a), "r"(v) : "memory"); }
FR_DEVI void bar_tokens() { asm volatile("bar.sync 1, 128;\n" ::: "memory"); }
FR_DEVI float redux_maxf(float x) {   // warp maximum through the order-preserving integer image of the float
  int i = __float_as_int(x);
  i ^= (i >> 31) & 0x7FFFFFFF;
  i = __reduce_max_sync(FULLMASK, i);
  i ^= (i >> 31) & 0x7FFFFFFF;
  return __int_as_float(i);
}
// bounded and abortable (tc5::mbar_wait_abortable); the first wait of the kernel that runs out names its line
FR_DEVI bool tc_wait_at(uint32_t bar, uint32_t parity, volatile uint32_t* abort, int line) {
  if (tc5::mbar_try(bar, parity)) return true;
  const bool was = *abort != 0;
  const bool ok = tc5::mbar_wait_abortable(bar, parity, abort);
  if (!ok && !was) atomicCAS(&g_status, 0, line);
  return ok;
}
#define tc_wait(bar, parity, abort) tc_wait_at(bar, parity, abort, __LINE__)

template <int NB, bool KO>
__global__ void __launch_bounds__(TC_THREADS, 2) k_decode_tc(const DecodeParams p) {
  static_assert(NB == 4, "INT4 pages");
  constexpr int NV = KO ? 3 : 1;
  using L = DLay<NB>;
  using S = TMap<NB, NV>;
  constexpr int NS = S::NS;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ int last_flag;
  const int tid = threadIdx.x, lane = tid & 31, w = __shfl_sync(FULLMASK, tid >> 5, 0);   // w: provably warp-uniform
  const int NT = (p.G + 3) >> 2;
  // grid z: rows 0 .. B - 1 run the page splits (y = split); rows B .. 2 B - 1 (only with BF16 rows, only y = 0) run the
  // window CTAs, so that these short CTAs are dealt last and fill the partly empty final wave of the page CTAs
  const bool wcta = static_cast<int>(blockIdx.z) >= p.B;
  if (wcta && blockIdx.y != 0) return;
  const int kvh = blockIdx.x / NT, qt = blockIdx.x % NT, split = wcta ? p.nsplit : static_cast<int>(blockIdx.y);
  const int b = wcta ? static_cast<int>(blockIdx.z) - p.B : static_cast<int>(blockIdx.z);
  const int has_tail = p.tail != nullptr;
  const int nsp = p.nsplit + has_tail;
  const int len = p.seq_lens[b];
  const int ns_b = len > 0 ? min(p.nsplit, max(1, (len + p.chunk - 1) / p.chunk)) : 0;
  const int nparts = ns_b + has_tail;
  float* scr = reinterpret_cast<float*>(smem + S::RAW);
  constexpr int WS = 4 * 128 + 8;

  if (split >= p.nsplit) {   // the BF16 window CTA
    tail_cta_mma(p, smem + S::RAW, scr, b, kvh, qt, min(p.tail_len[b], 256));
    cta_finish(p, scr, b, kvh, qt, NT, ns_b, nparts, nsp, &last_flag);
    return;
  }
  if (split >= ns_b) return;

  const int c0 = split * p.chunk, c1 = min(len, c0 + p.chunk);
  const int lo = max(c0, p.kv_start);
  const int ntok = c1 - c0, nsteps = (ntok + TC_STEP - 1) / TC_STEP;
  const uint32_t sb = smem_u32(smem);
  int16_t* qtab = reinterpret_cast<int16_t*>(smem + S::QT);
  int* sqs = reinterpret_cast<int*>(smem + S::SQ);
  float* sfs = reinterpret_cast<float*>(smem + S::SF);
  float* red = reinterpret_cast<float*>(smem + S::RED);
  int* pidx = reinterpret_cast<int*>(smem + S::PIDX);
  const uint32_t mb = sb + S::MBAR;
  const uint32_t mb_qk = mb + 8 * TC_ST, mb_pv = mb_qk + 8;
  volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(smem + S::MISC);
  volatile uint32_t* abortf = misc + 1;

  if (w == 0) {
    tc5::tmem_alloc(sb + S::MISC, S::TCOLS);
    tc5::tmem_relinquish();
  }
  if (tid == 32) {
    for (int s = 0; s < TC_ST; ++s) tc5::mbar_init(mb + 8 * s, 1);
    tc5::mbar_init(mb_qk, 1);
    tc5::mbar_init(mb_pv, 1);
    misc[1] = 0;
    tc5::mbar_init_fence();
  }
  {
    const int* bt = p.block_table + static_cast<size_t>(b) * p.bt_stride + c0 / L::P;
    const int npg = (ntok + L::P - 1) / L::P;
    for (int i = tid; i < npg && i < MAXPG; i += 128) pidx[i] = __ldg(bt + i);
  }
  q_prologue<NV>(p, b, kvh, qt, qtab, sqs, sfs);
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tbase = __shfl_sync(FULLMASK, misc[0], 0);
  const uint32_t tS = tbase, tO = tbase + 4 * NS;

  const uint8_t* poolh = p.pool + static_cast<size_t>(kvh) * L::CHUNK;
  const size_t pstride = static_cast<size_t>(p.Hkv) * L::CHUNK;
  auto issue = [&](int s) {                                   // thread 64: the pages of step s into their ring slot
    const int npages = min(8, (ntok - s * TC_STEP + L::P - 1) / L::P);
    const uint32_t bar = mb + 8 * (s % TC_ST), dst = sb + S::RAW + (s % TC_ST) * S::RAW_STAGE;
    tc5::mbar_expect(bar, npages * L::CHUNK);
    for (int i = 0; i < npages; ++i)
      tc5::bulk_g2s(dst + i * L::CHUNK, poolh + static_cast<size_t>(pidx[8 * s + i]) * pstride, L::CHUNK, bar);
  };
  if (tid == 64)
    for (int s = 0; s < TC_ST && s < nsteps; ++s) issue(s);

  // q operand: row n = base * 8 + head * 2 + part (part 0 = hi), K index = dim inside the group
  for (int i = tid; i < 4 * NS * 2; i += 128) {            // one 16-byte chunk (n, group, half) per iteration
    const int n = i % NS, g = (i / NS) & 3, hh = i / (4 * NS);
    uint32_t wd[4] = {0u, 0u, 0u, 0u};
    if (n < NV * 8) {
      const int c = n >> 3, hd = (n >> 1) & 3, part = n & 1;
#pragma unroll
      for (int k = 0; k < 16; ++k) {
        const int qi = qtab[(c * 4 + hd) * 128 + 32 * g + 16 * hh + k];
        const int hi = (qi + 64) >> 7, lw = qi - (hi << 7);
        wd[k >> 2] |= static_cast<uint32_t>((part ? lw : hi) & 0xFF) << (8 * (k & 3));
      }
    }
    sts128(sb + S::QB + g * NS * 32 + (n >> 3) * 256 + hh * 128 + (n & 7) * 16, wd[0], wd[1], wd[2], wd[3]);
  }
  float sf[4];
#pragma unroll
  for (int h = 0; h < 4; ++h) sf[h] = sfs[h];

  float m[4], l[4], of[4], zf[4][4], alpha[4], pstep4[4];
#pragma unroll
  for (int h = 0; h < 4; ++h) {
    m[h] = NEG_INF; l[h] = 0.f; of[h] = 0.f; alpha[h] = 0.f; pstep4[h] = 0.f;
#pragma unroll
    for (int g = 0; g < 4; ++g) zf[h][g] = 0.f;
  }
  const uint32_t lanebase = static_cast<uint32_t>(w * 32) << 16;
  const int pg = tid >> 4, pos = tid & 15;
  constexpr uint32_t id_qk = tc5::idesc(2, 0, 1, 128, NS), id_pv = tc5::idesc(2, 0, 0, 128, 32);
  // fold of a finished PV: this thread is dim d = tid (group w); its columns are (w * 4 + head) * 2 + part
  auto fold = [&](int s) {
    tc_wait(mb_pv, s & 1, abortf);
    tc5::fence_after_sync();
    uint32_t r[16];
    tc5::tmem_ld16(tO + (w >> 1) * 16 + lanebase, r);
    tc5::tmem_ld_wait();
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      const int o8 = (w & 1) * 8 + 2 * h;
      const int x = static_cast<int>(r[o8]) * 128 + static_cast<int>(r[o8 + 1]);
      of[h] = fmaf(of[h], alpha[h], pstep4[h] * static_cast<float>(x));
    }
  };

  for (int s = 0; s < nsteps; ++s) {
    const uint32_t raw = sb + S::RAW + (s % TC_ST) * S::RAW_STAGE;
    const int npages = min(8, (ntok - s * TC_STEP + L::P - 1) / L::P);
    tc_wait(mb + 8 * (s % TC_ST), (s / TC_ST) & 1, abortf);
    // ---- this thread's token: scale words and flags
    const int tok = c0 + s * TC_STEP + tid;
    const bool valid = tok < c1 && tok >= lo;
    uint2 ksw = make_uint2(0u, 0u);
    uint32_t vsw[4] = {0u, 0u, 0u, 0u};
    if (valid) {
      const uint32_t rp = raw + pg * L::CHUNK;
      ksw = lds64(rp + L::KS_OFF + 8 * pos);
#pragma unroll
      for (int j = 0; j < 4; ++j) vsw[j] = lds16(rp + L::VS_OFF + 2 * (j * 16 + 8 * (pos >> 3) + vslot8(pos)));
    }
    // ---- mask pass, K: item = (token, quarter tg): 16 stored bytes = words j = 0 .. 3 (the four groups)
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int item = tid + 128 * it, tk = item >> 2, tg = item & 3;
      if ((tk >> 4) < npages) {
        const uint4 v = lds128(raw + (tk >> 4) * L::CHUNK + 64 * (tk & 15) + 16 * tg);
        const uint32_t dst = sb + S::KA + (tk >> 3) * 256 + (tk & 7) * 16 + 4 * tg;
        const uint32_t wj[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          sts32(dst + j * 4096, wj[j] & 0x0F0F0F0Fu);
          sts32(dst + j * 4096 + 128, (wj[j] >> 4) & 0x0F0F0F0Fu);
        }
      }
    }
    tc5::fence_async_smem();
    tc5::fence_before_sync();
    bar_tokens();
    if (w == 0) {                 // issued under elect.sync: the operands stay in the uniform datapath
      tc5::fence_after_sync();
      if (tc5::elect_one()) {
#pragma unroll
        for (int g = 0; g < 4; ++g)
          tc5::mma_i8_ss(tS + g * NS, tc5::desc_plain(sb + S::KA + g * 4096, 128, 256),
                         tc5::desc_plain(sb + S::QB + g * NS * 32, 128, 256), id_qk, 0);
        tc5::mma_commit(mb_qk);
      }
      __syncwarp();
    }
    // ---- under the QK: fold of the previous step, then the V mask pass (the V and P' tiles are free once that PV is done)
    if (s > 0) fold(s - 1);
#pragma unroll
    for (int it = 0; it < 4; ++it) {   // item = one 16-byte entry e of a page: words s = 2 m + r8 <-> dim 64 m + 16 w + gid + 8 r8
      const int item = tid + 128 * it, vp = item >> 6, e = item & 63;
      if (vp < npages) {
        const uint4 v = lds128(raw + vp * L::CHUNK + L::V_OFF + 16 * e);
        const int c8 = e & 1, gid = (e >> 1) & 7, vw = e >> 4;
        const uint32_t dst = sb + S::VA + (vp >> 1) * 4096 + (vp & 1) * 128 + 4 * c8;
        const uint32_t ws[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int si = 0; si < 4; ++si) {
          const int d = 64 * (si >> 1) + 16 * vw + gid + 8 * (si & 1);
          const uint32_t a = dst + (d >> 3) * 256 + (d & 7) * 16;
          sts32(a, ws[si] & 0x0F0F0F0Fu);            // tokens 8 c8 + 0, 2, 4, 6
          sts32(a + 8, (ws[si] >> 4) & 0x0F0F0F0Fu); // tokens 8 c8 + 1, 3, 5, 7
        }
      }
    }
    // ---- scores of this thread's token
    tc_wait(mb_qk, s & 1, abortf);
    tc5::fence_after_sync();
    float sc4[4] = {0.f, 0.f, 0.f, 0.f};
    [[maybe_unused]] const bool ffl = (vsw[0] & 0x8000u) != 0;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      uint32_t r[NS];
      if constexpr (NS == 32) tc5::tmem_ld32(tS + g * NS + lanebase, r);
      else tc5::tmem_ld16(tS + g * NS + lanebase, r);
      tc5::tmem_ld_wait();
      const uint32_t kw = ((g & 2) ? ksw.y : ksw.x) >> (16 * (g & 1));
      const float ks = h2f(kw & 0x7FFFu);
      const int z = static_cast<int>(kw & 15u);
      int c = 0;
      if constexpr (KO) c = ffl ? 2 : static_cast<int>((kw >> 15) & 1u);
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        int hi = static_cast<int>(r[2 * h]), lw = static_cast<int>(r[2 * h + 1]);
        if constexpr (KO) {
          hi = c == 2 ? static_cast<int>(r[16 + 2 * h]) : (c == 1 ? static_cast<int>(r[8 + 2 * h]) : hi);
          lw = c == 2 ? static_cast<int>(r[17 + 2 * h]) : (c == 1 ? static_cast<int>(r[9 + 2 * h]) : lw);
        }
        const int y = hi * 128 + lw - z * sqs[(c * 4 + h) * 4 + g];
        sc4[h] = fmaf(ks, static_cast<float>(y), sc4[h]);
      }
    }
    uint32_t vmaxb = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) vmaxb = max(vmaxb, vsw[j] & 0x7FFFu);
    vmaxb = __reduce_max_sync(FULLMASK, vmaxb);
    float* rd = red + (s & 1) * 32 + w * 8;
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      sc4[h] = valid ? sc4[h] * sf[h] : NEG_INF;
      const float wm = redux_maxf(sc4[h]);
      if (lane == 0) rd[h] = wm;
    }
    if (lane == 0) rd[4] = __uint_as_float(vmaxb);
    tc5::fence_before_sync();
    bar_tokens();   // maxima visible; every thread is past its reads of the ring slot and of the S columns
    if (tid == 64 && s + TC_ST < nsteps) issue(s + TC_ST);
    const float* ra = red + (s & 1) * 32;
    // P' is quantised relative to the step's own maximum (14 bits below the largest term of the step); beta carries the
    // step into the running scale
    float beta[4], sbase[4];
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      const float ms = fmaxf(fmaxf(ra[h], ra[8 + h]), fmaxf(ra[16 + h], ra[24 + h]));
      const float mn = fmaxf(m[h], ms);
      const float base = mn == NEG_INF ? 0.f : mn;
      sbase[h] = ms == NEG_INF ? 0.f : ms;
      alpha[h] = ex2(m[h] - base);
      beta[h] = ex2(ms - base);
      m[h] = mn;
    }
    const uint32_t nmaxb = max(max(__float_as_uint(ra[4]), __float_as_uint(ra[12])), max(__float_as_uint(ra[20]), __float_as_uint(ra[28])));
    const float nmax = h2f(nmaxb);
    const float pstep1 = nmax * (1.0f / 16256.0f);
    const float pinv = nmax > 0.f ? 16256.0f / nmax : 0.f;
    float pr[4];
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      pr[h] = valid ? ex2(sc4[h] - sbase[h]) : 0.f;      // relative to the step's maximum
      l[h] = fmaf(l[h], alpha[h], pr[h] * beta[h]);
      pstep4[h] = pstep1 * beta[h];
    }
    // ---- P' operand: row n = (group * 4 + head) * 2 + part, K index = token inside its 32-token slice.  P' is an unsigned
    // 14-bit integer (two 7-bit digits, u8 operand); the zero-point term uses the same integer, so the rounding error of
    // P' meets (code - zero point) and not the bare code
    {
      const uint32_t pb = sb + S::PB + (pg >> 1) * 1024 + (pg & 1) * 128 + ((pos & 1) * 8 + (pos >> 1));
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const float vs = h2f(vsw[g] & 0x7FFFu) * pinv;
        const float vz = static_cast<float>(vsw[g] & 15u);
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          const uint32_t bits = __float_as_uint(fmaf(pr[h], vs, 8388608.0f));     // integer in the low mantissa bits
          const float pq = __uint_as_float(bits) - 8388608.0f;
          zf[h][g] = fmaf(zf[h][g], alpha[h], pq * vz * pstep4[h]);
          const int n = (g * 4 + h) * 2;
          sts8(pb + (n >> 3) * 256 + (n & 7) * 16, static_cast<int>(bits >> 7));
          sts8(pb + (n >> 3) * 256 + ((n + 1) & 7) * 16, static_cast<int>(bits & 127u));
        }
      }
    }
    tc5::fence_async_smem();
    bar_tokens();
    if (w == 0) {
      tc5::fence_after_sync();
      if (tc5::elect_one()) {
#pragma unroll
        for (int sl = 0; sl < 4; ++sl)
          tc5::mma_i8_ss(tO, tc5::desc_plain(sb + S::VA + sl * 4096, 128, 256), tc5::desc_plain(sb + S::PB + sl * 1024, 128, 256),
                         id_pv, sl > 0);
        tc5::mma_commit(mb_pv);
      }
      __syncwarp();
    }
  }
  fold(nsteps - 1);

  // ---- CTA epilogue: sums over the threads, zero-point term, hand-over to the split merge
  tc5::fence_before_sync();
  bar_tokens();   // every tensor-memory read is complete; the raw ring is free (all bulk copies were consumed)
  if (w == 0) tc5::tmem_dealloc(tbase, S::TCOLS);
  float* zs = scr + 4 * WS;            // [4 warps][20]
#pragma unroll
  for (int h = 0; h < 4; ++h) {
    float v = l[h];
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) v += __shfl_xor_sync(FULLMASK, v, o);
    if (lane == 0) zs[w * 20 + 16 + h] = v;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      float z = zf[h][g];
#pragma unroll
      for (int o = 16; o >= 1; o >>= 1) z += __shfl_xor_sync(FULLMASK, z, o);
      if (lane == 0) zs[w * 20 + h * 4 + g] = z;
    }
  }
  bar_tokens();
#pragma unroll
  for (int h = 0; h < 4; ++h) {
    const float zsum = zs[h * 4 + w] + zs[20 + h * 4 + w] + zs[40 + h * 4 + w] + zs[60 + h * 4 + w];
    scr[h * 128 + tid] = of[h] - zsum;
#pragma unroll
    for (int k = 1; k < NWARP; ++k) scr[k * WS + h * 128 + tid] = 0.f;
  }
  if (tid < 4) {
    scr[512 + tid] = m[tid];
    scr[516 + tid] = zs[16 + tid] + zs[36 + tid] + zs[56 + tid] + zs[76 + tid];
#pragma unroll
    for (int k = 1; k < NWARP; ++k) { scr[k * WS + 512 + tid] = NEG_INF; scr[k * WS + 516 + tid] = 0.f; }
  }
  cta_finish(p, scr, b, kvh, qt, NT, split, nparts, nsp, &last_flag);
}

template <int NB, bool KO> int launch_tc(const DecodeParams& p, cudaStream_t st) {
  constexpr int smem = TMap<NB, KO ? 3 : 1>::TOTAL;
  static bool set = false;
  if (!set) {
    if (cudaFuncSetAttribute(k_decode_tc<NB, KO>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -2;
    set = true;
  }
  const int NT = (p.G + 3) / 4;
  const dim3 grid(p.Hkv * NT, p.nsplit, p.B * (p.tail != nullptr ? 2 : 1));
  k_decode_tc<NB, KO><<<grid, TC_THREADS, smem, st>>>(p);
  return cudaPeekAtLastError() == cudaSuccess ? 0 : -1;
}
