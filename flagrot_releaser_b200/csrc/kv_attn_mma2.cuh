// KIVI paged decode on the tensor cores, CTA-synchronous variant of k_kv_attn_mma (same math, same page reads, same
// output format; included by kv_capi.cu after kv_attn_mma.cuh, whose helpers it uses).
//
// k_kv_attn_mma keeps a full set of output accumulators (8 heads x 128 channels x 3 storage classes = 96 registers per
// lane) in every warp, which caps the kernel at 2 CTAs per SM.  Here the four warps of a CTA advance together over four
// 32-token groups per step: warp w does QK and the value-tile expansion of group 4 it + w, the four group maxima are
// combined into ONE running maximum per head, every warp publishes its p (fp16) in shared memory, and warp w then does the PV
// products of all four groups for the 32-channel block w only.  One set of accumulators per CTA: 24 registers per lane.
// Three CTA barriers per step of 128 tokens.
#pragma once

namespace kvm {

constexpr int P_HSTR = 40;                                 // halves per (group, head) row of p: 32 tokens + 8 (bank spread)
constexpr int P_BYTES = 4 * 8 * P_HSTR * 2;                // p of the step: [group][head][token] fp16 (the PV A operand is fp16 anyway)
constexpr int SMEM2 = QB_BYTES + 4 * WARP_SMEM + P_BYTES + 256;   // + [4][8] group maxima, [4] flags
static_assert(3 * (SMEM2 + 1024) <= 227 * 1024, "three CTAs per SM");

template <int G, bool F8>
__global__ void __launch_bounds__(128, 3) k_kv_attn_mma2(const __nv_bfloat16* __restrict__ q, long long q_rs,
                                                          const uint8_t* __restrict__ pool, const int* __restrict__ bt, long long bt_rs,
                                                          const int* __restrict__ cached, int kv_start, int Hkv, int NS, int chunk,
                                                          float qscale, const __nv_bfloat16* __restrict__ ring,
                                                          const int* __restrict__ tail_len, const int* __restrict__ tail_idx, int T,
                                                          int B, float* __restrict__ opart, float* __restrict__ ml) {
  static_assert(G <= 8, "one M tile of q heads");
  using L = KLay<F8>;                            // kivi2p8 pages are read as stored: their FP8 pairs are converted at use
  extern __shared__ __align__(16) uint8_t smraw[];
  if (static_cast<int>(blockIdx.z) >= B) {       // the BF16 sink / window splits come last in the grid
    if (blockIdx.y == 0) kv_tail_mma<G>(smraw, blockIdx.x, static_cast<int>(blockIdx.z) - B, q, q_rs, Hkv, NS, qscale, ring, tail_len,
                                        tail_idx, T, opart, ml);
    return;
  }
  float (*qb)[8][D] = reinterpret_cast<float (*)[8][D]>(smraw);
  const int h = blockIdx.x, sp = blockIdx.y, b = blockIdx.z;
  if (sp >= NS) return;                          // NS == 0: the grid still has one y row, but there is no page split
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g8 = lane >> 2, c4 = lane & 3;
  const long long pidx = static_cast<long long>(b * Hkv + h) * (NS + 1) + sp;
  float* op = opart + pidx * G * D;
  float* mlp = ml + pidx * G * 2;
  const int t0 = max(sp * chunk, kv_start), t1 = min((sp + 1) * chunk, cached[b]);
  if (t1 <= t0) {
    for (int e = tid; e < G; e += 128) { mlp[2 * e] = KV_NEG_INF; mlp[2 * e + 1] = 0.f; }
    return;
  }
  // ---- q in three bases (rows >= G are zero), rows re-laid with a padded stride, times qscale * 16 (channels 8 - 15 of
  // every 16: times qscale / 16, their key codes enter the MMA 2^8 larger, see the QK step)
  {
    const __nv_bfloat16* qp = q + static_cast<long long>(b) * q_rs + static_cast<long long>(h) * G * D;
    for (int e = tid; e < 8 * D; e += 128) {
      const float v = e < G * D ? __bfloat162float(qp[e]) : 0.f;
      qb[0][e / D][e % D] = v; qb[1][e / D][e % D] = v; qb[2][e / D][e % D] = v;
    }
    __syncthreads();
    smem_hada<8>(qb[1], 32);
    smem_hada<8>(qb[2], 128);
    float v[24];
#pragma unroll
    for (int i = 0; i < 24; ++i) v[i] = reinterpret_cast<float*>(smraw)[tid + 128 * i];
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 24; ++i) {
      const int e = tid + 128 * i;
      reinterpret_cast<float*>(smraw)[(e / D) * QSTR + e % D] = v[i] * ((e & 8) ? qscale * (1.f / 16.f) : qscale * 16.f);
    }
    __syncthreads();
  }
  const uint32_t sb = smem_u32(smraw);
  const uint32_t wraw = sb + QB_BYTES + warp * WARP_SMEM;
  const uint32_t qbs = sb;
  const uint32_t pbuf = sb + QB_BYTES + 4 * WARP_SMEM;              // [group][head][token]
  float* gmax = reinterpret_cast<float*>(smraw + QB_BYTES + 4 * WARP_SMEM + P_BYTES);   // [group][head]
  int* gflag = reinterpret_cast<int*>(gmax + 32);                     // [group]: bit 0 the group exists, bit 1 it has a whole-head token
  const int* btb = bt + static_cast<long long>(b) * bt_rs;
  const int gfirst = t0 / GRP, gend = (t1 + GRP - 1) / GRP;
  auto load_group = [&](int g32, int buf) {
    const uint8_t* chA = pool + (static_cast<long long>(btb[2 * g32]) * Hkv + h) * L::CB;
    const uint8_t* chB = pool + (static_cast<long long>(btb[2 * g32 + 1]) * Hkv + h) * L::CB;
    const uint32_t dst = wraw + buf * RAW_GROUP;
    for (int i = lane; i < L::CB / 16; i += 32) {
      cp16(dst + 16 * i, chA + 16 * i);
      cp16(dst + RAW_PAGE + 16 * i, chB + 16 * i);
    }
    cp_commit();
  };

  // ---- accumulators of this warp: channel block `warp` (tile columns 32 warp ..), all heads, all groups of the split
  float accIH[4][4], accF[4][2];         // [n-tile of the block][head g8: plain cols 2 c4, +1 | H32 cols]; whole-head class
#pragma unroll
  for (int i = 0; i < 4; ++i) { accIH[i][0] = accIH[i][1] = accIH[i][2] = accIH[i][3] = 0.f; accF[i][0] = accF[i][1] = 0.f; }
  float zI = 0.f, zH = 0.f, zF = 0.f;    // p * min sums of block `warp`, head g8 (this lane's tokens)
  float m_run = KV_NEG_INF, l_run = 0.f; // m_run: the CTA's running maximum of head g8 (identical in every warp)
  bool sawF = false;

  const int nsteps = (gend - gfirst + 3) / 4;
  if (gfirst + warp < gend) load_group(gfirst + warp, 0);
  for (int it = 0; it < nsteps; ++it) {
    const int buf = it & 1;
    const int g32 = gfirst + 4 * it + warp;
    const bool have = g32 < gend;
    if (g32 + 4 < gend) { load_group(g32 + 4, buf ^ 1); cp_wait<1>(); } else { cp_wait<0>(); }
    __syncwarp();
    const uint32_t rA = wraw + buf * RAW_GROUP, rB = rA + RAW_PAGE;
    const uint32_t wvt = wraw + 2 * RAW_GROUP;
    const int base = g32 * GRP;
    float s[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
    float mx = KV_NEG_INF;
    bool anyF = false;
    if (have) {
      // ---- group flags
      uint32_t lmask = 0;
      bool useF;
      if (F8) {                                      // sign of slot 0 of cells 0 .. 3 | of cell 4
        const uint4 m0 = lds128(rA + L::KM), m1 = lds128(rA + L::KM + 16);
        lmask = ((m0.x >> 7) & 1u) | (((m0.z >> 7) & 1u) << 1) | (((m1.x >> 7) & 1u) << 2) | (((m1.z >> 7) & 1u) << 3);
        useF = ((lds32(rA + L::KM + 32) >> 7) & 1u) != 0;
      } else {
        const uint4 m0 = lds128(rA + L::KM);
        lmask = ((m0.x >> 15) & 1u) | (((m0.y >> 15) & 1u) << 1) | (((m0.z >> 15) & 1u) << 2) | (((m0.w >> 15) & 1u) << 3);
        useF = ((lds32(rA + L::KM + 16) >> 15) & 1u) != 0;
      }
      // ---- A fragments of QK: lane (head g8, c4) holds channels 16 kk + 2 c4 + {0, 1, 8, 9}
      uint32_t qa[8][2];
      float bias = 0.f, bias8 = 0.f;                 // bias8: the terms of channels 8 - 15 of every 16 (q there is 2^-8 small)
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const int which = useF ? 2 : static_cast<int>((lmask >> (kk >> 1)) & 1u);
        const int c0 = 16 * kk + 2 * c4;
        const uint32_t mp = (kk < 4 ? rA : rB) + L::KM + ((4 * kk + (c4 >> 1)) & 15) * L::MCELL + (L::MCELL / 2) * (c4 & 1);
        float2 a0, a1, b0, b1;                                                 // (scale | flag, min) of channels c0, c0 + 1 | c0 + 8, c0 + 9
        if (F8) {
          const uint32_t wa = lds32(mp), wb = lds32(mp + 2 * L::MCELL);
          a0 = e4m3x2_val(static_cast<uint16_t>(wa & 0xFF7Fu)); a1 = e4m3x2_val(static_cast<uint16_t>((wa >> 16) & 0xFF7Fu));
          b0 = e4m3x2_val(static_cast<uint16_t>(wb & 0xFF7Fu)); b1 = e4m3x2_val(static_cast<uint16_t>((wb >> 16) & 0xFF7Fu));
        } else {
          const uint2 ma = lds64(mp), mb = lds64(mp + 2 * L::MCELL);
          a0 = unpack_h2(ma.x); a1 = unpack_h2(ma.y); b0 = unpack_h2(mb.x); b1 = unpack_h2(mb.y);
        }
        const uint2 qx = lds64(qbs + ((which * 8 + g8) * QSTR + c0) * 4), qy = lds64(qbs + ((which * 8 + g8) * QSTR + c0 + 8) * 4);
        const float q0 = __uint_as_float(qx.x), q1 = __uint_as_float(qx.y), q2 = __uint_as_float(qy.x), q3 = __uint_as_float(qy.y);
        qa[kk][0] = pack_h2(q0 * fabsf(a0.x), q1 * fabsf(a1.x));      // q is stored times qscale * 16 | qscale / 16
        qa[kk][1] = pack_h2(q2 * fabsf(b0.x), q3 * fabsf(b1.x));
        bias = fmaf(q0, a0.y, fmaf(q1, a1.y, bias));
        bias8 = fmaf(q2, b0.y, fmaf(q3, b1.y, bias8));
      }
      bias = fmaf(bias8, 256.f, bias);
      bias += __shfl_xor_sync(FULLMASK, bias, 1);
      bias += __shfl_xor_sync(FULLMASK, bias, 2);
      bias *= 1.f / 16.f;
      // ---- QK: B = key codes of token 8 nt + g8, word kk rotated right by 2 c4: the pair (2 c4, 2 c4 + 1) then sits in
      // mantissa bits 0 - 1 of the two halves (code * 2^-24), the pair (2 c4 + 8, 2 c4 + 9) in bits 8 - 9 (code * 2^-16): two
      // masks, no further shifts; the 2^8 between them is in the q table, the common 2^20 in the score epilogue
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const uint32_t kp = (nt < 2 ? rA : rB) + ((8 * nt + g8) & 15) * 32;
        const uint4 w0 = lds128(kp), w1 = lds128(kp + 16);
        const uint32_t wd[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t r = __funnelshift_r(wd[kk], wd[kk], 2 * c4);
          mma(s[nt], qa[kk][0], 0u, qa[kk][1], 0u, r & 0x00030003u, r & 0x03000300u);
        }
      }
      // ---- scores of head g8 (this lane: tokens 8 nt + 2 c4 + e), the group's maximum
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int pos = base + 8 * nt + 2 * c4 + e;
          const float v = (pos >= t0 && pos < t1) ? fmaf(s[nt][e], 1048576.f, bias) : KV_NEG_INF;
          s[nt][e] = v;
          mx = fmaxf(mx, v);
        }
      mx = fmaxf(mx, __shfl_xor_sync(FULLMASK, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(FULLMASK, mx, 2));
      // ---- value tile: lane = token; word w -> pairs (i, i + 8) of its 16 channels.  The code stays where it is in the word
      // (fields 0 - 4) or where one shift by 10 puts it (fields 5 - 7): mantissa bits 2 i' .. 2 i' + 1, i' = i mod 5, i.e.
      // code * 2^(2 i' - 24); the power of two of a tile column is taken out once, in the epilogue
      {
        const uint32_t vp = (lane < 16 ? rA : rB) + L::VC + (lane & 15) * 32;
        const uint4 w0 = lds128(vp), w1 = lds128(vp + 16);
        const uint32_t wd[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int w = 0; w < 8; ++w) {
          uint32_t o[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = i < 5 ? (wd[w] & (0x00030003u << (2 * i))) : ((wd[w] >> 10) & (0x00030003u << (2 * (i - 5))));
          sts128(wvt + lane * VT_STRIDE + 32 * w, o[0], o[1], o[2], o[3]);
          sts128(wvt + lane * VT_STRIDE + 32 * w + 16, o[4], o[5], o[6], o[7]);
        }
      }
      // ---- value scales, once per token (lane = token).  Table [block][token]: plain scale, H32 scale, plain min, H32 min
      // (16 bytes), then [block][token]: whole-head scale, min (8 bytes); it goes over the group's consumed raw pages
      {
        const uint32_t pg = lane < 16 ? rA : rB;
        float2 smj[4];                              // (scale, min) of the token's four blocks
        uint32_t hbits = 0;                         // bit j: block j is stored as H32 x
        bool fF;
        if (F8) {
          const uint2 vm = lds64(pg + L::VM + (lane & 15) * L::MCELL);
          const uint32_t pr[4] = {vm.x & 0xFFFFu, vm.x >> 16, vm.y & 0xFFFFu, vm.y >> 16};
#pragma unroll
          for (int j = 0; j < 4; ++j) { smj[j] = e4m3x2_val(static_cast<uint16_t>(pr[j] & 0xFF7Fu)); hbits |= ((pr[j] >> 7) & 1u) << j; }
          fF = ((lds32(pg + L::KM + (lane & 15) * L::MCELL + 4) >> 23) & 1u) != 0u;    // bit 7 of the cell's slot-3 key scale
        } else {
          const uint4 vm = lds128(pg + L::VM + (lane & 15) * L::MCELL);
          const uint32_t wv[4] = {vm.x, vm.y, vm.z, vm.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) { smj[j] = unpack_h2(wv[j]); hbits |= ((wv[j] >> 15) & 1u) << j; }
          fF = ((lds32(pg + L::VF + (lane & 12)) >> (8 * (lane & 3))) & 0xFFu) != 0u;
        }
        anyF = __any_sync(FULLMASK, fF);
        __syncwarp();                               // every lane has read what it needs of the raw pages
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 sm = smj[j];
          const float sc = fabsf(sm.x) * 16.f;
          const bool fH = !fF && ((hbits >> j) & 1u), fI = !fF && !fH;
          sts128(rA + (j * 32 + lane) * 16, __float_as_uint(fI ? sc : 0.f), __float_as_uint(fH ? sc : 0.f),
                 __float_as_uint(fI ? sm.y : 0.f), __float_as_uint(fH ? sm.y : 0.f));
          asm volatile("st.shared.v2.u32 [%0], {%1,%2};\n" ::"r"(rA + 2048 + (j * 32 + lane) * 8), "r"(__float_as_uint(fF ? sc : 0.f)),
                       "r"(__float_as_uint(fF ? sm.y : 0.f))
                       : "memory");
        }
      }
    }
    if (c4 == 0) gmax[warp * 8 + g8] = mx;
    if (lane == 0) gflag[warp] = (have ? 1 : 0) | (anyF ? 2 : 0);
    __syncthreads();                                // (1) the four group maxima, value tiles and scale tables are in place
    // ---- one running maximum per head for the whole CTA; p of the own group goes to shared memory
    {
      const float gm = fmaxf(fmaxf(gmax[g8], gmax[8 + g8]), fmaxf(gmax[16 + g8], gmax[24 + g8]));
      const float mnew = fmaxf(m_run, gm);
      const float mb_ = mnew == KV_NEG_INF ? 0.f : mnew;
      const float alpha = m_run == KV_NEG_INF ? 0.f : ex2(m_run - mb_);
      m_run = mnew;
      float psum = 0.f;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const float p0 = have ? ex2(s[nt][0] - mb_) : 0.f, p1 = have ? ex2(s[nt][1] - mb_) : 0.f;
        psum += p0 + p1;
        asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(pbuf + ((warp * 8 + g8) * P_HSTR + 8 * nt + 2 * c4) * 2), "r"(pack_h2(p0, p1))
                     : "memory");
      }
      l_run = l_run * alpha + psum;
      if (alpha != 1.f) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          accIH[i][0] *= alpha; accIH[i][1] *= alpha; accIH[i][2] *= alpha; accIH[i][3] *= alpha;
          accF[i][0] *= alpha; accF[i][1] *= alpha;
        }
        zI *= alpha; zH *= alpha; zF *= alpha;
      }
    }
    __syncthreads();                                // (2) p of the four groups is in place
    // ---- PV of channel block `warp` over the step's groups: A = p * scale of this lane's tokens by class, B = the value tile
#pragma unroll 1
    for (int gq = 0; gq < 4; ++gq) {
      const int fl = gflag[gq];
      if (!(fl & 1)) continue;
      const bool gF = (fl & 2) != 0;
      sawF |= gF;
      const uint32_t gbase = sb + QB_BYTES + gq * WARP_SMEM;
      const uint32_t tab = gbase + buf * RAW_GROUP, tile = gbase + 2 * RAW_GROUP;
      uint32_t aI[2][2], aH[2][2], aF[2][2];          // [k-step][token pair 2 c4 | 8 + 2 c4]
#pragma unroll
      for (int kk = 0; kk < 2; ++kk)
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const int tk = 16 * kk + 8 * hf + 2 * c4;
          const float2 pp = unpack_h2(lds32(pbuf + ((gq * 8 + g8) * P_HSTR + tk) * 2));
          const float p0 = pp.x, p1 = pp.y;
          const uint4 x0 = lds128(tab + (warp * 32 + tk) * 16), x1 = lds128(tab + (warp * 32 + tk + 1) * 16);
          aI[kk][hf] = pack_h2(p0 * __uint_as_float(x0.x), p1 * __uint_as_float(x1.x));
          aH[kk][hf] = pack_h2(p0 * __uint_as_float(x0.y), p1 * __uint_as_float(x1.y));
          zI = fmaf(p0, __uint_as_float(x0.z), fmaf(p1, __uint_as_float(x1.z), zI));
          zH = fmaf(p0, __uint_as_float(x0.w), fmaf(p1, __uint_as_float(x1.w), zH));
          aF[kk][hf] = 0u;
          if (gF) {
            const uint4 y = lds128(tab + 2048 + (warp * 32 + tk) * 8);      // (scale, min) of tokens tk, tk + 1
            aF[kk][hf] = pack_h2(p0 * __uint_as_float(y.x), p1 * __uint_as_float(y.z));
            zF = fmaf(p0, __uint_as_float(y.y), fmaf(p1, __uint_as_float(y.w), zF));
          }
        }
#pragma unroll
      for (int kk = 0; kk < 2; ++kk)
#pragma unroll
        for (int np = 0; np < 2; ++np) {               // two n-tiles per ldmatrix
          uint32_t b0, b1, b2, b3;
          ldsm_x4_t(tile + (16 * kk + (lane & 7) + 8 * ((lane >> 3) & 1)) * VT_STRIDE + (32 * warp + 16 * np + 8 * (lane >> 4)) * 2, b0, b1,
                    b2, b3);
          mma(accIH[2 * np], aI[kk][0], aH[kk][0], aI[kk][1], aH[kk][1], b0, b1);
          mma(accIH[2 * np + 1], aI[kk][0], aH[kk][0], aI[kk][1], aH[kk][1], b2, b3);
          if (gF) {
            float t0_[4] = {accF[2 * np][0], accF[2 * np][1], 0.f, 0.f}, t1_[4] = {accF[2 * np + 1][0], accF[2 * np + 1][1], 0.f, 0.f};
            mma(t0_, aF[kk][0], 0u, aF[kk][1], 0u, b0, b1);
            mma(t1_, aF[kk][0], 0u, aF[kk][1], 0u, b2, b3);
            accF[2 * np][0] = t0_[0]; accF[2 * np][1] = t0_[1]; accF[2 * np + 1][0] = t1_[0]; accF[2 * np + 1][1] = t1_[1];
          }
        }
    }
    __syncthreads();                                // (3) tiles, tables and p may be overwritten by the next step
  }

  // ---- the CTA's result: every warp holds its channel block; sums of this lane's tokens go over the four c4 lanes
  float* red = reinterpret_cast<float*>(smraw);        // [4 warps][8 heads] m (all warps hold the same value) | then arrays
  float* accs = red + 64;                              // [3 classes][8 heads][128 channels]
  float* zs = accs + 3 * 8 * D;                        // [3][8][4]
  float* ls = zs + 96;                                 // [8]
  l_run += __shfl_xor_sync(FULLMASK, l_run, 1);
  l_run += __shfl_xor_sync(FULLMASK, l_run, 2);
  zI += __shfl_xor_sync(FULLMASK, zI, 1); zI += __shfl_xor_sync(FULLMASK, zI, 2);
  zH += __shfl_xor_sync(FULLMASK, zH, 1); zH += __shfl_xor_sync(FULLMASK, zH, 2);
  zF += __shfl_xor_sync(FULLMASK, zF, 1); zF += __shfl_xor_sync(FULLMASK, zF, 2);
  if (tid < 8) ls[tid] = 0.f;                          // (the step loop ended with a barrier: the q bases are no longer needed)
  if (c4 == 0) red[warp * 8 + g8] = m_run;
  __syncthreads();
  // tile column 16 w + 2 i + e is channel 16 w + i + 8 e; this lane holds columns 32 warp + 8 nt + 2 c4 + e of n-tile nt
#pragma unroll
  for (int nt = 0; nt < 4; ++nt)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int col = 32 * warp + 8 * nt + 2 * c4 + e;
      const int ch = (col & ~15) + ((col & 15) >> 1) + 8 * (col & 1);
      const int fi = (col & 15) >> 1;                      // field of the column's channel pair: code * 2^(2 (fi mod 5) - 24)
      const float cf = __int_as_float((127 + 8 - 2 * (fi < 5 ? fi : fi - 5)) << 23);   // relative to the 2^-16 the rest assumes
      accs[(0 * 8 + g8) * D + ch] = accIH[nt][e] * cf;
      accs[(1 * 8 + g8) * D + ch] = accIH[nt][2 + e] * cf;
      accs[(2 * 8 + g8) * D + ch] = sawF ? accF[nt][e] * cf : 0.f;
    }
  if (c4 == 0) {
    zs[(0 * 8 + g8) * 4 + warp] = zI;
    zs[(1 * 8 + g8) * 4 + warp] = zH;
    zs[(2 * 8 + g8) * 4 + warp] = zF;
    atomicAdd(&ls[g8], l_run);
  }
  __syncthreads();
  // ---- thread = channel: add the min terms, rotate the two rotated classes back (as k_kv_attn does), store
  {
    const int c = tid, blk = c >> 5;
    float oI[8], oH[8];
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      oI[g] = accs[(0 * 8 + g) * D + c] * 4096.f + zs[(0 * 8 + g) * 4 + blk];
      oH[g] = accs[(1 * 8 + g) * D + c] * 4096.f + zs[(1 * 8 + g) * 4 + blk];
    }
    float oF[8];
#pragma unroll
    for (int g = 0; g < 8; ++g) oF[g] = accs[(2 * 8 + g) * D + c] * 4096.f + zs[(2 * 8 + g) * 4 + blk];
    const float lsum[8] = {ls[0], ls[1], ls[2], ls[3], ls[4], ls[5], ls[6], ls[7]};
    const float mfin[8] = {red[0], red[1], red[2], red[3], red[4], red[5], red[6], red[7]};
    __syncthreads();
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      float v = oH[g];                                    // channel c: lane = c % 32 -> H32 over the block by shuffles
#pragma unroll
      for (int hh = 1; hh < 32; hh <<= 1) {
        const float o = __shfl_xor_sync(FULLMASK, v, hh);
        v = (lane & hh) ? __fsub_rn(o, v) : __fadd_rn(v, o);
      }
      oI[g] = __fadd_rn(oI[g], __fmul_rn(v, fr::C32));
      qb[2][g][c] = oF[g];
    }
    __syncthreads();
    smem_hada<8>(qb[2], 128);
#pragma unroll
    for (int g = 0; g < G; ++g) op[g * D + c] = __fadd_rn(oI[g], qb[2][g][c]);
    if (tid < G) { mlp[2 * tid] = mfin[tid]; mlp[2 * tid + 1] = lsum[tid]; }
  }
}

}  // namespace kvm
