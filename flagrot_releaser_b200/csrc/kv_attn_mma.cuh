// KIVI paged decode attention on the tensor cores (mma.sync m16n8k16 FP16, fp32 accumulation) for GQA groups of up to 8 q
// heads.  Included by kv_capi.cu inside its anonymous namespace; replaces the body CTAs of k_kv_attn (the BF16 sink /
// window CTA stays there) and the reference kernel k_attn (integrations/vllm_flagrot/csrc/kivi.cu).
//
// CTA = (kv head, split, row), 4 warps; warp w owns the 32-token key groups w, w + 4, ... of the split with its own
// running (m, l) and accumulators (merged once at the end), so there is no CTA barrier inside the loop.  Per group:
//   * the two page chunks (2 x 1 552 B) arrive by cp.async into the warp's double buffer;
//   * QK: A = q' * scale of the group's channels (q' = q in the base the group's flags name: identity / H32 per 32-channel
//     block / H128), built in registers per lane directly as the A fragment (rows = q heads, rows 8 - 15 zero); B = the 2-bit
//     key codes read in place: the stored word holds channel pairs (2 m, 2 m + 1) at bits (2 m, 2 m + 16), i.e. one
//     shift + mask per B register.  The code lands in mantissa bits 8 - 9 of an FP16 subnormal (code * 2^-16, exact); the
//     2^16 is split between the A operand (2^4) and the fp32 epilogue (2^12).  The q' . min term is a per-head scalar;
//   * softmax per warp in registers (the C fragment rows are the q heads);
//   * PV: the value codes of the 32 tokens are expanded to the same FP16 form into the warp's [32][128] tile (channel
//     pairs (i, i + 8) of every 16-channel word share a register, so the tile's columns are a fixed permutation of the
//     channels) and read back with ldmatrix.trans as B; A = p * value scale per (token, 32-channel block), rows 0 - 7 for
//     tokens / blocks stored plain, rows 8 - 15 for those stored as H32 (the sign of the scale), a second MMA with the
//     whole-head (H128) tokens only when the group has one (the 2^16 of the codes is again split 2^4 / 2^12).  The p * min terms are per (head, block, class) scalars;
//   * epilogue: warps merge in shared memory, columns are un-permuted, the two rotated classes are rotated back once.
#pragma once

namespace kvm {

constexpr int RAW_PAGE = 1568;                 // 1552 rounded to 32
constexpr int RAW_GROUP = 2 * RAW_PAGE;
constexpr int VT_STRIDE = 272;                 // bytes per token row of the FP16 value tile (256 + 16)
constexpr int VM_TAB = 4 * 32 * 24;             // per (block, token): plain / H32 scale * 16 and min (16 B), whole-head scale and min (8 B)
constexpr int WARP_SMEM = 2 * RAW_GROUP + 32 * VT_STRIDE;     // 14 976 (the scale table reuses the group's consumed raw pages)
static_assert(VM_TAB <= RAW_GROUP, "the scale table fits in a raw group buffer");
constexpr int QSTR = 136;                      // floats per q row (128 + 8: the eight head rows spread over the banks)
constexpr int QB_BYTES = 3 * 8 * QSTR * 4;     // q * qscale * 16 in three bases, fp32 [3][8][136]
constexpr int SMEM = QB_BYTES + 4 * WARP_SMEM; // 72 960: three CTAs per SM

FR_DEVI uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
FR_DEVI void cp16(uint32_t dst, const void* src) { asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory"); }
FR_DEVI void cp_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> FR_DEVI void cp_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }
FR_DEVI uint32_t lds32(uint32_t a) { uint32_t v; asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(a)); return v; }
FR_DEVI uint2 lds64(uint32_t a) { uint2 v; asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "r"(a)); return v; }
FR_DEVI uint4 lds128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
FR_DEVI void sts128(uint32_t a, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(a), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
FR_DEVI void ldsm_x4_t(uint32_t a, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
FR_DEVI void mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
FR_DEVI uint32_t pack_h2(float a, float b) {
  const __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}
FR_DEVI float2 unpack_h2(uint32_t v) { return __half22float2(*reinterpret_cast<const __half2*>(&v)); }
FR_DEVI float ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x)); return y; }

#ifndef KVM_MINB
#define KVM_MINB 2
#endif
template <int G>
FR_DEVI void kv_tail_mma(uint8_t* smraw, int h, int b, const __nv_bfloat16* __restrict__ q, long long q_rs, int Hkv, int NS, float qscale,
                         const __nv_bfloat16* __restrict__ ring, const int* __restrict__ tail_len,
                         const int* __restrict__ tail_idx, int T, float* __restrict__ opart, float* __restrict__ ml);

// grid (Hkv, NS, 2 B): z < B are the page splits; z >= B (y == 0 only) are the BF16 sink / window splits, dispatched last so
// that they fill the final, partly empty wave of the page splits
template <int G>
__global__ void __launch_bounds__(128, KVM_MINB) k_kv_attn_mma(const __nv_bfloat16* __restrict__ q, long long q_rs,
                                                        const uint8_t* __restrict__ pool, const int* __restrict__ bt, long long bt_rs,
                                                        const int* __restrict__ cached, int kv_start, int Hkv, int NS, int chunk,
                                                        float qscale, const __nv_bfloat16* __restrict__ ring,
                                                        const int* __restrict__ tail_len, const int* __restrict__ tail_idx, int T,
                                                        int B, float* __restrict__ opart, float* __restrict__ ml) {
  static_assert(G <= 8, "one M tile of q heads");
  extern __shared__ __align__(16) uint8_t smraw[];
  if (static_cast<int>(blockIdx.z) >= B) {
    if (blockIdx.y == 0) kv_tail_mma<G>(smraw, blockIdx.x, static_cast<int>(blockIdx.z) - B, q, q_rs, Hkv, NS, qscale, ring, tail_len,
                                        tail_idx, T, opart, ml);
    return;
  }
  float (*qb)[8][D] = reinterpret_cast<float (*)[8][D]>(smraw);
  const int h = blockIdx.x, sp = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g8 = lane >> 2, c4 = lane & 3;
  const long long pidx = static_cast<long long>(b * Hkv + h) * (NS + 1) + sp;
  float* op = opart + pidx * G * D;
  float* mlp = ml + pidx * G * 2;
  const int t0 = max(sp * chunk, kv_start), t1 = min((sp + 1) * chunk, cached[b]);
  if (t1 <= t0) {
    for (int e = tid; e < G; e += 128) { mlp[2 * e] = KV_NEG_INF; mlp[2 * e + 1] = 0.f; }
    return;
  }
  // ---- q in three bases (rows >= G are zero)
  {
    const __nv_bfloat16* qp = q + static_cast<long long>(b) * q_rs + static_cast<long long>(h) * G * D;
    for (int e = tid; e < 8 * D; e += 128) {
      const float v = e < G * D ? __bfloat162float(qp[e]) : 0.f;
      qb[0][e / D][e % D] = v; qb[1][e / D][e % D] = v; qb[2][e / D][e % D] = v;
    }
    __syncthreads();
    smem_hada<8>(qb[1], 32);
    smem_hada<8>(qb[2], 128);
    // re-lay the rows with a padded stride (back to front: the padded table is longer than the dense one)
    float v[24];
#pragma unroll
    for (int i = 0; i < 24; ++i) v[i] = reinterpret_cast<float*>(smraw)[tid + 128 * i];
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 24; ++i) {
      const int e = tid + 128 * i;
      reinterpret_cast<float*>(smraw)[(e / D) * QSTR + e % D] = v[i] * (qscale * 16.f);
    }
    __syncthreads();
  }
  const uint32_t sb = smem_u32(smraw);
  const uint32_t wraw = sb + QB_BYTES + warp * WARP_SMEM, wvt = wraw + 2 * RAW_GROUP;
  const uint32_t qbs = sb;
  const int* btb = bt + static_cast<long long>(b) * bt_rs;
  const int gfirst = t0 / GRP, gend = (t1 + GRP - 1) / GRP;
  auto load_group = [&](int g32, int buf) {
    const uint8_t* chA = pool + (static_cast<long long>(btb[2 * g32]) * Hkv + h) * CB;
    const uint8_t* chB = pool + (static_cast<long long>(btb[2 * g32 + 1]) * Hkv + h) * CB;
    const uint32_t dst = wraw + buf * RAW_GROUP;
    for (int i = lane; i < CB / 16; i += 32) {
      cp16(dst + 16 * i, chA + 16 * i);
      cp16(dst + RAW_PAGE + 16 * i, chB + 16 * i);
    }
    cp_commit();
  };

  float accIH[16][4], accF[16][2];       // O fragments: [n-tile][head g8: plain cols 2 c4, +1 | H32 cols]; whole-head class
#pragma unroll
  for (int i = 0; i < 16; ++i) { accIH[i][0] = accIH[i][1] = accIH[i][2] = accIH[i][3] = 0.f; accF[i][0] = accF[i][1] = 0.f; }
  float zI[4] = {0.f, 0.f, 0.f, 0.f}, zH[4] = {0.f, 0.f, 0.f, 0.f}, zF[4] = {0.f, 0.f, 0.f, 0.f};
  float m_run = KV_NEG_INF, l_run = 0.f;
  bool sawF = false;                      // a whole-head token occurred in one of this warp's groups

  int g32 = gfirst + warp;
  if (g32 < gend) load_group(g32, 0);
  for (int it = 0; g32 < gend; g32 += 4, ++it) {
    const int buf = it & 1;
    if (g32 + 4 < gend) { load_group(g32 + 4, buf ^ 1); cp_wait<1>(); } else { cp_wait<0>(); }
    __syncwarp();
    const uint32_t rA = wraw + buf * RAW_GROUP, rB = rA + RAW_PAGE;
    const int base = g32 * GRP;
    // ---- group flags
    uint32_t lmask = 0;
    {
      const uint4 m0 = lds128(rA + OFF_KM);
      lmask = ((m0.x >> 15) & 1u) | (((m0.y >> 15) & 1u) << 1) | (((m0.z >> 15) & 1u) << 2) | (((m0.w >> 15) & 1u) << 3);
    }
    const bool useF = ((lds32(rA + OFF_KM + 16) >> 15) & 1u) != 0;
    // ---- A fragments of QK: lane (head g8, c4) holds channels 16 kk + 2 c4 + {0, 1, 8, 9}
    uint32_t qa[8][2];
    float bias = 0.f;
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      const int which = useF ? 2 : static_cast<int>((lmask >> (kk >> 1)) & 1u);
      const int c0 = 16 * kk + 2 * c4;
      const uint32_t mp = (kk < 4 ? rA : rB) + OFF_KM + ((4 * kk + (c4 >> 1)) & 15) * 16 + 8 * (c4 & 1);
      const uint2 ma = lds64(mp), mb = lds64(mp + 32);                       // channels c0, c0 + 1 | c0 + 8, c0 + 9
      const uint2 qx = lds64(qbs + ((which * 8 + g8) * QSTR + c0) * 4), qy = lds64(qbs + ((which * 8 + g8) * QSTR + c0 + 8) * 4);
      const float2 a0 = unpack_h2(ma.x), a1 = unpack_h2(ma.y), b0 = unpack_h2(mb.x), b1 = unpack_h2(mb.y);   // (scale | flag, min)
      const float q0 = __uint_as_float(qx.x), q1 = __uint_as_float(qx.y), q2 = __uint_as_float(qy.x), q3 = __uint_as_float(qy.y);
      qa[kk][0] = pack_h2(q0 * fabsf(a0.x), q1 * fabsf(a1.x));      // q is stored times qscale * 16
      qa[kk][1] = pack_h2(q2 * fabsf(b0.x), q3 * fabsf(b1.x));
      bias = fmaf(q0, a0.y, fmaf(q1, a1.y, fmaf(q2, b0.y, fmaf(q3, b1.y, bias))));
    }
    bias += __shfl_xor_sync(FULLMASK, bias, 1);
    bias += __shfl_xor_sync(FULLMASK, bias, 2);
    bias *= 1.f / 16.f;
    // ---- QK: B = key codes of token 8 nt + g8, word kk: pairs (2 c4, 2 c4 + 1) and (2 c4 + 8, 2 c4 + 9) of the word
    float s[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
      const uint32_t kp = (nt < 2 ? rA : rB) + ((8 * nt + g8) & 15) * 32;
      const uint4 w0 = lds128(kp), w1 = lds128(kp + 16);
      const uint32_t wd[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)
        mma(s[nt], qa[kk][0], 0u, qa[kk][1], 0u, (wd[kk] << (8 - 2 * c4)) & 0x03000300u, (wd[kk] >> (2 * c4)) & 0x03000300u);
    }
    // ---- softmax of head g8 over the group's 32 tokens (this lane: tokens 8 nt + 2 c4 + e)
    float mx = KV_NEG_INF;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int pos = base + 8 * nt + 2 * c4 + e;
        const float v = (pos >= t0 && pos < t1) ? fmaf(s[nt][e], 4096.f, bias) : KV_NEG_INF;
        s[nt][e] = v;
        mx = fmaxf(mx, v);
      }
    mx = fmaxf(mx, __shfl_xor_sync(FULLMASK, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(FULLMASK, mx, 2));
    const float mnew = fmaxf(m_run, mx);
    const float mb_ = mnew == KV_NEG_INF ? 0.f : mnew;
    const float alpha = m_run == KV_NEG_INF ? 0.f : ex2(m_run - mb_);
    m_run = mnew;
    float psum = 0.f;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e) { s[nt][e] = ex2(s[nt][e] - mb_); psum += s[nt][e]; }
    l_run = l_run * alpha + psum;
    if (alpha != 1.f) {
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        accIH[i][0] *= alpha; accIH[i][1] *= alpha; accIH[i][2] *= alpha; accIH[i][3] *= alpha;
        accF[i][0] *= alpha; accF[i][1] *= alpha;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) { zI[j] *= alpha; zH[j] *= alpha; zF[j] *= alpha; }
    }
    // ---- value tile: lane = token; word w -> pairs (i, i + 8) of its 16 channels, code in mantissa bits 8 - 9
    {
      const uint32_t vp = (lane < 16 ? rA : rB) + OFF_VC + (lane & 15) * 32;
      const uint4 w0 = lds128(vp), w1 = lds128(vp + 16);
      const uint32_t wd[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
      for (int w = 0; w < 8; ++w) {
        uint32_t o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = (2 * i <= 8 ? (wd[w] << (8 - 2 * i)) : (wd[w] >> (2 * i - 8))) & 0x03000300u;
        sts128(wvt + lane * VT_STRIDE + 32 * w, o[0], o[1], o[2], o[3]);
        sts128(wvt + lane * VT_STRIDE + 32 * w + 16, o[4], o[5], o[6], o[7]);
      }
    }
    __syncwarp();
    // ---- value scales, once per token (lane = token): per 32-channel block (scale * 16, min) go to the slot of the class
    // the (token, block) is stored in (plain / H32 / whole head), zeros to the others.  Table [block][token]: plain scale,
    // H32 scale, plain min, H32 min (16 bytes), then [block][token]: whole-head scale, min (8 bytes)
    bool anyF;
    const uint32_t wtab = rA;
    {
      const uint32_t pg = lane < 16 ? rA : rB;
      const uint4 vm = lds128(pg + OFF_VM + (lane & 15) * 16);
      const bool fF = ((lds32(pg + OFF_VF + (lane & 12)) >> (8 * (lane & 3))) & 0xFFu) != 0u;
      anyF = __any_sync(FULLMASK, fF);
      sawF |= anyF;
      const uint32_t wv[4] = {vm.x, vm.y, vm.z, vm.w};
      __syncwarp();                               // every lane has read what it needs of the raw pages: the table goes over them
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 sm = unpack_h2(wv[j]);
        const float sc = fabsf(sm.x) * 16.f;
        const bool fH = !fF && signbit(sm.x), fI = !fF && !fH;
        sts128(wtab + (j * 32 + lane) * 16, __float_as_uint(fI ? sc : 0.f), __float_as_uint(fH ? sc : 0.f),
               __float_as_uint(fI ? sm.y : 0.f), __float_as_uint(fH ? sm.y : 0.f));
        asm volatile("st.shared.v2.u32 [%0], {%1,%2};\n" ::"r"(wtab + 2048 + (j * 32 + lane) * 8), "r"(__float_as_uint(fF ? sc : 0.f)),
                     "r"(__float_as_uint(fF ? sm.y : 0.f))
                     : "memory");
      }
    }
    __syncwarp();
    // ---- PV per 32-channel block: A = p * scale of this lane's 8 tokens by class, B = the value tile
#pragma unroll
    for (int blk = 0; blk < 4; ++blk) {
      uint32_t aI[2][2], aH[2][2], aF[2][2];          // [k-step][token pair 2 c4 | 8 + 2 c4]
#pragma unroll
      for (int kk = 0; kk < 2; ++kk)
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const int tk = 16 * kk + 8 * hf + 2 * c4;
          const float p0 = s[2 * kk + hf][0], p1 = s[2 * kk + hf][1];
          const uint4 x0 = lds128(wtab + (blk * 32 + tk) * 16), x1 = lds128(wtab + (blk * 32 + tk + 1) * 16);
          aI[kk][hf] = pack_h2(p0 * __uint_as_float(x0.x), p1 * __uint_as_float(x1.x));
          aH[kk][hf] = pack_h2(p0 * __uint_as_float(x0.y), p1 * __uint_as_float(x1.y));
          zI[blk] = fmaf(p0, __uint_as_float(x0.z), fmaf(p1, __uint_as_float(x1.z), zI[blk]));
          zH[blk] = fmaf(p0, __uint_as_float(x0.w), fmaf(p1, __uint_as_float(x1.w), zH[blk]));
          aF[kk][hf] = 0u;
          if (anyF) {
            const uint4 y = lds128(wtab + 2048 + (blk * 32 + tk) * 8);      // (scale, min) of tokens tk, tk + 1
            aF[kk][hf] = pack_h2(p0 * __uint_as_float(y.x), p1 * __uint_as_float(y.z));
            zF[blk] = fmaf(p0, __uint_as_float(y.y), fmaf(p1, __uint_as_float(y.w), zF[blk]));
          }
        }
#pragma unroll
      for (int kk = 0; kk < 2; ++kk)
#pragma unroll
        for (int np = 0; np < 2; ++np) {               // two n-tiles per ldmatrix
          uint32_t b0, b1, b2, b3;
          ldsm_x4_t(wvt + (16 * kk + (lane & 7) + 8 * ((lane >> 3) & 1)) * VT_STRIDE + (32 * blk + 16 * np + 8 * (lane >> 4)) * 2, b0, b1, b2,
                    b3);
          const int n0 = 4 * blk + 2 * np;
          mma(accIH[n0], aI[kk][0], aH[kk][0], aI[kk][1], aH[kk][1], b0, b1);
          mma(accIH[n0 + 1], aI[kk][0], aH[kk][0], aI[kk][1], aH[kk][1], b2, b3);
          if (anyF) {
            float t0_[4] = {accF[n0][0], accF[n0][1], 0.f, 0.f}, t1_[4] = {accF[n0 + 1][0], accF[n0 + 1][1], 0.f, 0.f};
            mma(t0_, aF[kk][0], 0u, aF[kk][1], 0u, b0, b1);
            mma(t1_, aF[kk][0], 0u, aF[kk][1], 0u, b2, b3);
            accF[n0][0] = t0_[0]; accF[n0][1] = t0_[1]; accF[n0 + 1][0] = t1_[0]; accF[n0 + 1][1] = t1_[1];
          }
        }
    }
    __syncwarp();
  }

  // ---- merge of the four warps: common maximum, then sums of scaled accumulators in shared memory
  __syncthreads();                                     // the q bases and the warp tiles are no longer needed
  float* red = reinterpret_cast<float*>(smraw);        // [4 warps][8 heads] m | then arrays
  float* accs = red + 64;                              // [3 classes][8 heads][128 channels]
  float* zs = accs + 3 * 8 * D;                        // [3][8][4]
  float* ls = zs + 96;                                 // [8]
  l_run += __shfl_xor_sync(FULLMASK, l_run, 1);
  l_run += __shfl_xor_sync(FULLMASK, l_run, 2);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    zI[j] += __shfl_xor_sync(FULLMASK, zI[j], 1); zI[j] += __shfl_xor_sync(FULLMASK, zI[j], 2);
    zH[j] += __shfl_xor_sync(FULLMASK, zH[j], 1); zH[j] += __shfl_xor_sync(FULLMASK, zH[j], 2);
    zF[j] += __shfl_xor_sync(FULLMASK, zF[j], 1); zF[j] += __shfl_xor_sync(FULLMASK, zF[j], 2);
  }
  if (c4 == 0) red[warp * 8 + g8] = m_run;
  for (int e = tid; e < 3 * 8 * D + 96 + 8; e += 128) accs[e] = 0.f;
  __syncthreads();
  const float M = fmaxf(fmaxf(red[g8], red[8 + g8]), fmaxf(red[16 + g8], red[24 + g8]));
  const float wgt = (m_run == KV_NEG_INF || M == KV_NEG_INF) ? 0.f : ex2(m_run - M);
  // tile column 16 w + 2 i + e is channel 16 w + i + 8 e; this lane holds columns 8 nt + 2 c4 + e of n-tile nt
#pragma unroll
  for (int nt = 0; nt < 16; ++nt)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int col = 8 * nt + 2 * c4 + e;
      const int ch = (col & ~15) + ((col & 15) >> 1) + 8 * (col & 1);
      atomicAdd(&accs[(0 * 8 + g8) * D + ch], wgt * accIH[nt][e]);
      atomicAdd(&accs[(1 * 8 + g8) * D + ch], wgt * accIH[nt][2 + e]);
      if (sawF) atomicAdd(&accs[(2 * 8 + g8) * D + ch], wgt * accF[nt][e]);
    }
  if (c4 == 0) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      atomicAdd(&zs[(0 * 8 + g8) * 4 + j], wgt * zI[j]);
      atomicAdd(&zs[(1 * 8 + g8) * 4 + j], wgt * zH[j]);
      atomicAdd(&zs[(2 * 8 + g8) * 4 + j], wgt * zF[j]);
    }
    atomicAdd(&ls[g8], wgt * l_run);
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
    const float mfin[8] = {fmaxf(fmaxf(red[0], red[8]), fmaxf(red[16], red[24])), fmaxf(fmaxf(red[1], red[9]), fmaxf(red[17], red[25])),
                           fmaxf(fmaxf(red[2], red[10]), fmaxf(red[18], red[26])), fmaxf(fmaxf(red[3], red[11]), fmaxf(red[19], red[27])),
                           fmaxf(fmaxf(red[4], red[12]), fmaxf(red[20], red[28])), fmaxf(fmaxf(red[5], red[13]), fmaxf(red[21], red[29])),
                           fmaxf(fmaxf(red[6], red[14]), fmaxf(red[22], red[30])), fmaxf(fmaxf(red[7], red[15]), fmaxf(red[23], red[31]))};
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

// ---- the BF16 sink / window split of a row on the tensor cores (mma.sync m16n8k16 BF16): warp w owns the 16-token slices
// w, w + 4, ... with its own (m, l) and accumulators, the four warps merge in shared memory.  q and K are BF16 already (exact
// products, fp32 sums); p goes in as two BF16 parts (hi + lo).  Writes the partial of split NS in k_kv_attn's format.
FR_DEVI void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
FR_DEVI uint32_t pack_bf2(float a, float b) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}
constexpr int TAIL_VSTR = 272;
constexpr int TAIL_SMEM = 4 * 16 * TAIL_VSTR + 4 * (8 * D + 16) * 4;      // V tiles + per-warp partials

template <int G>
FR_DEVI void kv_tail_mma(uint8_t* smraw, int h, int b, const __nv_bfloat16* __restrict__ q, long long q_rs, int Hkv, int NS, float qscale,
                         const __nv_bfloat16* __restrict__ ring, const int* __restrict__ tail_len,
                         const int* __restrict__ tail_idx, int T, float* __restrict__ opart, float* __restrict__ ml) {
  static_assert(G <= 8, "one M tile of q heads");
  const int tid = threadIdx.x, w = tid >> 5, lane = tid & 31, g8 = lane >> 2, c4 = lane & 3;
  const long long pidx = static_cast<long long>(b * Hkv + h) * (NS + 1) + NS;
  float* op = opart + pidx * G * D;
  float* mlp = ml + pidx * G * 2;
  const int tl = tail_len ? tail_len[b] : 0;
  if (tl <= 0) {
    for (int e = tid; e < G; e += 128) { mlp[2 * e] = KV_NEG_INF; mlp[2 * e + 1] = 0.f; }
    return;
  }
  const uint32_t vt = smem_u32(smraw) + w * 16 * TAIL_VSTR;
  float* part = reinterpret_cast<float*>(smraw + 4 * 16 * TAIL_VSTR) + w * (8 * D + 16);
  uint32_t qa[8][2];
  {
    const __nv_bfloat16* qp = q + static_cast<long long>(b) * q_rs + static_cast<long long>(h) * G * D;
    const bool on = g8 < G;
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      qa[kk][0] = on ? *reinterpret_cast<const uint32_t*>(qp + g8 * D + 16 * kk + 2 * c4) : 0u;
      qa[kk][1] = on ? *reinterpret_cast<const uint32_t*>(qp + g8 * D + 16 * kk + 2 * c4 + 8) : 0u;
    }
  }
  const long long rs = 2LL * Hkv * D;
  const __nv_bfloat16* rbase = ring + static_cast<long long>(tail_idx ? tail_idx[b] : 0) * T * rs;
  const __nv_bfloat16* kbase = rbase + static_cast<long long>(h) * D;
  const __nv_bfloat16* vbase = rbase + static_cast<long long>(Hkv + h) * D;
  float o[16][2];
#pragma unroll
  for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = 0.f;
  float m = KV_NEG_INF, l = 0.f;
  for (int t0 = 16 * w; t0 < tl; t0 += 64) {
    __syncwarp();
    for (int i = lane; i < 256; i += 32) {
      const int r = i >> 4, c16 = i & 15;
      const uint32_t dst = vt + r * TAIL_VSTR + 16 * c16;
      if (t0 + r < tl) cp16(dst, vbase + (t0 + r) * rs + 8 * c16);
      else sts128(dst, 0u, 0u, 0u, 0u);
    }
    cp_commit();
    uint32_t kb[2][8][2];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const int t = t0 + 8 * nt + g8;
      const __nv_bfloat16* kr = kbase + t * rs + 2 * c4;
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        kb[nt][kk][0] = t < tl ? __ldg(reinterpret_cast<const uint32_t*>(kr + 16 * kk)) : 0u;
        kb[nt][kk][1] = t < tl ? __ldg(reinterpret_cast<const uint32_t*>(kr + 16 * kk + 8)) : 0u;
      }
    }
    float s[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) mma_bf16(s[nt], qa[kk][0], 0u, qa[kk][1], 0u, kb[nt][kk][0], kb[nt][kk][1]);
    }
    float mx = KV_NEG_INF;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float v = (t0 + 8 * nt + 2 * c4 + e < tl) ? s[nt][e] * qscale : KV_NEG_INF;
        s[nt][e] = v;
        mx = fmaxf(mx, v);
      }
    mx = fmaxf(mx, __shfl_xor_sync(FULLMASK, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(FULLMASK, mx, 2));
    const float mn = fmaxf(m, mx), base = mn == KV_NEG_INF ? 0.f : mn;
    const float alpha = m == KV_NEG_INF ? 0.f : ex2(m - base);
    m = mn;
    float ps = 0.f;
    uint32_t ph[2], pl[2];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const float p0 = ex2(s[nt][0] - base), p1 = ex2(s[nt][1] - base);
      ps += p0 + p1;
      ph[nt] = pack_bf2(p0, p1);
      pl[nt] = pack_bf2(p0 - fr::bf16_lo(ph[nt]), p1 - fr::bf16_hi(ph[nt]));
    }
    l = l * alpha + ps;
#pragma unroll
    for (int i = 0; i < 16; ++i) { o[i][0] *= alpha; o[i][1] *= alpha; }
    cp_wait<0>();
    __syncwarp();
#pragma unroll
    for (int np = 0; np < 8; ++np) {
      uint32_t b0, b1, b2, b3;
      ldsm_x4_t(vt + ((lane & 7) + 8 * ((lane >> 3) & 1)) * TAIL_VSTR + (16 * np + 8 * (lane >> 4)) * 2, b0, b1, b2, b3);
      float c0[4] = {o[2 * np][0], o[2 * np][1], 0.f, 0.f}, c1[4] = {o[2 * np + 1][0], o[2 * np + 1][1], 0.f, 0.f};
      mma_bf16(c0, ph[0], 0u, ph[1], 0u, b0, b1);
      mma_bf16(c0, pl[0], 0u, pl[1], 0u, b0, b1);
      mma_bf16(c1, ph[0], 0u, ph[1], 0u, b2, b3);
      mma_bf16(c1, pl[0], 0u, pl[1], 0u, b2, b3);
      o[2 * np][0] = c0[0]; o[2 * np][1] = c0[1]; o[2 * np + 1][0] = c1[0]; o[2 * np + 1][1] = c1[1];
    }
  }
  l += __shfl_xor_sync(FULLMASK, l, 1);
  l += __shfl_xor_sync(FULLMASK, l, 2);
#pragma unroll
  for (int nt = 0; nt < 16; ++nt) *reinterpret_cast<float2*>(part + g8 * D + 8 * nt + 2 * c4) = make_float2(o[nt][0], o[nt][1]);
  if (c4 == 0) { part[8 * D + g8] = m; part[8 * D + 8 + g8] = l; }
  __syncthreads();
  // thread = channel: merge the four warps
  const float* p0 = reinterpret_cast<const float*>(smraw + 4 * 16 * TAIL_VSTR);
  constexpr int PS = 8 * D + 16;
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const float M = fmaxf(fmaxf(p0[8 * D + g], p0[PS + 8 * D + g]), fmaxf(p0[2 * PS + 8 * D + g], p0[3 * PS + 8 * D + g]));
    float acc = 0.f, L = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float mk = p0[k * PS + 8 * D + g];
      const float wk = (mk == KV_NEG_INF || M == KV_NEG_INF) ? 0.f : ex2(mk - M);
      acc = fmaf(wk, p0[k * PS + g * D + tid], acc);
      L = fmaf(wk, p0[k * PS + 8 * D + 8 + g], L);
    }
    op[g * D + tid] = acc;
    if (tid == 0) { mlp[2 * g] = M; mlp[2 * g + 1] = L; }
  }
}

}  // namespace kvm
