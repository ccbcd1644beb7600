// Shared pieces of the KIVI paged decode kernels (mma.sync m16n8k16, fp32 accumulation; GQA groups of up to 8 q heads):
// shared-memory geometry of a warp's page buffers and value tile, small PTX wrappers, and the BF16 sink / window split
// (kv_tail_mma).  Included by kv_capi.cu inside its anonymous namespace, before kv_attn_mma2.cuh (the page-split kernel).
//
// Operand forms both kernels rely on:
//   * key codes are read in place: the stored word holds channel pairs (2 m, 2 m + 1) at bits (2 m, 2 m + 16), so one
//     rotate + mask puts a code into the mantissa of an FP16 subnormal (code * 2^-24 or 2^-16, exact); the power of two
//     is split between the other operand and the fp32 epilogue;
//   * value codes of a 32-token group are expanded the same way into an FP16 tile [32 tokens][128 channels] (the
//     columns are a fixed permutation of the channels) that ldmatrix.trans reads as the B operand of P V;
//   * the three storage classes of a value (plain, H32 per block, whole-head H128) accumulate separately and are
//     rotated back once per CTA.
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
