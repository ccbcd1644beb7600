// Paged split-KV GQA decode attention over INT4 / INT2 FlagRot pages for sm_100a.
//
// Replaces the reference kernels k_attn2 / k_attn2g (kernels/csrc/attn_decode_v2.cu:687, attn_decode_v2g.cuh:276), k_cbk
// (kernels/csrc/attn_codebook_attn.cuh:2126), the BF16 window kernels k_tail_* (attn_tail.cuh) and the in-kernel split
// merge (attn_merge.cuh) for the formats int4a / int2a (static block flags) and konlya / konlya2 (per-token flags in the
// scale sign bits).  Same pages, same workspace contract, one launch.
//
// Design (B200): the path is HBM-bound, but 2.5 - 4.5-bit cells carry more multiply-accumulates per byte than the FP32
// lanes of an SM can retire at HBM speed, so the dot products run on the integer tensor path (mma.sync m16n8k32
// u8 x s8 -> s32) directly on the packed codes; everything that touches a scale, a flag or the softmax stays on the
// CUDA cores.
//   * grid (Hkv * ceil(G / 4), nsplit, B [x 2 with BF16 rows: the window CTAs come last and fill the final wave]),
//     128 threads; a CTA serves 4 q heads of one kv head;
//   * each warp owns every 4th 32-token block (two 16-token pages or one 32-token page) of the split and a private ring
//     of three stages; all 32 lanes copy 16-byte pieces of the page chunks with cp.async (one commit group per block).
//     A single lane issuing bulk copies was measured to stall its warp for about 460 cycles per block on the copy
//     engine's issue path; spread over the lanes the issue costs ten instructions per lane and no waiting loop at all
//     (cp.async.wait_group is a hardware wait);
//   * QK: A = the code bytes as stored (the K row layout is the m16n8k32 A fragment: one 128-bit shared load per
//     token gives all four groups), B = q in 15-bit fixed point split hi / lo, for key-only pages in three bases
//     (identity, per-group H32, whole-head H128); per (token, group) the flags select the variant, the zero point is
//     removed with the matching sum of q, the group scale is applied in fp32;
//   * PV: P' = p * V-scale is quantised to 14 bits per (token, group) with a running normaliser, transposed through
//     1 KB of shared memory per warp and multiplied with the V^T code bytes (again the stored bytes are the A
//     fragment); integer accumulators are folded into fp32 whenever the running maximum or the normaliser moves;
//   * the 4 warps merge in shared memory; splits merge through the caller's workspace, last arriving CTA wins.
#include <algorithm>
#include <cmath>
#include <functional>
#include <type_traits>
#include <vector>

#include "fr_common.cuh"
#include "fr_kernels.h"

namespace fr {

namespace {

constexpr int NWARP = 4;
constexpr int BLK = 32;            // tokens per warp step
constexpr int ST = 3;              // bulk-copy stages per warp
constexpr int MINB = 3;            // resident CTAs per SM the register budget is set for
constexpr int MAXPG = 512;         // pages per split (chunk <= 8192 tokens of 16)
#define NEG_INF (-INFINITY)


FR_DEVI uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
// 16-byte asynchronous copy global -> shared (L2 only), tracked by per-thread commit groups
FR_DEVI void cp16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
}
FR_DEVI void cp_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> FR_DEVI void cp_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }
// D = A * B with a zero accumulator (no register initialisation)
FR_DEVI void mma_u8s8_z(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
               : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
FR_DEVI void mma_u8u8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
FR_DEVI float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
FR_DEVI uint32_t prmt(uint32_t a, uint32_t b, uint32_t s) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;\n" : "=r"(r) : "r"(a), "r"(b), "r"(s));
  return r;
}
FR_DEVI uint4 lds128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
FR_DEVI uint2 lds64(uint32_t a) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "r"(a));
  return v;
}
FR_DEVI void sts128(uint32_t a, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(a), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
FR_DEVI float h2f(uint32_t bits16) { return __half2float(__ushort_as_half(static_cast<unsigned short>(bits16))); }
FR_DEVI float2 h2x2f(uint32_t v) {   // two packed fp16 -> two fp32
  __half2 h;
  *reinterpret_cast<uint32_t*>(&h) = v;
  return __half22float2(h);
}

template <int NB, int PG> struct DLay {
  static_assert(PG == 16 || PG == 32, "pages of 16 or 32 tokens");
  static constexpr int P = PG;                                // tokens per page; a warp step is always 32 tokens = 32 / P pages
  static constexpr int CHUNK = Lay<NB>::CELL * P;             // 2304 | 1280 (P 16), 4608 | 2560 (P 32)
  static constexpr int PG1 = CHUNK + 64;                      // P 16: second page of a stage (64-byte skew: bank spread)
  static constexpr int STAGE = P == 16 ? ((PG1 + CHUNK + 127) / 128) * 128 : ((CHUNK + 127) / 128) * 128;
  static constexpr int V_OFF = Lay<NB>::CBY * P, KS_OFF = 2 * Lay<NB>::CBY * P, VS_OFF = KS_OFF + 8 * P;
  static constexpr uint32_t ZM = NB == 4 ? 0xFu : 0x3u;
  // the tensor path reads the code fields in place, i.e. scaled by a power of two:
  // K fields of group j by KF(j) (INT4 16; INT2 4 for even, 64 for odd groups), V^T rows gid / gid + 8 by 1 / VF0, 1 / VF1
  __host__ __device__ static constexpr int kf(int j) { return NB == 4 ? 16 : ((j & 1) ? 64 : 4); }
  __host__ __device__ static constexpr float kfinv(int j) { return 1.0f / static_cast<float>(kf(j)); }
  static constexpr float VF0 = NB == 4 ? 1.0f / 16.0f : 1.0f / 4.0f, VF1 = NB == 4 ? 1.0f / 16.0f : 1.0f / 64.0f;
};
constexpr int PBUF_WORDS = 4 * 72;  // P' exchange per warp: [head] stride 72 words (18 x 16 B), [c][hl][e][j]
constexpr int KTAB_BYTES = 1024;    // K scale table per warp: [group pair][32 tokens] x (2 scales fp32, sign = H32 flag | 2 zero points)
constexpr float TAU = 2.0f;         // the softmax reference only moves when a score exceeds it by more than TAU (log2): p <= 4

// shared memory map (dynamic): ring | pbuf | K scale tables | q table | sums | page ids | merge scratch (aliases the ring)
template <int NB, int NV, int PG = 16> struct SMap {
  static constexpr int RING = 0;
  static constexpr int RING_BYTES = NWARP * ST * DLay<NB, PG>::STAGE;
  static constexpr int PBUF = RING + RING_BYTES;
  static constexpr int KTAB = PBUF + NWARP * PBUF_WORDS * 4;           // per warp: [2 group pairs][32 tokens] x 16 bytes
  static constexpr int QT = KTAB + NWARP * KTAB_BYTES;                 // int16 [NV][4][128]
  static constexpr int SQ = QT + NV * 4 * 128 * 2;                      // int [NV][4][4]
  static constexpr int SF = SQ + NV * 16 * 4;                           // float [4]
  static constexpr int PIDX = SF + 16;                                  // int [MAXPG]
  static constexpr int TOTAL = PIDX + MAXPG * 4;
  static_assert(RING_BYTES >= NWARP * (4 * 128 + 8) * 4, "merge scratch aliases the ring");
};

// ------------------------------------------------------------------------------------------------ split merge
// parts of (row b, kv head, q tile): slots base .. base + n - 1, each [4][128] floats of opart and [4][2] of mlpart.
// Warp w merges head w: (m, l) of the parts over the lanes, then the float4 rows.
FR_DEVI void merge_parts(const float* opart, const float* mlpart, int base, int n, int head, int lane, float (&x)[4],
                         float& Mo, float& Lo) {
  const float2* ml = reinterpret_cast<const float2*>(mlpart);
  float M = NEG_INF;
  for (int s = lane; s < n; s += 32) M = fmaxf(M, __ldcg(&ml[(base + s) * 4 + head]).x);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(FULLMASK, M, o));
  float l = 0.f;
  for (int s = lane; s < n; s += 32) {
    const float2 v = __ldcg(&ml[(base + s) * 4 + head]);
    l += v.x == NEG_INF ? 0.f : ex2(v.x - M) * v.y;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(FULLMASK, l, o);
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  const float4* op = reinterpret_cast<const float4*>(opart) + head * 32 + lane;
  int s = 0;
  for (; s + 4 <= n; s += 4) {
    float4 v[4];
    float wgt[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      v[k] = __ldcg(op + static_cast<size_t>(base + s + k) * 128);
      const float m = __ldcg(&ml[(base + s + k) * 4 + head]).x;
      wgt[k] = m == NEG_INF ? 0.f : ex2(m - M);
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      acc.x = fmaf(wgt[k], v[k].x, acc.x); acc.y = fmaf(wgt[k], v[k].y, acc.y);
      acc.z = fmaf(wgt[k], v[k].z, acc.z); acc.w = fmaf(wgt[k], v[k].w, acc.w);
    }
  }
  for (; s < n; ++s) {
    const float4 v = __ldcg(op + static_cast<size_t>(base + s) * 128);
    const float m = __ldcg(&ml[(base + s) * 4 + head]).x;
    const float wgt = m == NEG_INF ? 0.f : ex2(m - M);
    acc.x = fmaf(wgt, v.x, acc.x); acc.y = fmaf(wgt, v.y, acc.y); acc.z = fmaf(wgt, v.z, acc.z); acc.w = fmaf(wgt, v.w, acc.w);
  }
  x[0] = acc.x; x[1] = acc.y; x[2] = acc.z; x[3] = acc.w;
  Mo = M; Lo = l;
}

// orthonormal H32 of the flagged 32-blocks of a row held 4 elements per lane (mask: 4 bytes of this kv head)
FR_DEVI void rot_blocks(float (&x)[4], const uint8_t* mask, int lane) {
  if (mask == nullptr) return;
  const bool rot = mask[lane >> 3] != 0;
  if (!__any_sync(FULLMASK, rot)) return;
  float y[4] = {x[0], x[1], x[2], x[3]};
  fwht_row_stages(y, lane, 32);
#pragma unroll
  for (int i = 0; i < 4; ++i) if (rot) x[i] = y[i] * C32;
}

// final store of head `head` of the CTA's q tile: x = unnormalised row (4 dims per lane), l its denominator
FR_DEVI void store_row(const DecodeParams& p, int b, int kvh, int qt, int head, int lane, float (&x)[4], float M, float l) {
  const int g = qt * 4 + head;
  if (g >= p.G) return;
  const float rl = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) x[i] *= rl;
  rot_blocks(x, p.vmask ? p.vmask + kvh * 4 : nullptr, lane);      // static formats: back to the original V basis
  const int hq = kvh * p.G + g;
  if (p.part_out != nullptr) {   // extension: fp32 row + (m, l) for a merge across devices
    float* po = p.part_out + (static_cast<size_t>(b) * p.Hkv * p.G + hq) * 130;
    *reinterpret_cast<float2*>(po + 4 * lane) = make_float2(x[0], x[1]);
    *reinterpret_cast<float2*>(po + 4 * lane + 2) = make_float2(x[2], x[3]);
    if (lane == 0) { po[128] = M; po[129] = l; }
    return;
  }
  const __nv_bfloat162 o01 = __floats2bfloat162_rn(x[0], x[1]), o23 = __floats2bfloat162_rn(x[2], x[3]);
  uint2 ov;
  ov.x = *reinterpret_cast<const uint32_t*>(&o01);
  ov.y = *reinterpret_cast<const uint32_t*>(&o23);
  *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(p.out) + b * p.o_bs + hq * HD + 4 * lane) = ov;
}

// CTA epilogue.  scr: per warp [4][128] floats o (unnormalised, relative to the warp's m) then [4] m, [4] l.
// Combines the warps, then either stores the row (single part) or publishes the partial and, as last arriver of the
// (row, kv head), merges every part of every q tile.
FR_DEVI void cta_finish(const DecodeParams& p, float* scr, int b, int kvh, int qt, int NT, int part, int nparts, int nsp,
                        int* last_flag) {
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  constexpr int WS = 4 * 128 + 8;
  __syncthreads();
  // warp w combines head w over the 4 warps
  float M = NEG_INF;
#pragma unroll
  for (int k = 0; k < NWARP; ++k) M = fmaxf(M, scr[k * WS + 512 + w]);
  float x[4] = {0.f, 0.f, 0.f, 0.f}, l = 0.f;
#pragma unroll
  for (int k = 0; k < NWARP; ++k) {
    const float mk = scr[k * WS + 512 + w];
    const float wk = mk == NEG_INF ? 0.f : ex2(mk - M);
    const float4 v = *reinterpret_cast<const float4*>(scr + k * WS + w * 128 + 4 * lane);
    x[0] = fmaf(wk, v.x, x[0]); x[1] = fmaf(wk, v.y, x[1]); x[2] = fmaf(wk, v.z, x[2]); x[3] = fmaf(wk, v.w, x[3]);
    l = fmaf(wk, scr[k * WS + 516 + w], l);
  }
  if (nparts * NT == 1) {
    store_row(p, b, kvh, qt, w, lane, x, M, l);
    return;
  }
  const int slot = ((b * p.Hkv + kvh) * NT + qt) * nsp + part;
  *reinterpret_cast<float4*>(p.opart + static_cast<size_t>(slot) * 512 + w * 128 + 4 * lane) = make_float4(x[0], x[1], x[2], x[3]);
  if (lane == 0) *reinterpret_cast<float2*>(p.mlpart + slot * 8 + 2 * w) = make_float2(M, l);
  // publish: the CTA barrier orders every thread's stores before thread 0, whose fence (cumulative at device scope) and
  // ticket make them visible to the last arriver; that CTA's thread 0 fences again before the barrier that releases its
  // readers, which load through L2 (__ldcg).  One fence pair per CTA instead of one per thread.
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const int old = atomicAdd(p.counter + b * p.Hkv + kvh, 1);
    *last_flag = old == nparts * NT - 1;
    if (*last_flag) __threadfence();
  }
  __syncthreads();
  if (!*last_flag) return;
  for (int t = 0; t < NT; ++t) {
    float y[4], Mo, Lo;
    merge_parts(p.opart, p.mlpart, ((b * p.Hkv + kvh) * NT + t) * nsp, nparts, w, lane, y, Mo, Lo);
    store_row(p, b, kvh, t, w, lane, y, Mo, Lo);
  }
  if (tid == 0) p.counter[b * p.Hkv + kvh] = 0;
}

// ------------------------------------------------------------------------------------------------ BF16 window CTA
// One CTA per (row, kv head, q tile) over the <= 256 BF16 rows of the row's ring entry, on the tensor cores (mma.sync
// m16n8k16 BF16, fp32 accumulation).  Warp w owns the 16-token slices w, w + 4, ...
// of the window with its own running (m, l) and accumulators; rows 0 - 3 of the M tile are the q heads.  K fragments come
// straight from global memory (a lane's two registers of a k-step cover one whole 32-byte sector of a row), V rows go
// through the warp's shared-memory tile and ldmatrix.trans.  q and K are BF16 already, so the scores are exact products
// summed in fp32; p is split into two BF16 parts (hi + lo) so that P V keeps 16 bits of p.
constexpr int TAILM_VSTR = 272;                       // bytes per V row in the warp tile (256 + 16)
constexpr int TAILM_BYTES = NWARP * (4 * 128 + 8) * 4 + 128 + NWARP * 16 * TAILM_VSTR;
FR_DEVI void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
FR_DEVI uint32_t pack_bf2(float a, float b) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}
FR_DEVI void tail_cta_mma(const DecodeParams& p, uint8_t* smem, float* scr, int b, int kvh, int qt, int tl) {
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5, g8 = lane >> 2, c4 = lane & 3;
  constexpr int WS = 4 * 128 + 8;
  const uint32_t vt = smem_u32(smem) + NWARP * WS * 4 + 128 + w * 16 * TAILM_VSTR;
  // A fragments of q: rows 0 - 3 = the tile's heads
  uint32_t qa[8][2];
  {
    const __nv_bfloat16* qb = static_cast<const __nv_bfloat16*>(p.q) + b * p.q_bs + (kvh * p.G + qt * 4) * HD;
    const bool on = g8 < 4 && qt * 4 + g8 < p.G;
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      qa[kk][0] = on ? *reinterpret_cast<const uint32_t*>(qb + g8 * HD + 16 * kk + 2 * c4) : 0u;
      qa[kk][1] = on ? *reinterpret_cast<const uint32_t*>(qb + g8 * HD + 16 * kk + 2 * c4 + 8) : 0u;
    }
  }
  const __nv_bfloat16* tb = static_cast<const __nv_bfloat16*>(p.tail) + (p.tail_idx ? p.tail_idx[b] : b) * p.tail_bs;
  const __nv_bfloat16* kbase = tb + kvh * HD;
  const __nv_bfloat16* vbase = tb + (p.Hkv + kvh) * HD;
  float o[16][2];
#pragma unroll
  for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = 0.f;
  float m = NEG_INF, l = 0.f;
  for (int t0 = 16 * w; t0 < tl; t0 += 16 * NWARP) {
    // V rows of the slice -> shared tile (rows past the window are zeros: p = 0 must not meet stale bytes)
    __syncwarp();
    for (int i = lane; i < 16 * 16; i += 32) {
      const int r = i >> 4, c16 = i & 15;
      const uint32_t dst = vt + r * TAILM_VSTR + 16 * c16;
      if (t0 + r < tl) {
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(vbase + (t0 + r) * p.tail_ts + 8 * c16) : "memory");
      } else {
        sts128(dst, 0u, 0u, 0u, 0u);
      }
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
    // K fragments of tokens t0 + 8 nt + g8
    uint32_t kb[2][8][2];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const int t = t0 + 8 * nt + g8;
      const __nv_bfloat16* kr = kbase + t * p.tail_ts + 2 * c4;
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
    float mx = NEG_INF;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float v = (t0 + 8 * nt + 2 * c4 + e < tl) ? s[nt][e] * p.qscale : NEG_INF;
        s[nt][e] = v;
        mx = fmaxf(mx, v);
      }
    mx = fmaxf(mx, __shfl_xor_sync(FULLMASK, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(FULLMASK, mx, 2));
    const float mn = fmaxf(m, mx), base = mn == NEG_INF ? 0.f : mn;
    const float alpha = m == NEG_INF ? 0.f : ex2(m - base);
    m = mn;
    float ps = 0.f;
    uint32_t ph[2], pl[2];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const float p0 = ex2(s[nt][0] - base), p1 = ex2(s[nt][1] - base);
      ps += p0 + p1;
      ph[nt] = pack_bf2(p0, p1);
      pl[nt] = pack_bf2(p0 - bf16_lo(ph[nt]), p1 - bf16_hi(ph[nt]));
    }
    l = l * alpha + ps;
#pragma unroll
    for (int i = 0; i < 16; ++i) { o[i][0] *= alpha; o[i][1] *= alpha; }
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncwarp();
#pragma unroll
    for (int np = 0; np < 8; ++np) {
      uint32_t b0, b1, b2, b3;
      asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                   : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3)
                   : "r"(vt + ((lane & 7) + 8 * ((lane >> 3) & 1)) * TAILM_VSTR + (16 * np + 8 * (lane >> 4)) * 2));
      float c0[4] = {o[2 * np][0], o[2 * np][1], 0.f, 0.f}, c1[4] = {o[2 * np + 1][0], o[2 * np + 1][1], 0.f, 0.f};
      mma_bf16(c0, ph[0], 0u, ph[1], 0u, b0, b1);
      mma_bf16(c0, pl[0], 0u, pl[1], 0u, b0, b1);
      mma_bf16(c1, ph[0], 0u, ph[1], 0u, b2, b3);
      mma_bf16(c1, pl[0], 0u, pl[1], 0u, b2, b3);
      o[2 * np][0] = c0[0]; o[2 * np][1] = c0[1]; o[2 * np + 1][0] = c1[0]; o[2 * np + 1][1] = c1[1];
    }
  }
  // partial of this warp: [4 heads][128] o, [4] m, [4] l (lanes g8 < 4 hold the heads)
  l += __shfl_xor_sync(FULLMASK, l, 1);
  l += __shfl_xor_sync(FULLMASK, l, 2);
  if (g8 < 4) {
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) *reinterpret_cast<float2*>(scr + w * WS + g8 * 128 + 8 * nt + 2 * c4) = make_float2(o[nt][0], o[nt][1]);
    if (c4 == 0) { scr[w * WS + 512 + g8] = m; scr[w * WS + 516 + g8] = l; }
  }
  __syncwarp();
  if (p.vmask_tail != nullptr) {     // static formats with V flags: move the partial into the stored V basis
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      float4 v = *reinterpret_cast<float4*>(scr + w * WS + g * 128 + 4 * lane);
      float x[4] = {v.x, v.y, v.z, v.w};
      rot_blocks(x, p.vmask_tail + kvh * 4, lane);
      *reinterpret_cast<float4*>(scr + w * WS + g * 128 + 4 * lane) = make_float4(x[0], x[1], x[2], x[3]);
    }
  }
}

// ------------------------------------------------------------------------------------------------ q prologue
// warp g prepares q head g of the tile (row mapping): the NV variants in fixed point, their per-group sums, the scale.
template <int NV>
FR_DEVI void q_prologue(const DecodeParams& p, int b, int kvh, int qt, int16_t* qtab, int* sq, float* sf) {
  const int lane = threadIdx.x & 31, g = threadIdx.x >> 5;
  const __nv_bfloat16* qb = static_cast<const __nv_bfloat16*>(p.q) + b * p.q_bs + (kvh * p.G + qt * 4 + g) * HD;
  uint2 raw = make_uint2(0, 0);
  if (qt * 4 + g < p.G) raw = *reinterpret_cast<const uint2*>(qb + 4 * lane);
  float v[NV][4];
  v[0][0] = bf16_lo(raw.x); v[0][1] = bf16_hi(raw.x); v[0][2] = bf16_lo(raw.y); v[0][3] = bf16_hi(raw.y);
  if constexpr (NV == 3) {
#pragma unroll
    for (int i = 0; i < 4; ++i) { v[1][i] = v[0][i]; v[2][i] = v[0][i]; }
    fwht_row_stages(v[1], lane, 32);
    fwht_row_stages(v[2], lane, 128);
#pragma unroll
    for (int i = 0; i < 4; ++i) { v[1][i] *= C32; v[2][i] *= C128; }
  } else {
    rot_blocks(v[0], p.kmask ? p.kmask + kvh * 4 : nullptr, lane);   // static: q into the stored K basis
  }
  float am = 0.f;
#pragma unroll
  for (int c = 0; c < NV; ++c)
#pragma unroll
    for (int i = 0; i < 4; ++i) am = fmaxf(am, fabsf(v[c][i]));
  am = warp_max(am);
  const float step = am > 0.f ? am * (1.0f / 8128.0f) : 1.0f;
  const float inv = 1.0f / step;
#pragma unroll
  for (int c = 0; c < NV; ++c) {
    int s = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int qi = max(-8128, min(8128, __float2int_rn(v[c][i] * inv)));
      qtab[(c * 4 + g) * 128 + 4 * lane + i] = static_cast<int16_t>(qi);
      s += qi;
    }
    s += __shfl_xor_sync(FULLMASK, s, 1);
    s += __shfl_xor_sync(FULLMASK, s, 2);
    s += __shfl_xor_sync(FULLMASK, s, 4);
    if ((lane & 7) == 0) sq[(c * 4 + g) * 4 + (lane >> 3)] = s;
  }
  if (lane == 0) sf[g] = p.qscale * step;
}

// pieces of row b: the first rows_wide rows are cut into nsplit - 1 pieces of chunk_w tokens, the others into nsplit pieces
// of chunk tokens (both cover the same nominal length nsplit * chunk); returns the piece size, `np` = pieces of this row
FR_DEVI int row_pieces(const DecodeParams& p, int b, int& np) {
  const bool wide = b < p.rows_wide;
  np = wide ? p.nsplit - 1 : p.nsplit;
  return wide ? p.chunk_w : p.chunk;
}

// ------------------------------------------------------------------------------------------------ the kernel
// SYM (NB 4 only): the symmetric `int4` / `konly` pages (reference attn_decode_v2.cuh:26-28): sign-magnitude elements, plain
// FP16 scale words.  A code word is rewritten on the fly as the INT4A word of q + 8 (carry-free byte arithmetic) and every
// zero point is 8, after which the asymmetric path applies unchanged.
template <int NB, bool KO, int PG, bool SYM = false>
__global__ void __launch_bounds__(128, MINB) k_decode(const DecodeParams p) {
  constexpr int NV = KO ? 3 : 1;
  using L = DLay<NB, PG>;
  using S = SMap<NB, NV, PG>;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ int last_flag;
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5, gid = lane >> 2, tig = lane & 3;
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
  int np_b;
  const int chunk_b = row_pieces(p, b, np_b);
  const int ns_b = len > 0 ? min(np_b, max(1, (len + chunk_b - 1) / chunk_b)) : 0;
  const int nparts = ns_b + has_tail;
  float* scr = reinterpret_cast<float*>(smem + S::RING);
  constexpr int WS = 4 * 128 + 8;

  if (split >= p.nsplit) {   // the BF16 window CTA
    const int tl = min(p.tail_len[b], 256);
    if (len <= 0 && tl <= 0 && nparts * NT > 1) {
      // nothing to attend: still publish an empty part so that the tickets add up
    }
    tail_cta_mma(p, smem + S::RING, scr, b, kvh, qt, tl);
    cta_finish(p, scr, b, kvh, qt, NT, ns_b, nparts, nsp, &last_flag);
    return;
  }
  if (split >= ns_b) return;

  const int c0 = split * chunk_b, c1 = min(len, c0 + chunk_b);
  const int lo = max(c0, p.kv_start);                                 // first attended token
  const int ntok = c1 - c0, nblk = (ntok + BLK - 1) / BLK;
  int16_t* qtab = reinterpret_cast<int16_t*>(smem + S::QT);
  int* sqs = reinterpret_cast<int*>(smem + S::SQ);
  float* sfs = reinterpret_cast<float*>(smem + S::SF);
  int* pidx = reinterpret_cast<int*>(smem + S::PIDX);

  // ---- page loads: every lane copies 16-byte pieces of the block's page chunks (cp.async, one commit group per block), so
  // the issue is spread over the warp instead of stalling one lane on the copy engine.  The first ST - 1 blocks of a warp
  // are requested before anything else, with their page numbers straight from the global block table, so that the q
  // prologue and the staging of the table run under the latency of those loads.
  const int* bt = p.block_table + static_cast<size_t>(b) * p.bt_stride + c0 / L::P;
  const uint8_t* poolh = p.pool + static_cast<size_t>(kvh) * L::CHUNK + 16 * lane;
  const size_t pstride = static_cast<size_t>(p.Hkv) * L::CHUNK;
  const uint32_t ring = smem_u32(smem + S::RING) + w * ST * L::STAGE;
  // block n of this warp = CTA block w + 4 n
  const int nmine = nblk > w ? (nblk - w + NWARP - 1) / NWARP : 0;
  auto copy_chunk = [&](uint32_t dst, const uint8_t* src) {
    constexpr int NV16 = L::CHUNK / 16;                               // 144 | 80 (P 16), 288 | 160 (P 32)
#pragma unroll
    for (int v = 0; v < NV16 / 32; ++v) cp16(dst + 512 * v, src + 512 * v);
    if (NV16 % 32 != 0 && lane < NV16 % 32) cp16(dst + 512 * (NV16 / 32), src + 512 * (NV16 / 32));
  };
  auto issue = [&](int n, bool early) {                               // all lanes; n may lie past the warp's last block
    if (n < nmine) {
      const int blk = w + NWARP * n;
      const uint32_t dst = ring + (n % ST) * L::STAGE + 16 * lane;
      if constexpr (L::P == 16) {
        const bool two = ntok - blk * BLK > L::P;
        const int pg0 = early ? __ldg(bt + 2 * blk) : pidx[2 * blk];
        const int pg1 = two ? (early ? __ldg(bt + 2 * blk + 1) : pidx[2 * blk + 1]) : 0;
        copy_chunk(dst, poolh + static_cast<size_t>(pg0) * pstride);
        if (two) copy_chunk(dst + L::PG1, poolh + static_cast<size_t>(pg1) * pstride);
      } else {                          // one 32-token page per step
        copy_chunk(dst, poolh + static_cast<size_t>(early ? __ldg(bt + blk) : pidx[blk]) * pstride);
      }
    }
    cp_commit();                        // an empty group past the end keeps the group count in step with n
  };
#pragma unroll
  for (int n = 0; n < ST - 1; ++n) issue(n, true);
  {
    const int npg = (ntok + L::P - 1) / L::P;
    for (int i = tid; i < npg && i < MAXPG; i += 128) pidx[i] = __ldg(bt + i);
  }
  q_prologue<NV>(p, b, kvh, qt, qtab, sqs, sfs);
  __syncthreads();

  // ---- per-thread constants
  // q B fragments: column gid = (head gid >> 1, part gid & 1: hi / lo); k = 4 tig .. (b0), 16 + 4 tig .. (b1)
  uint32_t qf[NV][4][2];
  int SQ[NV][4];   // MINUS the per-group sums of the fixed-point q, pre-multiplied by the code scaling of the group (KF)
  {
    const int hd = gid >> 1, lo_part = gid & 1;
#pragma unroll
    for (int c = 0; c < NV; ++c)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          uint32_t word = 0;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int qi = qtab[(c * 4 + hd) * 128 + 32 * j + 16 * r + 4 * tig + k];
            const int hi = (qi + 64) >> 7, lw = qi - (hi << 7);
            word |= static_cast<uint32_t>((lo_part ? lw : hi) & 0xFF) << (8 * k);
          }
          qf[c][j][r] = word;
        }
        SQ[c][j] = -sqs[(c * 4 + tig) * 4 + j] * L::kf(j);
      }
  }
  const float sfac = NB == 4 ? sfs[tig] * L::kfinv(0) : sfs[tig];      // (INT2: the table's scales carry 1 / KF(j))
  // tokens of this lane inside a block: tau_i = 8 c + 2 i + e, (c, e) = (gid >> 1, gid & 1)
  const int tc = gid >> 1, te = gid & 1;
  const uint32_t tpoff = L::P == 16 ? (tc >> 1) * L::PG1 : 0;          // page of the block holding the lane's tokens
  const int tpos0 = (L::P == 16 ? 8 * (tc & 1) : 8 * tc) + te;         // position in the page of token i = 0 (+ 2 i)
  // P' exchange buffer: [head] 72 words, [part hi / lo] 36 words, [chunk c] 8 words, [e] 4 words, [j]
  const uint32_t pbuf = smem_u32(smem + S::PBUF) + w * PBUF_WORDS * 4;
  const uint32_t pw_dst = pbuf + 4 * (tig * 72 + tc * 8 + te * 4);               // + 144 bytes for the lo part
  const uint32_t pw_src = pbuf + 4 * ((gid >> 1) * 72 + (gid & 1) * 36 + tig * 8);   // 8 words: [e][j]
  // K scale table of the warp: lane = token writes, every lane reads its four tokens 8 tc + 2 i + te
  const uint32_t ktab = smem_u32(smem + S::KTAB) + w * KTAB_BYTES;
  const uint32_t kt_dst = ktab + 16 * lane, kt_src = ktab + 16 * (8 * tc + te);   // + 32 i; groups 2, 3: 512 bytes further
  const uint32_t kt_ld = L::P == 16 ? (lane >> 4) * L::PG1 + L::KS_OFF + 8 * (lane & 15)
                                    : L::KS_OFF + 8 * lane;                       // the token's four K scale words in a stage
  // byte offsets of this lane's shared-memory reads inside a stage
  const uint32_t vs_off = tpoff + L::VS_OFF + 2 * (8 * (L::P == 16 ? (tc & 1) : tc) + 4 * te);   // + 2 P j
  // K code row of token i: INT4 rows are 64 bytes apart in token order; INT2 rows are 32 bytes apart with physical row
  // pos ^ ((pos >> 1) & 2), which for pos = tpos0 + 2 i just swaps i = 2 and i = 3: a compile-time offset per i either way
  const uint32_t kc_base = tpoff + (NB == 4 ? 64 * tpos0 + 16 * tig : 32 * tpos0 + 8 * tig);
  auto kc_row = [](int i) { return NB == 4 ? 128 * i : 64 * (i < 2 ? i : 5 - i); };
  const uint32_t vc_off = L::P == 16 ? (tig >> 1) * L::PG1 + L::V_OFF + (NB == 4 ? 16 : 8) * (gid * (L::P / 8) + (tig & 1))
                                     : L::V_OFF + (NB == 4 ? 16 : 8) * (gid * (L::P / 8) + tig);

  // ---- running state (head tig)
  float m_run = NEG_INF, l_run = 0.f;
  uint32_t nmax16 = 0;                           // fp16 bits of the largest V scale admitted by the normaliser
  float nrm = 0.f, inrm = 0.f;                   // P~ = rint(p * sv * nrm), nrm = 2^14 / (2 max sv)
  int Oi[2][4][4];                               // [m][w][frag] integer PV accumulators
  float Of[2][4][2];                             // folded fp32 accumulators, rows gid / gid + 8 of tile (m, w), head tig
  int Zi[4];
  float Zf[4];
#pragma unroll
  for (int a = 0; a < 2; ++a)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
#pragma unroll
      for (int k = 0; k < 4; ++k) Oi[a][c][k] = 0;
      Of[a][c][0] = Of[a][c][1] = 0.f;
    }
#pragma unroll
  for (int j = 0; j < 4; ++j) { Zi[j] = 0; Zf[j] = 0.f; }

  auto fold = [&](float alpha) {   // integer accumulators -> fp32 (scaled by inrm), then everything times alpha
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        Of[a][c][0] = (Of[a][c][0] + fmaf(static_cast<float>(Oi[a][c][0]), 256.f, static_cast<float>(Oi[a][c][1])) * (inrm * L::VF0)) * alpha;
        Of[a][c][1] = (Of[a][c][1] + fmaf(static_cast<float>(Oi[a][c][2]), 256.f, static_cast<float>(Oi[a][c][3])) * (inrm * L::VF1)) * alpha;
#pragma unroll
        for (int k = 0; k < 4; ++k) Oi[a][c][k] = 0;
      }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      Zf[j] = (Zf[j] + static_cast<float>(Zi[j]) * inrm) * alpha;
      Zi[j] = 0;
    }
    l_run *= alpha;
  };

  // one 32-token block of this warp from stage memory `st`; PARTIAL: some tokens lie outside [lo, c1)
  auto process = [&](const uint32_t st, int tok0, auto partial_tag) {
    constexpr bool PARTIAL = decltype(partial_tag)::value;
    // ---- K scales of the block, decoded once per (token, group): lane = token converts its four words to fp32 (bit 15, the
    // H32 flag of a key-only page, simply becomes the sign) and splits off the zero points; the lanes that share a token
    // then read the same 16 + 16 bytes instead of decoding the words four times over
    {
      const uint2 t = lds64(st + kt_ld);
      float2 f01 = h2x2f(t.x), f23 = h2x2f(t.y);
      if (NB == 2) { f01.x *= L::kfinv(0); f01.y *= L::kfinv(1); f23.x *= L::kfinv(2); f23.y *= L::kfinv(3); }
      sts128(kt_dst, __float_as_uint(f01.x), __float_as_uint(f01.y), SYM ? 8u : t.x & L::ZM, SYM ? 8u : (t.x >> 16) & L::ZM);   // groups 0, 1
      sts128(kt_dst + 512, __float_as_uint(f23.x), __float_as_uint(f23.y), SYM ? 8u : t.y & L::ZM, SYM ? 8u : (t.y >> 16) & L::ZM);   // 2, 3
    }
    // ---- V scale words of the lane's 4 tokens (group j: tokens 0 1 | 2 3); group 0 now (it carries the whole-head flags
    // of the keys), groups 1 - 3 after the scores
    uint32_t vsw[4][2];
    {
      const uint2 t = lds64(st + vs_off);
      vsw[0][0] = t.x; vsw[0][1] = t.y;
    }
    __syncwarp();
    bool valid[4] = {true, true, true, true};
    [[maybe_unused]] bool ffl[4] = {false, false, false, false};
    if constexpr (KO) {   // whole-head flag of the key of token i: bit 15 of its V group-0 word
      ffl[0] = (vsw[0][0] & 0x8000u) != 0; ffl[1] = static_cast<int>(vsw[0][0]) < 0;
      ffl[2] = (vsw[0][1] & 0x8000u) != 0; ffl[3] = static_cast<int>(vsw[0][1]) < 0;
      vsw[0][0] &= 0x7FFF7FFFu; vsw[0][1] &= 0x7FFF7FFFu;
    }
    if constexpr (PARTIAL) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int pos = tok0 + 8 * tc + 2 * i + te;
        valid[i] = pos >= lo && pos < c1;
      }
    }
    // ---- QK
    float sc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      float skp[2][2];     // table entries of the current group pair, rows 2 u and 2 u + 1
      int kzp[2][2];
      uint32_t ka[2][4];   // code words of rows i = 2 u, 2 u + 1: INT4 4 words (group j), INT2 2 words (groups 2 jp, 2 jp + 1)
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        if (NB == 4) {
          const uint4 t = lds128(st + kc_base + kc_row(2 * u + r));
          ka[r][0] = t.x; ka[r][1] = t.y; ka[r][2] = t.z; ka[r][3] = t.w;
          if (SYM) {
#pragma unroll
            for (int k = 0; k < 4; ++k) ka[r][k] = sym_to_asym(ka[r][k]);
          }
        } else {
          const uint2 t = lds64(st + kc_base + kc_row(2 * u + r));
          ka[r][0] = t.x; ka[r][1] = t.y; ka[r][2] = 0; ka[r][3] = 0;
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        // group scale (key-only pages: negative = stored as H32 x) and zero point of the two rows: one 128-bit load per row
        // and group pair
        if ((j & 1) == 0) {
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            const uint4 e = lds128(kt_src + 32 * (2 * u + r) + 512 * (j >> 1));
            skp[r][0] = __uint_as_float(e.x); skp[r][1] = __uint_as_float(e.y);
            kzp[r][0] = static_cast<int>(e.z); kzp[r][1] = static_cast<int>(e.w);
          }
        }
        // A fragments: the code fields in place, scaled by KF(j) = 16 (INT4) | 4, 64 (INT2): no right shifts
        uint32_t a0, a1, a2, a3;
        if (NB == 4) {
          a0 = (ka[0][j] * 16u) & 0xF0F0F0F0u; a2 = ka[0][j] & 0xF0F0F0F0u;
          a1 = (ka[1][j] * 16u) & 0xF0F0F0F0u; a3 = ka[1][j] & 0xF0F0F0F0u;
        } else {
          const uint32_t msk = (j & 1) ? 0xC0C0C0C0u : 0x0C0C0C0Cu;
          a0 = (ka[0][j >> 1] * 4u) & msk; a2 = ka[0][j >> 1] & msk;
          a1 = (ka[1][j >> 1] * 4u) & msk; a3 = ka[1][j >> 1] & msk;
        }
        int acc[NV][4];
#pragma unroll
        for (int c = 0; c < NV; ++c) mma_u8s8_z(acc[c], a0, a1, a2, a3, qf[c][j][0], qf[c][j][1]);
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const int i = 2 * u + r;
          const float sk = skp[r][j & 1];
          const int z = kzp[r][j & 1];
          int val = acc[0][2 * r] * 128 + acc[0][2 * r + 1] + z * SQ[0][j];
          if constexpr (KO) {
            const int vh = acc[1][2 * r] * 128 + acc[1][2 * r + 1] + z * SQ[1][j];
            const int vf = acc[2][2 * r] * 128 + acc[2][2 * r + 1] + z * SQ[2][j];
            const bool hfl = __float_as_int(sk) < 0;
            val = ffl[i] ? vf : (hfl ? vh : val);
          }
          sc[i] = fmaf(KO ? fabsf(sk) : sk, static_cast<float>(val), sc[i]);
        }
      }
    }
#pragma unroll
    for (int j = 1; j < 4; ++j) {
      const uint2 t = lds64(st + vs_off + 2 * L::P * j);
      vsw[j][0] = t.x; vsw[j][1] = t.y;
    }
    if constexpr (PARTIAL) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {   // garbage beyond the sequence must not reach the normaliser / P'
        if (!valid[0]) vsw[j][0] &= 0xFFFF0000u;
        if (!valid[1]) vsw[j][0] &= 0x0000FFFFu;
        if (!valid[2]) vsw[j][1] &= 0xFFFF0000u;
        if (!valid[3]) vsw[j][1] &= 0x0000FFFFu;
      }
    }
    // ---- softmax step (head tig; the 8 lanes of a column hold the block's 32 tokens)
    float bm = NEG_INF;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      sc[i] = (!PARTIAL || valid[i]) ? sc[i] * sfac : NEG_INF;
      bm = fmaxf(bm, sc[i]);
    }
    bm = fmaxf(bm, __shfl_xor_sync(FULLMASK, bm, 4));
    bm = fmaxf(bm, __shfl_xor_sync(FULLMASK, bm, 8));
    bm = fmaxf(bm, __shfl_xor_sync(FULLMASK, bm, 16));
    // largest V scale of the lane's tokens (fp16 order = integer order of the 15-bit patterns)
    uint32_t vm = __vmaxu2(__vmaxu2(__vmaxu2(vsw[0][0], vsw[0][1]), __vmaxu2(vsw[1][0], vsw[1][1])),
                           __vmaxu2(__vmaxu2(vsw[2][0], vsw[2][1]), __vmaxu2(vsw[3][0], vsw[3][1])));
    vm = max(vm & 0xFFFFu, vm >> 16);
    // the reference m_run is lazy: it moves only when a score exceeds it by more than TAU, so p <= 2^TAU and the 16-bit P~
    // keeps two bits of headroom; every move folds the integer accumulators into fp32.  Without a move they cannot
    // overflow: a warp sees at most MAXPG / 8 = 64 blocks, each adding at most 32 x 240 x 128 < 2^20 to an accumulator
    if (__any_sync(FULLMASK, bm > m_run + TAU || vm > nmax16)) {
      uint32_t wm = vm;
      wm = max(wm, __shfl_xor_sync(FULLMASK, wm, 4));
      wm = max(wm, __shfl_xor_sync(FULLMASK, wm, 8));
      wm = max(wm, __shfl_xor_sync(FULLMASK, wm, 16));
      const float mn = bm > m_run + TAU ? bm : m_run;                  // (m_run = -inf: any finite score moves it)
      const float alpha = m_run == NEG_INF ? 0.f : (mn == m_run ? 1.f : ex2(m_run - mn));
      fold(alpha);
      m_run = mn;
      if (wm > nmax16) {     // twice the largest scale seen (one exponent step in fp16), capped below infinity
        nmax16 = min(wm + 0x0400u, 0x7BFFu);
        const float nf = h2f(nmax16);
        nrm = 16384.f / nf;
        inrm = nf * (1.0f / 16384.f);
      }
    }
    const float msafe = m_run == NEG_INF ? 0.f : m_run;
    float pn[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float pr = ex2(sc[i] - msafe);
      l_run += pr;
      pn[i] = pr * nrm;
    }
    // ---- P~ per (token, group): 14-bit fixed point (u8 hi, u8 lo), transposed through shared memory into the PV B fragments
    uint32_t hiw[4], low[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 s01 = h2x2f(vsw[j][0]), s23 = h2x2f(vsw[j][1]);
      const uint32_t t0 = __float_as_uint(fmaf(pn[0], s01.x, 8388608.f)), t1 = __float_as_uint(fmaf(pn[1], s01.y, 8388608.f));
      const uint32_t t2 = __float_as_uint(fmaf(pn[2], s23.x, 8388608.f)), t3 = __float_as_uint(fmaf(pn[3], s23.y, 8388608.f));
      const uint32_t x01 = prmt(t0, t1, 0x5410u), x23 = prmt(t2, t3, 0x5410u);
      hiw[j] = prmt(x01, x23, 0x7531u);
      low[j] = prmt(x01, x23, 0x6420u);
      // zero-point sums with the same integers the tensor path sees: bytes (z0, z1, z2, z3)
      const uint32_t zb = SYM ? 0x08080808u : prmt(vsw[j][0], vsw[j][1], 0x6420u) & (L::ZM * 0x01010101u);
      Zi[j] = __dp2a_hi(x23, zb, __dp2a_lo(x01, zb, static_cast<unsigned>(Zi[j])));
    }
    sts128(pw_dst, hiw[0], hiw[1], hiw[2], hiw[3]);
    sts128(pw_dst + 144, low[0], low[1], low[2], low[3]);
    __syncwarp();
    uint32_t pb[2][4];   // [e][j] of this lane's column (head gid >> 1, part gid & 1), tokens of chunk tig
    {
      const uint4 t0 = lds128(pw_src), t1 = lds128(pw_src + 16);
      pb[0][0] = t0.x; pb[0][1] = t0.y; pb[0][2] = t0.z; pb[0][3] = t0.w;
      pb[1][0] = t1.x; pb[1][1] = t1.y; pb[1][2] = t1.z; pb[1][3] = t1.w;
    }
    // ---- PV: A = V^T code fields of chunk tig (page tig >> 1, c8 = tig & 1) in place, 16 d rows per tile
#pragma unroll
    for (int ww = 0; ww < 4; ++ww) {
      uint32_t vw[4];
      if (NB == 4) {
        const uint4 t = lds128(st + vc_off + 16 * (ww * 8 * (L::P / 8)));
        vw[0] = t.x; vw[1] = t.y; vw[2] = t.z; vw[3] = t.w;
        if (SYM) {
#pragma unroll
          for (int k = 0; k < 4; ++k) vw[k] = sym_to_asym(vw[k]);
        }
      } else {
        const uint2 t = lds64(st + vc_off + 8 * (ww * 8 * (L::P / 8)));
        vw[0] = t.x; vw[1] = t.y; vw[2] = 0; vw[3] = 0;
      }
#pragma unroll
      for (int mm = 0; mm < 2; ++mm) {
        uint32_t a0, a1, a2, a3;
        if (NB == 4) {   // rows gid (word 2 mm) and gid + 8 (word 2 mm + 1), both scaled by 16
          a0 = (vw[2 * mm] * 16u) & 0xF0F0F0F0u; a2 = vw[2 * mm] & 0xF0F0F0F0u;
          a1 = (vw[2 * mm + 1] * 16u) & 0xF0F0F0F0u; a3 = vw[2 * mm + 1] & 0xF0F0F0F0u;
        } else {         // row gid scaled by 4, row gid + 8 by 64
          a0 = (vw[mm] * 4u) & 0x0C0C0C0Cu; a2 = vw[mm] & 0x0C0C0C0Cu;
          a1 = (vw[mm] * 4u) & 0xC0C0C0C0u; a3 = vw[mm] & 0xC0C0C0C0u;
        }
        const int j = 2 * mm + (ww >> 1);
        mma_u8u8(Oi[mm][ww], a0, a1, a2, a3, pb[0][j], pb[1][j]);
      }
    }
  };

  for (int n = 0; n < nmine; ++n) {
    const int blk = w + NWARP * n, s = n % ST;
    __syncwarp();                       // every lane is done with the stage that block n + ST - 1 overwrites
    issue(n + ST - 1, false);
    cp_wait<ST - 1>();                  // this lane's pieces of block n have landed ...
    __syncwarp();                       // ... and so have everybody else's
    const uint32_t st = ring + s * L::STAGE;
    const int tok0 = c0 + blk * BLK;                                   // absolute position of the block's token 0
    if (tok0 < lo || tok0 + BLK > c1) process(st, tok0, std::true_type{});
    else process(st, tok0, std::false_type{});
  }
  cp_wait<0>();

  // ---- warp epilogue: fold, reduce over the column's lanes, remove the zero points, park in shared memory
  fold(1.f);
  l_run += __shfl_xor_sync(FULLMASK, l_run, 4);
  l_run += __shfl_xor_sync(FULLMASK, l_run, 8);
  l_run += __shfl_xor_sync(FULLMASK, l_run, 16);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    Zf[j] += __shfl_xor_sync(FULLMASK, Zf[j], 4);
    Zf[j] += __shfl_xor_sync(FULLMASK, Zf[j], 8);
    Zf[j] += __shfl_xor_sync(FULLMASK, Zf[j], 16);
  }
  __syncthreads();   // every warp is done with its ring: the scratch aliases it
#pragma unroll
  for (int mm = 0; mm < 2; ++mm)
#pragma unroll
    for (int ww = 0; ww < 4; ++ww) {
      const int j = 2 * mm + (ww >> 1), d = 64 * mm + 16 * ww + gid;
      scr[w * WS + tig * 128 + d] = Of[mm][ww][0] - Zf[j];
      scr[w * WS + tig * 128 + d + 8] = Of[mm][ww][1] - Zf[j];
    }
  if (gid == 0) { scr[w * WS + 512 + tig] = m_run; scr[w * WS + 516 + tig] = l_run; }
  {
    // the slot arithmetic is redone from the block index and the length (read again) rather than kept in registers
    // across the main loop
    const int len_e = __ldcg(p.seq_lens + b);
    int np_e;
    const int chunk_e = row_pieces(p, b, np_e);
    const int nsb_e = len_e > 0 ? min(np_e, max(1, (len_e + chunk_e - 1) / chunk_e)) : 0;
    cta_finish(p, scr, static_cast<int>(blockIdx.z), static_cast<int>(blockIdx.x) / NT, static_cast<int>(blockIdx.x) % NT, NT,
               static_cast<int>(blockIdx.y), nsb_e + has_tail, p.nsplit + has_tail, &last_flag);
  }
}

// ---- host: wave packing.  A launch whose equal CTAs do not fill a whole number of waves of the GPU's resident CTA slots
// ends with a partly empty wave.  The kernel may cut the first `rows_wide` rows into nsplit - 1 wider pieces instead of
// nsplit (same nominal length; the workspace has room for nsplit pieces of every row), which gives two CTA sizes; CTAs are
// dispatched in grid order (rows ascending), i.e. the wide ones first, and a free slot takes the next CTA.  pack_rows
// simulates that dispatch (cost of a CTA = its tokens + a fixed part, window CTAs last) for a few values of rows_wide and
// returns the one with the earliest finish.  Pure host arithmetic, cached for the last shape seen.
constexpr int PACK_C0 = 640;      // fixed cost of a page CTA in token equivalents (q staging, pipeline fill, merge)
constexpr int PACK_CW = 900;      // a BF16 window CTA (<= 256 rows of 512 bytes per kv head) in token equivalents

long long pack_finish(int B, int X, int p, int chunk, int chunk_w, int rows_wide, int slots, bool tail, std::vector<long long>& heap) {
  heap.assign(static_cast<size_t>(slots), 0);                       // min-heap of slot finish times (all equal: a valid heap)
  auto run = [&](long long n, long long cost) {
    for (long long i = 0; i < n; ++i) {
      std::pop_heap(heap.begin(), heap.end(), std::greater<long long>());
      heap.back() += cost;
      std::push_heap(heap.begin(), heap.end(), std::greater<long long>());
    }
  };
  run(static_cast<long long>(rows_wide) * X * (p - 1), chunk_w + PACK_C0);
  run(static_cast<long long>(B - rows_wide) * X * p, chunk + PACK_C0);
  if (tail) run(static_cast<long long>(B) * X, PACK_CW);
  return *std::max_element(heap.begin(), heap.end());
}

int pack_rows(int B, int X, int p, int chunk, int slots, bool tail, int& chunk_w) {
  chunk_w = 0;
  if (p < 2 || slots < 1) return 0;
  const long long nominal = static_cast<long long>(p) * chunk;
  if (nominal % (p - 1) != 0) return 0;
  const long long cw = nominal / (p - 1);
  if (cw % BLK != 0 || cw > MAXPG * 16) return 0;               // pieces start on a 32-token block
  if (static_cast<long long>(B) * X * p > 200000) return 0;        // keep the simulation cheap; such launches have many waves anyway
  static struct { int B, X, p, chunk, slots, tail, rows, cw; } memo = {-1, 0, 0, 0, 0, 0, 0, 0};
  if (memo.B == B && memo.X == X && memo.p == p && memo.chunk == chunk && memo.slots == slots && memo.tail == static_cast<int>(tail)) {
    chunk_w = memo.cw;
    return memo.rows;
  }
  std::vector<long long> heap;
  int best = 0;
  long long best_t = pack_finish(B, X, p, chunk, static_cast<int>(cw), 0, slots, tail, heap);
  const int step = B > 32 ? B / 16 : 1;
  for (int pass = 0; pass < 2; ++pass) {
    const int lo = pass == 0 ? step : std::max(1, best - step + 1), hi = pass == 0 ? B : std::min(B, best + step - 1);
    const int st = pass == 0 ? step : 1;
    int cand_best = best;
    for (int r = lo; r <= hi; r += st) {
      const long long t = pack_finish(B, X, p, chunk, static_cast<int>(cw), r, slots, tail, heap);
      if (t < best_t) { best_t = t; cand_best = r; }
    }
    best = cand_best;
    if (step == 1) break;
  }
  memo = {B, X, p, chunk, slots, static_cast<int>(tail), best, static_cast<int>(cw)};
  chunk_w = static_cast<int>(cw);
  return best;
}

template <int NB, bool KO, int PG, bool SYM = false> int launch_k(DecodeParams p, cudaStream_t st) {
  constexpr int NV = KO ? 3 : 1;
  constexpr int smem = SMap<NB, NV, PG>::TOTAL > TAILM_BYTES ? SMap<NB, NV, PG>::TOTAL : TAILM_BYTES;
  static unsigned long long ready = 0;
  if (!smem_limit_ready(k_decode<NB, KO, PG, SYM>, smem, ready)) return -2;
  static int slots_of[64];                   // resident CTAs of this instantiation per device ordinal (0: not asked yet)
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  if (slots_of[dev] == 0) {
    int sms = 0, occ = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, k_decode<NB, KO, PG, SYM>, 128, smem) != cudaSuccess || occ < 1)
      return -2;
    slots_of[dev] = sms * occ;
  }
  const int NT = (p.G + 3) / 4;
  p.rows_wide = pack_rows(p.B, p.Hkv * NT, p.nsplit, p.chunk, slots_of[dev], p.tail != nullptr, p.chunk_w);
  const dim3 grid(p.Hkv * NT, p.nsplit, p.B * (p.tail != nullptr ? 2 : 1));
  k_decode<NB, KO, PG, SYM><<<grid, 128, smem, st>>>(p);
  return cudaPeekAtLastError() == cudaSuccess ? 0 : -1;
}

}  // namespace

int decode_launch(const DecodeParams& p, cudaStream_t st) {
  if (p.B <= 0) return 0;
  if (p.page != 16 && p.page != 32) return -5;
  if (p.chunk <= 0 || p.chunk % 64 != 0 || p.chunk > MAXPG * 16 || p.nsplit < 1) return -3;
  if (p.page == 32) {
    if (p.sym) return p.key_only ? launch_k<4, true, 32, true>(p, st) : launch_k<4, false, 32, true>(p, st);
    if (p.nb == 4) return p.key_only ? launch_k<4, true, 32>(p, st) : launch_k<4, false, 32>(p, st);
    return p.key_only ? launch_k<2, true, 32>(p, st) : launch_k<2, false, 32>(p, st);
  }
  if (p.sym) return p.key_only ? launch_k<4, true, 16, true>(p, st) : launch_k<4, false, 16, true>(p, st);
  if (p.nb == 4) return p.key_only ? launch_k<4, true, 16>(p, st) : launch_k<4, false, 16>(p, st);
  return p.key_only ? launch_k<2, true, 16>(p, st) : launch_k<2, false, 16>(p, st);
}

int decode_occupancy(int nb, int key_only) {
  int n = 0;
  cudaError_t e;
  if (nb == 4 && key_only) {
    cudaFuncSetAttribute(k_decode<4, true, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMap<4, 3>::TOTAL);
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, k_decode<4, true, 16>, 128, SMap<4, 3>::TOTAL);
  } else if (nb == 4) {
    cudaFuncSetAttribute(k_decode<4, false, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMap<4, 1>::TOTAL);
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, k_decode<4, false, 16>, 128, SMap<4, 1>::TOTAL);
  } else if (key_only) {
    cudaFuncSetAttribute(k_decode<2, true, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMap<2, 3>::TOTAL);
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, k_decode<2, true, 16>, 128, SMap<2, 3>::TOTAL);
  } else {
    cudaFuncSetAttribute(k_decode<2, false, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMap<2, 1>::TOTAL);
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, k_decode<2, false, 16>, 128, SMap<2, 1>::TOTAL);
  }
  return e == cudaSuccess ? n : 0;
}

int decode_status() { return 0; }      // the decode kernel has no device-side wait loop (hardware copy groups only)

}  // namespace fr
