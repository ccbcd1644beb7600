// libflagrot_mq.so for sm_100a: prefix-cached multi-query prefill attention straight from the FlagRot INT4 / INT2 pages.
// C ABI 7 of the reference's integrations/vllm_flagrot/csrc/mq_prefill.cu (declarations + citations:
// include/flagrot_mq.h).  A work item = one tile of query rows (rows / G tokens x the G q heads of a kv head) x a range
// of 64-key blocks; per item the kernel emits unnormalised O (fp32), the row maximum m (log2 units) and the sum l;
// frmq_merge combines the items of a tile.  Key j is visible to the query at position p iff
// kmin <= j <= max(p - shift, ext).
//
// Kernel k_mq<ROWS, NB, KO>: CTA = (item, kv head), ROWS / 16 warps, 16 query rows per warp.  Per 64-key block the four
// page chunks arrive by cp.async (double buffered); the CTA converts them into FP16 tiles K [64][128] (key-only pages:
// per-token inverse H32 / H128 in fp32, one rounding to FP16) and V^T [128][64] ((c - z) exact, one rounding at the
// scale); QK and PV run on the tensor cores (m16n8k16 FP16, fp32 accumulation), online softmax in fp32 (exp2).
#include <cmath>
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "fr_common.cuh"
#include "fr_tc5.cuh"
#include "../../include/flagrot_mq.h"

namespace {

using fr::FULLMASK;
constexpr int D = 128, PAGE = 16, BN = 64, PPB = BN / PAGE;
constexpr int TILE_INTS = 9, ITEM_INTS = 4;
constexpr int KSTR = 136;   // halves per K / q tile row (128 + 8: conflict-free ldmatrix)
constexpr int VSTR = 72;    // halves per V^T tile row (64 + 8)
#define MQ_NEG_INF (-INFINITY)

FR_DEVI uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
FR_DEVI float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
FR_DEVI uint32_t pack_h2(float a, float b) {
  const __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}
FR_DEVI void cp16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
}
FR_DEVI void cp_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
FR_DEVI void cp_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::: "memory"); }
FR_DEVI void ldsm_x4(uint32_t a, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
FR_DEVI void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
FR_DEVI float h16f(uint32_t bits) { return __half2float(__ushort_as_half(static_cast<unsigned short>(bits))); }

// ------------------------------------------------------------------------------------------------ q preparation
// q -> FP16 in the keys' stored basis, times softmax scale * log2(e).  Warp per (row, q head), 4 dims per lane.  Static
// formats: whole-head H128 / 8 on kfull[kv head], then orthonormal H32 on the kmask[kv head] groups (the writer's order).
__global__ void k_mq_prep(const void* q, int q_fp32, long long q_ts, const int* idx, int m, int Hq, int G, const uint8_t* kfull,
                          const uint8_t* kmask, float qscale, __half* q16) {
  const long long w = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= static_cast<long long>(m) * Hq) return;
  const int t = static_cast<int>(w / Hq), hq = static_cast<int>(w % Hq), hk = hq / G;
  const long long row = idx != nullptr ? idx[t] : t;
  float x[4];
  if (q_fp32) {
    const float4 v = *reinterpret_cast<const float4*>(static_cast<const float*>(q) + row * q_ts + hq * D + 4 * lane);
    x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
  } else {
    const uint2 raw = *reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(q) + row * q_ts + hq * D + 4 * lane);
    x[0] = fr::bf16_lo(raw.x); x[1] = fr::bf16_hi(raw.x); x[2] = fr::bf16_lo(raw.y); x[3] = fr::bf16_hi(raw.y);
  }
  if (kfull != nullptr && kfull[hk]) {
    fr::fwht_row_stages(x, lane, 128);
#pragma unroll
    for (int i = 0; i < 4; ++i) x[i] *= 0.125f;
  }
  if (kmask != nullptr) {
    const bool f = kmask[hk * 4 + (lane >> 3)] != 0;
    float y[4] = {x[0], x[1], x[2], x[3]};
    fr::fwht_row_stages(y, lane, 32);
#pragma unroll
    for (int i = 0; i < 4; ++i) x[i] = f ? y[i] * fr::C32 : x[i];
  }
  uint2 v;
  v.x = pack_h2(x[0] * qscale, x[1] * qscale);
  v.y = pack_h2(x[2] * qscale, x[3] * qscale);
  *reinterpret_cast<uint2*>(q16 + (static_cast<long long>(t) * Hq + hq) * D + 4 * lane) = v;
}

// ------------------------------------------------------------------------------------------------ item merge
// grid (tiles, kv heads, rows / 4), warp per query row: combines the items of the row's tile -> bf16 output row (or
// fp32 compact row) and optionally the natural-log LSE (-inf: no visible key).
__global__ void __launch_bounds__(128) k_mq_merge(const int* tiles, const float* opart, const float* ml, int Hkv, int G, int rows,
                                                  void* out, long long o_ts, int out_fp32, float* lse, long long lse_ts) {
  const int* tl = tiles + TILE_INTS * blockIdx.x;
  const int h = blockIdx.y;
  const int crow0 = tl[1], orow0 = tl[2], ntok = tl[3], item0 = tl[6], nitem = tl[7];
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.z * 4 + (threadIdx.x >> 5);
  const int TQ = rows / G, Hq = Hkv * G;
  const int t = r / G;
  if (r >= TQ * G || t >= ntok) return;
  const int hq = h * G + r % G;
  const long long b0 = (static_cast<long long>(item0) * Hkv + h) * rows + r;
  const long long bs = static_cast<long long>(Hkv) * rows;
  float M = MQ_NEG_INF;
  for (int s = lane; s < nitem; s += 32) M = fmaxf(M, ml[2 * (b0 + s * bs)]);
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) M = fmaxf(M, __shfl_xor_sync(FULLMASK, M, o));
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float L = 0.f;
  if (M != MQ_NEG_INF) {
    for (int s = lane; s < nitem; s += 32) {
      const float2 v = *reinterpret_cast<const float2*>(ml + 2 * (b0 + s * bs));
      L += ex2(v.x - M) * v.y;
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) L += __shfl_xor_sync(FULLMASK, L, o);
    for (int s = 0; s < nitem; ++s) {
      const long long b = b0 + s * bs;
      const float wgt = ex2(ml[2 * b] - M);
      const float4 x = *reinterpret_cast<const float4*>(opart + b * D + 4 * lane);
      acc.x += wgt * x.x; acc.y += wgt * x.y; acc.z += wgt * x.z; acc.w += wgt * x.w;
    }
    const float inv = L > 0.f ? 1.f / L : 0.f;
    acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
  }
  if (out_fp32) {
    *reinterpret_cast<float4*>(static_cast<float*>(out) + (static_cast<long long>(crow0 + t) * Hq + hq) * D + 4 * lane) = acc;
  } else {
    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(out) + static_cast<long long>(orow0 + t) * o_ts + hq * D + 4 * lane;
    const __nv_bfloat162 a = __floats2bfloat162_rn(acc.x, acc.y), b = __floats2bfloat162_rn(acc.z, acc.w);
    uint2 v;
    v.x = *reinterpret_cast<const uint32_t*>(&a);
    v.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>(dst) = v;
  }
  if (lse != nullptr && lane == 0)
    lse[hq * lse_ts + crow0 + t] = (M == MQ_NEG_INF || L <= 0.f) ? MQ_NEG_INF : (M + log2f(L)) * 0.6931471805599453f;
}

// ------------------------------------------------------------------------------------------------ BF16 window parts
// row d of the gathered K / V comes from map[d] = (kind << 32) | row: kind 0 sink rows, 1 earlier-window rows (both
// [*, 2 Hkv, 128], K rows then V rows), 2 the batch's own K / V rows (strided).
__global__ void __launch_bounds__(128) k_win_gather(const long long* map, int nk, const __nv_bfloat16* sinkb, const __nv_bfloat16* preb,
                                                    const __nv_bfloat16* kch, long long k_ts, const __nv_bfloat16* vch, long long v_ts,
                                                    int Hkv, __nv_bfloat16* kw, __nv_bfloat16* vw) {
  const int d = blockIdx.x;
  if (d >= nk) return;
  const long long code = map[d];
  const int kind = static_cast<int>(code >> 32);
  const long long row = code & 0xffffffffLL;
  const int nvec = Hkv * D / 8;
  const uint4 *ks, *vs;
  if (kind == 2) {
    ks = reinterpret_cast<const uint4*>(kch + row * k_ts);
    vs = reinterpret_cast<const uint4*>(vch + row * v_ts);
  } else {
    const __nv_bfloat16* b = (kind == 0 ? sinkb : preb) + row * 2LL * Hkv * D;
    ks = reinterpret_cast<const uint4*>(b);
    vs = reinterpret_cast<const uint4*>(b + Hkv * D);
  }
  uint4* kd = reinterpret_cast<uint4*>(kw + static_cast<long long>(d) * Hkv * D);
  uint4* vd = reinterpret_cast<uint4*>(vw + static_cast<long long>(d) * Hkv * D);
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) { kd[i] = ks[i]; vd[i] = vs[i]; }
}

// per (compact row c, q head): LSE merge (natural log) of the page part (fp32 o, lse), the window part (bf16 o, lse) and the
// sink part (fp32 softmax over the keys j < min(S, len) with j <= pos - W) -> bf16 output row idx[c]
__global__ void __launch_bounds__(128) k_bf_merge(int m, int Hq, int Hkv, const __nv_bfloat16* q, long long q_ts, const long long* idx,
                                                  const float* o_p, const float* lse_p, const __nv_bfloat16* o_w, const float* lse_w,
                                                  const __nv_bfloat16* sk, const long long* row_req, const long long* row_pos,
                                                  const long long* sk_len, int S, int W, float scale, __nv_bfloat16* out, long long o_ts) {
  const int c = blockIdx.x;
  const int hq = blockIdx.y * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (c >= m || hq >= Hq) return;
  const int G = Hq / Hkv, kvh = hq / G;
  const long long brow = idx[c];
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  float M = MQ_NEG_INF, L = 0.f;
  auto add = [&](float l, const float (&x)[4]) {     // running (acc, L) at log-scale M  (+)  normalised x at log-scale l
    if (l == MQ_NEG_INF || isinf(l) || l != l) return;
    const float nm = fmaxf(M, l);
    const float a = M == MQ_NEG_INF ? 0.f : expf(M - nm), b = expf(l - nm);
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[e] = acc[e] * a + x[e] * b;
    L = L * a + b;
    M = nm;
  };
  {
    const float4 v = *reinterpret_cast<const float4*>(o_p + (static_cast<long long>(c) * Hq + hq) * D + 4 * lane);
    const float x[4] = {v.x, v.y, v.z, v.w};
    add(lse_p[static_cast<long long>(hq) * m + c], x);
  }
  if (o_w != nullptr) {
    const uint2 raw = *reinterpret_cast<const uint2*>(o_w + (static_cast<long long>(c) * Hq + hq) * D + 4 * lane);
    const float x[4] = {fr::bf16_lo(raw.x), fr::bf16_hi(raw.x), fr::bf16_lo(raw.y), fr::bf16_hi(raw.y)};
    add(lse_w[static_cast<long long>(hq) * m + c], x);
  }
  if (sk != nullptr) {
    const long long rq = row_req[c], lim = row_pos[c] - W, nsk = sk_len[rq];
    const uint2 qr = *reinterpret_cast<const uint2*>(q + brow * q_ts + static_cast<long long>(hq) * D + 4 * lane);
    const float qv[4] = {fr::bf16_lo(qr.x), fr::bf16_hi(qr.x), fr::bf16_lo(qr.y), fr::bf16_hi(qr.y)};
    float sm = MQ_NEG_INF, sl = 0.f, so[4] = {0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < S; ++j) {
      if (j >= nsk || j > lim) break;
      const uint2 kr = *reinterpret_cast<const uint2*>(sk + ((rq * S + j) * 2LL * Hkv + kvh) * D + 4 * lane);
      const uint2 vr = *reinterpret_cast<const uint2*>(sk + ((rq * S + j) * 2LL * Hkv + Hkv + kvh) * D + 4 * lane);
      float dot = qv[0] * fr::bf16_lo(kr.x) + qv[1] * fr::bf16_hi(kr.x) + qv[2] * fr::bf16_lo(kr.y) + qv[3] * fr::bf16_hi(kr.y);
#pragma unroll
      for (int o = 16; o >= 1; o >>= 1) dot += __shfl_xor_sync(FULLMASK, dot, o);
      const float s = dot * scale;
      const float nm = fmaxf(sm, s);
      const float a = sm == MQ_NEG_INF ? 0.f : expf(sm - nm), b = expf(s - nm);
      so[0] = so[0] * a + fr::bf16_lo(vr.x) * b; so[1] = so[1] * a + fr::bf16_hi(vr.x) * b;
      so[2] = so[2] * a + fr::bf16_lo(vr.y) * b; so[3] = so[3] * a + fr::bf16_hi(vr.y) * b;
      sl = sl * a + b;
      sm = nm;
    }
    if (sm != MQ_NEG_INF) {
      const float inv = 1.f / sl;
#pragma unroll
      for (int e = 0; e < 4; ++e) so[e] *= inv;
      add(sm + logf(sl), so);
    }
  }
  const float inv = L > 0.f ? 1.f / L : 0.f;
  const __nv_bfloat162 a = __floats2bfloat162_rn(acc[0] * inv, acc[1] * inv), b = __floats2bfloat162_rn(acc[2] * inv, acc[3] * inv);
  uint2 v;
  v.x = *reinterpret_cast<const uint32_t*>(&a);
  v.y = *reinterpret_cast<const uint32_t*>(&b);
  *reinterpret_cast<uint2*>(out + brow * o_ts + static_cast<long long>(hq) * D + 4 * lane) = v;
}

// ------------------------------------------------------------------------------------------------ attention kernel
struct MqParams {
  const __half* q;          // [m, Hq, 128] FP16, stored basis, pre-scaled by softmax scale * log2(e)
  const uint8_t* pool;      // [pages, Hkv, chunk]
  long long page_stride;    // bytes
  const int* bt;            // block table [rows, bt_stride]
  long long bt_stride;
  const int* tiles;         // [ntiles, 9]: bt row, compact row 0, output row 0, tokens, position 0, page keys, item 0, items, ext
  const int* items;         // [nitems, 4]: tile, first key block, end key block, -
  int Hkv, G, shift, kmin;
  float* opart;             // [nitems, Hkv, ROWS, 128]
  float* ml;                // [nitems, Hkv, ROWS, 2]
};

template <int NB> struct MLay {
  static constexpr int CBY = NB == 4 ? 64 : 32;
  static constexpr int CHUNK = (2 * CBY + 16) * PAGE;            // 2304 | 1280
  static constexpr int V_OFF = CBY * PAGE, KS_OFF = 2 * CBY * PAGE, VS_OFF = KS_OFF + 8 * PAGE;
  static constexpr uint32_t ZM = NB == 4 ? 15u : 3u;
};
template <int ROWS, int NB> struct MSmem {
  static constexpr int QS = 0, KS = QS + ROWS * KSTR * 2, VT = KS + BN * KSTR * 2, RAW = VT + D * VSTR * 2;
  static constexpr int TOTAL = RAW + 2 * PPB * MLay<NB>::CHUNK;
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
FR_DEVI uint2 lds64(uint32_t a) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "r"(a));
  return v;
}
FR_DEVI uint4 lds128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
FR_DEVI void sts64(uint32_t a, uint32_t x, uint32_t y) { asm volatile("st.shared.v2.u32 [%0], {%1,%2};\n" ::"r"(a), "r"(x), "r"(y) : "memory"); }
FR_DEVI void sts128(uint32_t a, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(a), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
FR_DEVI uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;\n" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
FR_DEVI uint32_t hsub2u(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("sub.rn.f16x2 %0, %1, %2;\n" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
FR_DEVI uint32_t hmul2u(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.f16x2 %0, %1, %2;\n" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

// K tile [64 keys][128] FP16 from the raw pages: warp per key, lane = dims 4 l .. 4 l + 3.  (c - z) * s exactly in fp32;
// key-only pages: the token's inverse transform (whole-head H128 if its flag is set, else H32 of the flagged groups) in
// fp32; one rounding to FP16.  Keys >= nvalid are written as zeros.
template <int NB, bool KO, int NW>
FR_DEVI void convert_k(uint32_t raw, uint32_t ks, int nvalid, int warp, int lane) {
  using L = MLay<NB>;
  const int j = lane >> 3, isb = (lane >> 2) & 1, tg = lane & 3;
  for (int tok = warp; tok < BN; tok += NW) {
    const uint32_t dst = ks + tok * (KSTR * 2) + lane * 8;
    if (tok >= nvalid) { sts64(dst, 0u, 0u); continue; }
    const uint32_t rc = raw + (tok >> 4) * L::CHUNK;
    const int pos = tok & 15;
    uint32_t c[4];
    if (NB == 4) {
      const uint32_t w = lds32(rc + 64 * pos + 16 * tg + 4 * j) >> (4 * isb);
#pragma unroll
      for (int i = 0; i < 4; ++i) c[i] = (w >> (8 * i)) & 15u;
    } else {
      const uint32_t w = lds32(rc + 32 * (pos ^ ((pos >> 1) & 2)) + 8 * tg + 4 * (j >> 1)) >> (4 * (j & 1) + 2 * isb);
#pragma unroll
      for (int i = 0; i < 4; ++i) c[i] = (w >> (8 * i)) & 3u;
    }
    const uint32_t kw = lds16(rc + L::KS_OFF + 8 * pos + 2 * j);
    const float sc = h16f(kw & 0x7FFFu);
    const int z = static_cast<int>(kw & L::ZM);
    float x[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) x[i] = static_cast<float>(static_cast<int>(c[i]) - z) * sc;
    if constexpr (KO) {
      const bool ffl = (lds16(rc + L::VS_OFF + 2 * (8 * (pos >> 3) + fr::vslot8(pos))) & 0x8000u) != 0;   // warp-uniform
      const bool hfl = (kw & 0x8000u) != 0;
      if (ffl) {
        fr::fwht_row_stages(x, lane, 128);
#pragma unroll
        for (int i = 0; i < 4; ++i) x[i] *= fr::C128;
      } else if (__any_sync(FULLMASK, hfl)) {
        float y[4] = {x[0], x[1], x[2], x[3]};
        fr::fwht_row_stages(y, lane, 32);
#pragma unroll
        for (int i = 0; i < 4; ++i) x[i] = hfl ? y[i] * fr::C32 : x[i];
      }
    }
    sts64(dst, pack_h2(x[0], x[1]), pack_h2(x[2], x[3]));
  }
}

// V^T tile [128 dims][64 keys] FP16: one work unit = the 8 tokens of one (page, dim) code word -> 16 contiguous bytes.
// (c - z) exact in FP16, one rounding at the scale.  Keys >= nvalid are zeros.
template <int NB, int NT>
FR_DEVI void convert_v(uint32_t raw, uint32_t vt, int nvalid, int tid) {
  using L = MLay<NB>;
  for (int it = tid; it < PPB * 64 * 4; it += NT) {
    const int pg = it >> 8, e = (it >> 2) & 63, s = it & 3;
    const int c8 = e & 1, gid = (e >> 1) & 7, w = e >> 4;
    const int m = s >> 1, r8 = s & 1;
    const int d = 64 * m + 16 * w + gid + 8 * r8, j = 2 * m + (w >> 1);
    const uint32_t rc = raw + pg * L::CHUNK;
    uint32_t word;
    if (NB == 4) word = lds32(rc + L::V_OFF + 16 * e + 4 * s);
    else word = lds32(rc + L::V_OFF + 8 * e + 4 * m) >> (4 * r8);
    const uint4 sw = lds128(rc + L::VS_OFF + 2 * (j * PAGE + 8 * c8));     // scale words of tokens 0 2 4 6 | 1 3 5 7
    const uint32_t sp[4] = {prmt(sw.x, sw.z, 0x5410u), prmt(sw.x, sw.z, 0x7632u), prmt(sw.y, sw.w, 0x5410u), prmt(sw.y, sw.w, 0x7632u)};
    uint32_t o[4];
    const int t0 = 16 * pg + 8 * c8;
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
    sts128(vt + d * (VSTR * 2) + t0 * 2, o[0], o[1], o[2], o[3]);
  }
}

template <int ROWS, int NB, bool KO>
__global__ void __launch_bounds__(ROWS * 2) k_mq(const MqParams p) {
  using L = MLay<NB>;
  using S = MSmem<ROWS, NB>;
  constexpr int NW = ROWS / 16, NT = ROWS * 2;
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t sb = smem_u32(smem);
  const uint32_t qs = sb + S::QS, ks = sb + S::KS, vt = sb + S::VT;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g8 = lane >> 2, c4 = lane & 3;
  const int item = blockIdx.x, h = blockIdx.y;
  const int* it = p.items + ITEM_INTS * item;
  const int* tl = p.tiles + TILE_INTS * it[0];
  const int req = tl[0], crow0 = tl[1], ntok = tl[3], pos0 = tl[4], nk = tl[5], ext = tl[8];
  const int G = p.G, Hq = p.Hkv * G, TQ = ROWS / G;
  const int* bt = p.bt + static_cast<long long>(req) * p.bt_stride;
  // keys of this item: blocks [kb0, kb1), clipped to the pages and to the last token's causal limit
  const int kend = min(min(nk, it[2] * BN), max(pos0 + ntok - p.shift, ext + 1));
  const int kb0 = it[1];
  const int kb1 = kend > kb0 * BN ? (kend + BN - 1) / BN : kb0;
  int rpos[2];
  bool rval[2];
#pragma unroll
  for (int rh = 0; rh < 2; ++rh) {
    const int r = warp * 16 + g8 + 8 * rh;
    const int t = r / G;
    rval[rh] = r < TQ * G && t < ntok;
    rpos[rh] = max(pos0 + t - p.shift, ext);        // last visible key of the row
  }
  for (int c = tid; c < ROWS * (D / 8); c += NT) {   // q tile (zero rows for padding)
    const int r = c >> 4, c16 = c & 15, t = r / G;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r < TQ * G && t < ntok)
      v = *reinterpret_cast<const uint4*>(p.q + (static_cast<long long>(crow0 + t) * Hq + h * G + r % G) * D + 8 * c16);
    sts128(qs + r * (KSTR * 2) + c16 * 16, v.x, v.y, v.z, v.w);
  }
  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float mrow[2] = {MQ_NEG_INF, MQ_NEG_INF}, lrow[2] = {0.f, 0.f};

  const uint8_t* poolh = p.pool + static_cast<long long>(h) * L::CHUNK;
  auto load_raw = [&](int kb, int buf) {
    const int npg = min(PPB, (kend - kb * BN + PAGE - 1) / PAGE);
    const uint32_t dst = sb + S::RAW + buf * (PPB * L::CHUNK);
    for (int s = tid; s < npg * (L::CHUNK / 16); s += NT) {
      const int pg = s / (L::CHUNK / 16), off = (s % (L::CHUNK / 16)) * 16;
      cp16(dst + pg * L::CHUNK + off, poolh + static_cast<long long>(bt[kb * PPB + pg]) * p.page_stride + off);
    }
    cp_commit();
  };
  if (kb0 < kb1) load_raw(kb0, 0);
  for (int kb = kb0; kb < kb1; ++kb) {
    const int buf = (kb - kb0) & 1;
    cp_wait_all();
    __syncthreads();                                  // raw block landed; the previous block's tiles are consumed
    if (kb + 1 < kb1) load_raw(kb + 1, buf ^ 1);
    const uint32_t raw = sb + S::RAW + buf * (PPB * L::CHUNK);
    const int nvalid = kend - kb * BN;
    convert_k<NB, KO, NW>(raw, ks, nvalid, warp, lane);
    convert_v<NB, NT>(raw, vt, nvalid, tid);
    __syncthreads();
    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      uint32_t qa[4];
      ldsm_x4(qs + (warp * 16 + (lane & 15)) * (KSTR * 2) + (16 * kk + 8 * (lane >> 4)) * 2, qa[0], qa[1], qa[2], qa[3]);
#pragma unroll
      for (int nt = 0; nt < 8; nt += 2) {
        const int mi = lane >> 3, ri = lane & 7;
        uint32_t b0, b1, b2, b3;
        ldsm_x4(ks + (8 * (nt + (mi >> 1)) + ri) * (KSTR * 2) + (16 * kk + 8 * (mi & 1)) * 2, b0, b1, b2, b3);
        mma16816(s[nt], qa, b0, b1);
        mma16816(s[nt + 1], qa, b2, b3);
      }
    }
    const int j0 = kb * BN + 2 * c4;
    float alpha[2];
#pragma unroll
    for (int rh = 0; rh < 2; ++rh) {
      const int lim = min(kend - 1, rpos[rh]);
      float mx = MQ_NEG_INF;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int j = j0 + 8 * nt + e;
          float& x = s[nt][2 * rh + e];
          x = (rval[rh] && j <= lim && j >= p.kmin) ? x : MQ_NEG_INF;
          mx = fmaxf(mx, x);
        }
      mx = fmaxf(mx, __shfl_xor_sync(FULLMASK, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(FULLMASK, mx, 2));
      const float mn = fmaxf(mrow[rh], mx);
      const float base = mn == MQ_NEG_INF ? 0.f : mn;
      alpha[rh] = ex2(mrow[rh] - base);
      mrow[rh] = mn;
      float sum = 0.f;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          float& x = s[nt][2 * rh + e];
          x = ex2(x - base);
          sum += x;
        }
      lrow[rh] = lrow[rh] * alpha[rh] + sum;
    }
#pragma unroll
    for (int dn = 0; dn < 16; ++dn) { o[dn][0] *= alpha[0]; o[dn][1] *= alpha[0]; o[dn][2] *= alpha[1]; o[dn][3] *= alpha[1]; }
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      uint32_t pa[4];
      pa[0] = pack_h2(s[2 * kk][0], s[2 * kk][1]);
      pa[1] = pack_h2(s[2 * kk][2], s[2 * kk][3]);
      pa[2] = pack_h2(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      pa[3] = pack_h2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int dn = 0; dn < 16; dn += 2) {
        const int mi = lane >> 3, ri = lane & 7;
        uint32_t b0, b1, b2, b3;
        ldsm_x4(vt + (8 * (dn + (mi >> 1)) + ri) * (VSTR * 2) + (16 * kk + 8 * (mi & 1)) * 2, b0, b1, b2, b3);
        mma16816(o[dn], pa, b0, b1);
        mma16816(o[dn + 1], pa, b2, b3);
      }
    }
  }
#pragma unroll
  for (int rh = 0; rh < 2; ++rh) {   // partials: unnormalised O, m (log2 units), l
    float l = lrow[rh];
    l += __shfl_xor_sync(FULLMASK, l, 1);
    l += __shfl_xor_sync(FULLMASK, l, 2);
    if (!rval[rh]) continue;
    const int r = warp * 16 + g8 + 8 * rh;
    const long long base = (static_cast<long long>(item) * p.Hkv + h) * ROWS + r;
    float* op = p.opart + base * D + 2 * c4;
#pragma unroll
    for (int dn = 0; dn < 16; ++dn) *reinterpret_cast<float2*>(op + 8 * dn) = make_float2(o[dn][2 * rh], o[dn][2 * rh + 1]);
    if (c4 == 0) *reinterpret_cast<float2*>(p.ml + base * 2) = make_float2(mrow[rh], l);
  }
}

template <int ROWS, int NB, bool KO>
int launch_mq(const MqParams& p, int nitems, cudaStream_t st) {
  constexpr int smem = MSmem<ROWS, NB>::TOTAL;
  static bool set = false;
  if (!set) {
    if (cudaFuncSetAttribute(k_mq<ROWS, NB, KO>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -2;
    set = true;
  }
  k_mq<ROWS, NB, KO><<<dim3(nitems, p.Hkv), ROWS * 2, smem, st>>>(p);
  return cudaPeekAtLastError() == cudaSuccess ? 0 : -1;
}

#include "mq_tc.cuh"

}  // namespace

extern "C" {

int frmq_abi_version() { return 7; }
const char* frmq_last_error() { return cudaGetErrorString(cudaGetLastError()); }
int frmq_smem_bytes() { return TQMap<4, 3>::TOTAL; }
/* no counterpart in the reference: 0, or the source line of a bounded device-side wait that gave up (sticky) */
int frmq_device_status() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_mq_status, sizeof(int));
  return v;
}

int frmq_prep_q(const void* q, int q_fp32, long long q_ts, const int* idx, int m, int Hq, int G, const uint8_t* kfull,
                const uint8_t* kmask, float qscale, void* q16, int Dh, void* stream) {
  if (m <= 0) return 0;
  if (Dh != D) return -4;
  const long long warps = static_cast<long long>(m) * Hq;
  k_mq_prep<<<static_cast<unsigned>((warps * 32 + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      q, q_fp32, q_ts, idx, m, Hq, G, kfull, kmask, qscale, static_cast<__half*>(q16));
  return cudaPeekAtLastError() == cudaSuccess ? 0 : -1;
}

int frmq_attn(const void* q16, const uint8_t* pool, long long page_stride, const int* bt, long long bt_stride, const int* tiles,
              const int* items, int nitems, int Hkv, int G, int shift, int konly, float* opart, float* ml, int kernel, int Dh,
              void* stream, int kmin) {
  if (nitems <= 0) return 0;
  if (Dh != D) return -4;
  if (G < 1 || G > 64) return -3;
  if (kernel < 1 || kernel > 3) return -3;
  MqParams p{static_cast<const __half*>(q16), pool, page_stride, bt, bt_stride, tiles, items, Hkv, G, shift, kmin, opart, ml};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool ko = (konly & 1) != 0, b2 = (konly & 2) != 0;
  if (kernel == 1) {          // 64 rows per tile
    if (b2) return ko ? launch_mq<64, 2, true>(p, nitems, st) : launch_mq<64, 2, false>(p, nitems, st);
    return ko ? launch_mq<64, 4, true>(p, nitems, st) : launch_mq<64, 4, false>(p, nitems, st);
  }
  if (kernel == 3) {          // tcgen05 / tensor memory
    if (b2) return ko ? launch_mq_tc<2, true>(p, nitems, st) : launch_mq_tc<2, false>(p, nitems, st);
    return ko ? launch_mq_tc<4, true>(p, nitems, st) : launch_mq_tc<4, false>(p, nitems, st);
  }
  if (b2) return ko ? launch_mq<128, 2, true>(p, nitems, st) : launch_mq<128, 2, false>(p, nitems, st);
  return ko ? launch_mq<128, 4, true>(p, nitems, st) : launch_mq<128, 4, false>(p, nitems, st);
}

int frmq_merge(const int* tiles, int ntiles, const float* opart, const float* ml, int Hkv, int G, int rows, void* out,
               long long o_ts, int out_fp32, float* lse, long long lse_ts, int Dh, void* stream) {
  if (ntiles <= 0) return 0;
  if (Dh != D) return -4;
  k_mq_merge<<<dim3(ntiles, Hkv, rows / 4), 128, 0, static_cast<cudaStream_t>(stream)>>>(tiles, opart, ml, Hkv, G, rows, out, o_ts,
                                                                                        out_fp32, lse, lse_ts);
  return cudaPeekAtLastError() == cudaSuccess ? 0 : -1;
}

int frmq_win_gather(const long long* map, int nk, const void* sinkb, const void* preb, const void* kch, long long k_ts,
                    const void* vch, long long v_ts, int Hkv, void* kw, void* vw, int Dh, void* stream) {
  if (nk <= 0) return 0;
  if (Dh != D) return -4;
  using B = __nv_bfloat16;
  k_win_gather<<<nk, 128, 0, static_cast<cudaStream_t>(stream)>>>(map, nk, static_cast<const B*>(sinkb), static_cast<const B*>(preb),
                                                                 static_cast<const B*>(kch), k_ts, static_cast<const B*>(vch), v_ts,
                                                                 Hkv, static_cast<B*>(kw), static_cast<B*>(vw));
  return cudaPeekAtLastError() == cudaSuccess ? 0 : -1;
}

int frmq_bf_merge(int m, int Hq, int Hkv, const void* q, long long q_ts, const long long* idx, const float* o_p, const float* lse_p,
                  const void* o_w, const float* lse_w, const void* sk, const long long* row_req, const long long* row_pos,
                  const long long* sk_len, int S, int W, float scale, void* out, long long o_ts, int Dh, void* stream) {
  if (m <= 0) return 0;
  if (Dh != D) return -4;
  using B = __nv_bfloat16;
  k_bf_merge<<<dim3(m, (Hq + 3) / 4), 128, 0, static_cast<cudaStream_t>(stream)>>>(
      m, Hq, Hkv, static_cast<const B*>(q), q_ts, idx, o_p, lse_p, static_cast<const B*>(o_w), lse_w, static_cast<const B*>(sk),
      row_req, row_pos, sk_len, S, W, scale, static_cast<B*>(out), o_ts);
  return cudaPeekAtLastError() == cudaSuccess ? 0 : -1;
}

}  // extern "C"
