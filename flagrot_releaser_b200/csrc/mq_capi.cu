// libflagrot_mq.so for sm_100a: prefix-cached multi-query prefill attention straight from the FlagRot INT4 / INT2 pages.
// C ABI 7 of the reference's integrations/vllm_flagrot/csrc/mq_prefill.cu (declarations + citations:
// include/flagrot_mq.h).  A work item = one tile of query rows (rows / G tokens x the G q heads of a kv head) x a range
// of 64-key blocks; per item the attention kernel emits unnormalised O (fp32), the row maximum m (log2 units) and the
// sum l; frmq_merge combines the items of a tile.  Key j is visible to the query at position p iff
// kmin <= j <= max(p - shift, ext).
//
// Kernels of this file: k_q_stage (q -> FP16 in the keys' stored basis), k_item_fold (single-pass combine of a tile's
// items), k_rows_collect (BF16 window rows from three sources), k_bf_merge (page + window + sink parts).  The attention
// kernel itself is k_mq_tc (mq_tc.cuh, tcgen05 / tensor memory) for every plan: the plan's `kernel` number only decides
// how many query rows a tile has (64 or 128), which the host planner and the partial layout fix, not the instruction set.
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
#define MQ_NEG_INF (-INFINITY)

FR_DEVI uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
FR_DEVI float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
FR_DEVI uint32_t bf2_bits(float a, float b) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// ------------------------------------------------------------------------------------------------ q staging
// One CTA per query token, warp w takes q heads w, w + 8, ...; a head row sits 4 dims per lane.  The row is read as fp32
// or bf16 (FP32IN), moved into the basis the keys are stored in and written as FP16 times `gain` (softmax scale * log2 e).
// Static formats: heads with kfull[kv head] take the whole-head transform H128 / 8 (the writer's bf16(H128 x / 16) times
// 2: q . k is then unchanged up to the key's own rounding), and groups with kmask[kv head][group] the orthonormal H32,
// in the writer's order (whole head first).  `pick` maps the compact row to the caller's row of q (null: identity).
template <bool FP32IN>
__global__ void __launch_bounds__(256) k_q_stage(const void* __restrict__ src, long long src_ts, const int* __restrict__ pick,
                                                 int Hq, int G, const uint8_t* __restrict__ kfull, const uint8_t* __restrict__ kmask,
                                                 float gain, __half* __restrict__ dst) {
  const int tok = blockIdx.x, lane = threadIdx.x & 31;
  const long long srow = pick != nullptr ? pick[tok] : tok;
  for (int hq = threadIdx.x >> 5; hq < Hq; hq += 8) {
    const int kvh = hq / G;
    float v[4];
    if constexpr (FP32IN) {
      const float4 f = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(src) + srow * src_ts + hq * D) + lane);
      v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    } else {
      const uint2 u = __ldg(reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(src) + srow * src_ts + hq * D) + lane);
      v[0] = fr::bf16_lo(u.x); v[1] = fr::bf16_hi(u.x); v[2] = fr::bf16_lo(u.y); v[3] = fr::bf16_hi(u.y);
    }
    if (kfull != nullptr && kfull[kvh] != 0) {           // warp-uniform
      fr::fwht_row_stages(v, lane, 128);
#pragma unroll
      for (int i = 0; i < 4; ++i) v[i] *= 0.125f;        // exact (power of two)
    }
    const bool blockrot = kmask != nullptr && kmask[kvh * 4 + (lane >> 3)] != 0;
    if (__any_sync(FULLMASK, blockrot)) {                // the butterflies stay inside a group's 8 lanes
      float r[4] = {v[0], v[1], v[2], v[3]};
      fr::fwht_row_stages(r, lane, 32);
      if (blockrot) {
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = r[i] * fr::C32;
      }
    }
    const __half2 lo = __floats2half2_rn(v[0] * gain, v[1] * gain), hi = __floats2half2_rn(v[2] * gain, v[3] * gain);
    uint2 o;
    o.x = *reinterpret_cast<const uint32_t*>(&lo);
    o.y = *reinterpret_cast<const uint32_t*>(&hi);
    reinterpret_cast<uint2*>(dst + (static_cast<long long>(tok) * Hq + hq) * D)[lane] = o;
  }
}

// ------------------------------------------------------------------------------------------------ item fold
// Combines the partials of a tile's items in ONE pass: a running reference m, denominator and row that are rescaled
// whenever an item brings a larger m (the same recurrence the attention kernel runs over key blocks), so no separate
// maximum pass and no cross-lane traffic: every lane of a warp reads the item's (m, l) pair itself (one broadcast load)
// and owns 4 dims of the row.  CTA = (tile, kv head), 8 warps striding over the tile's query rows; the next item's
// row is requested before the current one is folded in.
__global__ void __launch_bounds__(256) k_item_fold(const int* __restrict__ tiles, const float* __restrict__ opart,
                                                   const float* __restrict__ ml, int Hkv, int G, int rows, void* __restrict__ out,
                                                   long long o_ts, int out_fp32, float* __restrict__ lse, long long lse_ts) {
  const int* tl = tiles + TILE_INTS * blockIdx.x;
  const int kvh = blockIdx.y, lane = threadIdx.x & 31;
  const int crow0 = __ldg(tl + 1), orow0 = __ldg(tl + 2), ntok = __ldg(tl + 3), first = __ldg(tl + 6), count = __ldg(tl + 7);
  const int used = min(ntok, rows / G) * G;                          // query rows of the tile that carry a token
  const long long istride = static_cast<long long>(Hkv) * rows;      // partial rows between consecutive items
  for (int r = threadIdx.x >> 5; r < used; r += 8) {
    const long long prow = (static_cast<long long>(first) * Hkv + kvh) * rows + r;
    float m = MQ_NEG_INF, den = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 nxt = count > 0 ? __ldcs(reinterpret_cast<const float4*>(opart + prow * D) + lane) : acc;
    for (int s = 0; s < count; ++s) {
      const float4 cur = nxt;
      const long long pr = prow + s * istride;
      if (s + 1 < count) nxt = __ldcs(reinterpret_cast<const float4*>(opart + (pr + istride) * D) + lane);
      const float2 st = __ldcs(reinterpret_cast<const float2*>(ml) + pr);
      if (st.x == MQ_NEG_INF) continue;                               // the item saw no visible key for this row
      float wgt = 1.f;
      if (st.x > m) {                                                 // new reference: bring what has been folded so far down to it
        const float down = ex2(m - st.x);                             // m = -inf: 0
        acc.x *= down; acc.y *= down; acc.z *= down; acc.w *= down;
        den *= down;
        m = st.x;
      } else {
        wgt = ex2(st.x - m);
      }
      acc.x = fmaf(wgt, cur.x, acc.x); acc.y = fmaf(wgt, cur.y, acc.y);
      acc.z = fmaf(wgt, cur.z, acc.z); acc.w = fmaf(wgt, cur.w, acc.w);
      den = fmaf(wgt, st.y, den);
    }
    const float norm = den > 0.f ? 1.f / den : 0.f;
    acc.x *= norm; acc.y *= norm; acc.z *= norm; acc.w *= norm;
    const int t = r / G, hq = kvh * G + r % G, Hq = Hkv * G;
    if (out_fp32) {
      reinterpret_cast<float4*>(static_cast<float*>(out) + (static_cast<long long>(crow0 + t) * Hq + hq) * D)[lane] = acc;
    } else {
      uint2 o;
      o.x = bf2_bits(acc.x, acc.y);
      o.y = bf2_bits(acc.z, acc.w);
      reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(out) + static_cast<long long>(orow0 + t) * o_ts + hq * D)[lane] = o;
    }
    if (lse != nullptr && lane == 0)                                  // natural log; -inf: the row had no visible key at all
      lse[hq * lse_ts + crow0 + t] = den > 0.f ? (m + log2f(den)) * 0.6931471805599453f : MQ_NEG_INF;
  }
}

// ------------------------------------------------------------------------------------------------ BF16 window parts
// Collects the K and V rows of the window attention call.  Destination row d takes its K row and its V row from the
// source that where[d] = (kind << 32) | row names: kind 0 the sink rows, kind 1 the window rows gathered by the cache
// update (both [*, 2 Hkv, 128]: K heads then V heads), kind 2 the step's own K / V rows (token strides k_ts / v_ts).
// Flat grid-stride copy: one 16-byte vector per thread and step over all (row, K | V, vector) triples, so a launch with
// few rows still spreads over the SMs.
__global__ void __launch_bounds__(256) k_rows_collect(const long long* __restrict__ where, long long total, int vecs,
                                                      const __nv_bfloat16* __restrict__ sinks, const __nv_bfloat16* __restrict__ prior,
                                                      const __nv_bfloat16* __restrict__ knew, long long k_ts,
                                                      const __nv_bfloat16* __restrict__ vnew, long long v_ts,
                                                      __nv_bfloat16* __restrict__ kdst, __nv_bfloat16* __restrict__ vdst) {
  const long long step = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; e < total; e += step) {
    const int vec = static_cast<int>(e % vecs);
    const long long dv = e / vecs;
    const int isv = static_cast<int>(dv & 1);
    const long long d = dv >> 1;
    const long long w = __ldg(where + d);
    const long long row = w & 0xffffffffLL;
    const uint4* from;
    if ((w >> 32) == 2) from = reinterpret_cast<const uint4*>(isv ? vnew + row * v_ts : knew + row * k_ts);
    else from = reinterpret_cast<const uint4*>(((w >> 32) == 0 ? sinks : prior) + (row * 2 + isv) * (vecs * 8LL));
    reinterpret_cast<uint4*>((isv ? vdst : kdst) + d * (vecs * 8LL))[vec] = __ldg(from + vec);
  }
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
  int rows;                 // query rows per tile in the partial layout: 128 (plan kernels 2, 3) or 64 (plan kernel 1)
  float* opart;             // [nitems, Hkv, rows, 128]
  float* ml;                // [nitems, Hkv, rows, 2]
};

template <int NB> struct MLay {
  static constexpr int CBY = NB == 4 ? 64 : 32;
  static constexpr int CHUNK = (2 * CBY + 16) * PAGE;            // 2304 | 1280
  static constexpr int V_OFF = CBY * PAGE, KS_OFF = 2 * CBY * PAGE, VS_OFF = KS_OFF + 8 * PAGE;
  static constexpr uint32_t ZM = NB == 4 ? 15u : 3u;
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
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (q_fp32) k_q_stage<true><<<m, 256, 0, st>>>(q, q_ts, idx, Hq, G, kfull, kmask, qscale, static_cast<__half*>(q16));
  else k_q_stage<false><<<m, 256, 0, st>>>(q, q_ts, idx, Hq, G, kfull, kmask, qscale, static_cast<__half*>(q16));
  return cudaPeekAtLastError() == cudaSuccess ? 0 : -1;
}

int frmq_attn(const void* q16, const uint8_t* pool, long long page_stride, const int* bt, long long bt_stride, const int* tiles,
              const int* items, int nitems, int Hkv, int G, int shift, int konly, float* opart, float* ml, int kernel, int Dh,
              void* stream, int kmin) {
  if (nitems <= 0) return 0;
  if (Dh != D) return -4;
  if (G < 1 || G > 64) return -3;
  if (kernel < 1 || kernel > 3) return -3;
  const int rows = kernel == 1 ? 64 : 128;      // the reference's plan kernels: 64-row tiles (1) or 128-row tiles (2, 3)
  if (G > rows) return -3;
  MqParams p{static_cast<const __half*>(q16), pool, page_stride, bt, bt_stride, tiles, items, Hkv, G, shift, kmin, rows, opart, ml};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool ko = (konly & 1) != 0, b2 = (konly & 2) != 0;
  if (b2) return ko ? launch_mq_tc<2, true>(p, nitems, st) : launch_mq_tc<2, false>(p, nitems, st);
  return ko ? launch_mq_tc<4, true>(p, nitems, st) : launch_mq_tc<4, false>(p, nitems, st);
}

int frmq_merge(const int* tiles, int ntiles, const float* opart, const float* ml, int Hkv, int G, int rows, void* out,
               long long o_ts, int out_fp32, float* lse, long long lse_ts, int Dh, void* stream) {
  if (ntiles <= 0) return 0;
  if (Dh != D) return -4;
  if (G < 1 || rows < G) return -3;
  k_item_fold<<<dim3(ntiles, Hkv), 256, 0, static_cast<cudaStream_t>(stream)>>>(tiles, opart, ml, Hkv, G, rows, out, o_ts, out_fp32,
                                                                               lse, lse_ts);
  return cudaPeekAtLastError() == cudaSuccess ? 0 : -1;
}

int frmq_win_gather(const long long* map, int nk, const void* sinkb, const void* preb, const void* kch, long long k_ts,
                    const void* vch, long long v_ts, int Hkv, void* kw, void* vw, int Dh, void* stream) {
  if (nk <= 0) return 0;
  if (Dh != D) return -4;
  using B = __nv_bfloat16;
  const int vecs = Hkv * D / 8;                                  // 16-byte vectors per K (or V) row
  const long long total = static_cast<long long>(nk) * 2 * vecs;
  const long long want = (total + 255) / 256;
  const unsigned blocks = static_cast<unsigned>(want < 148 * 8 ? want : 148 * 8);   // grid-stride beyond eight CTAs per SM
  k_rows_collect<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(map, total, vecs, static_cast<const B*>(sinkb),
                                                                       static_cast<const B*>(preb), static_cast<const B*>(kch), k_ts,
                                                                       static_cast<const B*>(vch), v_ts, static_cast<B*>(kw),
                                                                       static_cast<B*>(vw));
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
