// libflagrot_kivi.so for sm_100a: FlagRot-KIVI INT2 pages (keys per channel over 32-token groups, values per token,
// FP16 scale / min, selective identity / H32 / whole-head Hadamard by the attention-weighted rule).  C ABI 9 of the
// reference's integrations/vllm_flagrot/csrc/kivi.cu (declarations + citations: include/flagrot_kivi.h).
//
// Page layout (unchanged, part of the ABI; reference kivi.cu:15-26): per (16-token page, kv head) 12 D + 16 bytes =
//   KC [16][D/4] key codes (16-channel words, channel i at bit 2 (i >> 1) + 16 (i & 1)) | KM [16][D/32] half2
//   (scale | flag sign, min) of the token's GROUP (cell i = position % 32 holds channels [4 i, 4 i + 4)) | VC [16][D/4] |
//   VM [16][D/32] half2 (scale | H32 sign, min) | VF [16] u8.
// Quantizer: s = (max - min) * fp32(1/3), code = rint(clamp((x - min) / s, 0, 3)), x^ = code * s + min, every
// operation rounded separately (reference kivi.cu:99-109).
//
// Kernels: k_v_write (warp per (token, head)), k_k_encode (CTA per (group, head); fp32 CUDA cores: the selection is
// defined by fp32 sums), kvm::k_kv_attn_mma2 (kv_attn_mma2.cuh: page splits and the BF16 sink / window split on the tensor
// cores, GQA groups <= 8, one launch), k_kv_merge, k_kv_dequant, k_kv_lse_merge.
//
// kivi2p8 pages (f8 bit 0 of every entry; reference kivi.cu:28-35, 83-88): scale and minimum stored as FP8 E4M3 (round to
// nearest even, saturating at +-448), the codes computed from the STORED values; chunk of 10 D bytes:
//   KC [16][D/4] | KM [16][D/32][2] u8 (s8 | flag << 7, m8) of the GROUP | VC [16][D/4] | VM [16][D/32][2] u8 (s8 | H32 << 7, m8).
// Flags sit in the sign bits of the non-negative scales: key sub-vector j -> cell j slot 0, key whole head -> cell 4 slot 0,
// the VALUE whole-head flag of the token in cell i -> key scale of cell i slot 3 (set by the value writer, kept by the key
// encoder).  Every kernel is templated on the page kind; f8 bit 1 (the reference's "fast" kernel variants, same values)
// selects nothing here.  Head dim 256 answers code 2 with a message.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include "fr_common.cuh"
#include "../../include/flagrot_kivi.h"

namespace {

using fr::FULLMASK;
constexpr int D = 128, NV = 4, PAGE = 16, GRP = 32;
template <bool F8> struct KLay {              // byte offsets inside a (page, kv head) chunk
  static constexpr int CB = F8 ? 10 * D : 12 * D + 16;
  static constexpr int KM = 4 * D, VC = F8 ? 5 * D : 6 * D, VM = F8 ? 9 * D : 10 * D;
  static constexpr int VF = 12 * D;           // kivi2 only
  static constexpr int MCELL = F8 ? 2 * NV : 4 * NV;   // bytes of (scale, min) pairs per cell
};
#define KV_NEG_INF (-INFINITY)

char g_err[512];
int fail(const char* fmt, int a = 0, int b = 0) {
  std::snprintf(g_err, sizeof(g_err), fmt, a, b);
  return 2;
}
int check_launch(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    std::snprintf(g_err, sizeof(g_err), "%s: %s", what, cudaGetErrorString(e));
    return 1;
  }
  return 0;
}

FR_DEVI int kbit(int i) { return 2 * (i >> 1) + 16 * (i & 1); }
FR_DEVI float kivi_scale(float mn, float mx) { return __fmul_rn(__fsub_rn(mx, mn), 1.0f / 3.0f); }
FR_DEVI int kivi_code(float x, float mn, float s) {
  const float d = s == 0.f ? 1.f : s;
  return static_cast<int>(rintf(fminf(fmaxf(__fdiv_rn(__fsub_rn(x, mn), d), 0.f), 3.f)));
}
FR_DEVI float kivi_rec(int code, float mn, float s) { return __fadd_rn(__fmul_rn(static_cast<float>(code), s), mn); }
// FP8 E4M3, round to nearest even, saturating at +-448 (reference kivi.cu:110-119)
FR_DEVI uint8_t e4m3_bits(float x) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(fminf(fmaxf(x, -448.f), 448.f), __NV_SATFINITE, __NV_E4M3));
}
FR_DEVI float e4m3_val(uint8_t b) { return __half2float(__half(__nv_cvt_fp8_to_halfraw(b, __NV_E4M3))); }
FR_DEVI float2 e4m3x2_val(uint16_t pair) {    // (low byte, high byte)
  return __half22float2(__half2(__nv_cvt_fp8x2_to_halfraw2(pair, __NV_E4M3)));
}
// (scale, min) the quantizer works with: fp32 for kivi2, the stored E4M3 values for kivi2p8 (reference kivi.cu:120-125)
template <bool F8> FR_DEVI void qparams(float mn, float mx, float& s, float& m) {
  s = kivi_scale(mn, mx);
  m = mn;
  if (F8) { s = e4m3_val(e4m3_bits(s)); m = e4m3_val(e4m3_bits(mn)); }
}
// orthonormal H_n (n = 32 | 128) of a row held 4 elements per lane
FR_DEVI void hada_row(float (&v)[4], int lane, int n) {
  fr::fwht_row_stages(v, lane, n);
  const float c = n == 32 ? fr::C32 : fr::C128;
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = __fmul_rn(v[i], c);
}

// ------------------------------------------------------------------------------------------------ value writer
// WMAT: the selection weighted by a full matrix M (its own instantiation: the error vectors in shared memory and the row
// loops cost registers and occupancy that the diagonal weighting must not pay)
template <bool F8, bool WMAT>
__global__ void __launch_bounds__(128) k_v_write(const __nv_bfloat16* __restrict__ kv, long long kv_rs, int n, int Hkv,
                                                 const long long* __restrict__ slots, const float* __restrict__ co,
                                                 const float* __restrict__ M, uint8_t* __restrict__ pool, int ident,
                                                 const int* __restrict__ vfix) {
  __shared__ float esh[WMAT ? 4 : 1][3][WMAT ? D : 1];   // matrix weighting: the warp's error vectors (I, H32, whole head)
  const int lane = threadIdx.x & 31;
  const long long item = static_cast<long long>(blockIdx.x) * 4 + (threadIdx.x >> 5);
  if (item >= static_cast<long long>(n) * Hkv) return;
  const int t = static_cast<int>(item / Hkv), h = static_cast<int>(item % Hkv);
  const long long slot = slots[t];
  if (slot < 0) return;
  const uint2 raw = *reinterpret_cast<const uint2*>(kv + t * kv_rs + static_cast<long long>(Hkv + h) * D + 4 * lane);
  const float x[4] = {fr::bf16_lo(raw.x), fr::bf16_hi(raw.x), fr::bf16_lo(raw.y), fr::bf16_hi(raw.y)};
  float rec[3][4], sc[3], mnv[3];
  int code[3][4];
#pragma unroll
  for (int c = 0; c < 3; ++c) {
    if (c > 0 && ident) break;
    float y[4] = {x[0], x[1], x[2], x[3]};
    if (c > 0) hada_row(y, lane, c == 1 ? 32 : 128);
    const float mn = fr::group_min8(fminf(fminf(y[0], y[1]), fminf(y[2], y[3])));
    const float mx = fr::group_max8(fmaxf(fmaxf(y[0], y[1]), fmaxf(y[2], y[3])));
    float s, m0;
    qparams<F8>(mn, mx, s, m0);
    sc[c] = s; mnv[c] = m0;
#pragma unroll
    for (int i = 0; i < 4; ++i) { code[c][i] = kivi_code(y[i], m0, s); y[i] = kivi_rec(code[c][i], m0, s); }
    if (c > 0) hada_row(y, lane, c == 1 ? 32 : 128);
#pragma unroll
    for (int i = 0; i < 4; ++i) rec[c][i] = y[i];
  }
  int cand = 0;
  bool useF = false;
  if (!ident && vfix != nullptr) {   // frozen choice of this kv head: bits 0..3 = H32 per sub-vector, bit 16 = whole head
    useF = (vfix[h] >> 16) & 1;
    cand = useF ? 2 : ((vfix[h] >> (lane >> 3)) & 1);
  } else if (WMAT && !ident && M != nullptr) {
    // weighting by a full matrix M [Hkv, D, D] (e^T M e): the I / H32 errors of a sub-vector use its diagonal 32 x 32 block,
    // the whole-head error and the error of the chosen combination the whole matrix (reference kivi.cu:222-275; sums in
    // the reference's order, products contracted as its compiler contracts them)
    const int wp = threadIdx.x >> 5, jb = lane >> 3;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      esh[wp][0][4 * lane + i] = __fsub_rn(rec[0][i], x[i]);
      esh[wp][1][4 * lane + i] = __fsub_rn(rec[1][i], x[i]);
      esh[wp][2][4 * lane + i] = __fsub_rn(rec[2][i], x[i]);
    }
    __syncwarp();
    const float* Mh = M + static_cast<long long>(h) * D * D;
    float eI = 0.f, eH = 0.f, eF = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = 4 * lane + i;
      const float* row = Mh + static_cast<long long>(r) * D;
      float a0 = 0.f, a1 = 0.f, a2 = 0.f;
      for (int k = jb * 32; k < jb * 32 + 32; ++k) {
        const float m = row[k];
        a0 = fmaf(m, esh[wp][0][k], a0);
        a1 = fmaf(m, esh[wp][1][k], a1);
      }
      for (int k = 0; k < D; ++k) a2 = fmaf(row[k], esh[wp][2][k], a2);
      eI = fmaf(esh[wp][0][r], a0, eI);
      eH = fmaf(esh[wp][1][r], a1, eH);
      eF = fmaf(esh[wp][2][r], a2, eF);
    }
#pragma unroll
    for (int m = 1; m < 8; m <<= 1) {
      eI = __fadd_rn(eI, __shfl_xor_sync(FULLMASK, eI, m));
      eH = __fadd_rn(eH, __shfl_xor_sync(FULLMASK, eH, m));
    }
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) eF = __fadd_rn(eF, __shfl_xor_sync(FULLMASK, eF, m));
    const bool useH = eH < eI;
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 4; ++i) esh[wp][0][4 * lane + i] = useH ? esh[wp][1][4 * lane + i] : esh[wp][0][4 * lane + i];
    __syncwarp();
    float a = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = 4 * lane + i;
      const float* row = Mh + static_cast<long long>(r) * D;
      float sacc = 0.f;
      for (int k = 0; k < D; ++k) sacc = fmaf(row[k], esh[wp][0][k], sacc);
      a = fmaf(esh[wp][0][r], sacc, a);
    }
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) a = __fadd_rn(a, __shfl_xor_sync(FULLMASK, a, m));
    useF = eF < a;
    cand = useF ? 2 : (useH ? 1 : 0);
  } else if (!ident) {
    const float4 cw4 = *reinterpret_cast<const float4*>(co + static_cast<long long>(h) * D + 4 * lane);
    const float cw[4] = {cw4.x, cw4.y, cw4.z, cw4.w};
    float eI = 0.f, eH = 0.f, eF = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float d0 = __fsub_rn(rec[0][i], x[i]), d1 = __fsub_rn(rec[1][i], x[i]), d2 = __fsub_rn(rec[2][i], x[i]);
      eI = fmaf(__fmul_rn(d0, d0), cw[i], eI);
      eH = fmaf(__fmul_rn(d1, d1), cw[i], eH);
      eF = fmaf(__fmul_rn(d2, d2), cw[i], eF);
    }
#pragma unroll
    for (int m = 1; m < 8; m <<= 1) {
      eI = __fadd_rn(eI, __shfl_xor_sync(FULLMASK, eI, m));
      eH = __fadd_rn(eH, __shfl_xor_sync(FULLMASK, eH, m));
    }
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) eF = __fadd_rn(eF, __shfl_xor_sync(FULLMASK, eF, m));
    const bool useH = eH < eI;                       // identity on ties
    float eB = (lane & 7) == 0 ? (useH ? eH : eI) : 0.f;
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) eB = __fadd_rn(eB, __shfl_xor_sync(FULLMASK, eB, m));
    useF = eF < eB;                                  // base on ties
    cand = useF ? 2 : (useH ? 1 : 0);
  }
  const long long blk = slot / PAGE;
  const int off = static_cast<int>(slot % PAGE);
  using L = KLay<F8>;
  uint8_t* chunk = pool + (blk * Hkv + h) * static_cast<long long>(L::CB);
  int cc[4];
  float s_, m_;
  if (cand == 0) { cc[0] = code[0][0]; cc[1] = code[0][1]; cc[2] = code[0][2]; cc[3] = code[0][3]; s_ = sc[0]; m_ = mnv[0]; }
  else if (cand == 1) { cc[0] = code[1][0]; cc[1] = code[1][1]; cc[2] = code[1][2]; cc[3] = code[1][3]; s_ = sc[1]; m_ = mnv[1]; }
  else { cc[0] = code[2][0]; cc[1] = code[2][1]; cc[2] = code[2][2]; cc[3] = code[2][3]; s_ = sc[2]; m_ = mnv[2]; }
  chunk[L::VC + off * (D / 4) + lane] = static_cast<uint8_t>((cc[0] & 3) | ((cc[1] & 3) << 2) | ((cc[2] & 3) << 4) | ((cc[3] & 3) << 6));
  if (F8) {
    if ((lane & 7) == 0)
      *reinterpret_cast<uint16_t*>(chunk + L::VM + off * L::MCELL + 2 * (lane >> 3)) =
          static_cast<uint16_t>((e4m3_bits(s_) & 0x7F) | (cand == 1 ? 0x80 : 0) | (e4m3_bits(m_) << 8));
    if (lane == 0) {                                 // the token's whole-head flag: bit 7 of its cell's slot-3 key scale
      uint8_t* kb = chunk + L::KM + off * L::MCELL + 2 * (NV - 1);
      *kb = static_cast<uint8_t>((*kb & 0x7F) | (useF ? 0x80 : 0));
    }
    return;
  }
  if ((lane & 7) == 0) {
    __half sh = __float2half_rn(s_);
    if (cand == 1) sh = __hneg(__habs(sh));          // sign bit = this sub-vector is stored as H32 x
    reinterpret_cast<__half2*>(chunk + L::VM + off * (D / 8))[lane >> 3] = __halves2half2(sh, __float2half_rn(m_));
  }
  if (lane == 0) chunk[L::VF + off] = useF ? 1 : 0;
}

// ------------------------------------------------------------------------------------------------ key group encoder
constexpr int LD = D + 4, QT = 64;
constexpr size_t KENC_SMEM = sizeof(float) * (32 * LD + 3 * 32 * LD + QT * LD + QT);

template <bool F8>
__global__ void __launch_bounds__(256) k_k_encode(const __nv_bfloat16* __restrict__ src, long long src_rs,
                                                  const __nv_bfloat16* __restrict__ src2, long long src2_rs,
                                                  const long long* __restrict__ sidx, const long long* __restrict__ dslot,
                                                  int Hkv, const float* __restrict__ qs, const float* __restrict__ lz,
                                                  int NQ, float qsc, uint8_t* __restrict__ pool, int ident,
                                                  const int* __restrict__ kfix) {
  extern __shared__ float sm[];
  float* xs = sm;                            // [32][LD] keys
  float* es = xs + 32 * LD;                  // [3][32][LD] candidates, then their errors
  float* qt = es + 3 * 32 * LD;              // [QT][LD] calibration query tile
  float* lzt = qt + QT * LD;                 // [QT]
  __shared__ int s_valid[32];
  __shared__ float s_par[3][2][D];           // per candidate (min, scale) per channel
  __shared__ int s_choice[NV + 1];
  const int item = blockIdx.x, h = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const long long* si = sidx + static_cast<long long>(item) * 32;
  const long long* ds = dslot + static_cast<long long>(item) * 32;
  if (ds[0] < 0) return;
  if (tid < 32) s_valid[tid] = si[tid] != -1;
  for (int e = tid; e < 32 * D; e += 256) {
    const int t = e / D, c = e % D;
    const long long r = si[t];
    xs[t * LD + c] = r >= 0 ? __bfloat162float(src[r * src_rs + static_cast<long long>(h) * D + c])
                   : r <= -2 ? __bfloat162float(src2[(-r - 2) * src2_rs + static_cast<long long>(h) * D + c]) : 0.f;
  }
  __syncthreads();
  if (ident) {
    for (int c = tid; c < D; c += 256) {
      float mn = INFINITY, mx = -INFINITY;
      for (int t = 0; t < 32; ++t)
        if (s_valid[t]) { const float v = xs[t * LD + c]; mn = fminf(mn, v); mx = fmaxf(mx, v); }
      qparams<F8>(mn, mx, s_par[0][1][c], s_par[0][0][c]);
    }
    if (tid <= NV) s_choice[tid] = 0;
    __syncthreads();
  } else {
    for (int t = warp; t < 32; t += 8) {       // the three transformed views of every token
      float x[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) x[i] = xs[t * LD + 4 * lane + i];
#pragma unroll
      for (int c = 0; c < 3; ++c) {
        float y[4] = {x[0], x[1], x[2], x[3]};
        if (c > 0) hada_row(y, lane, c == 1 ? 32 : 128);
#pragma unroll
        for (int i = 0; i < 4; ++i) es[(c * 32 + t) * LD + 4 * lane + i] = y[i];
      }
    }
    __syncthreads();
    for (int e = tid; e < 3 * D; e += 256) {   // per channel over the group's valid tokens: range, scale, reconstruction
      const int c3 = e / D, c = e % D;
      float* col = es + c3 * 32 * LD + c;
      float mn = INFINITY, mx = -INFINITY;
      for (int t = 0; t < 32; ++t)
        if (s_valid[t]) { const float v = col[t * LD]; mn = fminf(mn, v); mx = fmaxf(mx, v); }
      float s, m0;
      qparams<F8>(mn, mx, s, m0);
      s_par[c3][0][c] = m0;
      s_par[c3][1][c] = s;
      for (int t = 0; t < 32; ++t)
        if (s_valid[t]) col[t * LD] = kivi_rec(kivi_code(col[t * LD], m0, s), m0, s);
    }
    __syncthreads();
    if (kfix != nullptr) {
      if (tid <= NV) s_choice[tid] = tid < NV ? (kfix[h] >> tid) & 1 : (kfix[h] >> 16) & 1;
      __syncthreads();
    } else {
      for (int t = warp; t < 32; t += 8) {     // back to the original basis, errors (0 for tokens outside the group)
#pragma unroll
        for (int c = 0; c < 3; ++c) {
          float y[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) y[i] = es[(c * 32 + t) * LD + 4 * lane + i];
          if (c > 0) hada_row(y, lane, c == 1 ? 32 : 128);
#pragma unroll
          for (int i = 0; i < 4; ++i)
            es[(c * 32 + t) * LD + 4 * lane + i] = s_valid[t] ? __fsub_rn(y[i], xs[t * LD + 4 * lane + i]) : 0.f;
        }
      }
      __syncthreads();
      // Pooled attention-weighted errors in ONE pass over the calibration queries.  Lane = token, warp w takes the
      // queries w, w + 8, ... of a staged tile.  Per (token, query): weight min(1, exp(qsc x.q - lz)), the projections of
      // the I / H32 errors per 32-dim sub-vector (a_I[j], a_H[j]) and of the whole-head error (a_F).  The error of the
      // "base" candidate for ANY combination of sub-vector choices is w (sum_j pick_j)^2, so all 16 combinations are
      // accumulated and the one matching the final choices is read afterwards: no second pass, no weight recomputation.
      const int tk = lane;
      const bool vt = s_valid[tk] != 0;
      float EI[NV], EH[NV], EF = 0.f, EB[16];
#pragma unroll
      for (int j = 0; j < NV; ++j) { EI[j] = 0.f; EH[j] = 0.f; }
#pragma unroll
      for (int m = 0; m < 16; ++m) EB[m] = 0.f;
      const float* qh = qs + static_cast<long long>(h) * NQ * D;
      const float* lzh = lz + static_cast<long long>(h) * NQ;
      const float4* xr = reinterpret_cast<const float4*>(xs + tk * LD);
      const float4* e0 = reinterpret_cast<const float4*>(es + (0 * 32 + tk) * LD);
      const float4* e1 = reinterpret_cast<const float4*>(es + (1 * 32 + tk) * LD);
      const float4* e2 = reinterpret_cast<const float4*>(es + (2 * 32 + tk) * LD);
      auto dot4 = [](float acc, float4 a, float4 b) {
        acc = fmaf(a.x, b.x, acc); acc = fmaf(a.y, b.y, acc); acc = fmaf(a.z, b.z, acc); return fmaf(a.w, b.w, acc);
      };
      for (int q0 = 0; q0 < NQ; q0 += QT) {
        __syncthreads();
        for (int e = tid; e < QT * (D / 4); e += 256) {
          const int qq = e / (D / 4), c4 = e % (D / 4);
          *reinterpret_cast<float4*>(qt + qq * LD + 4 * c4) =
              q0 + qq < NQ ? reinterpret_cast<const float4*>(qh + static_cast<long long>(q0 + qq) * D)[c4] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        for (int e = tid; e < QT; e += 256) lzt[e] = q0 + e < NQ ? lzh[q0 + e] : 0.f;
        __syncthreads();
        for (int qq = warp; qq < QT && q0 + qq < NQ; qq += 8) {
          const float4* qv = reinterpret_cast<const float4*>(qt + qq * LD);   // same address on every lane: broadcast
          float lg = 0.f, aI[NV], aH[NV], aF = 0.f;
#pragma unroll
          for (int j = 0; j < NV; ++j) {
            aI[j] = 0.f; aH[j] = 0.f;
#pragma unroll 2
            for (int c4 = 8 * j; c4 < 8 * j + 8; ++c4) {   // (a full unroll makes ptxas hoist 160 loads and spill)
              const float4 qc = qv[c4];
              lg = dot4(lg, xr[c4], qc);
              aI[j] = dot4(aI[j], e0[c4], qc);
              aH[j] = dot4(aH[j], e1[c4], qc);
              aF = dot4(aF, e2[c4], qc);
            }
          }
          const float wt = vt ? fminf(expf(__fsub_rn(__fmul_rn(qsc, lg), lzt[qq])), 1.f) : 0.f;
#pragma unroll
          for (int j = 0; j < NV; ++j) { EI[j] = fmaf(wt * aI[j], aI[j], EI[j]); EH[j] = fmaf(wt * aH[j], aH[j], EH[j]); }
          EF = fmaf(wt * aF, aF, EF);
          const float s01[4] = {aI[0] + aI[1], aH[0] + aI[1], aI[0] + aH[1], aH[0] + aH[1]};   // bit 0 = choice of j = 0, bit 1 of j = 1
          const float s23[4] = {aI[2] + aI[3], aH[2] + aI[3], aI[2] + aH[3], aH[2] + aH[3]};
#pragma unroll
          for (int m = 0; m < 16; ++m) {
            const float sb = s01[m & 3] + s23[m >> 2];
            EB[m] = fmaf(wt * sb, sb, EB[m]);
          }
        }
      }
      // fixed-order reduction: lanes (tokens) by shuffles, then the 8 warps in order
      float* redv = qt;                                   // the query tile is free now: [8][25]
      __syncthreads();
#pragma unroll
      for (int j = 0; j < NV; ++j)
        for (int m = 16; m >= 1; m >>= 1) {
          EI[j] += __shfl_xor_sync(FULLMASK, EI[j], m);
          EH[j] += __shfl_xor_sync(FULLMASK, EH[j], m);
        }
      for (int m = 16; m >= 1; m >>= 1) EF += __shfl_xor_sync(FULLMASK, EF, m);
#pragma unroll
      for (int k = 0; k < 16; ++k)
        for (int m = 16; m >= 1; m >>= 1) EB[k] += __shfl_xor_sync(FULLMASK, EB[k], m);
      if (lane == 0) {
#pragma unroll
        for (int j = 0; j < NV; ++j) { redv[warp * 25 + j] = EI[j]; redv[warp * 25 + NV + j] = EH[j]; }
        redv[warp * 25 + 8] = EF;
#pragma unroll
        for (int k = 0; k < 16; ++k) redv[warp * 25 + 9 + k] = EB[k];
      }
      __syncthreads();
      if (tid == 0) {
        float tot[25];
#pragma unroll
        for (int k = 0; k < 25; ++k) {
          float a = 0.f;
          for (int w_ = 0; w_ < 8; ++w_) a += redv[w_ * 25 + k];
          tot[k] = a;
        }
        int mask = 0;
        for (int j = 0; j < NV; ++j) {
          const int ch = tot[NV + j] < tot[j] ? 1 : 0;    // H32 only if strictly better: identity on ties
          s_choice[j] = ch;
          mask |= ch << j;
        }
        s_choice[NV] = tot[8] < tot[9 + mask] ? 1 : 0;     // whole head only if strictly better than the base
      }
      __syncthreads();
    }
  }
  // codes of the chosen candidate for the group's tokens, (scale | flag, min) slices of all 32 cells
  const bool useF = s_choice[NV] != 0;
  for (int t = warp; t < 32; t += 8) {
    if (!s_valid[t]) continue;
    float x[4], yh[4], yf[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) { x[i] = xs[t * LD + 4 * lane + i]; yh[i] = x[i]; yf[i] = x[i]; }
    hada_row(yh, lane, 32);
    hada_row(yf, lane, 128);
    const int cand = useF ? 2 : s_choice[lane >> 3];
    const long long slot = ds[t];
    uint8_t* chunk = pool + ((slot / PAGE) * Hkv + h) * static_cast<long long>(KLay<F8>::CB);
    const int off = static_cast<int>(slot % PAGE);
    uint32_t word = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = 4 * lane + i;
      const float y = cand == 0 ? x[i] : cand == 1 ? yh[i] : yf[i];
      word |= static_cast<uint32_t>(kivi_code(y, s_par[cand][0][c], s_par[cand][1][c]) & 3) << kbit(c % 16);
    }
    word |= __shfl_xor_sync(FULLMASK, word, 1);
    word |= __shfl_xor_sync(FULLMASK, word, 2);
    if ((lane & 3) == 0) reinterpret_cast<uint32_t*>(chunk + off * (D / 4))[lane >> 2] = word;
  }
  if constexpr (F8) {     // (s8 | flag << 7, m8) byte pairs; bit 7 of a cell's slot-3 scale is the value writer's and stays
    for (int c = tid; c < D; c += 256) {
      const int cand = useF ? 2 : s_choice[c / 32];
      const int cell = c / NV, k = c % NV;
      const bool neg = k == 0 && (cell < NV ? (!useF && s_choice[cell] != 0) : (cell == NV && useF));
      const long long slot = ds[cell];
      uint8_t* km = pool + ((slot / PAGE) * Hkv + h) * static_cast<long long>(KLay<true>::CB) + KLay<true>::KM +
                    static_cast<int>(slot % PAGE) * KLay<true>::MCELL + 2 * k;
      uint8_t sb = static_cast<uint8_t>((e4m3_bits(s_par[cand][1][c]) & 0x7F) | (neg ? 0x80 : 0));
      if (k == NV - 1) sb = static_cast<uint8_t>((sb & 0x7F) | (km[0] & 0x80));
      km[0] = sb;
      km[1] = e4m3_bits(s_par[cand][0][c]);
    }
  } else {
  for (int c = tid; c < D; c += 256) {
    const int cand = useF ? 2 : s_choice[c / 32];
    __half sh = __float2half_rn(s_par[cand][1][c]);
    const bool neg = c < NV ? (!useF && s_choice[c] != 0) : (c == NV ? useF : false);
    sh = neg ? __hneg(__habs(sh)) : __habs(sh);
    const int cell = c / NV, k = c % NV;
    const long long slot = ds[cell];
    uint8_t* chunk = pool + ((slot / PAGE) * Hkv + h) * static_cast<long long>(KLay<false>::CB);
    reinterpret_cast<__half2*>(chunk + KLay<false>::KM + static_cast<int>(slot % PAGE) * (D / 8))[k] =
        __halves2half2(sh, __float2half_rn(s_par[cand][0][c]));
  }
  }
}

// ------------------------------------------------------------------------------------------------ decode attention
// (the page-split kernel and the BF16 sink / window split live in kv_attn_mma2.cuh / kv_attn_mma.cuh)
template <int G>
__device__ void smem_hada(float (*x)[D], int n) {   // orthonormal H_n of G rows in shared memory (all 128 threads)
  const int tid = threadIdx.x;
  for (int hh = 1; hh < n; hh <<= 1) {
    for (int e = tid; e < G * D / 2; e += 128) {
      const int g = e / (D / 2), k = e % (D / 2);
      const int lo = ((k & ~(hh - 1)) << 1) | (k & (hh - 1)), hi = lo + hh;
      const float a = x[g][lo], b = x[g][hi];
      x[g][lo] = __fadd_rn(a, b);
      x[g][hi] = __fsub_rn(a, b);
    }
    __syncthreads();
  }
  const float c = n == 32 ? fr::C32 : fr::C128;
  for (int e = tid; e < G * D; e += 128) x[e / D][e % D] = __fmul_rn(x[e / D][e % D], c);
  __syncthreads();
}

__global__ void __launch_bounds__(128) k_kv_merge(const float* __restrict__ opart, const float* __restrict__ ml, int Hkv, int G,
                                                  int NS, __nv_bfloat16* __restrict__ out, long long out_rs) {
  const int b = blockIdx.x, hq = blockIdx.y;
  const int h = hq / G, g = hq % G;
  const long long p0 = static_cast<long long>(b * Hkv + h) * (NS + 1);
  float M = KV_NEG_INF;
  for (int s = 0; s <= NS; ++s) M = fmaxf(M, ml[((p0 + s) * G + g) * 2]);
  float o = 0.f, L = 0.f;
  if (M != KV_NEG_INF) {
    for (int s = 0; s <= NS; ++s) {
      const float m = ml[((p0 + s) * G + g) * 2];
      if (m == KV_NEG_INF) continue;
      const float f = exp2f(m - M);
      L += f * ml[((p0 + s) * G + g) * 2 + 1];
      o = fmaf(f, opart[((p0 + s) * G + g) * D + threadIdx.x], o);
    }
  }
  out[static_cast<long long>(b) * out_rs + static_cast<long long>(hq) * D + threadIdx.x] = __float2bfloat16(o * (L > 0.f ? 1.f / L : 0.f));
}

// ------------------------------------------------------------------------------------------------ page dequantisation
// positions [32 g0, 32 g1) of one request -> K, V rows in the writers' basis (inverse H32 / H_D applied); warp per token
template <typename OT, bool F8>
__global__ void __launch_bounds__(128) k_kv_dequant(const uint8_t* __restrict__ pool, const int* __restrict__ bt, int g0, int Hkv,
                                                    int nvalid, OT* __restrict__ ok, OT* __restrict__ ov) {
  using L = KLay<F8>;
  const int gi = blockIdx.x, h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = g0 + gi;
  const uint8_t* chA = pool + (static_cast<long long>(bt[2 * g]) * Hkv + h) * L::CB;
  const uint8_t* chB = pool + (static_cast<long long>(bt[2 * g + 1]) * Hkv + h) * L::CB;
  // (scale with its flag, min) of pair k of a cell as floats; the flag comes back as the sign of the scale
  auto meta = [](const uint8_t* cellp, int k) -> float2 {
    if (F8) {
      const uint16_t pr = reinterpret_cast<const uint16_t*>(cellp)[k];
      const float2 v = e4m3x2_val(static_cast<uint16_t>(pr & 0xFF7Fu));
      return make_float2((pr & 0x80u) ? -v.x : v.x, v.y);            // (a zero scale loses the flag: callers test the byte)
    }
    const uint32_t wv = reinterpret_cast<const uint32_t*>(cellp)[k];
    const __half2 hv = *reinterpret_cast<const __half2*>(&wv);
    return make_float2(__low2float(hv), __high2float(hv));
  };
  auto flag = [](const uint8_t* cellp, int k) -> uint32_t {
    return F8 ? (cellp[2 * k] >> 7) & 1u : (reinterpret_cast<const uint32_t*>(cellp)[k] >> 15) & 1u;
  };
  uint32_t lm = 0;                                                     // key flags of the group
  for (int j = 0; j < NV; ++j) lm |= (F8 ? flag(chA + L::KM + j * L::MCELL, 0) : flag(chA + L::KM, j)) << j;
  const uint32_t fF = F8 ? flag(chA + L::KM + NV * L::MCELL, 0) : flag(chA + L::KM + L::MCELL, 0);
  const uint8_t* cm = lane < 16 ? chA : chB;       // this lane's channels 4 lane .. 4 lane + 3 = cell `lane`
  float ks[4], kmn[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 m = meta(cm + L::KM + (lane % 16) * L::MCELL, i);
    ks[i] = fabsf(m.x);
    kmn[i] = m.y;
  }
  auto store = [&](OT* dst, const float (&x)[4]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) dst[i] = static_cast<OT>(x[i]);
  };
  for (int t = warp; t < 32; t += 4) {
    const uint8_t* ch = t < 16 ? chA : chB;
    const long long o = static_cast<long long>(gi) * 32 + t;
    float x[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = 4 * lane + i;
      const int code = (reinterpret_cast<const uint32_t*>(ch + (t % 16) * (D / 4))[c / 16] >> kbit(c % 16)) & 3;
      x[i] = __fadd_rn(__fmul_rn(static_cast<float>(code), ks[i]), kmn[i]);
    }
    if (fF) hada_row(x, lane, 128);
    else if (lm) {
      float y[4] = {x[0], x[1], x[2], x[3]};
      hada_row(y, lane, 32);
      if ((lm >> (lane >> 3)) & 1u) { x[0] = y[0]; x[1] = y[1]; x[2] = y[2]; x[3] = y[3]; }
    }
    if (o < nvalid) store(ok + (o * Hkv + h) * D + 4 * lane, x);
    const int cell = t % 16;
    const uint8_t* vmc = ch + L::VM + cell * L::MCELL;
    uint32_t l = 0;
    for (int j = 0; j < NV; ++j) l |= flag(vmc, j) << j;
    const bool f = F8 ? flag(ch + L::KM + cell * L::MCELL, NV - 1) != 0 : ch[L::VF + cell] != 0;
    const float2 vmeta = meta(vmc, lane >> 3);
    const float vs = fabsf(vmeta.x), vmn = vmeta.y;
    const uint8_t byte = ch[L::VC + cell * (D / 4) + lane];
#pragma unroll
    for (int i = 0; i < 4; ++i) x[i] = __fadd_rn(__fmul_rn(static_cast<float>((byte >> (2 * i)) & 3), vs), vmn);
    if (f) hada_row(x, lane, 128);
    else if (l) {
      float y[4] = {x[0], x[1], x[2], x[3]};
      hada_row(y, lane, 32);
      if ((l >> (lane >> 3)) & 1u) { x[0] = y[0]; x[1] = y[1]; x[2] = y[2]; x[3] = y[3]; }
    }
    if (o < nvalid) store(ov + (o * Hkv + h) * D + 4 * lane, x);
  }
}

// LSE merge of two partial attentions, every operation rounded separately (reference kivi.cu:2290-2313)
__global__ void k_kv_lse_merge(const __nv_bfloat16* __restrict__ oa, const float* __restrict__ la, long long la_hs,
                               const __nv_bfloat16* __restrict__ ob, const float* __restrict__ lb, long long lb_hs,
                               __nv_bfloat16* __restrict__ out, long long out_rs, int na, int H, int Dd) {
  const long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= static_cast<long long>(na) * H * Dd) return;
  const int c = static_cast<int>(e % Dd);
  const long long rh = e / Dd;
  const int hh = static_cast<int>(rh % H);
  const long long r = rh / H;
  float a = la[hh * la_hs + r], b = lb[hh * lb_hs + r];
  if (a == INFINITY) a = -INFINITY;
  if (b == INFINITY) b = -INFINITY;
  const float m = (a != a || b != b) ? NAN : fmaxf(a, b);
  const float wa = expf(__fsub_rn(a, m)), wb = expf(__fsub_rn(b, m));
  const float va = __bfloat162float(oa[(r * H + hh) * Dd + c]), vb = __bfloat162float(ob[(r * H + hh) * Dd + c]);
  const float num = __fadd_rn(__fmul_rn(va, wa), __fmul_rn(vb, wb));
  out[r * out_rs + static_cast<long long>(hh) * Dd + c] = __float2bfloat16_rn(__fdiv_rn(num, __fadd_rn(wa, wb)));
}

#include "kv_attn_mma.cuh"
#include "kv_attn_mma2.cuh"

// one launch: grid (Hkv, max(NS, 1), 2 B); z < B are the page splits (y >= NS exits: a call with NS == 0 has only BF16
// rows), z >= B (y == 0) the BF16 sink / window splits.
template <int G, bool F8>
int launch_attn(const void* q, long long q_rs, const void* pool, const void* bt, long long bt_rs, const void* cached,
                int kv_start, int B, int Hkv, int NS, int chunk, float qscale, const void* ring, const void* tail_len,
                const void* tail_idx, int T, void* opart, void* ml, cudaStream_t st) {
  static_assert(kvm::TAIL_SMEM <= kvm::SMEM2, "the window split runs in the page-split kernel's shared memory");
  static unsigned long long ready = 0;
  if (!fr::smem_limit_ready(kvm::k_kv_attn_mma2<G, F8>, kvm::SMEM2, ready)) return 1;
  kvm::k_kv_attn_mma2<G, F8><<<dim3(Hkv, NS > 0 ? NS : 1, 2 * B), 128, kvm::SMEM2, st>>>(
      static_cast<const __nv_bfloat16*>(q), q_rs, static_cast<const uint8_t*>(pool), static_cast<const int*>(bt), bt_rs,
      static_cast<const int*>(cached), kv_start, Hkv, NS, chunk, qscale, static_cast<const __nv_bfloat16*>(ring),
      static_cast<const int*>(tail_len), static_cast<const int*>(tail_idx), T, B, static_cast<float*>(opart), static_cast<float*>(ml));
  return 0;
}

}  // namespace

extern "C" {

const char* kv_last_error() { return g_err; }
int kv_abi_version() { return 9; }
int kv_chunk_bytes(int Dd) { return 12 * Dd + 16; }
int kv_chunk_bytes8(int Dd) { return 10 * Dd; }

int kv_v_write(const void* kv, long long kv_rs, int n, int Hkv, int Dd, const void* slots, const void* co, const void* M,
               void* pool, int ident, const void* vfix, int f8, void* stream) {
  if (n <= 0) return 0;
  if (Dd != D) return fail("kv_v_write: D %d (head dim 128 only)", Dd);
  const unsigned blocks = static_cast<unsigned>((static_cast<long long>(n) * Hkv + 3) / 4);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool wmat = M != nullptr && !ident && vfix == nullptr;
#define KV_VW(F, W) k_v_write<F, W><<<blocks, 128, 0, st>>>(static_cast<const __nv_bfloat16*>(kv), kv_rs, n, Hkv, \
      static_cast<const long long*>(slots), static_cast<const float*>(co), static_cast<const float*>(M), \
      static_cast<uint8_t*>(pool), ident, static_cast<const int*>(vfix))
  if (f8 & 1) { if (wmat) KV_VW(true, true); else KV_VW(true, false); }
  else { if (wmat) KV_VW(false, true); else KV_VW(false, false); }
#undef KV_VW
  return check_launch("kv_v_write");
}

int kv_k_encode(const void* src, long long src_rs, const void* src2, long long src2_rs, const void* sidx, const void* dslot,
                int N, int Hkv, int Dd, const void* qs, const void* lz, int NQ, float qsc, void* pool, int ident,
                const void* kfix, int f8, void* stream) {
  if (N <= 0) return 0;
  if (Dd != D) return fail("kv_k_encode: D %d (head dim 128 only)", Dd);
  static unsigned long long ready = 0, ready8 = 0;
  if (!((f8 & 1) ? fr::smem_limit_ready(k_k_encode<true>, static_cast<int>(KENC_SMEM), ready8)
                 : fr::smem_limit_ready(k_k_encode<false>, static_cast<int>(KENC_SMEM), ready)))
    return check_launch("kv_k_encode (shared memory)") ? 1 : 1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define KV_ENC(F) k_k_encode<F><<<dim3(N, Hkv), 256, KENC_SMEM, st>>>( \
      static_cast<const __nv_bfloat16*>(src), src_rs, static_cast<const __nv_bfloat16*>(src2), src2_rs, \
      static_cast<const long long*>(sidx), static_cast<const long long*>(dslot), Hkv, static_cast<const float*>(qs), \
      static_cast<const float*>(lz), NQ, qsc, static_cast<uint8_t*>(pool), ident, static_cast<const int*>(kfix))
  if (f8 & 1) KV_ENC(true); else KV_ENC(false);
#undef KV_ENC
  return check_launch("kv_k_encode");
}

int kv_attn(const void* q, long long q_rs, const void* pool, const void* bt, long long bt_rs, const void* cached, int kv_start,
            int B, int Hkv, int G, int Dd, int NS, int chunk, float qscale, const void* ring, const void* tail_len,
            const void* tail_idx, int T, void* opart, void* ml, void* out, long long out_rs, int f8, void* stream) {
  if (B <= 0) return 0;
  if (G > 8 || G < 1 || chunk % GRP) return fail("kv_attn: G %d chunk %d", G, chunk);
  if (Dd != D) return fail("kv_attn: D %d (head dim 128 only)", Dd);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int rc = 0;
#define KV_CASE(GG) case GG: rc = (f8 & 1) ? launch_attn<GG, true>(q, q_rs, pool, bt, bt_rs, cached, kv_start, B, Hkv, NS, chunk, qscale, ring, \
                                                                    tail_len, tail_idx, T, opart, ml, st) \
                                           : launch_attn<GG, false>(q, q_rs, pool, bt, bt_rs, cached, kv_start, B, Hkv, NS, chunk, qscale, ring, \
                                                                     tail_len, tail_idx, T, opart, ml, st); break;
  switch (G) { KV_CASE(1) KV_CASE(2) KV_CASE(3) KV_CASE(4) KV_CASE(5) KV_CASE(6) KV_CASE(7) KV_CASE(8) }
#undef KV_CASE
  if (rc) return check_launch("kv_attn (shared memory)") ? 1 : 1;
  k_kv_merge<<<dim3(B, Hkv * G), 128, 0, st>>>(static_cast<const float*>(opart), static_cast<const float*>(ml), Hkv, G, NS,
                                               static_cast<__nv_bfloat16*>(out), out_rs);
  return check_launch("kv_attn");
}

int kv_dequant(const void* pool, const void* bt, int g0, int g1, int nvalid, int Hkv, int Dd, int fp32, void* ok, void* ov,
               int f8, void* stream) {
  if (g1 <= g0) return 0;
  if (Dd != D) return fail("kv_dequant: D %d (head dim 128 only)", Dd);
  const dim3 grid(g1 - g0, Hkv);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define KV_DQ(T, F) k_kv_dequant<T, F><<<grid, 128, 0, st>>>(static_cast<const uint8_t*>(pool), static_cast<const int*>(bt), g0, Hkv, \
                                                             nvalid, static_cast<T*>(ok), static_cast<T*>(ov))
  if (fp32) { if (f8 & 1) KV_DQ(float, true); else KV_DQ(float, false); }
  else { if (f8 & 1) KV_DQ(__nv_bfloat16, true); else KV_DQ(__nv_bfloat16, false); }
#undef KV_DQ
  return check_launch("kv_dequant");
}

int kv_lse_merge(const void* oa, const void* la, long long la_hs, const void* ob, const void* lb, long long lb_hs, void* out,
                 long long out_rs, int na, int H, int Dd, void* stream) {
  if (na <= 0) return 0;
  const long long tot = static_cast<long long>(na) * H * Dd;
  k_kv_lse_merge<<<static_cast<unsigned>((tot + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(oa), static_cast<const float*>(la), la_hs, static_cast<const __nv_bfloat16*>(ob),
      static_cast<const float*>(lb), lb_hs, static_cast<__nv_bfloat16*>(out), out_rs, na, H, Dd);
  return check_launch("kv_lse_merge");
}

}  // extern "C"
