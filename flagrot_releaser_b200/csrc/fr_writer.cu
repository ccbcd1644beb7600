// Paged cache writers for sm_100a: whole-head Hadamard, static writer (block flags, whole-head flags, key centring) and
// the dynamic key-only 2x2 writer (per 32-vector {I, H32} x per head {base, H128} chosen by the calibrated
// attention-weighted error; flags in the sign bits of the scale words).
//
// Replaces, byte for byte, the reference kernels k_paged_write (kernels/csrc/attn_decode_v2.cu:1717-1881), k_head_fwht
// and k_head_fwht256 (integrations/vllm_flagrot/csrc/flagrot_capi.cu:167-245), k_cb_write (kernels/csrc/attn_codebook.cu:46-361) and the
// fused v3 writers (kernels/csrc/attn_cb_write3.cuh) for the kinds konlya / konlya2 and the formats int4a / int2a.
//
// Structure: two kernels for appends and small writes, three more for bulk writes.
//   k_rows      one warp per (token, K or V row): load 4 bf16 per lane, optional whole-head H128 (+ bf16 rounding),
//               key centring, per-block H32, group quantizer, scatter into the page.  Used for the static formats
//               (all rows) and for the value rows of the dynamic kinds.
//   k_dyn_keys  one CTA of 128 threads per (kv head, TG tokens).  Thread i owns dimension i, so the 32 x 32 and
//               128 x 128 weighted-error products read C_q^T rows fully coalesced (L1 / L2 resident, 64 KB per head; for a
//               decode append of a few tokens the head's C_q^T is first staged in shared memory by a bulk copy, which
//               takes the L2 latency out of the 128-step sums) and accumulate in the reference's sequential fp32 order;
//               the whole-head candidate is evaluated by one warp per token in the row mapping.  No tensor cores here:
//               the criterion is defined by its fp32 operation order.
//   k_rows8 / k_rows8v   bulk rows: a warp per (8 consecutive tokens, row), whole V^T words where the slots allow;
//               k_rows8v computes transformed rows with a lane per 32-vector.
//   k_dyn_keys_bulk      bulk keys: 8 tokens per CTA; the head choice is first estimated on the tensor cores with a
//               rigorous error bar, and only the undecided tokens take the fixed-order fp32 sums (same bytes).
// V^T code words are shared by 8 tokens; a token only ever flips the bits of its own field (fr::put_field), so tokens
// of one word may be written by different warps, kernels or streams in any order.
#include "fr_common.cuh"
#include "fr_kernels.h"
#include "fr_tc5.cuh"

namespace fr {

// ------------------------------------------------------------------------------------------------ whole-head Hadamard
// One warp per (token, head).  NH = head dim / 128: lane l holds d = 128 s + 4 l .. + 3 of every 128-half s; the
// butterflies of strides 1 .. 64 run inside each half, the stride-128 one (NH = 2) between the two register sets.
template <int NH>
__global__ void __launch_bounds__(256) k_head_fwht(const __nv_bfloat16* __restrict__ x, long long x_ts,
                                                   __nv_bfloat16* out, long long o_ts, int T, int H,
                                                   const uint8_t* __restrict__ flags, float scale) {
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= static_cast<long long>(T) * H) return;
  const int t = static_cast<int>(warp / H), h = static_cast<int>(warp % H);
  const __nv_bfloat16* src = x + t * x_ts + h * (HD * NH) + 4 * lane;
  __nv_bfloat16* dst = out + t * o_ts + h * (HD * NH) + 4 * lane;
  uint2 res[NH];
#pragma unroll
  for (int s = 0; s < NH; ++s) res[s] = *reinterpret_cast<const uint2*>(src + HD * s);
  if (flags[h]) {
    float v[NH][4];
#pragma unroll
    for (int s = 0; s < NH; ++s) {
      v[s][0] = bf16_lo(res[s].x); v[s][1] = bf16_hi(res[s].x); v[s][2] = bf16_lo(res[s].y); v[s][3] = bf16_hi(res[s].y);
      fwht_row_stages(v[s], lane, 128);
    }
    if (NH == 2) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float a = v[0][i], b = v[NH - 1][i];
        v[0][i] = __fadd_rn(a, b);
        v[NH - 1][i] = __fsub_rn(a, b);
      }
    }
#pragma unroll
    for (int s = 0; s < NH; ++s) {
      const __nv_bfloat162 r0 = __floats2bfloat162_rn(__fmul_rn(v[s][0], scale), __fmul_rn(v[s][1], scale));
      const __nv_bfloat162 r1 = __floats2bfloat162_rn(__fmul_rn(v[s][2], scale), __fmul_rn(v[s][3], scale));
      res[s].x = *reinterpret_cast<const uint32_t*>(&r0);
      res[s].y = *reinterpret_cast<const uint32_t*>(&r1);
    }
  }
#pragma unroll
  for (int s = 0; s < NH; ++s) *reinterpret_cast<uint2*>(dst + HD * s) = res[s];
}

// ------------------------------------------------------------------------------------------------ page stores
// K row of one token from the 128 codes of the row (row mapping: lane l holds d = 4 l .. 4 l + 3)
template <int NB, bool SYM = false>
FR_DEVI void store_k_row(uint8_t* chunk, int P, int pos, int lane, const unsigned (&code)[4], unsigned word) {
  unsigned cb[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) cb[i] = __shfl_down_sync(FULLMASK, code[i], 4);   // the B elements (d + 16)
  const int tg = lane & 7, j = lane >> 3;
  if (NB == 4) {
    unsigned wd = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i)
      wd |= SYM ? sym_bits(code[i], false, i) | sym_bits(cb[i], true, i) : (code[i] << (8 * i)) | (cb[i] << (8 * i + 4));
    if (tg < 4) *reinterpret_cast<uint32_t*>(chunk + Lay<4>::krow(pos) + 16 * tg + 4 * j) = wd;
  } else {
    unsigned hw = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) hw |= (code[i] << (8 * i)) | (cb[i] << (8 * i + 2));
    const unsigned hw1 = __shfl_down_sync(FULLMASK, hw, 8);                     // group j + 1
    if (tg < 4 && !(j & 1)) *reinterpret_cast<uint32_t*>(chunk + Lay<2>::krow(pos) + 8 * tg + 4 * (j >> 1)) = hw | (hw1 << 4);
  }
  if (tg == 0) *reinterpret_cast<uint16_t*>(chunk + Lay<NB>::ks_off(P) + 8 * pos + 2 * j) = static_cast<uint16_t>(word);
}

// V^T codes + V scale of one token (row mapping).  shared15: bit 15 of the group-0 word belongs to the key writer.
template <int NB, bool SYM = false>
FR_DEVI void store_v_row(uint8_t* chunk, int P, int pos, int lane, const unsigned (&code)[4], unsigned word, bool shared15) {
  const int c8 = pos >> 3, ii = (pos & 7) >> 1, b = pos & 1;
  const int w = (lane & 15) >> 2, r8 = (lane & 3) >> 1, m = lane >> 4;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gid = 4 * (lane & 1) + i;
    const int e = (w * 8 + gid) * (P >> 3) + c8;
    if (SYM) put_bits(chunk, Lay<4>::v_off(P) + 16 * e + 4 * (2 * m + r8), sym_mask(b != 0, ii), sym_bits(code[i], b != 0, ii));
    else if (NB == 4) put_field(chunk, Lay<4>::v_off(P) + 16 * e + 4 * (2 * m + r8) + ii, 4 * b, 0xFu, code[i]);
    else put_field(chunk, Lay<2>::v_off(P) + 8 * e + 4 * m + ii, 4 * r8 + 2 * b, 0x3u, code[i]);
  }
  if ((lane & 7) == 0) {
    const int j = lane >> 3;
    const int off = Lay<NB>::vs_off(P) + 2 * (j * P + 8 * c8 + vslot8(pos));
    if (shared15 && j == 0) put_word_low15(chunk, off, word);
    else *reinterpret_cast<uint16_t*>(chunk + off) = static_cast<uint16_t>(word);
  }
}

// ------------------------------------------------------------------------------------------------ row writer
struct RowParams {
  const __nv_bfloat16* kv; long long kv_ts;
  const long long* slots; int slot_ph;
  int T, Hkv, page;
  const uint8_t* mask;      // [2 Hkv, 4] H32 block flags (K rows first) or null
  const uint8_t* hfull;     // [2 Hkv] whole-head flags or null
  const float* kmu;         // [Hkv, 128] or null
  uint8_t* pool;
  int row0, nrow;           // rows [row0, row0 + nrow) of the 2 Hkv rows of a token
  int shared15;
};

// codes and scale word of row hr of token t (row mapping: lane l holds d = 4 l .. 4 l + 3): bf16 -> fp32, whole-head H128 / 16
// rounded to bf16, key centering, H32 of the flagged 32-blocks, stored-form quantiser
template <int NB, bool SYM = false>
FR_DEVI void row_codes(const RowParams& p, int t, int hr, int lane, unsigned (&code)[4], unsigned& word) {
  const bool isv = hr >= p.Hkv;
  const uint2 raw = *reinterpret_cast<const uint2*>(p.kv + t * p.kv_ts + hr * HD + 4 * lane);
  float v[4] = {bf16_lo(raw.x), bf16_hi(raw.x), bf16_lo(raw.y), bf16_hi(raw.y)};
  if (p.hfull != nullptr && p.hfull[hr]) {   // whole-head H128 x / 16, rounded to bf16 once
    fwht_row_stages(v, lane, 128);
    const __nv_bfloat162 r0 = __floats2bfloat162_rn(__fmul_rn(v[0], 0.0625f), __fmul_rn(v[1], 0.0625f));
    const __nv_bfloat162 r1 = __floats2bfloat162_rn(__fmul_rn(v[2], 0.0625f), __fmul_rn(v[3], 0.0625f));
    const uint32_t a = *reinterpret_cast<const uint32_t*>(&r0), b = *reinterpret_cast<const uint32_t*>(&r1);
    v[0] = bf16_lo(a); v[1] = bf16_hi(a); v[2] = bf16_lo(b); v[3] = bf16_hi(b);
  }
  if (p.kmu != nullptr && !isv) {
    const float4 m = *reinterpret_cast<const float4*>(p.kmu + hr * HD + 4 * lane);
    v[0] = __fsub_rn(v[0], m.x); v[1] = __fsub_rn(v[1], m.y); v[2] = __fsub_rn(v[2], m.z); v[3] = __fsub_rn(v[3], m.w);
  }
  const bool rot = p.mask != nullptr && p.mask[hr * 4 + (lane >> 3)];
  {  // H32 of the flagged 32-blocks (the shuffles run on every lane; unflagged groups keep their values)
    float y[4] = {v[0], v[1], v[2], v[3]};
    if (p.mask != nullptr && __any_sync(FULLMASK, rot)) {
      fwht_row_stages(y, lane, 32);
#pragma unroll
      for (int i = 0; i < 4; ++i) if (rot) v[i] = __fmul_rn(y[i], C32);
    }
  }
  const float mn = group_min8(fminf(fminf(v[0], v[1]), fminf(v[2], v[3])));
  const float mx = group_max8(fmaxf(fmaxf(v[0], v[1]), fmaxf(v[2], v[3])));
  word = 0;
  if (SYM) {
    const float amax = fmaxf(-mn, mx);                 // = max |v| of the 32-group (exact)
#pragma unroll
    for (int i = 0; i < 4; ++i) quant_store_sym(v[i], amax, code[i], word);
    return;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) quant_store<NB>(v[i], mn, mx, code[i], word);
}

// one (token, row) of a warp: quantise and store at `slot` (the whole warp takes part; slot < 0: nothing is written)
template <int NB, bool SYM = false>
FR_DEVI void row_write(const RowParams& p, int t, int hr, long long slot, int lane) {
  if (slot < 0) return;
  const bool isv = hr >= p.Hkv;
  const int head = isv ? hr - p.Hkv : hr;
  const int P = p.page;
  const long long page = slot / P;
  const int pos = static_cast<int>(slot % P);
  uint8_t* chunk = p.pool + (page * p.Hkv + head) * static_cast<long long>(Lay<NB>::chunk(P));
  unsigned code[4], word;
  row_codes<NB, SYM>(p, t, hr, lane, code, word);
  if (!isv) store_k_row<NB, SYM>(chunk, P, pos, lane, code, word);
  else store_v_row<NB, SYM>(chunk, P, pos, lane, code, word, p.shared15 != 0);
}

template <int NB, bool SYM = false>
FR_DEVI void rows_block(const RowParams& p, long long block) {
  const int lane = threadIdx.x & 31;
  const long long item = block * 4 + (threadIdx.x >> 5);
  if (item >= static_cast<long long>(p.T) * p.nrow) return;
  const int t = static_cast<int>(item / p.nrow), hr = p.row0 + static_cast<int>(item % p.nrow);
  const int head = hr >= p.Hkv ? hr - p.Hkv : hr;
  row_write<NB, SYM>(p, t, hr, p.slot_ph ? p.slots[static_cast<long long>(t) * p.Hkv + head] : p.slots[t], lane);
}

template <int NB, bool SYM = false>
__global__ void __launch_bounds__(128) k_rows(const RowParams p) { rows_block<NB, SYM>(p, blockIdx.x); }

// Bulk writes: warp = (8 consecutive tokens, row).  A V^T code word holds ONE dim of the 8 tokens of an aligned 8-slot run of
// a page (INT2: two dims), so when the group's slots are such a run the warp assembles whole words in registers and stores
// them plainly (4 words per lane and 16 bytes of scale words per 32-group) instead of flipping 128 four-bit fields per token
// with atomics.  Any other group (ragged end, holes, scattered slots) and every K row take the per-token path.
template <int NB, bool SYM = false>
__global__ void __launch_bounds__(128) k_rows8(const RowParams p) {
  const int lane = threadIdx.x & 31;
  const long long item = static_cast<long long>(blockIdx.x) * 4 + (threadIdx.x >> 5);
  const int groups = (p.T + 7) >> 3;
  if (item >= static_cast<long long>(groups) * p.nrow) return;
  const int g = static_cast<int>(item / p.nrow), hr = p.row0 + static_cast<int>(item % p.nrow);
  const bool isv = hr >= p.Hkv;
  const int head = isv ? hr - p.Hkv : hr;
  const int t0 = 8 * g, nt = min(8, p.T - t0);
  long long sl = -1;
  if (lane < nt) sl = p.slot_ph ? p.slots[static_cast<long long>(t0 + lane) * p.Hkv + head] : p.slots[t0 + lane];
  const long long s0 = __shfl_sync(FULLMASK, sl, 0);
  const bool run = nt == 8 && s0 >= 0 && (s0 & 7) == 0 && __all_sync(FULLMASK, lane >= 8 || sl == s0 + lane);
  if (!isv || !run) {
    for (int i = 0; i < nt; ++i) row_write<NB, SYM>(p, t0 + i, hr, __shfl_sync(FULLMASK, sl, i), lane);
    return;
  }
  const int P = p.page;
  const int pos0 = static_cast<int>(s0 % P), c8 = pos0 >> 3;
  uint8_t* chunk = p.pool + ((s0 / P) * p.Hkv + head) * static_cast<long long>(Lay<NB>::chunk(P));
  unsigned acc[4] = {0u, 0u, 0u, 0u};       // per dim of the lane: the 8 tokens' codes (byte i >> 1, field i & 1)
  unsigned sw[4] = {0u, 0u, 0u, 0u};        // the 8 scale words of the lane's 32-group in page order (tokens 0 2 4 6 1 3 5 7)
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    unsigned code[4], word;
    row_codes<NB, SYM>(p, t0 + i, hr, lane, code, word);
#pragma unroll
    for (int k = 0; k < 4; ++k) acc[k] |= SYM ? sym_bits(code[k], (i & 1) != 0, i >> 1) : code[k] << (8 * (i >> 1) + NB * (i & 1));
    const int idx = (i & 1) ? 4 + (i >> 1) : (i >> 1);
    sw[idx >> 1] |= (word & 0xFFFFu) << (16 * (idx & 1));
  }
  const int w = (lane & 15) >> 2, r8 = (lane & 3) >> 1, m = lane >> 4;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int gid = 4 * (lane & 1) + k;
    const int e = (w * 8 + gid) * (P >> 3) + c8;
    if (NB == 4) {
      *reinterpret_cast<uint32_t*>(chunk + Lay<4>::v_off(P) + 16 * e + 4 * (2 * m + r8)) = acc[k];
    } else {                                  // dims d (r8 = 0, this lane) and d + 8 (lane + 2) share the word
      const unsigned hi = __shfl_down_sync(FULLMASK, acc[k], 2);
      if (r8 == 0) *reinterpret_cast<uint32_t*>(chunk + Lay<2>::v_off(P) + 8 * e + 4 * m) = acc[k] | (hi << 4);
    }
  }
  if ((lane & 7) == 0) {
    const int j = lane >> 3;
    const int off = Lay<NB>::vs_off(P) + 2 * (j * P + 8 * c8);
    if (p.shared15 && j == 0) {               // bit 15 of these words belongs to the key writer
#pragma unroll
      for (int x = 0; x < 8; ++x) put_word_low15(chunk, off + 2 * x, (sw[x >> 1] >> (16 * (x & 1))) & 0xFFFFu);
    } else {
      *reinterpret_cast<uint4*>(chunk + off) = make_uint4(sw[0], sw[1], sw[2], sw[3]);
    }
  }
}

// rintf(__fdiv_rn(a, b)) for a whole vector with one multiplication per element where that is provably the same:
// y = __frcp_rn(b), 1e-30 < b < 1e30, |a / b| < 2^20.  q0 = RN(a y) and RN(a / b) both lie within 3 * 2^-24 |a / b| of a / b,
// so they round to the same integer unless q0 is within 2.4e-7 |q0| of a half-integer (`near` collects that; the caller
// then redoes the vector with divisions).  The rounding itself is an addition of 1.5 * 2^23 (round to nearest even).
constexpr float RMAGIC = 12582912.f;
FR_DEVI float rint_mul(float a, float y, bool& near) {
  const float q0 = __fmul_rn(a, y);
  const float r = __fsub_rn(__fadd_rn(q0, RMAGIC), RMAGIC);
  near |= !(fabsf(__fsub_rn(fabsf(__fsub_rn(q0, r)), 0.5f)) > fmaf(fabsf(q0), 2.4e-7f, 1e-30f));
  return r;
}

// "vector" mapping of the bulk writer: a lane holds one whole 32-vector of a row in registers, so the H32 butterflies,
// the range and the quantizer need no shuffles (lane = 4 * token + vector of a group of 8 tokens; the whole-head H128
// takes its two outer stages from the neighbouring lanes).  Same operations in the same order as row_codes.
// Out: the 32 stored codes as bytes (cw[r] = codes 4 r .. 4 r + 3) and the scale word of the vector.
template <int NB, bool SYM>
FR_DEVI void vec_codes(const RowParams& p, int t, bool live, int hr, int b, unsigned (&cw)[8], unsigned& word) {
  float v[32];
  if (live) {
    const uint4* src = reinterpret_cast<const uint4*>(p.kv + t * p.kv_ts + hr * HD + 32 * b);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const uint4 w = src[r];
      v[8 * r + 0] = bf16_lo(w.x); v[8 * r + 1] = bf16_hi(w.x); v[8 * r + 2] = bf16_lo(w.y); v[8 * r + 3] = bf16_hi(w.y);
      v[8 * r + 4] = bf16_lo(w.z); v[8 * r + 5] = bf16_hi(w.z); v[8 * r + 6] = bf16_lo(w.w); v[8 * r + 7] = bf16_hi(w.w);
    }
  } else {
#pragma unroll
    for (int r = 0; r < 32; ++r) v[r] = 0.f;
  }
  const bool hf = p.hfull != nullptr && p.hfull[hr];                  // uniform over the warp
  const bool rot = p.mask != nullptr && p.mask[hr * 4 + b];           // per lane
  const bool ctr = p.kmu != nullptr && hr < p.Hkv;
  // pass 0: whole-head H128 x / 16 rounded to bf16 once (if hf); pass 1: key centring, then H32 of a flagged vector.
  // One copy of the 32-point butterflies serves both (the loop is kept rolled: the code stays small).
#pragma unroll 1
  for (int pass = 0; pass < 2; ++pass) {
    if (pass == 1 && ctr) {
      const float4* mu = reinterpret_cast<const float4*>(p.kmu + hr * HD + 32 * b);
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const float4 m = __ldg(mu + r);
        v[4 * r] = __fsub_rn(v[4 * r], m.x); v[4 * r + 1] = __fsub_rn(v[4 * r + 1], m.y);
        v[4 * r + 2] = __fsub_rn(v[4 * r + 2], m.z); v[4 * r + 3] = __fsub_rn(v[4 * r + 3], m.w);
      }
    }
    const bool act = pass == 0 ? hf : rot;
    if (!__any_sync(FULLMASK, act)) continue;
    float w[32];
#pragma unroll
    for (int r = 0; r < 32; ++r) w[r] = v[r];
#pragma unroll
    for (int h = 1; h < 32; h <<= 1)            // unnormalised butterflies h = 1 .. 16 inside the vector
#pragma unroll
      for (int r = 0; r < 32; ++r)
        if (!(r & h)) {
          const float x = w[r], y = w[r + h];
          w[r] = __fadd_rn(x, y);
          w[r + h] = __fsub_rn(x, y);
        }
    if (pass == 0) {                            // (uniform) h = 32, 64: the other vectors of the token sit in the lanes b ^ 1, b ^ 2
#pragma unroll
      for (int m = 1; m < 4; m <<= 1)
#pragma unroll
        for (int r = 0; r < 32; ++r) {
          const float o = __shfl_xor_sync(FULLMASK, w[r], m);
          w[r] = (b & m) ? __fsub_rn(o, w[r]) : __fadd_rn(w[r], o);
        }
#pragma unroll
      for (int r = 0; r < 32; r += 2) {
        const __nv_bfloat162 q = __floats2bfloat162_rn(__fmul_rn(w[r], 0.0625f), __fmul_rn(w[r + 1], 0.0625f));
        const uint32_t u = *reinterpret_cast<const uint32_t*>(&q);
        v[r] = bf16_lo(u);
        v[r + 1] = bf16_hi(u);
      }
    } else {
#pragma unroll
      for (int r = 0; r < 32; ++r) v[r] = act ? __fmul_rn(w[r], C32) : v[r];
    }
  }
  float mn = v[0], mx = v[0];
#pragma unroll
  for (int r = 1; r < 32; ++r) { mn = fminf(mn, v[r]); mx = fmaxf(mx, v[r]); }
#pragma unroll
  for (int r = 0; r < 8; ++r) cw[r] = 0u;
  const float amax = fmaxf(-mn, mx);
  if (SYM) {                                   // quant_store_sym
    const __half sh = __float2half_rn(__fmul_rn(amax, 1.0f / 7.0f));
    const float sf = __half2float(sh);
    word = __half_as_ushort(sh);
    if (sf == 0.f) return;                     // all codes 0
    bool slow = !(sf > 1e-30f && sf < 1e30f && amax < __fmul_rn(sf, 1048576.f));
    if (!slow) {
      const float y = __frcp_rn(sf);
#pragma unroll
      for (int r = 0; r < 32; ++r) {
        const float q = fminf(fmaxf(rint_mul(v[r], y, slow), -7.f), 7.f);
        // sign-magnitude: 8 | |q| for q < 0; |q| <= 7 sits in the low bits of |q| + 1.5 * 2^23
        const unsigned mag = __float_as_uint(__fadd_rn(fabsf(q), RMAGIC)) & 7u;
        cw[r >> 2] |= (mag | (q < 0.f ? 8u : 0u)) << (8 * (r & 3));
      }
    }
    if (slow) {                                // (rare) some quotient sits on a rounding boundary: every element by division
#pragma unroll
      for (int r = 0; r < 8; ++r) cw[r] = 0u;
#pragma unroll
      for (int r = 0; r < 32; ++r) {
        unsigned c, w2;
        quant_store_sym(v[r], amax, c, w2);
        cw[r >> 2] |= c << (8 * (r & 3));
      }
    }
    return;
  }
  float sc, z;                                 // quant_store: the range widened to include 0
  asym_params<NB>(fminf(mn, 0.f), fmaxf(mx, 0.f), sc, z);
  word = scale_word<NB>(sc, static_cast<unsigned>(z));
  constexpr float LV = static_cast<float>((1 << NB) - 1);
  bool slow = !(sc > 1e-30f && sc < 1e30f && amax < __fmul_rn(sc, 1048576.f));
  if (!slow) {
    const float y = __frcp_rn(sc);
#pragma unroll
    for (int r = 0; r < 32; ++r) {
      const float q = fminf(fmaxf(__fadd_rn(rint_mul(v[r], y, slow), z), 0.f), LV);
      cw[r >> 2] |= (__float_as_uint(__fadd_rn(q, RMAGIC)) & 0xFu) << (8 * (r & 3));
    }
  }
  if (slow) {
#pragma unroll
    for (int r = 0; r < 8; ++r) cw[r] = 0u;
#pragma unroll
    for (int r = 0; r < 32; ++r) cw[r >> 2] |= static_cast<unsigned>(asym_code<NB>(v[r], sc, z)) << (8 * (r & 3));
  }
}

// k_rows8 for rows that are transformed before they are quantised (static formats with block flags or whole-head flags):
// warp = (8 consecutive tokens, row); the codes are computed in the vector mapping (vec_codes), handed over through shared
// memory and stored in the row mapping (lane l: d = 4 l .. 4 l + 3 of one token) exactly as k_rows8 stores them.  A V^T code word holds ONE
// dim of the 8 tokens of an aligned 8-slot run of a page (INT2: two dims), so when the group's slots are such a run the warp
// assembles whole words in registers and stores them plainly (4 words per lane and 16 bytes of scale words per 32-group)
// instead of flipping 128 four-bit fields per token with atomics.  Any other group (ragged end, holes, scattered slots) and
// every K row are stored token by token.
template <int NB, bool SYM = false>
__global__ void __launch_bounds__(128) k_rows8v(const RowParams p) {
  __shared__ __align__(16) uint8_t cs8[4][8][HD];     // per warp: stored codes [token][dim]
  __shared__ uint16_t ws8[4][8][4];                   // and scale words [token][vector]
  const int lane = threadIdx.x & 31, wp = threadIdx.x >> 5;
  const long long item = static_cast<long long>(blockIdx.x) * 4 + wp;
  const int groups = (p.T + 7) >> 3;
  if (item >= static_cast<long long>(groups) * p.nrow) return;
  const int g = static_cast<int>(item / p.nrow), hr = p.row0 + static_cast<int>(item % p.nrow);
  const bool isv = hr >= p.Hkv;
  const int head = isv ? hr - p.Hkv : hr;
  const int t0 = 8 * g, nt = min(8, p.T - t0);
  long long sl = -1;
  if (lane < nt) sl = p.slot_ph ? p.slots[static_cast<long long>(t0 + lane) * p.Hkv + head] : p.slots[t0 + lane];
  const long long s0 = __shfl_sync(FULLMASK, sl, 0);
  const bool run = nt == 8 && s0 >= 0 && (s0 & 7) == 0 && __all_sync(FULLMASK, lane >= 8 || sl == s0 + lane);
  {
    const int tl = lane >> 2, b = lane & 3;
    unsigned cw[8], word;
    vec_codes<NB, SYM>(p, t0 + tl, tl < nt, hr, b, cw, word);
    uint4* dst = reinterpret_cast<uint4*>(&cs8[wp][tl][32 * b]);
    dst[0] = make_uint4(cw[0], cw[1], cw[2], cw[3]);
    dst[1] = make_uint4(cw[4], cw[5], cw[6], cw[7]);
    ws8[wp][tl][b] = static_cast<uint16_t>(word);
  }
  __syncwarp();
  if (!isv || !run) {
    const int P = p.page;
    for (int i = 0; i < nt; ++i) {
      const long long slot = __shfl_sync(FULLMASK, sl, i);
      if (slot < 0) continue;
      uint8_t* chunk = p.pool + ((slot / P) * p.Hkv + head) * static_cast<long long>(Lay<NB>::chunk(P));
      const int pos = static_cast<int>(slot % P);
      const unsigned c4 = *reinterpret_cast<const uint32_t*>(&cs8[wp][i][4 * lane]);
      const unsigned code[4] = {c4 & 0xFFu, (c4 >> 8) & 0xFFu, (c4 >> 16) & 0xFFu, c4 >> 24};
      const unsigned word = ws8[wp][i][lane >> 3];
      if (!isv) store_k_row<NB, SYM>(chunk, P, pos, lane, code, word);
      else store_v_row<NB, SYM>(chunk, P, pos, lane, code, word, p.shared15 != 0);
    }
    return;
  }
  const int P = p.page;
  const int pos0 = static_cast<int>(s0 % P), c8 = pos0 >> 3;
  uint8_t* chunk = p.pool + ((s0 / P) * p.Hkv + head) * static_cast<long long>(Lay<NB>::chunk(P));
  unsigned acc[4] = {0u, 0u, 0u, 0u};       // per dim of the lane: the 8 tokens' codes (byte i >> 1, field i & 1)
  unsigned sw[4] = {0u, 0u, 0u, 0u};        // the 8 scale words of the lane's 32-group in page order (tokens 0 2 4 6 1 3 5 7)
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const unsigned c4 = *reinterpret_cast<const uint32_t*>(&cs8[wp][i][4 * lane]);
    const unsigned code[4] = {c4 & 0xFFu, (c4 >> 8) & 0xFFu, (c4 >> 16) & 0xFFu, c4 >> 24};
    const unsigned word = ws8[wp][i][lane >> 3];
#pragma unroll
    for (int k = 0; k < 4; ++k) acc[k] |= SYM ? sym_bits(code[k], (i & 1) != 0, i >> 1) : code[k] << (8 * (i >> 1) + NB * (i & 1));
    const int idx = (i & 1) ? 4 + (i >> 1) : (i >> 1);
    sw[idx >> 1] |= (word & 0xFFFFu) << (16 * (idx & 1));
  }
  const int w = (lane & 15) >> 2, r8 = (lane & 3) >> 1, m = lane >> 4;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int gid = 4 * (lane & 1) + k;
    const int e = (w * 8 + gid) * (P >> 3) + c8;
    if (NB == 4) {
      *reinterpret_cast<uint32_t*>(chunk + Lay<4>::v_off(P) + 16 * e + 4 * (2 * m + r8)) = acc[k];
    } else {                                  // dims d (r8 = 0, this lane) and d + 8 (lane + 2) share the word
      const unsigned hi = __shfl_down_sync(FULLMASK, acc[k], 2);
      if (r8 == 0) *reinterpret_cast<uint32_t*>(chunk + Lay<2>::v_off(P) + 8 * e + 4 * m) = acc[k] | (hi << 4);
    }
  }
  if ((lane & 7) == 0) {
    const int j = lane >> 3;
    const int off = Lay<NB>::vs_off(P) + 2 * (j * P + 8 * c8);
    if (p.shared15 && j == 0) {               // bit 15 of these words belongs to the key writer
#pragma unroll
      for (int x = 0; x < 8; ++x) put_word_low15(chunk, off + 2 * x, (sw[x >> 1] >> (16 * (x & 1))) & 0xFFFFu);
    } else {
      *reinterpret_cast<uint4*>(chunk + off) = make_uint4(sw[0], sw[1], sw[2], sw[3]);
    }
  }
}

// ------------------------------------------------------------------------------------------------ dynamic key writer
struct DynParams {
  const __nv_bfloat16* kv; long long kv_ts;
  const long long* slots; int slot_ph;
  int T, Hkv, page;
  const float* CT;          // [Hkv, 128 (k), 128 (i)] = C_q[h][i][k]
  const float* kmu;
  uint8_t* pool;
};

static __device__ __forceinline__ uint32_t wsmem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ int g_wstatus;                   // != 0: the staging copy of C_q^T did not arrive in time (the kernel then read global memory)

// rows.T > 0 (STAGED launches only): the grid has extra rows y >= ceil(T / TG) whose CTAs write the value rows of the same
// tokens (rows_block), so that an append is one launch; key and value writers only flip bits of their own fields
template <int NB, int TG, bool STAGED, bool SYM = false>
__global__ void __launch_bounds__(128) k_dyn_keys(const DynParams p, const RowParams rows) {
  if (STAGED && rows.T > 0) {
    const int groups = (p.T + TG - 1) / TG;
    if (static_cast<int>(blockIdx.y) >= groups) {
      rows_block<NB, SYM>(rows, static_cast<long long>(blockIdx.y - groups) * gridDim.x + blockIdx.x);
      return;
    }
  }
  extern __shared__ __align__(128) float cts[];   // STAGED: C_q^T of this head [128 (k)][128 (i)]
  __shared__ __align__(8) uint64_t ctbar;
  __shared__ float xs[TG][HD];              // centred key rows
  __shared__ float es[TG][2][HD];           // reconstruction errors of the head candidates (base, F)
  __shared__ float ps[TG][2][HD];           // e_i * u_i
  __shared__ uint8_t cs[TG][2][HD];         // stored codes of the head candidates
  __shared__ uint16_t ws[TG][2][4];         // stored scale words (base: with the H32 flag)
  __shared__ float herr[TG][2];
  const int i = threadIdx.x, lane = i & 31, j = i >> 5;
  const int h = blockIdx.x;
  const float* CT = p.CT + static_cast<size_t>(h) * HD * HD;
  if (STAGED && i == 0) {
    tc5::mbar_init(wsmem_u32(&ctbar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    tc5::mbar_expect(wsmem_u32(&ctbar), HD * HD * 4);
#pragma unroll
    for (int c = 0; c < 4; ++c)
      tc5::bulk_g2s(wsmem_u32(cts) + c * (HD * HD), reinterpret_cast<const uint8_t*>(CT) + c * (HD * HD), HD * HD,
                    wsmem_u32(&ctbar));
  }
  if (STAGED) __syncthreads();
  bool staged = !STAGED;
  bool stage_lost = false;             // the staging wait ran out: the sums read C_q^T from global memory instead
  for (int t0 = blockIdx.y * TG; t0 < p.T; t0 += gridDim.y * TG) {
  const int ntok = min(TG, p.T - t0);

  // ---- A1: local candidates I / H32 of 32-vector j (dim mapping), block-diagonal weighted error, first argmin
#pragma unroll
  for (int t = 0; t < TG; ++t) {
    if (t >= ntok) break;
    float z = __bfloat162float(p.kv[(t0 + t) * p.kv_ts + h * HD + i]);
    if (p.kmu != nullptr) z = __fsub_rn(z, __ldg(p.kmu + h * HD + i));
    xs[t][i] = z;
    const float y1 = fwht32_lane(z, lane);
    const float mn0 = warp_min(z), mx0 = warp_max(z), mn1 = warp_min(y1), mx1 = warp_max(y1);
    const float e0 = __fsub_rn(dyn_err_deq<NB, SYM>(z, mn0, mx0), z);
    const float e1 = __fsub_rn(fwht32_lane(dyn_err_deq<NB, SYM>(y1, mn1, mx1), lane), z);
    float u0 = 0.f, u1 = 0.f;
    if (!staged) {                     // first use of C_q^T: the copy has had the loads and the Hadamard above to arrive
      staged = true;
      if (tc5::mbar_wait(wsmem_u32(&ctbar), 0)) CT = cts;
      else { stage_lost = true; if (i == 0) atomicExch(&g_wstatus, __LINE__); }
    }
#pragma unroll
    for (int k = 0; k < 32; ++k) {   // fully unrolled: the 32 loads do not depend on the sum chain and go out together
      const float cv = STAGED ? CT[(32 * j + k) * HD + i] : __ldg(CT + (32 * j + k) * HD + i);   // C[i][32 j + k]
      const float p0 = __fmul_rn(cv, __shfl_sync(FULLMASK, e0, k));
      const float p1 = __fmul_rn(cv, __shfl_sync(FULLMASK, e1, k));
      u0 = k == 0 ? p0 : __fadd_rn(u0, p0);
      u1 = k == 0 ? p1 : __fadd_rn(u1, p1);
    }
    const float err0 = tree32(__fmul_rn(e0, u0)), err1 = tree32(__fmul_rn(e1, u1));
    const bool ch = err1 < err0;
    unsigned code, word;
    dyn_store<NB, SYM>(ch ? y1 : z, ch ? mn1 : mn0, ch ? mx1 : mx0, code, word);
    es[t][0][i] = ch ? e1 : e0;
    cs[t][0][i] = static_cast<uint8_t>(code);
    if (lane == 0) ws[t][0][j] = static_cast<uint16_t>(word | (ch ? 0x8000u : 0u));
  }
  __syncthreads();
  // ---- A2: whole-head candidate F = H128 (row mapping, warp j = token j)
  if (j < ntok) {
    const int t = j;
    float x[4], y[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) { x[k] = xs[t][4 * lane + k]; y[k] = x[k]; }
    fwht_row_stages(y, lane, 128);
#pragma unroll
    for (int k = 0; k < 4; ++k) y[k] = __fmul_rn(y[k], C128);
    const float mn = group_min8(fminf(fminf(y[0], y[1]), fminf(y[2], y[3])));
    const float mx = group_max8(fmaxf(fmaxf(y[0], y[1]), fmaxf(y[2], y[3])));
    float d[4];
    unsigned word = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      unsigned code;
      d[k] = dyn_err_deq<NB, SYM>(y[k], mn, mx);
      dyn_store<NB, SYM>(y[k], mn, mx, code, word);
      cs[t][1][4 * lane + k] = static_cast<uint8_t>(code);
    }
    fwht_row_stages(d, lane, 128);
#pragma unroll
    for (int k = 0; k < 4; ++k) es[t][1][4 * lane + k] = __fsub_rn(__fmul_rn(d[k], C128), x[k]);
    if ((lane & 7) == 0) ws[t][1][lane >> 3] = static_cast<uint16_t>(word);
  }
  __syncthreads();
  // ---- B: u_i = ((U0 + U1) + U2) + U3, U_b = seq_{k in block b} C[i][k] e_k, for every (token, head candidate)
  {
    float u[TG][2];
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      float U[TG][2];
#pragma unroll 16
      for (int k = 0; k < 32; ++k) {
        const float cv = STAGED ? CT[(32 * b + k) * HD + i] : __ldg(CT + (32 * b + k) * HD + i);
#pragma unroll
        for (int t = 0; t < TG; ++t)
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const float pr = __fmul_rn(cv, es[t][c][32 * b + k]);
            U[t][c] = k == 0 ? pr : __fadd_rn(U[t][c], pr);
          }
      }
#pragma unroll
      for (int t = 0; t < TG; ++t)
#pragma unroll
        for (int c = 0; c < 2; ++c) u[t][c] = b == 0 ? U[t][c] : __fadd_rn(u[t][c], U[t][c]);
    }
#pragma unroll
    for (int t = 0; t < TG; ++t)
#pragma unroll
      for (int c = 0; c < 2; ++c) ps[t][c][i] = __fmul_rn(es[t][c][i], u[t][c]);
  }
  __syncthreads();
  // ---- C: halving tree of e * u over the 128 dims (warp per (token, candidate))
  for (int it = j; it < 2 * ntok; it += 4) {
    const int t = it >> 1, c = it & 1;
    const float a = __fadd_rn(ps[t][c][lane], ps[t][c][lane + 64]);
    const float b = __fadd_rn(ps[t][c][lane + 32], ps[t][c][lane + 96]);
    const float e = tree32(__fadd_rn(a, b));
    if (lane == 0) herr[t][c] = e;
  }
  __syncthreads();
  // ---- D: head choice and page write (warp j = token j)
  if (j < ntok) {
    const int t = j;
    const long long slot = p.slot_ph ? p.slots[static_cast<long long>(t0 + t) * p.Hkv + h] : p.slots[t0 + t];
    if (slot >= 0) {
    const bool F = herr[t][1] < herr[t][0];
    const int c = F ? 1 : 0;
    const int P = p.page;
    const long long page = slot / P;
    const int pos = static_cast<int>(slot % P);
    uint8_t* chunk = p.pool + (page * p.Hkv + h) * static_cast<long long>(Lay<NB>::chunk(P));
    unsigned code[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) code[k] = cs[t][c][4 * lane + k];
    store_k_row<NB, SYM>(chunk, P, pos, lane, code, ws[t][c][lane >> 3]);
    if (lane == 0)   // the key's whole-head flag rides in bit 15 of the token's V group-0 scale word
      put_word_bit15(chunk, Lay<NB>::vs_off(P) + 2 * (8 * (pos >> 3) + vslot8(pos)), F);
    }
  }
  __syncthreads();                     // the next group of tokens reuses the shared arrays
  }
  // a bulk copy that is still in flight must not land in shared memory the next CTA on this SM already owns: give it one
  // more bounded wait before the CTA leaves (the status word is set; the step's pages are to be rewritten by the caller)
  if (STAGED && stage_lost) tc5::mbar_wait(wsmem_u32(&ctbar), 0);
}

// ------------------------------------------------------------------------------------------------ dynamic key writer, bulk
// Same arithmetic as k_dyn_keys, arranged for many tokens: 8 tokens per CTA share every C_q^T value read, and the two
// candidates of a choice (I / H32 of a 32-vector, base / F of the head) ride in the halves of packed fp32 pairs
// (mul.f32x2 / add.f32x2 round each half like the scalar instruction, so the sequential sums are unchanged), which halves
// the arithmetic instructions and lets one 16-byte shared load feed four products.  CTAs are numbered head-major, so the
// CTAs resident on an SM at one time read the same 64 KB of C_q^T through L1.
FR_DEVI float2 tree32x2(float2 v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    v = __fadd2_rn(v, make_float2(__shfl_xor_sync(FULLMASK, v.x, o), __shfl_xor_sync(FULLMASK, v.y, o)));
  return v;
}

// one quantizer evaluation for both forms of the dynamic writer: the error form (unwidened range) gives the
// dequantized value of the criterion, the stored form (range widened to include 0) the code and the scale word.  When
// the group's range already contains 0 the two forms have the same parameters, so the second evaluation is skipped.
template <int NB, bool SYM> struct DynQ {
  float s, z, s2, z2;
  bool same;
  FR_DEVI DynQ(float mn, float mx) {
    if (SYM) {
      s = mn; z = mx; same = true; s2 = z2 = 0.f;     // (the symmetric quantizer has a single form; keeps the range)
    } else {
      asym_params<NB>(mn, mx, s, z);
      same = mn <= 0.f && mx >= 0.f;
      s2 = s; z2 = z;
      if (!same) asym_params<NB>(fminf(mn, 0.f), fmaxf(mx, 0.f), s2, z2);
    }
  }
  FR_DEVI void element(float y, float& deq, unsigned& code) const {
    if (SYM) {
      unsigned word;
      quant_store_sym(y, fmaxf(-s, z), code, word);
      deq = sym_deq(code, word);
    } else {
      const float q = asym_code<NB>(y, s, z);
      deq = __fmul_rn(__fsub_rn(q, z), s);
      code = static_cast<unsigned>(same ? q : asym_code<NB>(y, s2, z2));
    }
  }
  FR_DEVI unsigned word() const {
    if (SYM) return __half_as_ushort(__float2half_rn(__fmul_rn(fmaxf(-s, z), 1.0f / 7.0f)));
    return scale_word<NB>(s2, static_cast<unsigned>(z2));
  }
};

// counters of the bulk key writer: [0] (token, head) pairs written, [1] those whose head choice needed the exact sums
__device__ unsigned long long g_dynstat[2];
// relative half-width of the estimate's error bar, in units of sum |e_i| |C_ik| |e_k| (see the kernel's phase B)
constexpr float DYN_DELTA = 0.003f;

FR_DEVI void mma_tf32(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int NB, bool SYM>
__global__ void __launch_bounds__(128) k_dyn_keys_bulk(const DynParams p, int groups, int exact_only) {
  constexpr int TG = 8;
  // reconstruction errors of the head candidates (x: base, y: F); rows padded by 4 floats: the 8-byte operand loads of
  // the MMA phase (a half warp = 2 tokens x 4 k) then fall into 16 different banks
  __shared__ __align__(16) float2 es[TG][HD + 2];
  __shared__ __align__(16) float ef[TG][HD];         // errors of the F candidate as the row mapping produces them
  __shared__ float est[4][2 * TG][2];                // per warp: partial (estimate, bound) of row 2 t + c
  __shared__ int hsel[TG];                           // head choice of token t: 0 base, 1 F, 2 undecided (exact sums needed)
  __shared__ __align__(16) float2 ps[TG][HD];        // first the errors of the local candidates (x: I, y: H32), then e * u
  __shared__ __align__(4) uint8_t cs[TG][2][HD];     // stored codes of the head candidates
  __shared__ __align__(8) uint16_t lc[TG][HD];       // stored codes of the local candidates (low byte I, high byte H32)
  __shared__ uint16_t lw[TG][2][4];                  // and their scale words
  __shared__ uint16_t ws[TG][2][4];                  // stored scale words of the head candidates (base: with the H32 flag)
  const int i = threadIdx.x, lane = i & 31, j = i >> 5;
  const int h = blockIdx.x / groups, t0 = (blockIdx.x % groups) * TG;
  const int ntok = min(TG, p.T - t0);
  const float* CT = p.CT + static_cast<size_t>(h) * HD * HD;

  // ---- A: candidates of every token in the row mapping (warp j takes tokens j, j + 4; lane l holds d = 4 l .. 4 l + 3,
  //         32-vector = 8 lanes): both local candidates I / H32 (errors, stored codes, words) and the whole-head candidate F
  for (int t = j; t < TG; t += 4) {
    float x[4] = {0.f, 0.f, 0.f, 0.f};
    if (t < ntok) {
      const uint2 raw = *reinterpret_cast<const uint2*>(p.kv + (t0 + t) * p.kv_ts + h * HD + 4 * lane);
      x[0] = bf16_lo(raw.x); x[1] = bf16_hi(raw.x); x[2] = bf16_lo(raw.y); x[3] = bf16_hi(raw.y);
    }
    if (p.kmu != nullptr) {
      const float4 m = __ldg(reinterpret_cast<const float4*>(p.kmu + h * HD + 4 * lane));
      x[0] = __fsub_rn(x[0], m.x); x[1] = __fsub_rn(x[1], m.y); x[2] = __fsub_rn(x[2], m.z); x[3] = __fsub_rn(x[3], m.w);
    }
    float e0[4], e1[4];
    unsigned c0 = 0, c1 = 0;
    {   // I
      const DynQ<NB, SYM> q(group_min8(fminf(fminf(x[0], x[1]), fminf(x[2], x[3]))),
                            group_max8(fmaxf(fmaxf(x[0], x[1]), fmaxf(x[2], x[3]))));
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float d; unsigned c;
        q.element(x[k], d, c);
        e0[k] = __fsub_rn(d, x[k]);
        c0 |= c << (8 * k);
      }
      if ((lane & 7) == 0) lw[t][0][lane >> 3] = static_cast<uint16_t>(q.word());
    }
    {   // H32
      float y[4] = {x[0], x[1], x[2], x[3]};
      fwht_row_stages(y, lane, 32);
#pragma unroll
      for (int k = 0; k < 4; ++k) y[k] = __fmul_rn(y[k], C32);
      const DynQ<NB, SYM> q(group_min8(fminf(fminf(y[0], y[1]), fminf(y[2], y[3]))),
                            group_max8(fmaxf(fmaxf(y[0], y[1]), fmaxf(y[2], y[3]))));
      float d[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        unsigned c;
        q.element(y[k], d[k], c);
        c1 |= c << (8 * k);
      }
      fwht_row_stages(d, lane, 32);
#pragma unroll
      for (int k = 0; k < 4; ++k) e1[k] = __fsub_rn(__fmul_rn(d[k], C32), x[k]);
      if ((lane & 7) == 0) lw[t][1][lane >> 3] = static_cast<uint16_t>(q.word());
    }
    *reinterpret_cast<float4*>(&ps[t][4 * lane]) = make_float4(e0[0], e1[0], e0[1], e1[1]);
    *reinterpret_cast<float4*>(&ps[t][4 * lane + 2]) = make_float4(e0[2], e1[2], e0[3], e1[3]);
    {   // byte k of c0 / c1 -> 16-bit cells (I low, H32 high)
      const unsigned lo = __byte_perm(c0, c1, 0x5140), hi = __byte_perm(c0, c1, 0x7362);
      *reinterpret_cast<uint2*>(&lc[t][4 * lane]) = make_uint2(lo, hi);
    }
    {   // F = H128
      float y[4] = {x[0], x[1], x[2], x[3]};
      fwht_row_stages(y, lane, 128);
#pragma unroll
      for (int k = 0; k < 4; ++k) y[k] = __fmul_rn(y[k], C128);
      const DynQ<NB, SYM> q(group_min8(fminf(fminf(y[0], y[1]), fminf(y[2], y[3]))),
                            group_max8(fmaxf(fmaxf(y[0], y[1]), fmaxf(y[2], y[3]))));
      float d[4];
      unsigned cf = 0;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        unsigned c;
        q.element(y[k], d[k], c);
        cf |= c << (8 * k);
      }
      fwht_row_stages(d, lane, 128);
#pragma unroll
      for (int k = 0; k < 4; ++k) d[k] = __fsub_rn(__fmul_rn(d[k], C128), x[k]);
      *reinterpret_cast<float4*>(&ef[t][4 * lane]) = make_float4(d[0], d[1], d[2], d[3]);
      *reinterpret_cast<uint32_t*>(&cs[t][1][4 * lane]) = cf;
      if ((lane & 7) == 0) ws[t][1][lane >> 3] = static_cast<uint16_t>(q.word());
    }
  }
  __syncthreads();
  {   // ---- A1 (dim mapping, thread i = dim i, 32-vector j = warp j): block-diagonal weighted error u_i = seq_k C[i][32 j + k] e_k
    //      of both local candidates, first argmin
    float2 U[TG];
#pragma unroll
    for (int k = 0; k < 32; k += 2) {
      const float ca = __ldg(CT + (32 * j + k) * HD + i), cb = __ldg(CT + (32 * j + k + 1) * HD + i);
#pragma unroll
      for (int t = 0; t < TG; ++t) {
        const float4 e = *reinterpret_cast<const float4*>(&ps[t][32 * j + k]);
        const float2 pa = __fmul2_rn(make_float2(ca, ca), make_float2(e.x, e.y));
        U[t] = k == 0 ? pa : __fadd2_rn(U[t], pa);
        U[t] = __fadd2_rn(U[t], __fmul2_rn(make_float2(cb, cb), make_float2(e.z, e.w)));
      }
    }
#pragma unroll
    for (int t = 0; t < TG; ++t) {
      const float2 own = ps[t][i];
      const float2 err = tree32x2(__fmul2_rn(own, U[t]));
      const bool ch = err.y < err.x;
      es[t][i] = make_float2(ch ? own.y : own.x, ef[t][i]);
      const unsigned c = lc[t][i];
      cs[t][0][i] = static_cast<uint8_t>(ch ? c >> 8 : c & 0xFFu);
      if (lane == 0) ws[t][0][j] = static_cast<uint16_t>(ch ? (lw[t][1][j] | 0x8000u) : lw[t][0][j]);
    }
  }
  __syncthreads();
  // ---- B: head choice.  The criterion is herr_c = fl(sum_i e_i u_i), u_i = fl(sum_k C[i][k] e_k), summed in a fixed fp32
  //      order; F is chosen when herr_1 < herr_0.  First an estimate on the tensor cores: with T_c = e^T C e and
  //      S_c = sum_ik |e_i| |C_ik| |e_k| in real arithmetic, the fixed-order value satisfies |herr_c - T_c| <= 2^-18 S_c (43
  //      roundings on the path of a term), and E_c = sum_i e_i (C~ e~)_i with TF32 operands (each within 2^-10 of its
  //      value) and fp32 accumulation satisfies |E_c - T_c| <= 0.0020 S_c; B_c = sum_i |e_i| (|C~| |e~|)_i >= 0.9979 S_c.
  //      So |herr_c - E_c| < DYN_DELTA B_c with a margin of 1.5, and the choice is certain whenever the two error bars do
  //      not overlap.  Only the undecided tokens (non-finite values included: every comparison is then false) take the
  //      exact sums u_i = ((U0 + U1) + U2) + U3, U_b = seq_{k in block b} C[i][k] e_k.
  {
    const int g = lane >> 2, q = lane & 3;
    // MMA rows: row g = (token g >> 1, candidate g & 1), row g + 8 = (token (g >> 1) + 4, same candidate): row = 2 t + c.
    // The B operand is read as B[k][n] = CT[i][k] = C[k][i], i.e. the transpose of C: e^T C^T e = e^T C e and the bound
    // is the same sum, while a thread's values for two MMA steps are then 16 contiguous bytes (k = 16 d + 4 q .. + 3:
    // the k slots (q, q + 4) of step 0 stand for k, k + 1, those of step 1 for k + 2, k + 3).
    const int t_lo = g >> 1, c = g & 1;
    float acc[4][4], bnd[4][4];
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
      for (int r = 0; r < 4; ++r) { acc[n][r] = 0.f; bnd[n][r] = 0.f; }
    if (!exact_only) {
#pragma unroll 2
      for (int k0 = 0; k0 < HD; k0 += 16) {
        uint32_t a[2][4], aa[2][4];
#pragma unroll
        for (int s2 = 0; s2 < 4; ++s2) {
          const float2 lo = es[t_lo][k0 + 4 * q + s2], hi = es[t_lo + 4][k0 + 4 * q + s2];
          a[s2 >> 1][2 * (s2 & 1)] = __float_as_uint(c ? lo.y : lo.x);
          a[s2 >> 1][2 * (s2 & 1) + 1] = __float_as_uint(c ? hi.y : hi.x);
        }
#pragma unroll
        for (int st = 0; st < 2; ++st)
#pragma unroll
          for (int r = 0; r < 4; ++r) aa[st][r] = a[st][r] & 0x7FFFFFFFu;
#pragma unroll
        for (int n = 0; n < 4; ++n) {
          const float4 v = __ldg(reinterpret_cast<const float4*>(CT + (32 * j + 8 * n + g) * HD + k0 + 4 * q));
          const uint32_t b[4] = {__float_as_uint(v.x), __float_as_uint(v.y), __float_as_uint(v.z), __float_as_uint(v.w)};
          mma_tf32(acc[n], a[0], b[0], b[1]);
          mma_tf32(bnd[n], aa[0], b[0] & 0x7FFFFFFFu, b[1] & 0x7FFFFFFFu);
          mma_tf32(acc[n], a[1], b[2], b[3]);
          mma_tf32(bnd[n], aa[1], b[2] & 0x7FFFFFFFu, b[3] & 0x7FFFFFFFu);
        }
      }
    }
    float E0 = 0.f, B0 = 0.f, E1 = 0.f, B1 = 0.f;    // rows g and g + 8 over this thread's 8 columns
    const float* ea = reinterpret_cast<const float*>(&es[t_lo][0]) + c;
    const float* eb = reinterpret_cast<const float*>(&es[t_lo + 4][0]) + c;
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      const int i0 = 32 * j + 8 * n + 2 * q;
      const float x0 = ea[2 * i0], x1 = ea[2 * i0 + 2], y0 = eb[2 * i0], y1 = eb[2 * i0 + 2];
      E0 = fmaf(x0, acc[n][0], fmaf(x1, acc[n][1], E0));
      B0 = fmaf(fabsf(x0), bnd[n][0], fmaf(fabsf(x1), bnd[n][1], B0));
      E1 = fmaf(y0, acc[n][2], fmaf(y1, acc[n][3], E1));
      B1 = fmaf(fabsf(y0), bnd[n][2], fmaf(fabsf(y1), bnd[n][3], B1));
    }
#pragma unroll
    for (int o = 1; o < 4; o <<= 1) {
      E0 += __shfl_xor_sync(FULLMASK, E0, o); B0 += __shfl_xor_sync(FULLMASK, B0, o);
      E1 += __shfl_xor_sync(FULLMASK, E1, o); B1 += __shfl_xor_sync(FULLMASK, B1, o);
    }
    if (q == 0) { est[j][g][0] = E0; est[j][g][1] = B0; est[j][g + 8][0] = E1; est[j][g + 8][1] = B1; }
  }
  __syncthreads();
  if (i < TG) {
    float E[2], D[2];
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      E[c] = (est[0][2 * i + c][0] + est[1][2 * i + c][0]) + (est[2][2 * i + c][0] + est[3][2 * i + c][0]);
      D[c] = (est[0][2 * i + c][1] + est[1][2 * i + c][1]) + (est[2][2 * i + c][1] + est[3][2 * i + c][1]);
    }
    // (bounds below 1e-20: products may have been flushed on the way, no estimate)
    const bool usable = !exact_only && D[0] > 1e-20f && D[1] > 1e-20f;
    const bool surelyF = usable && E[1] + DYN_DELTA * D[1] < E[0] - DYN_DELTA * D[0];
    const bool surelyBase = usable && E[1] - DYN_DELTA * D[1] > E[0] + DYN_DELTA * D[0];
    hsel[i] = surelyF ? 1 : surelyBase ? 0 : 2;
  }
  __syncthreads();
  {
    int nexact = 0;
    for (int t = 0; t < ntok; ++t) {
      if (hsel[t] != 2) continue;
      ++nexact;
      float2 u;
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        float2 U;
#pragma unroll 8
        for (int k = 0; k < 32; k += 2) {
          const float ca = __ldg(CT + (32 * b + k) * HD + i), cb = __ldg(CT + (32 * b + k + 1) * HD + i);
          const float4 e = *reinterpret_cast<const float4*>(&es[t][32 * b + k]);
          const float2 pa = __fmul2_rn(make_float2(ca, ca), make_float2(e.x, e.y));
          U = k == 0 ? pa : __fadd2_rn(U, pa);
          U = __fadd2_rn(U, __fmul2_rn(make_float2(cb, cb), make_float2(e.z, e.w)));
        }
        u = b == 0 ? U : __fadd2_rn(u, U);
      }
      ps[t][i] = __fmul2_rn(es[t][i], u);
    }
    if (i == 0) {
      atomicAdd(&g_dynstat[0], static_cast<unsigned long long>(ntok));
      if (nexact) atomicAdd(&g_dynstat[1], static_cast<unsigned long long>(nexact));
    }
  }
  __syncthreads();
  // ---- C + D: undecided tokens: halving tree of e * u over the 128 dims; page write (warp j takes tokens j, j + 4)
  for (int t = j; t < ntok; t += 4) {
    bool F = hsel[t] == 1;
    if (hsel[t] == 2) {
      const float2 a = __fadd2_rn(ps[t][lane], ps[t][lane + 64]), b = __fadd2_rn(ps[t][lane + 32], ps[t][lane + 96]);
      const float2 herr = tree32x2(__fadd2_rn(a, b));
      F = herr.y < herr.x;
    }
    const long long slot = p.slot_ph ? p.slots[static_cast<long long>(t0 + t) * p.Hkv + h] : p.slots[t0 + t];
    if (slot < 0) continue;
    const int c = F ? 1 : 0;
    const int P = p.page;
    const long long page = slot / P;
    const int pos = static_cast<int>(slot % P);
    uint8_t* chunk = p.pool + (page * p.Hkv + h) * static_cast<long long>(Lay<NB>::chunk(P));
    const unsigned cw = *reinterpret_cast<const uint32_t*>(&cs[t][c][4 * lane]);
    const unsigned code[4] = {cw & 0xFFu, (cw >> 8) & 0xFFu, (cw >> 16) & 0xFFu, cw >> 24};
    store_k_row<NB, SYM>(chunk, P, pos, lane, code, ws[t][c][lane >> 3]);
    if (lane == 0)   // the key's whole-head flag rides in bit 15 of the token's V group-0 scale word
      put_word_bit15(chunk, Lay<NB>::vs_off(P) + 2 * (8 * (pos >> 3) + vslot8(pos)), F);
  }
}

// ------------------------------------------------------------------------------------------------ launchers
static int check_launch() { return cudaPeekAtLastError() == cudaSuccess ? 0 : -1; }

int head_fwht_launch(const void* x, long long x_ts, void* out, long long o_ts, int T, int H, const uint8_t* flags,
                     float scale, cudaStream_t st, int D) {
  const long long warps = static_cast<long long>(T) * H;
  const unsigned blocks = static_cast<unsigned>((warps * 32 + 255) / 256);
  const auto* xi = static_cast<const __nv_bfloat16*>(x);
  auto* xo = static_cast<__nv_bfloat16*>(out);
  if (D == 256) k_head_fwht<2><<<blocks, 256, 0, st>>>(xi, x_ts, xo, o_ts, T, H, flags, scale);
  else k_head_fwht<1><<<blocks, 256, 0, st>>>(xi, x_ts, xo, o_ts, T, H, flags, scale);
  return check_launch();
}

// quantise-and-pack of whole rows: token groups of 8 for a bulk write, one warp per row for an append
template <int NB, bool SYM = false>
static void rows_kernel_launch(const RowParams& p, cudaStream_t st) {
  if (p.T >= 256) {                            // bulk write: groups of 8 tokens, whole V^T words where the slots allow
    const long long items = static_cast<long long>((p.T + 7) / 8) * p.nrow;
    // rows with transforms in front of the quantizer: a lane per 32-vector (322 against 385 us for 65 536 tokens x 16 rows on
    // consecutive slots); plain rows (the values of the key-only kinds): a warp per row is faster (233 against 308 us)
    if (p.mask != nullptr || p.hfull != nullptr) k_rows8v<NB, SYM><<<static_cast<unsigned>((items + 3) / 4), 128, 0, st>>>(p);
    else k_rows8<NB, SYM><<<static_cast<unsigned>((items + 3) / 4), 128, 0, st>>>(p);
  } else {
    const long long items = static_cast<long long>(p.T) * p.nrow;
    k_rows<NB, SYM><<<static_cast<unsigned>((items + 3) / 4), 128, 0, st>>>(p);
  }
}

int rows_launch(int nb, const void* kv, long long kv_ts, const long long* slots, int slot_ph, int T, int Hkv, int page,
                const uint8_t* mask, const uint8_t* hfull, const float* kmu, uint8_t* pool, int row0, int nrow,
                int shared15, cudaStream_t st, int sym) {
  if (T <= 0 || nrow <= 0) return 0;
  RowParams p{static_cast<const __nv_bfloat16*>(kv), kv_ts, slots, slot_ph, T, Hkv, page, mask, hfull, kmu, pool, row0,
              nrow, shared15};
  if (sym) rows_kernel_launch<4, true>(p, st);       // symmetric INT4: sign-magnitude codes, plain FP16 scale words
  else if (nb == 4) rows_kernel_launch<4>(p, st);
  else rows_kernel_launch<2>(p, st);
  return check_launch();
}

constexpr int DYN_SMEM = HD * HD * 4;        // the staged C_q^T

// a decode append (a few tokens per head): one wave of CTAs with C_q^T staged in shared memory, the latency of the
// 128-step sums is then shared-memory latency; returns 1 when the shape does not fit one wave
template <int NB, int TG, bool SYM>
static int dyn_keys_staged(const DynParams& p, const RowParams& rows, cudaStream_t st) {
  static int slots_of[64];                   // resident CTAs of the staged kernel, per device ordinal (0: not asked yet)
  static unsigned long long ready = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -2;
  if (slots_of[dev] == 0) {
    int sms = 0, occ = 0;
    if (!smem_limit_ready(k_dyn_keys<NB, TG, true, SYM>, DYN_SMEM, ready) ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, k_dyn_keys<NB, TG, true, SYM>, 128, DYN_SMEM) != cudaSuccess || occ < 1)
      return -2;
    slots_of[dev] = sms * occ;
  }
  const int slots = slots_of[dev];
  const int groups = (p.T + TG - 1) / TG;
  if (static_cast<long long>(groups) * p.Hkv > slots) return 1;
  const long long rblocks = (static_cast<long long>(rows.T) * rows.nrow + 3) / 4;
  const int extra = static_cast<int>((rblocks + p.Hkv - 1) / p.Hkv);
  k_dyn_keys<NB, TG, true, SYM><<<dim3(p.Hkv, groups + extra), 128, DYN_SMEM, st>>>(p, rows);
  return check_launch();
}

static int g_dyn_exact_only = 0;          // test switch: the bulk writer skips the tensor-core estimate (same bytes, slower)
void dyn_writer_exact_only(int on) { g_dyn_exact_only = on ? 1 : 0; }
int dyn_writer_stats(unsigned long long* out2, int reset) {
  if (out2 != nullptr && cudaMemcpyFromSymbol(out2, g_dynstat, 2 * sizeof(unsigned long long)) != cudaSuccess) return -1;
  if (reset) {
    const unsigned long long z[2] = {0ull, 0ull};
    if (cudaMemcpyToSymbol(g_dynstat, z, sizeof(z)) != cudaSuccess) return -1;
  }
  return 0;
}

// rows.T > 0: also write those value rows (in the same launch when the append path takes it, else in a second launch)
template <int NB, bool SYM = false>
static int dyn_keys_nb(const DynParams& p, const RowParams& rows, cudaStream_t st) {
  const long long items = static_cast<long long>(p.T) * p.Hkv;
  if (items <= 1024) {
    const int rc = items <= 256 ? dyn_keys_staged<NB, 1, SYM>(p, rows, st) : dyn_keys_staged<NB, 2, SYM>(p, rows, st);
    if (rc != 1) return rc;
  }
  if (rows.T > 0) rows_kernel_launch<NB, SYM>(rows, st);
  RowParams none = rows;
  none.T = 0;
  // many tokens: C_q^T through L1 / L2 (coalesced rows), more resident CTAs, groups of up to 4 tokens share every value read
  const int tg = items <= 1024 ? 1 : items <= 4096 ? 2 : 8;
  const dim3 grid(p.Hkv, (p.T + tg - 1) / tg);
  if (tg == 1) k_dyn_keys<NB, 1, false, SYM><<<grid, 128, 0, st>>>(p, none);
  else if (tg == 2) k_dyn_keys<NB, 2, false, SYM><<<grid, 128, 0, st>>>(p, none);
  else {
    const long long groups = (p.T + 7) / 8;
    if (groups * p.Hkv > 0x7FFFFFFFll) return -3;
    k_dyn_keys_bulk<NB, SYM><<<static_cast<unsigned>(groups * p.Hkv), 128, 0, st>>>(p, static_cast<int>(groups), g_dyn_exact_only);
  }
  return check_launch();
}

int writer_status() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_wstatus, sizeof(int));
  return v;
}

// with_values: also the value rows [Hkv, 2 Hkv) of the same tokens (one launch for a decode append, else two)
int dyn_keys_launch(int nb, const void* kv, long long kv_ts, const long long* slots, int slot_ph, int T, int Hkv, int page,
                    const float* CT, const float* kmu, uint8_t* pool, cudaStream_t st, int with_values, int sym) {
  if (T <= 0) return 0;
  DynParams p{static_cast<const __nv_bfloat16*>(kv), kv_ts, slots, slot_ph, T, Hkv, page, CT, kmu, pool};
  RowParams rows{static_cast<const __nv_bfloat16*>(kv), kv_ts, slots, slot_ph, with_values ? T : 0, Hkv, page, nullptr, nullptr,
                 nullptr, pool, Hkv, Hkv, 1};
  if (sym) return dyn_keys_nb<4, true>(p, rows, st);          // konly: symmetric INT4 quantiser in the criterion and the pages
  return nb == 4 ? dyn_keys_nb<4>(p, rows, st) : dyn_keys_nb<2>(p, rows, st);
}

}  // namespace fr
