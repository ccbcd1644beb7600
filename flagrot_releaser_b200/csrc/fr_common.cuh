// Shared device helpers of the FlagRot KV-cache kernels for sm_100a: the asymmetric INT4 / INT2 group quantizer, the
// scale word, Walsh-Hadamard butterflies in the reference's fp32 operation order, and the paged byte layout.
//
// Arithmetic contract (what makes the packed codes and scale / flag words bit-exact against the reference):
//   * every product and sum of the quantizer and of the selection criterion is a separately rounded fp32 operation
//     (__fmul_rn / __fadd_rn / __fsub_rn, IEEE division __fdiv_rn): no FMA contraction, no reassociation;
//   * the scale is (max - min) * fp32(1 / lv) (reference: kernels/csrc/attn_cb_common.cuh:55-58);
//   * Hadamard stages run h = 1, 2, 4, ... as (a + b, a - b) followed by one multiply by fp32(1 / sqrt(n))
//     (reference: kernels/ref.py:22-33).
// Page layout: one contiguous chunk per (page, kv head), 144 P bytes (INT4) or 80 P bytes (INT2)
// (reference: kernels/csrc/attn_decode_v2.cuh:14-46).
#pragma once
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#define FR_DEVI __device__ __forceinline__

namespace fr {

constexpr int HD = 128;                        // head dim handled by these kernels
constexpr unsigned FULLMASK = 0xffffffffu;
constexpr float C32 = 0.17677669529663687f;    // fp32(1 / sqrt(32))
constexpr float C128 = 0.08838834764831845f;   // fp32(1 / sqrt(128))

// ------------------------------------------------------------------------------------------------ layout
// NB = code bits (4 | 2).  Offsets inside a (page, head) chunk of a page of P tokens.
template <int NB> struct Lay {
  static constexpr int CBY = NB == 4 ? 64 : 32;             // code bytes per (token, K or V row)
  static constexpr int CELL = 2 * CBY + 16;                 // bytes per (token, kv head): 144 | 80
  FR_DEVI static int chunk(int P) { return CELL * P; }
  FR_DEVI static int v_off(int P) { return CBY * P; }
  FR_DEVI static int ks_off(int P) { return 2 * CBY * P; }
  FR_DEVI static int vs_off(int P) { return 2 * CBY * P + 8 * P; }
  // byte offset of token pos's K row
  FR_DEVI static int krow(int pos) { return NB == 4 ? 64 * pos : 32 * (pos ^ ((pos >> 1) & 2)); }
};
// position of token pos's V scale inside its 8-token chunk: tokens 0 2 4 6 1 3 5 7
FR_DEVI int vslot8(int pos) { const int r = pos & 7; return (r & 1) ? 4 + (r >> 1) : (r >> 1); }

// ------------------------------------------------------------------------------------------------ quantizer
// FP16 bit pattern nearest (integer distance, ties up) to RN_fp16(s) whose NB low bits are z
// (reference: blockflag/formats.py:135-146,168-174)
template <int NB> FR_DEVI unsigned scale_word(float s, unsigned z) {
  constexpr int M = (1 << NB) - 1;
  const int h = static_cast<int>(__half_as_ushort(__float2half_rn(s)));
  const int x = min(max(h - static_cast<int>(z) + (1 << (NB - 1)), 0) & ~M, 0x7C00 - (1 << NB));
  return static_cast<unsigned>(x) + z;
}
template <int NB> FR_DEVI void asym_params(float mn, float mx, float& s, float& z) {
  s = fmaxf(__fmul_rn(__fsub_rn(mx, mn), 1.0f / static_cast<float>((1 << NB) - 1)), 1e-12f);
  z = rintf(__fdiv_rn(-mn, s));
}
template <int NB> FR_DEVI float asym_code(float y, float s, float z) {
  return fminf(fmaxf(__fadd_rn(rintf(__fdiv_rn(y, s)), z), 0.f), static_cast<float>((1 << NB) - 1));
}
// stored form: the group's range widened to include 0 (reference: kernels/csrc/attn_decode_v2.cu:1704-1715)
template <int NB> FR_DEVI void quant_store(float y, float mn, float mx, unsigned& code, unsigned& word) {
  float s, z;
  asym_params<NB>(fminf(mn, 0.f), fmaxf(mx, 0.f), s, z);
  code = static_cast<unsigned>(asym_code<NB>(y, s, z));
  word = scale_word<NB>(s, static_cast<unsigned>(z));
}
// error form: unwidened range, unbounded zero point, deq = (q - z) s (reference: kernels/codebook_ref.py:99-108)
// symmetric INT4 (`int4` pages): s = fp16(amax * fp32(1 / 7)), q = clamp(rne(y / s), -7, 7), 0 where s = 0 (reference
// attn_decode_v2.cu:1769-1781).  code = sign-magnitude (8 | |q| for q < 0), word = FP16 bits of s.
FR_DEVI void quant_store_sym(float y, float amax, unsigned& code, unsigned& word) {
  const __half sh = __float2half_rn(__fmul_rn(amax, 1.0f / 7.0f));
  const float sf = __half2float(sh);
  float q = sf != 0.f ? rintf(__fdiv_rn(y, sf)) : 0.f;
  q = fminf(fmaxf(q, -7.f), 7.f);
  const int qi = static_cast<int>(q);
  code = static_cast<unsigned>(qi < 0 ? (8 | -qi) : qi);
  word = __half_as_ushort(sh);
}
// bits of a sign-magnitude element in its 32-bit word (byte i holds A_i): A_i: sign -> bit 8 i + 7, |q| -> bits 8 i .. + 2;
// B_i: sign -> bit 8 i + 3, |q| -> bits 4 .. 6 of byte (i + 3) % 4 (reference attn_decode_v2.cuh:26-28)
FR_DEVI unsigned sym_bits(unsigned c, bool isB, int i) {
  const unsigned s = (c >> 3) & 1u, mag = c & 7u;
  return isB ? (s << (8 * i + 3)) | (mag << (8 * ((i + 3) & 3) + 4)) : ((s << 7) | mag) << (8 * i);
}
FR_DEVI unsigned sym_mask(bool isB, int i) { return isB ? (0x08u << (8 * i)) | (0x70u << (8 * ((i + 3) & 3))) : 0x87u << (8 * i); }
// the bits `mask` of the 32-bit word at chunk + word_off (4-byte aligned) := bits, whatever other threads do to the rest
FR_DEVI void put_bits(uint8_t* chunk, int word_off, unsigned mask, unsigned bits) {
  uint32_t* wp = reinterpret_cast<uint32_t*>(chunk + word_off);
  const unsigned delta = (*reinterpret_cast<volatile uint32_t*>(wp) ^ bits) & mask;
  if (delta) atomicXor(wp, delta);
}

// sign-magnitude bytes (sign bit 7, |q| bits 0 - 2) -> q + 8 per byte (1 .. 15): no carry leaves a byte
FR_DEVI uint32_t sym_offset_bytes(uint32_t x) {
  const uint32_t n7 = ((x >> 7) & 0x01010101u) * 7u;
  return ((x & 0x07070707u) ^ n7) + (0x08080808u - n7);
}
// a word of 4 A + 4 B sign-magnitude elements -> the INT4A word (A low, B high nibble of byte i) of q + 8
FR_DEVI uint32_t sym_to_asym(uint32_t w) {
  return sym_offset_bytes(w & 0x87878787u) | (sym_offset_bytes(__funnelshift_l(w, w, 4) & 0x87878787u) << 4);
}

// quantiser of the dynamic writer by page kind: the symmetric one has a single form (its error form is its stored form)
FR_DEVI float sym_deq(unsigned code, unsigned word) {
  const float q = static_cast<float>(static_cast<int>(code & 7u));
  return __fmul_rn((code & 8u) ? -q : q, __half2float(__ushort_as_half(static_cast<unsigned short>(word))));
}
template <int NB> FR_DEVI float quant_err_deq(float y, float mn, float mx);
template <int NB, bool SYM> FR_DEVI float dyn_err_deq(float y, float mn, float mx) {
  if (SYM) {
    unsigned code, word;
    quant_store_sym(y, fmaxf(-mn, mx), code, word);
    return sym_deq(code, word);
  }
  return quant_err_deq<NB>(y, mn, mx);
}
template <int NB, bool SYM> FR_DEVI void dyn_store(float y, float mn, float mx, unsigned& code, unsigned& word) {
  if (SYM) quant_store_sym(y, fmaxf(-mn, mx), code, word);
  else quant_store<NB>(y, mn, mx, code, word);
}

template <int NB> FR_DEVI float quant_err_deq(float y, float mn, float mx) {
  float s, z;
  asym_params<NB>(mn, mx, s, z);
  return __fmul_rn(__fsub_rn(asym_code<NB>(y, s, z), z), s);
}

// ------------------------------------------------------------------------------------------------ warp helpers
// "row" mapping: a warp holds one 128-vector, lane l the elements 4 l .. 4 l + 3 (32-group j = lanes 8 j .. 8 j + 7)
FR_DEVI void fwht_row_stages(float (&x)[4], int lane, int n) {  // unnormalised butterflies h = 1 .. n / 2 (n = 32 | 128)
  {
    const float a = x[0], b = x[1], c = x[2], d = x[3];
    x[0] = __fadd_rn(a, b); x[1] = __fsub_rn(a, b); x[2] = __fadd_rn(c, d); x[3] = __fsub_rn(c, d);
  }
  {
    const float a = x[0], b = x[1], c = x[2], d = x[3];
    x[0] = __fadd_rn(a, c); x[1] = __fadd_rn(b, d); x[2] = __fsub_rn(a, c); x[3] = __fsub_rn(b, d);
  }
  for (int h = 4; h < n; h <<= 1) {
    const int lm = h >> 2;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float o = __shfl_xor_sync(FULLMASK, x[i], lm);
      x[i] = (lane & lm) ? __fsub_rn(o, x[i]) : __fadd_rn(x[i], o);
    }
  }
}
FR_DEVI float group_min8(float a) {  // over the 8 lanes of a 32-group
#pragma unroll
  for (int o = 1; o < 8; o <<= 1) a = fminf(a, __shfl_xor_sync(FULLMASK, a, o));
  return a;
}
FR_DEVI float group_max8(float a) {
#pragma unroll
  for (int o = 1; o < 8; o <<= 1) a = fmaxf(a, __shfl_xor_sync(FULLMASK, a, o));
  return a;
}
// "dim" mapping: thread i of a 128-thread CTA holds element i (32-group j = warp j)
FR_DEVI float warp_min(float a) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) a = fminf(a, __shfl_xor_sync(FULLMASK, a, o));
  return a;
}
FR_DEVI float warp_max(float a) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(FULLMASK, a, o));
  return a;
}
FR_DEVI float fwht32_lane(float v, int lane) {  // orthonormal H32 of the warp's 32 elements
#pragma unroll
  for (int h = 1; h < 32; h <<= 1) {
    const float o = __shfl_xor_sync(FULLMASK, v, h);
    v = (lane & h) ? __fsub_rn(o, v) : __fadd_rn(v, o);
  }
  return __fmul_rn(v, C32);
}
FR_DEVI float tree32(float v) {  // halving tree over the lanes
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(FULLMASK, v, o));
  return v;
}

FR_DEVI float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
FR_DEVI float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// one nibble / 2-bit field of a shared 32-bit word: only this field's bits change, whatever other threads do to the
// rest of the word (the field itself has a single writer)
FR_DEVI void put_field(uint8_t* chunk, int byte_off, int shift, unsigned fmask, unsigned code) {
  const unsigned old = (static_cast<unsigned>(*reinterpret_cast<volatile uint8_t*>(chunk + byte_off)) >> shift) & fmask;
  const unsigned delta = old ^ code;
  if (delta) {
    uint32_t* wp = reinterpret_cast<uint32_t*>(chunk + (byte_off & ~3));
    atomicXor(wp, delta << (8 * (byte_off & 3) + shift));
  }
}
// 16-bit scale word whose bit 15 belongs to another writer (key-only kinds: the key's whole-head flag rides in the V
// group-0 scale word): replace the low 15 bits / bit 15 only
FR_DEVI void put_word_low15(uint8_t* chunk, int byte_off, unsigned w15) {
  const unsigned old = *reinterpret_cast<volatile uint16_t*>(chunk + byte_off) & 0x7FFFu;
  const unsigned delta = old ^ (w15 & 0x7FFFu);
  if (delta) atomicXor(reinterpret_cast<uint32_t*>(chunk + (byte_off & ~3)), delta << (8 * (byte_off & 2)));
}
FR_DEVI void put_word_bit15(uint8_t* chunk, int byte_off, bool on) {
  uint32_t* wp = reinterpret_cast<uint32_t*>(chunk + (byte_off & ~3));
  const uint32_t bit = 0x8000u << (8 * (byte_off & 2));
  if (on) atomicOr(wp, bit); else atomicAnd(wp, ~bit);
}


// ------------------------------------------------------------------------------------------------ host: launch set-up
// The dynamic shared-memory limit of a kernel is a per-device attribute: a process that drives several GPUs has to raise
// it on each of them.  `done` is one bit per device ordinal (a function-local static of the launcher).
template <typename Kern> inline bool smem_limit_ready(Kern kernel, int bytes, unsigned long long& done) {
  int dev = 0;
  const bool known = cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64;
  if (known && ((done >> dev) & 1ull)) return true;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return false;
  if (known) done |= 1ull << dev;
  return true;
}

}  // namespace fr
