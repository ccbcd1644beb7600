// Page dequantiser of libflagrot_kernels.so: positions [start, n) of one request's INT4 / INT2 FlagRot pages -> K and V rows
// [n - start, Hkv, 128] in bf16 or fp32, in the ORIGINAL basis.  It is the step on the cache side of the plugin's "fa"
// prefill path, which the reference does in PyTorch (integrations/vllm_flagrot/vllm_flagrot/attention/backend.py:1744-1789:
// kernels.dequant_cb_pages / dequant_v2_pages + unrotate_cached); fr_dequant_pages has no counterpart in the reference's
// C ABI.
//
// x^ = (code - zero point) * fp16(word & 0x7FFF) in fp32 (exact product of an integer and an fp16 value), then the inverse
// transform in fp32 butterflies: key-only pages carry the choice per token (bit 15 of a K scale word: group stored as
// H32 x; bit 15 of the V group-0 word: the key stored as H128 x, orthonormal), static pages per kv head (block masks
// [Hkv, 4] for K and V, whole-head flags [Hkv]: stored bf16(H128 x / 16), so x = H128 y / 8).
//
// CTA = (page, kv head), 128 threads: the chunk (2304 / 1280 bytes at page 16) is staged in shared memory with 16-byte
// loads, then warp w takes tokens w, w + 4, ... with 4 dims per lane (the row mapping of the writers).
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "fr_common.cuh"
#include "fr_kernels.h"

namespace fr {

namespace {

struct DqParams {
  const uint8_t* pool;        // [pages, Hkv, chunk]
  const int* bt;              // block-table row of the request
  int start, n, Hkv, page, pg0;
  int key_only, sym;
  const uint8_t *kmask, *vmask, *kfull, *vfull;   // static formats; any may be null
  void *ok, *ov;              // [n - start, Hkv, 128]
  int fp32;
};

FR_DEVI void store_row4(void* base, long long row_elems, int fp32, int lane, const float (&x)[4]) {
  if (fp32) {
    reinterpret_cast<float4*>(static_cast<float*>(base) + row_elems)[lane] = make_float4(x[0], x[1], x[2], x[3]);
  } else {
    const __nv_bfloat162 a = __floats2bfloat162_rn(x[0], x[1]), b = __floats2bfloat162_rn(x[2], x[3]);
    uint2 v;
    v.x = *reinterpret_cast<const uint32_t*>(&a);
    v.y = *reinterpret_cast<const uint32_t*>(&b);
    reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(base) + row_elems)[lane] = v;
  }
}

// inverse of the static transforms of one row: block flags (orthonormal H32, its own inverse), then the whole head
FR_DEVI void unrotate_static(float (&x)[4], const uint8_t* mask4, bool full, int lane) {
  if (mask4 != nullptr) {
    const bool rot = mask4[lane >> 3] != 0;
    if (__any_sync(FULLMASK, rot)) {
      float y[4] = {x[0], x[1], x[2], x[3]};
      fwht_row_stages(y, lane, 32);
      if (rot) {
#pragma unroll
        for (int i = 0; i < 4; ++i) x[i] = y[i] * C32;
      }
    }
  }
  if (full) {
    fwht_row_stages(x, lane, 128);
#pragma unroll
    for (int i = 0; i < 4; ++i) x[i] *= 0.125f;
  }
}

template <int NB, bool SYM = false>
__global__ void __launch_bounds__(128) k_dequant_pages(const DqParams p) {
  extern __shared__ __align__(16) uint8_t chunk[];
  const int P = p.page, h = blockIdx.y, pg = p.pg0 + blockIdx.x;
  const int CH = Lay<NB>::CELL * P;
  const uint8_t* src = p.pool + (static_cast<long long>(__ldg(p.bt + pg)) * p.Hkv + h) * CH;
  for (int i = threadIdx.x; i < CH / 16; i += 128) reinterpret_cast<uint4*>(chunk)[i] = __ldg(reinterpret_cast<const uint4*>(src) + i);
  __syncthreads();
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int j = lane >> 3, isb = (lane >> 2) & 1, tg = lane & 3;           // dims 4 lane .. 4 lane + 3: group j, half isb, word tg
  constexpr unsigned FM = (1u << NB) - 1;
  const int v_off = Lay<NB>::CBY * P, ks_off = 2 * Lay<NB>::CBY * P, vs_off = ks_off + 8 * P;
  for (int pos = w; pos < P; pos += 4) {
    const long long t = static_cast<long long>(pg) * P + pos;
    if (t < p.start || t >= p.n) continue;                                 // warp-uniform
    const long long row = ((t - p.start) * p.Hkv + h) * HD;
    // ---- key row
    const unsigned kw = *reinterpret_cast<const uint16_t*>(chunk + ks_off + 8 * pos + 2 * j);
    const unsigned vw0 = *reinterpret_cast<const uint16_t*>(chunk + vs_off + 2 * (8 * (pos >> 3) + vslot8(pos)));
    float x[4];
    {
      unsigned word;
      if (NB == 4) {
        word = *reinterpret_cast<const uint32_t*>(chunk + 64 * pos + 16 * tg + 4 * j);
        if (SYM) word = sym_to_asym(word);                                   // symmetric pages: the INT4A word of q + 8
        word >>= 4 * isb;
      }
      else word = *reinterpret_cast<const uint32_t*>(chunk + Lay<2>::krow(pos) + 8 * tg + 4 * (j >> 1)) >> (4 * (j & 1) + 2 * isb);
      const float s = __half2float(__ushort_as_half(static_cast<unsigned short>(kw & 0x7FFFu)));
      const int z = SYM ? 8 : static_cast<int>(kw & FM);
#pragma unroll
      for (int i = 0; i < 4; ++i) x[i] = static_cast<float>(static_cast<int>((word >> (8 * i)) & FM) - z) * s;
    }
    if (p.key_only) {
      if (vw0 & 0x8000u) {                                                 // warp-uniform: the key is stored as H128 x
        fwht_row_stages(x, lane, 128);
#pragma unroll
        for (int i = 0; i < 4; ++i) x[i] *= C128;
      } else {
        const bool hfl = (kw & 0x8000u) != 0;
        if (__any_sync(FULLMASK, hfl)) {
          float y[4] = {x[0], x[1], x[2], x[3]};
          fwht_row_stages(y, lane, 32);
          if (hfl) {
#pragma unroll
            for (int i = 0; i < 4; ++i) x[i] = y[i] * C32;
          }
        }
      }
    } else {
      unrotate_static(x, p.kmask ? p.kmask + h * 4 : nullptr, p.kfull != nullptr && p.kfull[h] != 0, lane);
    }
    store_row4(p.ok, row, p.fp32, lane, x);
    // ---- value row: dim d = 4 lane + i lives in the V^T entry of (w = (d % 64) / 16, gid = d % 8), word 2 (d / 64) + (d % 16) / 8
    {
      const unsigned sw = *reinterpret_cast<const uint16_t*>(chunk + vs_off + 2 * (j * P + 8 * (pos >> 3) + vslot8(pos)));
      const float s = __half2float(__ushort_as_half(static_cast<unsigned short>(sw & 0x7FFFu)));
      const int z = SYM ? 8 : static_cast<int>(sw & FM);
      const int c8 = pos >> 3, ii = (pos & 7) >> 1, odd = pos & 1;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int d = 4 * lane + i, m = d >> 6, ww = (d & 63) >> 4, gid = d & 7, r8 = (d & 15) >> 3;
        const int e = (ww * 8 + gid) * (P / 8) + c8;
        unsigned c;
        if (NB == 4 && SYM) c = (sym_to_asym(*reinterpret_cast<const uint32_t*>(chunk + v_off + 16 * e + 4 * (2 * m + r8))) >> (8 * ii + 4 * odd)) & 15u;
        else if (NB == 4) c = (chunk[v_off + 16 * e + 4 * (2 * m + r8) + ii] >> (4 * odd)) & 15u;
        else c = (chunk[v_off + 8 * e + 4 * m + ii] >> (4 * r8 + 2 * odd)) & 3u;
        x[i] = static_cast<float>(static_cast<int>(c) - z) * s;
      }
    }
    if (!p.key_only) unrotate_static(x, p.vmask ? p.vmask + h * 4 : nullptr, p.vfull != nullptr && p.vfull[h] != 0, lane);
    store_row4(p.ov, row, p.fp32, lane, x);
  }
}

}  // namespace

int dequant_pages_launch(int nb, int key_only, const uint8_t* pool, const int* bt_row, int start, int n, int Hkv, int page,
                         const uint8_t* kmask, const uint8_t* vmask, const uint8_t* kfull, const uint8_t* vfull, void* ok, void* ov,
                         int fp32, cudaStream_t st, int sym) {
  if (n <= start) return 0;
  const int pg0 = start / page, npg = (n + page - 1) / page - pg0;
  DqParams p{pool, bt_row, start, n, Hkv, page, pg0, key_only, sym, kmask, vmask, kfull, vfull, ok, ov, fp32};
  const dim3 grid(npg, Hkv);
  const int smem = (nb == 4 ? 144 : 80) * page;
  if (sym) k_dequant_pages<4, true><<<grid, 128, smem, st>>>(p);
  else if (nb == 4) k_dequant_pages<4><<<grid, 128, smem, st>>>(p);
  else k_dequant_pages<2><<<grid, 128, smem, st>>>(p);
  return cudaPeekAtLastError() == cudaSuccess ? 0 : -1;
}

}  // namespace fr
