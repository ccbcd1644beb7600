// Known-answer kernels for the tcgen05 building blocks of fr_tc5.cuh: one CTA computes D[128][N] = A[128][K] * B[N][K]^T
// through tensor memory with each operand path the product kernels use, so that descriptor encodings and tensor-memory
// layouts are pinned by a test instead of being inferred from a wrong attention result.
//   mode 0  FP16 operands in shared memory, 128-byte swizzle            (K a multiple of 64, fp32 accumulators)
//   mode 1  FP16 A operand in tensor memory, B as in mode 0             (K a multiple of 64)
//   mode 2  u8 x s8 operands in shared memory, no swizzle, K = 32 steps (K a multiple of 32, s32 accumulators)
// Built into the test-only library libflagrot_tc5test.so; not part of any C ABI, no counterpart in the reference.
//   int fr_tc5_selftest(int mode, const void* A, const void* B, void* D, int N, int K, void* stream)
// N a multiple of 16 <= 128; K a multiple of 64 <= 256 (modes 0 / 1) or of 32 <= 512 (mode 2).  Synchronises the stream.
// Returns 0, -1 launch error, -3 bad shape, or the source line of a bounded wait that gave up.
#include <cstdint>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "fr_tc5.cuh"

namespace {

__device__ int g_tc5_status;

FR_DEVI uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__global__ void __launch_bounds__(128) k_tc5_selftest(int mode, const void* A, const void* B, void* Dout, int N, int K) {
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ uint64_t mbar;
  __shared__ uint32_t tbase_slot;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t sb = (smem_u32(smem) + 1023u) & ~1023u;
  const bool f16 = mode != 2;
  // operand tiles: A 128 rows, B N rows; FP16: one 128-byte-row slab per 64 elements of K; u8: [rows / 8][K / 16][8][16]
  const uint32_t a_bytes = f16 ? 128u * K * 2 : 128u * K;
  const uint32_t sa = sb, sbb = sb + a_bytes;
  if (warp == 0) {
    tc5::tmem_alloc(smem_u32(&tbase_slot), 256);
    tc5::tmem_relinquish();
  }
  if (tid == 0) {
    tc5::mbar_init(smem_u32(&mbar), 1);
    tc5::mbar_init_fence();
  }
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tbase = tbase_slot;
  const uint32_t td = tbase, ta = tbase + 128;     // accumulators: columns 0 .. N - 1; TS operand: columns 128 ..

  if (f16) {
    const int kch = K / 8;                          // 16-byte chunks per row
    for (int op = 0; op < 2; ++op) {
      if (op == 0 && mode == 1) continue;
      const int rows = op == 0 ? 128 : N;
      const uint4* src = static_cast<const uint4*>(op == 0 ? A : B);
      const uint32_t dst = op == 0 ? sa : sbb;
      for (int i = tid; i < rows * kch; i += 128) {
        const int r = i / kch, c = i % kch;
        const uint4 v = src[i];
        const uint32_t a = dst + (c >> 3) * rows * 128 + tc5::sw128_off(r, c & 7);
        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(a), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
      }
    }
    if (mode == 1) {                                // A row = this thread's lane: K / 2 packed columns, 16 at a time
      const uint32_t* arow = static_cast<const uint32_t*>(A) + static_cast<size_t>(tid) * (K / 2);
      for (int c0 = 0; c0 < K / 2; c0 += 16) {
        uint32_t v[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = arow[c0 + i];
        tc5::tmem_st16(ta + c0 + (static_cast<uint32_t>(warp * 32) << 16), v);
      }
      tc5::tmem_st_wait();
    }
  } else {
    const int kch = K / 16;
    for (int op = 0; op < 2; ++op) {
      const int rows = op == 0 ? 128 : N;
      const uint4* src = static_cast<const uint4*>(op == 0 ? A : B);
      const uint32_t dst = op == 0 ? sa : sbb;
      for (int i = tid; i < rows * kch; i += 128) {
        const int r = i / kch, c = i % kch;
        const uint4 v = src[i];
        const uint32_t a = dst + ((r >> 3) * kch + c) * 128 + (r & 7) * 16;
        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(a), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
      }
    }
  }
  tc5::fence_async_smem();
  tc5::fence_before_sync();
  __syncthreads();
  if (tid == 0) {
    tc5::fence_after_sync();
    if (f16) {
      const uint32_t id = tc5::idesc(1, 0, 0, 128, N);
      for (int k = 0; k < K / 16; ++k) {
        const uint32_t koff = (k >> 2) * 128 * 128 + (k & 3) * 32, koffb = (k >> 2) * N * 128 + (k & 3) * 32;
        const uint64_t db = tc5::desc_sw128(sbb + koffb, 1024);
        if (mode == 0) tc5::mma_f16_ss(td, tc5::desc_sw128(sa + koff, 1024), db, id, k > 0);
        else tc5::mma_f16_ts(td, ta + k * 8, db, id, k > 0);
      }
    } else {
      const uint32_t id = tc5::idesc(2, 0, 1, 128, N);
      const int kch = K / 16;
      for (int k = 0; k < K / 32; ++k)
        tc5::mma_i8_ss(td, tc5::desc_plain(sa + k * 256, 128, kch * 128), tc5::desc_plain(sbb + k * 256, 128, kch * 128), id, k > 0);
    }
    tc5::mma_commit(smem_u32(&mbar));
  }
  const bool ok = tc5::mbar_wait(smem_u32(&mbar), 0);
  tc5::fence_after_sync();
  if (ok) {
    uint32_t* drow = static_cast<uint32_t*>(Dout) + static_cast<size_t>(tid) * N;
    for (int c0 = 0; c0 < N; c0 += 16) {
      uint32_t v[16];
      tc5::tmem_ld16(td + c0 + (static_cast<uint32_t>(warp * 32) << 16), v);
      tc5::tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 16; ++i) drow[c0 + i] = v[i];
    }
  } else if (lane == 0) {
    atomicExch(&g_tc5_status, __LINE__);
  }
  tc5::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc5::tmem_dealloc(tbase, 256);
}

}  // namespace

// A, B, D device pointers (FP16 / u8 / s8 row-major inputs, fp32 / s32 row-major [128][N] output).  Returns 0, -1 (launch),
// -3 (shape), and after a synchronising read of the status word the line of a wait that gave up.
extern "C" int fr_tc5_selftest(int mode, const void* A, const void* B, void* D, int N, int K, void* stream) {
  if (mode < 0 || mode > 2 || N < 16 || N > 128 || N % 16) return -3;
  if (mode == 2 ? (K % 32 || K > 512) : (K % 64 || K > 256)) return -3;
  const int smem = (mode == 2 ? (128 + N) * K : (128 + N) * K * 2) + 1024;
  static unsigned long long ready = 0;
  if (!fr::smem_limit_ready(k_tc5_selftest, 200 * 1024, ready)) return -2;
  int zero = 0;
  cudaMemcpyToSymbolAsync(g_tc5_status, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream));
  k_tc5_selftest<<<1, 128, smem, static_cast<cudaStream_t>(stream)>>>(mode, A, B, D, N, K);
  if (cudaPeekAtLastError() != cudaSuccess) return -1;
  if (cudaStreamSynchronize(static_cast<cudaStream_t>(stream)) != cudaSuccess) return -1;
  int st = 0;
  cudaMemcpyFromSymbol(&st, g_tc5_status, sizeof(int));
  return st;
}
