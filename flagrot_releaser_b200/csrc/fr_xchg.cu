// KV-sequence shards: exchange of the per-shard partial rows over peer memory and their merge, in ONE kernel per rank.
// No counterpart in the reference (its ABI has no multi-GPU entry); the plain path for the same job is
// fr_attn_partial -> NCCL all-gather -> fr_merge_partials, three launches and a collective for 16.6 KB per rank.
//
// Every rank owns one exchange buffer (device memory, mapped into the other ranks of the node through CUDA IPC) with the
// same layout:
//   [0, 512)            uint32 step[128]            launches done so far, per CTA index (local use only)
//   [512, 512 + 8 KB)   uint32 flag[2][8][128]      flag[parity][source rank][CTA]: the step whose rows are in place
//   [XCH_DATA, ...)     float  data[2][8][rows][130] data[parity][source rank]: that rank's partial rows (16-byte aligned slabs)
// CTA c of every rank handles rows [8 c, 8 c + 8) (one warp per row).  Per launch, with s = step[c] + 1 and parity s & 1:
//   1. it copies its rows of the local partial into data[parity][rank] of every peer (16-byte peer stores),
//   2. fences system-wide and writes s into flag[parity][rank][c] of every peer,
//   3. waits until its own flag[parity][r][c] reads s for every peer r (bounded: after XWAIT_CYCLES the status word is set
//      and the launch finishes with whatever arrived; its output must then be discarded),
//   4. merges the R partials (its own straight from the local partial) with the rule of fr_merge_partials,
//   5. records step[c] = s.
// Two parities suffice: a rank leaves step s only after every rank's step-s rows arrived, so nobody can be two steps ahead
// of a rank that still reads step s.  A CTA waits only for the CTA of the same index on other GPUs, never for a CTA of
// its own launch, so nothing depends on which CTAs of a grid are resident.  The step counters live on the device: a
// captured launch replays correctly.  All ranks must make the same sequence of calls (rows, R) on a buffer, like a
// collective.
//
// fr_xchg_selftest runs the same device code for R emulated ranks as ONE cooperative launch on one GPU (grid.y = rank): the
// protocol can be tested without a second GPU and without kernels of different launches waiting on one another.
#include <cstdint>
#include <cstdio>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "fr_common.cuh"
#include "fr_kernels.h"

namespace fr {
namespace {

constexpr int XR = 8;                          // ranks of a node
constexpr int XCTA = 128;                      // CTAs (8 rows each): rows <= 1024
constexpr int XCH_FLAGS = 512;
constexpr int XCH_DATA = 512 + 2 * XR * XCTA * 4;
constexpr long long XWAIT_CYCLES = 1ll << 34;  // about nine seconds of SM clock: the peers' launches may trail by host time

__device__ int g_xstatus;

struct XchgParams {
  const float* part[XR];     // local partial rows [rows][130] of the rank run by grid row y (entry 0 in a real launch)
  void* out[XR];             // merged rows of that rank
  uint8_t* buf[XR];          // exchange buffer of rank r as mapped HERE (buf[rank] is the local one)
  int rank0, R, rows, out_fp32;
};

__host__ __device__ inline size_t slab_bytes(int rows) { return (static_cast<size_t>(rows) * 520 + 15) / 16 * 16; }
FR_DEVI size_t data_off(int par, int src, int rows) { return XCH_DATA + (static_cast<size_t>(par) * XR + src) * slab_bytes(rows); }
// rows written by a peer are read past L1 (which peer stores do not invalidate); the rank's own partial is an ordinary load
FR_DEVI float ldx(const float* p, bool remote) { return remote ? __ldcg(p) : *p; }
FR_DEVI float2 ldx2(const float* p, bool remote) { return remote ? __ldcg(reinterpret_cast<const float2*>(p)) : *reinterpret_cast<const float2*>(p); }

FR_DEVI uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}
FR_DEVI void st_release_sys(uint32_t* p, uint32_t v) { asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory"); }

__global__ void __launch_bounds__(256) k_xchg_merge(const XchgParams p) {
  const int y = blockIdx.y, rank = p.rank0 + y, c = blockIdx.x, tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int R = p.R, rows = p.rows;
  uint8_t* mine = p.buf[rank];
  uint32_t* step = reinterpret_cast<uint32_t*>(mine) + c;
  const uint32_t s = *step + 1;
  const int par = static_cast<int>(s & 1u);
  const int r0 = 8 * c, nr = min(8, rows - r0);
  const float* part = p.part[y];
  // 1. my rows -> every peer (the rows of a CTA are contiguous: nr * 520 bytes from a 16-byte aligned offset)
  {
    const uint4* src = reinterpret_cast<const uint4*>(part + static_cast<size_t>(r0) * 130);
    const int n16 = nr * 130 * 4 / 16;
    for (int r = 0; r < R; ++r) {
      if (r == rank) continue;
      uint4* dst = reinterpret_cast<uint4*>(p.buf[r] + data_off(par, rank, rows) + static_cast<size_t>(r0) * 520);
      for (int i = tid; i < n16; i += 256) dst[i] = src[i];
    }
    if ((nr * 520) % 16 != 0) {                  // an odd row count leaves 8 bytes
      const int o = n16 * 4;                     // in floats
      for (int r = 0; r < R; ++r) {
        if (r == rank || tid >= 2) continue;
        reinterpret_cast<float*>(p.buf[r] + data_off(par, rank, rows))[static_cast<size_t>(r0) * 130 + o + tid] = part[static_cast<size_t>(r0) * 130 + o + tid];
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  // 2. tell every peer, 3. wait for every peer
  if (tid < R && tid != rank) {
    st_release_sys(reinterpret_cast<uint32_t*>(p.buf[tid] + XCH_FLAGS) + (par * XR + rank) * XCTA + c, s);
    const uint32_t* f = reinterpret_cast<const uint32_t*>(mine + XCH_FLAGS) + (par * XR + tid) * XCTA + c;
    const long long t0 = clock64();
    bool ok = ld_acquire_sys(f) == s;
    while (!ok && clock64() - t0 < XWAIT_CYCLES) {
      __nanosleep(100);
      ok = ld_acquire_sys(f) == s;
    }
    if (!ok) atomicCAS(&g_xstatus, 0, __LINE__);
  }
  __syncthreads();
  // 4. merge: one warp per row, o = sum_r w_r l_r o_r / sum_r w_r l_r, w_r = 2^(m_r - max m)
  if (w < nr) {
    const int row = r0 + w;
    const float* src[XR];
#pragma unroll
    for (int r = 0; r < XR; ++r)
      src[r] = r == rank ? part + static_cast<size_t>(row) * 130
                         : reinterpret_cast<const float*>(mine + data_off(par, r < R ? r : 0, rows)) + static_cast<size_t>(row) * 130;
    float M = -INFINITY;
#pragma unroll
    for (int r = 0; r < XR; ++r)
      if (r < R && ldx(src[r] + 129, r != rank) > 0.f) M = fmaxf(M, ldx(src[r] + 128, r != rank));
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float den = 0.f;
#pragma unroll
    for (int r = 0; r < XR; ++r) {
      if (r >= R) continue;
      const float l = ldx(src[r] + 129, r != rank);
      if (!(l > 0.f)) continue;
      const float wgt = exp2f(ldx(src[r] + 128, r != rank) - M) * l;
      const float2 a = ldx2(src[r] + 4 * lane, r != rank), b = ldx2(src[r] + 4 * lane + 2, r != rank);
      acc.x = fmaf(wgt, a.x, acc.x); acc.y = fmaf(wgt, a.y, acc.y); acc.z = fmaf(wgt, b.x, acc.z); acc.w = fmaf(wgt, b.y, acc.w);
      den += wgt;
    }
    const float inv = den > 0.f ? 1.f / den : 0.f;
    acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
    if (p.out_fp32) {
      *reinterpret_cast<float4*>(static_cast<float*>(p.out[y]) + static_cast<size_t>(row) * 128 + 4 * lane) = acc;
    } else {
      const __nv_bfloat162 x = __floats2bfloat162_rn(acc.x, acc.y), z = __floats2bfloat162_rn(acc.z, acc.w);
      uint2 v;
      v.x = *reinterpret_cast<const uint32_t*>(&x);
      v.y = *reinterpret_cast<const uint32_t*>(&z);
      *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(p.out[y]) + static_cast<size_t>(row) * 128 + 4 * lane) = v;
    }
  }
  // 5.
  if (tid == 0) *step = s;
}

int check_args(int R, int rows, int rank) {
  if (R < 1 || R > XR || rank < 0 || rank >= R || rows < 1 || rows > 8 * XCTA) return -3;
  return 0;
}

}  // namespace

size_t xchg_bytes(int rows) { return XCH_DATA + 2ull * XR * slab_bytes(rows); }

int xchg_launch(const float* part, void* const* bufs, int rank, int R, int rows, void* out, int out_fp32, cudaStream_t st) {
  if (check_args(R, rows, rank) != 0) return -3;
  XchgParams p{};
  p.part[0] = part;
  p.out[0] = out;
  for (int r = 0; r < R; ++r) p.buf[r] = static_cast<uint8_t*>(bufs[r]);
  p.rank0 = rank; p.R = R; p.rows = rows; p.out_fp32 = out_fp32;
  k_xchg_merge<<<dim3((rows + 7) / 8, 1), 256, 0, st>>>(p);
  return cudaPeekAtLastError() == cudaSuccess ? 0 : -1;
}

// R emulated ranks on this device as one cooperative launch (all CTAs resident: they wait on one another)
int xchg_selftest_launch(const float* const* parts, void* const* bufs, int R, int rows, void* const* outs, int out_fp32, cudaStream_t st) {
  if (check_args(R, rows, 0) != 0) return -3;
  XchgParams p{};
  for (int r = 0; r < R; ++r) { p.part[r] = parts[r]; p.out[r] = outs[r]; p.buf[r] = static_cast<uint8_t*>(bufs[r]); }
  p.rank0 = 0; p.R = R; p.rows = rows; p.out_fp32 = out_fp32;
  int dev = 0, sms = 0, occ = 0, coop = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev) != cudaSuccess || !coop ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, k_xchg_merge, 256, 0) != cudaSuccess)
    return -2;
  const dim3 grid((rows + 7) / 8, R);
  if (static_cast<long long>(grid.x) * grid.y > static_cast<long long>(sms) * occ) return -3;    // must all be resident
  void* args[] = {&p};
  return cudaLaunchCooperativeKernel(reinterpret_cast<void*>(k_xchg_merge), grid, dim3(256), args, 0, st) == cudaSuccess ? 0 : -1;
}

int xchg_status() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_xstatus, sizeof(int));
  return v;
}

}  // namespace fr
