// sm_100a 5th-generation tensor-core primitives used by the FlagRot kernels: tensor-memory allocation, shared-memory
// matrix descriptors, instruction descriptors, tcgen05.mma issue / commit, tensor-memory loads and stores, and bounded
// mbarrier waits.  Inline PTX only; nothing here allocates or synchronises on the host.
//
// Shared-memory operand layouts (both "K-major": the reduction dimension is contiguous):
//   SW128   rows of 128 bytes; 8-row groups of 1024 bytes (stride SBO); inside a group the 16-byte chunk c of row r lives at
//           r * 128 + ((c ^ r) * 16); the tile base must be 1024-byte aligned.  One tcgen05.mma consumes 32 bytes of K per
//           row: the k-th step of a 128-byte row starts at base + 32 k (the hardware applies the XOR on the address bits).
//   PLAIN   no swizzle: 8 x 16-byte core matrices of 128 contiguous bytes (row r at r * 16); the next core matrix along K
//           is LBO bytes away, the next 8 rows SBO bytes away.
// Tensor memory: 128 lanes x 512 columns of 32 bits per SM; address = lane << 16 | column.  With M = 128 accumulator row i
// is lane i, and a warp can only touch lanes 32 (warp % 4) .. + 31.
#pragma once
#include <cstdint>

#include "fr_common.cuh"

namespace tc5 {

// ---------------------------------------------------------------------------------------------- mbarrier (bounded)
constexpr long long WAIT_CYCLES = 1ll << 30;   // SM clock cycles (about half a second) before a wait gives up

FR_DEVI void mbar_init(uint32_t a, int n) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(a), "r"(n)); }
FR_DEVI void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory"); }
FR_DEVI void mbar_arrive(uint32_t a) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(a) : "memory"); }
FR_DEVI void mbar_expect(uint32_t a, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(a), "r"(bytes) : "memory");
}
FR_DEVI bool mbar_try(uint32_t a, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(ok)
               : "r"(a), "r"(parity)
               : "memory");
  return ok != 0;
}
// false after WAIT_CYCLES: the caller records the failure and leaves without touching what it waited for.  The clock is
// read once per 32 probes: a waiting warp should cost as few issue slots as possible.
FR_DEVI bool mbar_wait(uint32_t a, uint32_t parity) {
  if (mbar_try(a, parity)) return true;
  const long long t0 = clock64();
  do {
#pragma unroll 1
    for (int i = 0; i < 32; ++i)
      if (mbar_try(a, parity)) return true;
  } while (clock64() - t0 < WAIT_CYCLES);
  return false;
}
// the same, ended early when another thread of the CTA has set *abort; a wait that runs out sets *abort itself
FR_DEVI bool mbar_wait_abortable(uint32_t a, uint32_t parity, volatile uint32_t* abort) {
  if (mbar_try(a, parity)) return true;
  const long long t0 = clock64();
  do {
#pragma unroll 1
    for (int i = 0; i < 32; ++i)
      if (mbar_try(a, parity)) return true;
    if (*abort) return false;
  } while (clock64() - t0 < WAIT_CYCLES);
  *abort = 1;
  return false;
}
// for roles that run ahead of the critical path (producers): between probes the warp sleeps, so that its waiting does not
// take issue slots from the warps everything else waits for
FR_DEVI bool mbar_wait_relaxed(uint32_t a, uint32_t parity, volatile uint32_t* abort) {
  if (mbar_try(a, parity)) return true;
  const long long t0 = clock64();
  do {
#pragma unroll 1
    for (int i = 0; i < 32; ++i) {
      __nanosleep(200);
      if (mbar_try(a, parity)) return true;
    }
    if (*abort) return false;
  } while (clock64() - t0 < WAIT_CYCLES);
  *abort = 1;
  return false;
}
FR_DEVI void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t mbar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst), "l"(src),
               "r"(bytes), "r"(mbar)
               : "memory");
}

// ---------------------------------------------------------------------------------------------- fences
FR_DEVI void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }   // st.shared -> tensor core
FR_DEVI void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
FR_DEVI void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }

// ---------------------------------------------------------------------------------------------- tensor memory
// one full warp; ncols a power of two in [32, 512]; the base address is written to *slot (shared memory)
FR_DEVI void tmem_alloc(uint32_t slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(slot), "r"(ncols) : "memory");
}
FR_DEVI void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory"); }
FR_DEVI void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(ncols) : "memory");
}

// ---------------------------------------------------------------------------------------------- descriptors
constexpr uint64_t DESC_VERSION = 1ull << 46;          // descriptor version of this architecture
constexpr uint64_t DESC_SW128 = 2ull << 61;            // layout type: 128-byte swizzle
// K-major, 128-byte swizzle: sbo = bytes between 8-row groups (1024 when rows are 128 bytes apart)
FR_DEVI uint64_t desc_sw128(uint32_t saddr, uint32_t sbo) {
  return DESC_VERSION | DESC_SW128 | (static_cast<uint64_t>(sbo >> 4) << 32) | (1ull << 16) | ((saddr & 0x3FFFFu) >> 4);
}
// K-major, no swizzle: lbo = bytes between core matrices along K, sbo = bytes between 8-row groups
FR_DEVI uint64_t desc_plain(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  return DESC_VERSION | (static_cast<uint64_t>(sbo >> 4) << 32) | (static_cast<uint64_t>(lbo >> 4) << 16) | ((saddr & 0x3FFFFu) >> 4);
}
// instruction descriptor: D format (0 f16, 1 f32, 2 s32), A / B formats (kind::f16: 0 f16, 1 bf16; kind::i8: 0 u8, 1 s8),
// both operands K-major, M x N tile
__host__ __device__ constexpr uint32_t idesc(int dfmt, int afmt, int bfmt, int M, int N) {
  return (static_cast<uint32_t>(dfmt) << 4) | (static_cast<uint32_t>(afmt) << 7) | (static_cast<uint32_t>(bfmt) << 10) |
         (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}

// ---------------------------------------------------------------------------------------------- MMA issue (one thread)
// true in exactly one lane of a converged warp.  Issuing under this predicate (instead of lane == 0) keeps the operands
// of tcgen05.mma in the uniform datapath: descriptors built from warp-uniform values need no per-instruction transfer.
FR_DEVI bool elect_one() {
  uint32_t pred;
  asm volatile("{\n .reg .pred P;\n elect.sync _|P, 0xffffffff;\n selp.u32 %0, 1, 0, P;\n}\n" : "=r"(pred));
  return pred != 0;
}
// D[tmem] (+)= A[smem] * B[smem]^T; accumulate = 0 overwrites D
FR_DEVI void mma_f16_ss(uint32_t d, uint64_t a, uint64_t b, uint32_t id, uint32_t accumulate) {
  asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d), "l"(a),
               "l"(b), "r"(id), "r"(accumulate)
               : "memory");
}
// A from tensor memory (row i = lane i, 16-bit elements packed two per column)
FR_DEVI void mma_f16_ts(uint32_t d, uint32_t a, uint64_t b, uint32_t id, uint32_t accumulate) {
  asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n" ::"r"(d), "r"(a),
               "l"(b), "r"(id), "r"(accumulate)
               : "memory");
}
FR_DEVI void mma_i8_ss(uint32_t d, uint64_t a, uint64_t b, uint32_t id, uint32_t accumulate) {
  asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}\n" ::"r"(d), "l"(a),
               "l"(b), "r"(id), "r"(accumulate)
               : "memory");
}
// arrives on the mbarrier when every MMA issued so far by this thread has finished (implies fence::before_thread_sync)
FR_DEVI void mma_commit(uint32_t mbar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(mbar) : "memory");
}

// ---------------------------------------------------------------------------------------------- tensor memory <-> registers
// 32 lanes x N consecutive columns: thread i of the warp gets lane (lane field of taddr) + i
#define TC5_R4(v, o) "=r"(v[o]), "=r"(v[o + 1]), "=r"(v[o + 2]), "=r"(v[o + 3])
#define TC5_R16(v, o) TC5_R4(v, o), TC5_R4(v, o + 4), TC5_R4(v, o + 8), TC5_R4(v, o + 12)
#define TC5_W4(v, o) "r"(v[o]), "r"(v[o + 1]), "r"(v[o + 2]), "r"(v[o + 3])
#define TC5_W16(v, o) TC5_W4(v, o), TC5_W4(v, o + 4), TC5_W4(v, o + 8), TC5_W4(v, o + 12)
FR_DEVI void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : TC5_R16(v, 0)
      : "r"(taddr)
      : "memory");
}
FR_DEVI void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,"
      "%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : TC5_R16(v, 0), TC5_R16(v, 16)
      : "r"(taddr)
      : "memory");
}
FR_DEVI void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15};\n" ::TC5_W16(v, 0),
      "r"(taddr)
      : "memory");
}
FR_DEVI void tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,"
      "%23,%24,%25,%26,%27,%28,%29,%30,%31};\n" ::TC5_W16(v, 0),
      TC5_W16(v, 16), "r"(taddr)
      : "memory");
}
FR_DEVI void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
FR_DEVI void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

// byte offset of element (row, 16-byte chunk) inside a SW128 tile whose rows are 128 bytes
FR_DEVI uint32_t sw128_off(int row, int chunk) { return (row >> 3) * 1024 + (row & 7) * 128 + ((chunk ^ (row & 7)) << 4); }

}  // namespace tc5
