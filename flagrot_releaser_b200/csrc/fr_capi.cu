// C ABI of libflagrot_kernels.so (ABI 9): the entry points, argument orders and return codes of the reference's
// integrations/vllm_flagrot/csrc/flagrot_capi.cu, implemented on the sm_100a kernels of this directory.
// Declarations with the reference citation of every entry: include/flagrot_kernels.h.
//
// Conventions (as the reference): raw device pointers, element strides, the caller's cudaStream_t as void*; every
// launch is asynchronous and allocation-free; 0 = ok, -1 launch error, -2 shared memory, -3 unsupported variant,
// -4 unknown format / kind, -5 page size, -8 head dim.  Formats built here: int4a (5), int2a (8), konlya (7 / kind 10),
// konlya2 (9 / kind 11); the symmetric INT4 formats and the ablation codebooks answer -4.
#include <cstdint>
#include <cstring>
#include <cstdio>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "fr_kernels.h"
#include "../../include/flagrot_kernels.h"

namespace {
enum { FMT_INT4 = 4, FMT_INT4A = 5, FMT_KONLY = 6, FMT_KONLYA = 7, FMT_INT2A = 8, FMT_KONLYA2 = 9 };
enum { KIND_KONLY = 6, KIND_KONLYA = 10, KIND_KONLYA2 = 11 };
constexpr int VAR_HD256 = 4096;

// nb = code bits, ko bit 0 = key-only kind (per-token flags), ko bit 1 = symmetric INT4 (sign-magnitude codes)
bool fmt_info(int fmt, int& nb, int& ko) {
  switch (fmt) {
    case FMT_INT4: nb = 4; ko = 2; return true;
    case FMT_KONLY: nb = 4; ko = 3; return true;
    case FMT_INT4A: nb = 4; ko = 0; return true;
    case FMT_INT2A: nb = 2; ko = 0; return true;
    case FMT_KONLYA: nb = 4; ko = 1; return true;
    case FMT_KONLYA2: nb = 2; ko = 1; return true;
    default: return false;
  }
}
bool kind_info(int kind, int& nb, int* sym = nullptr) {      // konly (symmetric INT4) only where the caller takes `sym`
  if (sym != nullptr) *sym = 0;
  if (kind == KIND_KONLY && sym != nullptr) { nb = 4; *sym = 1; return true; }
  if (kind == KIND_KONLYA) { nb = 4; return true; }
  if (kind == KIND_KONLYA2) { nb = 2; return true; }
  return false;
}
int attn_common(int nb, int ko, const void* q, long long q_bs, const uint8_t* pool, const int* block_table, int bt_stride,
                const int* seq_lens, int B, int Hkv, int G, int page, int nsplit, int chunk, float qscale,
                const uint8_t* kmask, const uint8_t* vmask, const uint8_t* vmask_tail, float* opart, float* mlpart,
                int* counter, void* out, long long o_bs, const void* tail, const int* tail_len, const int* tail_idx,
                long long tail_bs, long long tail_ts, void* stream, int kv_start, float* part_out) {
  fr::DecodeParams p{};
  p.q = q; p.q_bs = q_bs; p.pool = pool; p.block_table = block_table; p.bt_stride = bt_stride; p.seq_lens = seq_lens;
  p.B = B; p.Hkv = Hkv; p.G = G; p.page = page; p.nsplit = nsplit; p.chunk = chunk; p.qscale = qscale;
  p.kmask = kmask; p.vmask = vmask; p.vmask_tail = vmask_tail;
  p.opart = opart; p.mlpart = mlpart; p.counter = counter; p.out = out; p.o_bs = o_bs;
  p.tail = tail; p.tail_len = tail_len; p.tail_idx = tail_idx; p.tail_bs = tail_bs; p.tail_ts = tail_ts;
  p.kv_start = kv_start; p.nb = nb; p.key_only = ko & 1; p.sym = ko >> 1; p.part_out = part_out;
  return fr::decode_launch(p, static_cast<cudaStream_t>(stream));
}
}  // namespace

extern "C" {

int fr_abi_version() { return 9; }

int fr_v2_attn(int fmt, const void* q, long long q_bs, const uint8_t* pool, const int* block_table, int bt_stride,
               const int* seq_lens, int B, int Hkv, int page, int nsplit, int chunk, float qscale,
               const uint8_t* kmask, const uint8_t* vmask, int rb, int qrot, int vrot, int variant, int stages,
               float* opart, float* mlpart, int* counter, void* out, long long o_bs, const void* tail,
               const int* tail_len, const int* tail_idx, long long tail_bs, long long tail_ts, void* stream, int gqa,
               int kv_start) {
  (void)stages;
  int nb, ko;
  if (!fmt_info(fmt, nb, ko)) return -4;
  if (variant & VAR_HD256) return -8;
  const bool kon = (ko & 1) != 0;
  const uint8_t* km = (!kon && qrot) ? kmask : nullptr;
  const uint8_t* vm = (!kon && vrot) ? vmask : nullptr;
  const uint8_t* vt = (!kon && (vrot || tail != nullptr)) ? vmask : nullptr;
  if ((km || vm || vt) && rb != 32) return -3;
  return attn_common(nb, ko, q, q_bs, pool, block_table, bt_stride, seq_lens, B, Hkv, gqa > 0 ? gqa : 4, page, nsplit,
                     chunk, qscale, km, vm, vt, opart, mlpart, counter, out, o_bs, tail, tail_len, tail_idx, tail_bs,
                     tail_ts, stream, kv_start, nullptr);
}

int fr_v2_write(int fmt, const void* kv, long long kv_ts, const long long* slots, int T, int Hkv, int page,
                const uint8_t* mask, int rb, uint8_t* pool, void* stream, int hd, const float* kmu) {
  if (T <= 0) return 0;
  if (hd != 0 && hd != 128 && hd != 256) return -8;
  if (fmt != FMT_INT4 && fmt != FMT_INT4A && fmt != FMT_INT2A) return -4;
  if (page != 16 && page != 32) return -5;
  if (mask != nullptr && rb != 32) return -3;
  // head dim 256: the two 128-d halves of a head are two half heads -- kv [T, 2 Hkv, 256] = [T, 4 Hkv, 128], mask
  // [2 Hkv, 8] = [4 Hkv, 4], kmu [Hkv, 256] = [2 Hkv, 128], pool [., Hkv, 2 chunk] = [., 2 Hkv, chunk]
  if (hd == 256) Hkv *= 2;
  return fr::rows_launch(fmt == FMT_INT2A ? 2 : 4, kv, kv_ts, slots, 0, T, Hkv, page, mask, nullptr, kmu, pool, 0, 2 * Hkv, 0,
                         static_cast<cudaStream_t>(stream), fmt == FMT_INT4);
}

int fr_v2_occupancy(int fmt, int variant, int stages, int page) {
  (void)variant; (void)stages; (void)page;
  int nb, ko;
  if (!fmt_info(fmt, nb, ko)) return 0;
  return fr::decode_occupancy(nb, ko & 1);
}
int fr_v2_chunk_bytes(int fmt, int page) { return page * ((fmt == FMT_INT2A || fmt == FMT_KONLYA2) ? 80 : 144); }

int fr_cb_nsg() { return 15; }

int fr_cb_write(const void* kv, long long kv_ts, const long long* slots, int slot_ph, int T, int Hkv, int page, int tg,
                const float* CT, const float* co, const unsigned* sg, int kind, uint8_t* pool, void* stream, int hd,
                const float* kmu) {
  (void)tg; (void)co; (void)sg;
  if (T <= 0) return 0;
  if (hd != 0 && hd != 128) return -8;
  int nb, sym;
  if (!kind_info(kind, nb, &sym)) return -4;
  if (page != 16 && page != 32) return -5;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return fr::dyn_keys_launch(nb, kv, kv_ts, slots, slot_ph, T, Hkv, page, CT, kmu, pool, st, 1, sym);   // keys and value rows
}

int fr_cb_write3(const void* kv, long long kv_ts, const long long* slots, int slot_ph, int T, int Hkv, int page,
                 const float* CT, const float* co, const void* C1, const float* beta, const unsigned* sg, int kind,
                 uint8_t* pool, int nchunk, int nchunk_v, void* stream, const float* kmu) {
  (void)co; (void)C1; (void)beta; (void)sg;   // C1 / beta are the reference's ranking tables: the bytes do not depend on them
  if (T <= 0) return 0;
  int nb, sym;
  if (!kind_info(kind, nb, &sym)) return -4;
  if (page != 16 && page != 32) return -5;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (nchunk >= 0 && nchunk_v >= 0) return fr::dyn_keys_launch(nb, kv, kv_ts, slots, slot_ph, T, Hkv, page, CT, kmu, pool, st, 1, sym);
  if (nchunk >= 0) return fr::dyn_keys_launch(nb, kv, kv_ts, slots, slot_ph, T, Hkv, page, CT, kmu, pool, st, 0, sym);
  if (nchunk_v >= 0)
    return fr::rows_launch(nb, kv, kv_ts, slots, slot_ph, T, Hkv, page, nullptr, nullptr, nullptr, pool, Hkv, Hkv, 1, st, sym);
  return 0;
}

int fr_w3_static_write(const void* kv, long long kv_ts, const long long* slots, int T, int Hkv, int page,
                       const uint8_t* mask, const uint8_t* hfull, int asym, uint8_t* pool, int path, void* stream,
                       const float* kmu) {
  (void)path;
  if (T <= 0) return 0;
  if (asym < 0 || asym > 2) return -4;
  if (page != 16 && page != 32) return -5;
  return fr::rows_launch(asym == 2 ? 2 : 4, kv, kv_ts, slots, 0, T, Hkv, page, mask, hfull, kmu, pool, 0, 2 * Hkv, 0,
                         static_cast<cudaStream_t>(stream), asym == 0);
}

int fr_cb_attn(const void* q, long long q_bs, const uint8_t* pool, const int* block_table, int bt_stride,
               const int* seq_lens, int B, int Hkv, int page, int nsplit, int chunk, float qscale, const unsigned* sg,
               int kind, int variant, int stages, float* opart, float* mlpart, int* counter, void* out, long long o_bs,
               const void* tail, const int* tail_len, const int* tail_idx, long long tail_bs, long long tail_ts,
               void* stream, int kv_start) {
  (void)sg; (void)variant; (void)stages;
  int nb, sym;
  if (!kind_info(kind, nb, &sym)) return -4;
  return attn_common(nb, sym ? 3 : 1, q, q_bs, pool, block_table, bt_stride, seq_lens, B, Hkv, 4, page, nsplit, chunk,
                     qscale, nullptr, nullptr, nullptr, opart, mlpart, counter, out, o_bs, tail, tail_len, tail_idx, tail_bs,
                     tail_ts, stream, kv_start, nullptr);
}

int fr_cb_occupancy(int kind, int variant, int stages, int page) {
  (void)variant; (void)stages; (void)page;
  int nb, sym;
  if (!kind_info(kind, nb, &sym)) return 0;
  return fr::decode_occupancy(nb, 1);
}
int fr_cb_chunk_bytes(int kind, int page) { return page * (kind == KIND_KONLYA2 ? 80 : 144); }
int fr_cb_write_smem(int kind, int tg, int hd) {
  (void)kind; (void)hd;
  const int t = tg < 1 ? 1 : (tg > 4 ? 4 : tg);
  return t * (128 * 4 + 2 * 128 * 4 * 2 + 2 * 128 + 2 * 4 * 2 + 2 * 4);   // static shared memory of the key writer
}

const char* fr_last_error() { return cudaGetErrorString(cudaGetLastError()); }

int fr_head_fwht(const void* x, long long x_ts, void* out, long long o_ts, int T, int H, const uint8_t* flags,
                 float scale, void* stream, int D) {
  if (T <= 0) return 0;
  if (D != 128 && D != 256) return -8;
  return fr::head_fwht_launch(x, x_ts, out, o_ts, T, H, flags, scale, static_cast<cudaStream_t>(stream), D);
}

// ---- extensions (no counterpart in the reference ABI)
int fr_attn_partial(int fmt, const void* q, long long q_bs, const uint8_t* pool, const int* block_table, int bt_stride,
                    const int* seq_lens, int B, int Hkv, int page, int nsplit, int chunk, float qscale,
                    const uint8_t* kmask, const uint8_t* vmask, float* opart, float* mlpart, int* counter, float* part,
                    const void* tail, const int* tail_len, const int* tail_idx, long long tail_bs, long long tail_ts,
                    void* stream, int gqa, int kv_start) {
  int nb, ko;
  if (!fmt_info(fmt, nb, ko)) return -4;
  return attn_common(nb, ko, q, q_bs, pool, block_table, bt_stride, seq_lens, B, Hkv, gqa > 0 ? gqa : 4, page, nsplit, chunk,
                     qscale, (ko & 1) ? nullptr : kmask, (ko & 1) ? nullptr : vmask, (ko & 1) ? nullptr : vmask, opart, mlpart, counter,
                     nullptr, 0, tail, tail_len, tail_idx, tail_bs, tail_ts, stream, kv_start, part);
}

int fr_dequant_pages(int fmt, const uint8_t* pool, const int* bt_row, int start, int n, int Hkv, int page, const uint8_t* kmask,
                     const uint8_t* vmask, const uint8_t* kfull, const uint8_t* vfull, void* ok, void* ov, int out_fp32,
                     void* stream) {
  int nb, ko;
  if (!fmt_info(fmt, nb, ko)) return -4;
  if (page != 16 && page != 32) return -5;
  if (start < 0 || Hkv <= 0) return -3;
  if (n > start && (pool == nullptr || bt_row == nullptr || ok == nullptr || ov == nullptr)) return -3;
  const bool kon = (ko & 1) != 0;
  return fr::dequant_pages_launch(nb, kon, pool, bt_row, start, n, Hkv, page, kon ? nullptr : kmask, kon ? nullptr : vmask,
                                  kon ? nullptr : kfull, kon ? nullptr : vfull, ok, ov, out_fp32, static_cast<cudaStream_t>(stream),
                                  ko >> 1);
}

// bulk key writer of fr_cb_write / fr_cb_write3: counters {(token, head) pairs, pairs whose head choice took the exact sums}
// since the last reset (device-wide), and a test switch that makes every choice take the exact sums (same bytes)
int fr_dyn_writer_stats(unsigned long long* out2, int reset) { return fr::dyn_writer_stats(out2, reset); }
void fr_dyn_writer_exact_only(int on) { fr::dyn_writer_exact_only(on); }

int fr_device_status() {
  const int d = fr::decode_status();
  if (d != 0) return d;
  const int w = fr::writer_status();
  return w != 0 ? w : fr::xchg_status();
}

}  // extern "C"

namespace {
// one warp per (row, q head): o = sum_r w_r l_r o_r / sum_r w_r l_r with w_r = 2^(m_r - max m); parts [R][rows][130]
__global__ void __launch_bounds__(128) k_merge_partials(const float* parts, int R, int rows, void* out, int out_fp32) {
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  float M = -INFINITY;
  for (int r = 0; r < R; ++r) {
    const float* p = parts + (static_cast<size_t>(r) * rows + row) * 130;
    if (p[129] > 0.f) M = fmaxf(M, p[128]);
  }
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float den = 0.f;
  for (int r = 0; r < R; ++r) {
    const float* p = parts + (static_cast<size_t>(r) * rows + row) * 130;
    const float l = p[129];
    if (!(l > 0.f)) continue;
    const float wgt = exp2f(p[128] - M) * l;
    const float2 a = *reinterpret_cast<const float2*>(p + 4 * lane), b = *reinterpret_cast<const float2*>(p + 4 * lane + 2);
    acc.x = fmaf(wgt, a.x, acc.x); acc.y = fmaf(wgt, a.y, acc.y); acc.z = fmaf(wgt, b.x, acc.z); acc.w = fmaf(wgt, b.y, acc.w);
    den += wgt;
  }
  const float inv = den > 0.f ? 1.f / den : 0.f;
  acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
  if (out_fp32) {
    *reinterpret_cast<float4*>(static_cast<float*>(out) + static_cast<size_t>(row) * 128 + 4 * lane) = acc;
  } else {
    const __nv_bfloat162 x = __floats2bfloat162_rn(acc.x, acc.y), y = __floats2bfloat162_rn(acc.z, acc.w);
    uint2 v;
    v.x = *reinterpret_cast<const uint32_t*>(&x);
    v.y = *reinterpret_cast<const uint32_t*>(&y);
    *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(out) + static_cast<size_t>(row) * 128 + 4 * lane) = v;
  }
}
}  // namespace

extern "C" {

int fr_merge_partials(const float* parts, int R, int rows, void* out, int out_fp32, void* stream) {
  if (rows <= 0 || R <= 0) return 0;
  k_merge_partials<<<(rows + 3) / 4, 128, 0, static_cast<cudaStream_t>(stream)>>>(parts, R, rows, out, out_fp32);
  return cudaPeekAtLastError() == cudaSuccess ? 0 : -1;
}

// ---- KV-sequence shards: exchange + merge over peer memory (csrc/fr_xchg.cu)
long long fr_xchg_bytes(int rows) { return static_cast<long long>(fr::xchg_bytes(rows)); }

int fr_xchg_alloc(int rows, void** ptr, void* handle64) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle travels as 64 bytes");
  void* d = nullptr;
  const size_t n = fr::xchg_bytes(rows);
  if (cudaMalloc(&d, n) != cudaSuccess) return -1;
  if (cudaMemset(d, 0, n) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess ||
      cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle64), d) != cudaSuccess) {
    cudaFree(d);
    return -1;
  }
  *ptr = d;
  return 0;
}

int fr_xchg_open(const void* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle64, sizeof(h));
  return cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess ? 0 : -1;
}

int fr_xchg_close(void* ptr) { return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? 0 : -1; }
int fr_xchg_free(void* ptr) { return cudaFree(ptr) == cudaSuccess ? 0 : -1; }

int fr_xchg_merge(const float* part, void* const* bufs, int rank, int R, int rows, void* out, int out_fp32, void* stream) {
  return fr::xchg_launch(part, bufs, rank, R, rows, out, out_fp32, static_cast<cudaStream_t>(stream));
}

int fr_xchg_selftest(const float* const* parts, void* const* bufs, int R, int rows, void* const* outs, int out_fp32, void* stream) {
  return fr::xchg_selftest_launch(parts, bufs, R, rows, outs, out_fp32, static_cast<cudaStream_t>(stream));
}

// ---- decode attention for callers that may not allocate device memory
// Some hosts of this library cannot hand over a workspace: a serving worker whose memory pool was sized and frozen at
// start-up (every later cudaMalloc would fail or fragment it), or a C / C++ host that owns no allocator at all and only
// forwards pointers it was given.  For them the split partials and the merge tickets live in one array compiled into
// the library.  Every GPU that loads the library carries these 16 MiB until the process exits.
// The host sees `g_noalloc_scratch` only as a handle of the symbol; the device address is looked up per device.
namespace {
constexpr size_t NOALLOC_SCRATCH_BYTES = 16u << 20;
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_SCRATCH_BYTES];
constexpr int NOALLOC_MAX_DEVICES = 64;
unsigned char* g_noalloc_ptr[NOALLOC_MAX_DEVICES];   // device address of the array on each device (0: not looked up yet)
}  // namespace

int fr_cb_attn_noalloc(const void* q, long long q_bs, const uint8_t* pool, const int* block_table, int bt_stride,
                       const int* seq_lens, int B, int Hkv, int page, int nsplit, int chunk, float qscale, int kind,
                       void* out, long long o_bs, const void* tail, const int* tail_len, const int* tail_idx,
                       long long tail_bs, long long tail_ts, void* stream, int kv_start) {
  int nb, sym;
  if (!kind_info(kind, nb, &sym)) return -4;
  if (B <= 0) return 0;
  if (Hkv <= 0 || nsplit < 1) return -3;
  // layout: tickets int32 [B * Hkv] (rounded up to 256 bytes) | (max, sum) pairs | partial rows
  const size_t parts = static_cast<size_t>(B) * Hkv * (static_cast<size_t>(nsplit) + 1);
  const size_t cnt_bytes = (static_cast<size_t>(B) * Hkv * sizeof(int) + 255) & ~static_cast<size_t>(255);
  const size_t ml_bytes = (parts * 8 * sizeof(float) + 255) & ~static_cast<size_t>(255);
  const size_t need = cnt_bytes + ml_bytes + parts * 512 * sizeof(float);
  if (need > NOALLOC_SCRATCH_BYTES) {
    std::fprintf(stderr, "fr_cb_attn_noalloc: batch %d x %d kv heads x %d splits needs %zu bytes of scratch, the built-in "
                         "array holds %zu; use fr_cb_attn with a caller workspace or fewer splits\n",
                 B, Hkv, nsplit, need, static_cast<size_t>(NOALLOC_SCRATCH_BYTES));
    return -9;
  }
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES) return -1;
  if (g_noalloc_ptr[dev] == nullptr) {   // first call on this device (do it before any stream capture)
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || p == nullptr) return -1;
    g_noalloc_ptr[dev] = static_cast<unsigned char*>(p);
  }
  unsigned char* base = g_noalloc_ptr[dev];
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // the array keeps whatever the previous call (or an aborted one) left: the tickets must start at zero
  if (cudaMemsetAsync(base, 0, cnt_bytes, st) != cudaSuccess) return -1;
  return attn_common(nb, sym ? 3 : 1, q, q_bs, pool, block_table, bt_stride, seq_lens, B, Hkv, 4, page, nsplit, chunk, qscale, nullptr,
                     nullptr, nullptr, reinterpret_cast<float*>(base + cnt_bytes + ml_bytes),
                     reinterpret_cast<float*>(base + cnt_bytes), reinterpret_cast<int*>(base), out, o_bs, tail, tail_len,
                     tail_idx, tail_bs, tail_ts, stream, kv_start, nullptr);
}

}  // extern "C"
