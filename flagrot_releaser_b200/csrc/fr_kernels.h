// Internal launcher declarations shared by the translation units of libflagrot_kernels.so (not part of the C ABI).
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace fr {

int head_fwht_launch(const void* x, long long x_ts, void* out, long long o_ts, int T, int H, const uint8_t* flags,
                     float scale, cudaStream_t st, int D = 128);
// rows [row0, row0 + nrow) of every token through the static row writer (nb = 4 | 2 code bits)
int rows_launch(int nb, const void* kv, long long kv_ts, const long long* slots, int slot_ph, int T, int Hkv, int page,
                const uint8_t* mask, const uint8_t* hfull, const float* kmu, uint8_t* pool, int row0, int nrow,
                int shared15, cudaStream_t st, int sym = 0);
int dyn_keys_launch(int nb, const void* kv, long long kv_ts, const long long* slots, int slot_ph, int T, int Hkv, int page,
                    const float* CT, const float* kmu, uint8_t* pool, cudaStream_t st, int with_values = 0, int sym = 0);

// positions [start, n) of one request's pages -> K / V rows in the original basis (fr_dequant.cu)
int dequant_pages_launch(int nb, int key_only, const uint8_t* pool, const int* bt_row, int start, int n, int Hkv, int page,
                         const uint8_t* kmask, const uint8_t* vmask, const uint8_t* kfull, const uint8_t* vfull, void* ok, void* ov,
                         int fp32, cudaStream_t st, int sym = 0);

// paged decode attention (fr_decode.cu)
struct DecodeParams {
  const void* q; long long q_bs;             // bf16 [B, G * Hkv, 128], row stride in elements
  const uint8_t* pool;                       // [num_pages, Hkv, chunk]
  const int* block_table; int bt_stride;     // int32 [B, bt_stride] (stride 0: every row reads row 0)
  const int* seq_lens;                       // int32 [B]
  int B, Hkv, G, page, nsplit, chunk;        // nsplit body splits of `chunk` tokens
  float qscale;                              // softmax scale * log2(e)
  const uint8_t* kmask; const uint8_t* vmask;  // static formats: [Hkv, 4] block flags or null (q rotation / output back-rotation)
  const uint8_t* vmask_tail;                 // V flags applied to the BF16 window partial (stored V basis) or null
  float* opart; float* mlpart; int* counter;
  void* out; long long o_bs;                 // bf16 [B, G * Hkv * 128]
  const void* tail; const int* tail_len; const int* tail_idx; long long tail_bs, tail_ts;
  int kv_start;
  int nb;                                    // code bits 4 | 2
  int key_only;                              // 1: per-token flags in the scale sign bits (konlya / konlya2 / konly)
  int sym;                                   // 1: symmetric INT4 pages (int4 / konly): sign-magnitude codes, no zero points
  float* part_out;                           // optional: unmerged (m, l, o) of the whole row (extension entry)
  int rows_wide, chunk_w;                    // set by decode_launch: rows [0, rows_wide) use nsplit - 1 pieces of chunk_w tokens
};
int decode_launch(const DecodeParams& p, cudaStream_t st);
int decode_occupancy(int nb, int key_only);
// exchange + merge of KV-sequence shard partials over peer memory (fr_xchg.cu)
size_t xchg_bytes(int rows);
int xchg_launch(const float* part, void* const* bufs, int rank, int R, int rows, void* out, int out_fp32, cudaStream_t st);
int xchg_selftest_launch(const float* const* parts, void* const* bufs, int R, int rows, void* const* outs, int out_fp32, cudaStream_t st);
int xchg_status();     // 0, or the source line of the peer wait that gave up (sticky)
void dyn_writer_exact_only(int on);                          // test switch of the bulk key writer (host state, not per stream)
int dyn_writer_stats(unsigned long long* out2, int reset);   // {(token, head) pairs, pairs that took the exact sums} of the bulk key writer
int writer_status();   // 0, or the source line of the staging wait that gave up (sticky; results stay correct)
int decode_status();   // 0, or the source line of a bounded wait that gave up (sticky)

}  // namespace fr
