/* C ABI of libflagrot_kernels.so for NVIDIA B200 (sm_100a), ABI version 9.
 *
 * Drop-in for the library the reference builds from integrations/vllm_flagrot/csrc/flagrot_capi.cu and that its vLLM
 * plugin loads through ctypes (integrations/vllm_flagrot/vllm_flagrot/kernels.py:140-177): same symbols, argument
 * orders, page byte layouts and return codes.  Every entry takes raw DEVICE pointers, element strides and the caller's
 * cudaStream_t (as void*); launches are asynchronous, allocate nothing and may be captured in CUDA graphs.
 * Return: 0 ok, -1 launch error, -2 shared memory, -3 unsupported variant, -4 unknown format / kind, -5 page size not
 * 16 | 32, -8 head dim not 128.
 *
 * Formats (fmt of fr_v2_*):  5 int4a, 8 int2a (static block flags), 7 konlya, 9 konlya2 (key-only 2x2 flags), and the
 *                            symmetric INT4 ones: 4 int4 (static), 6 konly (key-only).
 * Kinds   (kind of fr_cb_*): 10 konlya (INT4), 11 konlya2 (INT2), 6 konly (symmetric INT4).
 * The ablation codebooks (kinds 1-5, 7-9) answer -4.
 * Page layout: one chunk per (page, kv head), 144 * page bytes (INT4) or 80 * page bytes (INT2), as specified in the
 * reference's kernels/csrc/attn_decode_v2.cuh:14-46.
 */
#ifndef FLAGROT_KERNELS_H
#define FLAGROT_KERNELS_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* replaces flagrot_capi.cu:21 */
int fr_abi_version(void);

/* Paged decode attention over static pages or (fmt 7 / 9) key-only pages, any GQA group.
 * q bf16 [B, gqa*Hkv, 128] (row stride q_bs elements); pool [num_pages, Hkv, chunk]; block_table int32 [B, bt_stride]
 * (bt_stride 0: every row reads row 0); seq_lens int32 [B]; qscale = softmax scale * log2(e); kmask / vmask uint8
 * [Hkv, 4] honoured when qrot / vrot (rb must be 32); workspace opart / mlpart for B * Hkv * ceil(gqa/4) * (nsplit + 1)
 * partials of 4*128 + 8 floats, counter int32 [B * Hkv] zero-initialised once (left zero); out bf16 [B, gqa*Hkv*128]
 * (row stride o_bs); tail: BF16 rows [R, W, 2*Hkv, 128] (strides tail_bs / tail_ts elements), tail_len int32 [B]
 * (clipped to 256), tail_idx int32 [B] or null; kv_start: tokens [0, kv_start) masked in the pages.
 * variant / stages are accepted and ignored (variant bit 4096 = head dim 256: -8).
 * replaces flagrot_capi.cu:42-64 */
int fr_v2_attn(int fmt, const void* q, long long q_bs, const uint8_t* pool, const int* block_table, int bt_stride,
               const int* seq_lens, int B, int Hkv, int page, int nsplit, int chunk, float qscale,
               const uint8_t* kmask, const uint8_t* vmask, int rb, int qrot, int vrot, int variant, int stages,
               float* opart, float* mlpart, int* counter, void* out, long long o_bs, const void* tail,
               const int* tail_len, const int* tail_idx, long long tail_bs, long long tail_ts, void* stream, int gqa,
               int kv_start);

/* Static writer: kv bf16 [T, 2*Hkv, hd] (token stride kv_ts elements, 8-byte aligned rows) -> pool at slots int64 [T]
 * (slot = page_id * page + offset; < 0 skipped); mask uint8 [2*Hkv, hd/32] (K rows first) or null; kmu fp32 [Hkv, hd] or
 * null.  hd = 128 (or 0), or 256: a (page, kv head) chunk is then two 128-d half chunks, dims 0-127 first.
 * replaces flagrot_capi.cu:66-77 */
int fr_v2_write(int fmt, const void* kv, long long kv_ts, const long long* slots, int T, int Hkv, int page,
                const uint8_t* mask, int rb, uint8_t* pool, void* stream, int hd, const float* kmu);

/* resident CTAs per SM of the decode kernel (input of the host split planner); replaces flagrot_capi.cu:79 */
int fr_v2_occupancy(int fmt, int variant, int stages, int page);
/* replaces flagrot_capi.cu:80 */
int fr_v2_chunk_bytes(int fmt, int page);
/* replaces flagrot_capi.cu:84 (15 sign-table entries; the key-only kinds do not use the table) */
int fr_cb_nsg(void);

/* Dynamic key-only 2x2 writer: keys choose per 32-vector {I, H32} and per head {base, H128} by the C_q-weighted error,
 * values are stored untransformed.  CT fp32 [Hkv, 128, 128] = C_q transposed, co fp32 [Hkv, 128] (unused by these
 * kinds), sg HOST pointer to 60 sign words (unused), slot_ph 1: slots int64 [T, Hkv].  tg is accepted and ignored.
 * replaces flagrot_capi.cu:86-99 */
int fr_cb_write(const void* kv, long long kv_ts, const long long* slots, int slot_ph, int T, int Hkv, int page, int tg,
                const float* CT, const float* co, const unsigned* sg, int kind, uint8_t* pool, void* stream, int hd,
                const float* kmu);

/* Same bytes as fr_cb_write.  nchunk < 0 skips the key kernel, nchunk_v < 0 the value kernel (the two halves may run on
 * two streams in any order: bit 15 of the V group-0 scale word belongs to the key half).  C1 / beta are ignored.
 * replaces flagrot_capi.cu:104-116 */
int fr_cb_write3(const void* kv, long long kv_ts, const long long* slots, int slot_ph, int T, int Hkv, int page,
                 const float* CT, const float* co, const void* C1, const float* beta, const unsigned* sg, int kind,
                 uint8_t* pool, int nchunk, int nchunk_v, void* stream, const float* kmu);

/* Static writer fused with the whole-head rotation: rows of heads with hfull set become bf16(H128 x / 16) first;
 * asym 0 int4 (symmetric), 1 int4a, 2 int2a; path is accepted and ignored.  replaces flagrot_capi.cu:121-131 */
int fr_w3_static_write(const void* kv, long long kv_ts, const long long* slots, int T, int Hkv, int page,
                       const uint8_t* mask, const uint8_t* hfull, int asym, uint8_t* pool, int path, void* stream,
                       const float* kmu);

/* Decode attention over key-only pages at GQA 4; arguments as fr_v2_attn without masks.  replaces flagrot_capi.cu:133-149 */
int fr_cb_attn(const void* q, long long q_bs, const uint8_t* pool, const int* block_table, int bt_stride,
               const int* seq_lens, int B, int Hkv, int page, int nsplit, int chunk, float qscale, const unsigned* sg,
               int kind, int variant, int stages, float* opart, float* mlpart, int* counter, void* out, long long o_bs,
               const void* tail, const int* tail_len, const int* tail_idx, long long tail_bs, long long tail_ts,
               void* stream, int kv_start);

/* replaces flagrot_capi.cu:151-153 */
int fr_cb_occupancy(int kind, int variant, int stages, int page);
int fr_cb_chunk_bytes(int kind, int page);
int fr_cb_write_smem(int kind, int tg, int hd);
/* text of the last CUDA error of the calling thread; replaces flagrot_capi.cu:155 */
const char* fr_last_error(void);

/* out[t, h, :] = flags[h] ? bf16(scale * H_D x[t, h, :]) : x[t, h, :] (unnormalised Sylvester matrix, fp32
 * butterflies in ascending stride order, one rounding); x and out may alias; D = 128 or 256, anything else -8.
 * replaces flagrot_capi.cu:160-265 */
int fr_head_fwht(const void* x, long long x_ts, void* out, long long o_ts, int T, int H, const uint8_t* flags,
                 float scale, void* stream, int D);

/* ---- additions: no counterpart in the reference ABI ---- */

/* fr_v2_attn that emits, instead of bf16 rows, fp32 [B, gqa*Hkv, 130] = normalised row (128) + log2-domain maximum m +
 * denominator l, so that rows of KV-sequence shards held by different devices can be merged
 * (o = sum_r w_r l_r o_r / sum_r w_r l_r, w_r = 2^(m_r - max m)). */
int fr_attn_partial(int fmt, const void* q, long long q_bs, const uint8_t* pool, const int* block_table, int bt_stride,
                    const int* seq_lens, int B, int Hkv, int page, int nsplit, int chunk, float qscale,
                    const uint8_t* kmask, const uint8_t* vmask, float* opart, float* mlpart, int* counter, float* part,
                    const void* tail, const int* tail_len, const int* tail_idx, long long tail_bs, long long tail_ts,
                    void* stream, int gqa, int kv_start);

/* No counterpart in the reference.  Merges the rows of R KV-sequence shards written by fr_attn_partial: parts fp32
 * [R, rows, 130] (rows = B * q heads; 128 normalised values, m in log2 units, l; l = 0: the shard saw no key) -> out
 * [rows, 128] bf16 (or fp32 when out_fp32).  o = sum_r w_r l_r o_r / sum_r w_r l_r, w_r = 2^(m_r - max m). */
int fr_merge_partials(const float* parts, int R, int rows, void* out, int out_fp32, void* stream);

/* No counterpart in the reference's C ABI: the reference does this step of its "fa" prefill path in PyTorch
 * (vllm_flagrot/attention/backend.py:1744-1789, kernels.py dequant_cb_pages / dequant_v2_pages + unrotate_cached).
 * Positions [start, n) of the request whose block-table row is bt_row -> ok / ov [n - start, Hkv, 128] (bf16, or fp32 when
 * out_fp32) in the ORIGINAL basis.  fmt as fr_v2_attn (5 int4a, 7 konlya, 8 int2a, 9 konlya2).  Key-only formats take the
 * per-token flags from the pages; static formats take kmask / vmask uint8 [Hkv, 4] (block flags) and kfull / vfull uint8
 * [Hkv] (whole-head flags: stored as bf16(H128 x / 16)), any of which may be null. */
int fr_dequant_pages(int fmt, const uint8_t* pool, const int* bt_row, int start, int n, int Hkv, int page, const uint8_t* kmask,
                     const uint8_t* vmask, const uint8_t* kfull, const uint8_t* vfull, void* ok, void* ov, int out_fp32,
                     void* stream);

/* No counterpart in the reference.  KV-sequence shards on the GPUs of one node: exchange of the partial rows written by
 * fr_attn_partial over peer memory and their merge, one kernel per rank instead of an all-gather collective plus
 * fr_merge_partials.  Every rank allocates one exchange buffer (fr_xchg_alloc: device memory of fr_xchg_bytes(rows) bytes,
 * zeroed, and its 64-byte CUDA IPC handle), hands the handle to the other ranks (any host channel) and maps theirs
 * (fr_xchg_open).  fr_xchg_merge(part, bufs, rank, R, rows, out, ...): part fp32 [rows, 130] of this rank, bufs = HOST array
 * of the R buffers as mapped in this process (bufs[rank] the own one), R <= 8, rows <= 1024 -> out [rows, 128] bf16 (fp32
 * when out_fp32) = the merge over all ranks.  Collective semantics: every rank makes the same sequence of calls on the
 * buffers; the step counters live in the buffers, so a captured launch replays correctly.  The wait for the peers' rows is
 * bounded (about nine seconds: a peer's launch may trail by host time); if it runs out, fr_device_status reports it and the
 * output must be discarded.
 * fr_xchg_selftest runs the same protocol for R emulated ranks on ONE device as one cooperative launch (parts / bufs / outs:
 * host arrays of R device pointers). */
long long fr_xchg_bytes(int rows);
int fr_xchg_alloc(int rows, void** ptr, void* handle64);
int fr_xchg_open(const void* handle64, void** ptr);
int fr_xchg_close(void* ptr);
int fr_xchg_free(void* ptr);
int fr_xchg_merge(const float* part, void* const* bufs, int rank, int R, int rows, void* out, int out_fp32, void* stream);
int fr_xchg_selftest(const float* const* parts, void* const* bufs, int R, int rows, void* const* outs, int out_fp32,
                     void* stream);

/* 0, or the source line of a bounded device-side wait that gave up (sticky; synchronises the device). */
int fr_device_status(void);

/* Bulk key writer of fr_cb_write / fr_cb_write3 (more than 4096 (token, kv head) pairs per call): the head choice
 * base / H128 is first estimated on the tensor cores with a rigorous error bar and only the undecided pairs evaluate the
 * criterion's fixed-order fp32 sums, so the pages are the same bytes either way.  out2 = {pairs written, pairs that took
 * the exact sums} since the last reset, on the current device (synchronises it); reset != 0 clears the counters.
 * fr_dyn_writer_exact_only(1) makes every pair take the exact sums (a test switch: process-wide host state). */
int fr_dyn_writer_stats(unsigned long long* out2, int reset);
void fr_dyn_writer_exact_only(int on);

/* No counterpart in the reference.  fr_cb_attn (GQA 4, kinds 10 / 11) for a caller that cannot supply a workspace
 * because it cannot allocate device memory: a serving worker whose memory pool is frozen after start-up, or a plain C
 * host that only forwards the pointers it was handed.  The split partials and merge tickets live in a 16 MiB array
 * built into the library (held by every GPU that loads it, until exit); inputs and outputs are still the caller's.
 * Needs 256-rounded 4 * B * Hkv + 32 * parts bytes plus 2048 * parts bytes, parts = B * Hkv * (nsplit + 1); a larger
 * request returns -9 and prints the sizes to stderr.  The call allocates nothing.  The first call on a device looks up
 * the array's device address (this is also when the driver loads the module and sets the 16 MiB aside: on a device whose
 * memory is already full that first call answers -1): make that call before any stream capture.  The array is chosen
 * by the CURRENT device, so the current device must be the one `stream` belongs to.  All calls share the array, so two calls that
 * overlap on the GPU (two streams, or two host threads) corrupt each other: serialise them.  Each call clears its
 * tickets first; nothing else in the array is assumed. */
int fr_cb_attn_noalloc(const void* q, long long q_bs, const uint8_t* pool, const int* block_table, int bt_stride,
                       const int* seq_lens, int B, int Hkv, int page, int nsplit, int chunk, float qscale, int kind,
                       void* out, long long o_bs, const void* tail, const int* tail_len, const int* tail_idx,
                       long long tail_bs, long long tail_ts, void* stream, int kv_start);

#ifdef __cplusplus
}
#endif
#endif
