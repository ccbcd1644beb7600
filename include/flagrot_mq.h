/* C ABI of libflagrot_mq.so for NVIDIA B200 (sm_100a), ABI version 7: prefix-cached multi-query prefill attention over
 * FlagRot INT4 / INT2 pages.
 *
 * Drop-in for the library the reference builds from integrations/vllm_flagrot/csrc/mq_prefill.cu and loads through ctypes
 * (integrations/vllm_flagrot/vllm_flagrot/prefill_mq.py:57-86).  Raw DEVICE pointers, the caller's cudaStream_t as void*;
 * asynchronous, allocation-free.  Return 0 ok, -1 launch error, -2 shared memory, -3 bad G / kernel, -4 head dim not 128.
 * kernel 1 = 64 query rows per tile (mma.sync), kernel 2 = 128 rows (mma.sync), kernel 3 = 128 rows on tcgen05 / tensor memory (the partial buffers are [nitems, Hkv, rows, 128]).
 */
#ifndef FLAGROT_MQ_H
#define FLAGROT_MQ_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* replaces mq_prefill.cu:1470, 1600, 1598 */
int frmq_abi_version(void);
const char* frmq_last_error(void);
int frmq_smem_bytes(void);
/* no counterpart in the reference: 0, or the source line of a bounded device-side wait that gave up (sticky;
 * synchronises the device) */
int frmq_device_status(void);

/* q (bf16, or fp32 when q_fp32; row stride q_ts elements; rows idx[0..m) or 0..m) -> FP16 [m, Hq, 128] in the keys' stored
 * basis (kfull uint8 [Hkv]: whole-head H128 / 8; kmask uint8 [Hkv, 4]: H32 per group; either may be null) times qscale.
 * replaces mq_prefill.cu:1473-1488 */
int frmq_prep_q(const void* q, int q_fp32, long long q_ts, const int* idx, int m, int Hq, int G, const uint8_t* kfull,
                const uint8_t* kmask, float qscale, void* q16, int Dh, void* stream);

/* partial attention of every (item, kv head): tiles int32 [nt, 9], items int32 [ni, 4] (layouts: prefill_mq.py:106-126);
 * key j visible to the query at position p iff kmin <= j <= max(p - shift, ext); konly bit 0: key-only 2x2 pages (per-token
 * flags), bit 1: INT2 pages.  opart fp32 [ni, Hkv, rows, 128] unnormalised, ml fp32 [ni, Hkv, rows, 2] = (max in log2
 * units, sum).  replaces mq_prefill.cu:1490-1546 */
int frmq_attn(const void* q16, const uint8_t* pool, long long page_stride, const int* bt, long long bt_stride, const int* tiles,
              const int* items, int nitems, int Hkv, int G, int shift, int konly, float* opart, float* ml, int kernel, int Dh,
              void* stream, int kmin);

/* combines the items of each tile: bf16 rows (row stride o_ts) at the tiles' output rows, or fp32 [m, Hq, 128] compact
 * rows when out_fp32; lse (optional) fp32 [Hq, lse_ts] natural log, -inf = no visible key.  replaces mq_prefill.cu:1548-1559 */
int frmq_merge(const int* tiles, int ntiles, const float* opart, const float* ml, int Hkv, int G, int rows, void* out,
               long long o_ts, int out_fp32, float* lse, long long lse_ts, int Dh, void* stream);

/* gathers the K / V rows of the BF16 window call: map int64 [nk] = (kind << 32) | row, kind 0 sinkb, 1 preb (both
 * [*, 2 Hkv, 128]), 2 the batch rows kch / vch.  replaces mq_prefill.cu:1561-1578 */
int frmq_win_gather(const long long* map, int nk, const void* sinkb, const void* preb, const void* kch, long long k_ts,
                    const void* vch, long long v_ts, int Hkv, void* kw, void* vw, int Dh, void* stream);

/* three-way LSE merge of the page part (fp32), the window part (bf16 + lse; may be null) and the sink part (fp32 softmax
 * over <= S BF16 keys with j <= pos - W; may be null) into the bf16 output rows idx[c].  replaces mq_prefill.cu:1580-1596 */
int frmq_bf_merge(int m, int Hq, int Hkv, const void* q, long long q_ts, const long long* idx, const float* o_p, const float* lse_p,
                  const void* o_w, const float* lse_w, const void* sk, const long long* row_req, const long long* row_pos,
                  const long long* sk_len, int S, int W, float scale, void* out, long long o_ts, int Dh, void* stream);

#ifdef __cplusplus
}
#endif
#endif
