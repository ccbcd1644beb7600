/* C ABI of libflagrot_kivi.so for NVIDIA B200 (sm_100a), ABI version 9: FlagRot-KIVI INT2 pages.
 *
 * Drop-in for the library the reference builds from integrations/vllm_flagrot/csrc/kivi.cu and loads through ctypes
 * (integrations/vllm_flagrot/vllm_flagrot/kivi.py:49-77): same symbols, argument orders and page byte layout
 * (kivi.cu:15-26: 12 D + 16 bytes per (16-token page, kv head)).  Raw DEVICE pointers, element strides, the caller's
 * cudaStream_t as void*; asynchronous, allocation-free.  Return 0 ok, 1 launch error, 2 unsupported argument; text in
 * kv_last_error().  Built: head dim 128; the kivi2 pages (FP16 scale / min) and, with f8 bit 0 set in every entry, the
 * kivi2p8 pages (kivi.cu:28-35: FP8 E4M3 scale / min, 10 D bytes per (page, kv head), flags in the scale sign bits, codes
 * computed from the stored values).  f8 bit 1 (the reference's "fast" / "v2" kernel variants, which compute the same
 * values) is accepted everywhere and selects nothing.  Not built (code 2): head dim 256.
 */
#ifndef FLAGROT_KIVI_H
#define FLAGROT_KIVI_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* replaces kivi.cu:74-75 */
const char* kv_last_error(void);
int kv_abi_version(void);
/* replaces kivi.cu:97-98 */
int kv_chunk_bytes(int D);
int kv_chunk_bytes8(int D);

/* Per-token value encoder: kv bf16 [n, 2 Hkv, D] (row stride kv_rs elements, V rows Hkv .. 2 Hkv - 1) -> pool at slots
 * int64 [n] (< 0 skipped); candidates identity / H32 per 32-dim sub-vector / whole-head H_D chosen by sum d^2 co
 * (co fp32 [Hkv, D]) or, when M fp32 [Hkv, D, D] is given, by e^T M e; ident 1: identity only; vfix int32 [Hkv]: frozen choice
 * (bits 0..3 H32, bit 16 whole head).
 * replaces kivi.cu:1934-1948 */
int kv_v_write(const void* kv, long long kv_rs, int n, int Hkv, int D, const void* slots, const void* co, const void* M,
               void* pool, int ident, const void* vfix, int f8, void* stream);

/* Per-(32-token group, kv head) key encoder (per-channel INT2 over the group's valid tokens): src / src2 bf16 rows,
 * sidx int64 [N, 32] (r >= 0: src row r; r <= -2: src2 row -r - 2; -1: not in the group), dslot int64 [N, 32] page slots
 * (dslot[n][0] < 0: item skipped); selection by the attention-weighted rule with the calibration queries qs fp32
 * [Hkv, NQ, D], lz fp32 [Hkv, NQ], scaling qsc; ident / kfix as above.  replaces kivi.cu:1950-1979 */
int kv_k_encode(const void* src, long long src_rs, const void* src2, long long src2_rs, const void* sidx, const void* dslot,
                int N, int Hkv, int D, const void* qs, const void* lz, int NQ, float qsc, void* pool, int ident,
                const void* kfix, int f8, void* stream);

/* Paged split decode attention + BF16 sink / window rows + merge.  q bf16 [B, Hkv G, D] (row stride q_rs), bt int32
 * [B, bt_rs], cached int32 [B] (page tokens read: [kv_start, cached)), NS splits of `chunk` tokens (multiple of 32),
 * qscale = softmax scale * log2(e), ring bf16 [(R + 1) T, 2 Hkv, D] with tail_len / tail_idx int32 [B], workspace
 * opart fp32 [B Hkv (NS + 1) G D], ml fp32 [B Hkv (NS + 1) G 2], out bf16 (row stride out_rs); G <= 8.
 * replaces kivi.cu:1983-2060 */
int kv_attn(const void* q, long long q_rs, const void* pool, const void* bt, long long bt_rs, const void* cached, int kv_start,
            int B, int Hkv, int G, int D, int NS, int chunk, float qscale, const void* ring, const void* tail_len,
            const void* tail_idx, int T, void* opart, void* ml, void* out, long long out_rs, int f8, void* stream);

/* K, V rows [(g1 - g0) 32, Hkv, D] (bf16, or fp32 when fp32 != 0) of groups [g0, g1) of one request in the writers'
 * basis.  replaces kivi.cu:2320-2342 */
int kv_dequant(const void* pool, const void* bt, int g0, int g1, int nvalid, int Hkv, int D, int fp32, void* ok, void* ov,
               int f8, void* stream);

/* LSE merge of two partial attentions, every operation rounded separately.  replaces kivi.cu:2290-2318 */
int kv_lse_merge(const void* oa, const void* la, long long la_hs, const void* ob, const void* lb, long long lb_hs, void* out,
                 long long out_rs, int na, int H, int D, void* stream);

#ifdef __cplusplus
}
#endif
#endif
