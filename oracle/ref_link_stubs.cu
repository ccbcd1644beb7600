// Link stubs for the reference entry points whose definitions live in translation units that only build for sm_90a
// (they use wgmma).  The writer-only reference library built by build_ref.sh exports fr_cb_write3,
// fr_w3_static_write and fr_head_fwht; every other fr_* entry resolves to one of these stubs and reports
// "variant unsupported" (-3).  Test infrastructure only: nothing in the shipped libraries links this file.
#include "attn_codebook.cuh"
#include "attn_decode_v2.cuh"

int attn2_launch(int, int, int, const PagedParams&, cudaStream_t) { return -3; }
int attn2_occupancy(int, int, int, int) { return 0; }
int attn2_chunk_bytes(int fmt, int page) { return page * ((fmt == A2_INT2A || fmt == A2_KONLYA2) ? 80 : 144); }
int paged_write_launch(int, const PagedWriteParams&, cudaStream_t) { return -3; }
int cb_attn_launch(int, int, int, const CbAttnParams&, cudaStream_t) { return -3; }
int cb_attn_occupancy(int, int, int, int) { return 0; }
int cb_chunk_bytes(int kind, int page) { return page * (kind == CB_KONLYA2 ? 80 : 144); }
int cb_write_launch(int, const CbWriteParams&, cudaStream_t) { return -3; }
int cb_write_smem_hd(int, int, int) { return 0; }
