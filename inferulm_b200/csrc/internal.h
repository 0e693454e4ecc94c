// Internal launchers shared between the translation units of libwein_b200.so (not part of the C-ABI).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

enum { WB_GEMM_AUTO = 0, WB_GEMM_TC = 1 };  // kernel choice of a product: by row count (<= 32: skinny), or the tensor-memory kernel always
int32_t wb_gemm_wt(const void *a, const void *w, void *c, uint32_t m, uint32_t n, uint32_t k, uint32_t lda, uint32_t ldc,
                   void *scratch, uint64_t scratch_bytes, uint32_t path, cudaStream_t st);
int32_t wb_gemm_swiglu(const void *a, const void *w_gate_up, void *out, uint32_t m, uint32_t inter, uint32_t k, uint32_t lda,
                       uint32_t ldc, void *scratch, uint64_t scratch_bytes, uint32_t path, cudaStream_t st);
int32_t wb_ugemm(const void *a, const void *w, void *c, uint32_t m, uint32_t n, uint32_t k, uint32_t lda, uint32_t ldc, bool swiglu,
                 cudaStream_t st);  // tensor-memory GEMM (gemm_umma.cu), arguments already validated
int32_t wb_tensor_map_2d(void *tm, bool f32, const void *base, uint64_t inner, uint64_t rows, uint64_t row_bytes, uint32_t box_inner,
                         uint32_t box_rows);   // 128-byte-swizzled 2-d map; tm -> CUtensorMap
int32_t wb_ugemm_init();  // driver entry point and shared-memory opt-in of the current device, outside any stream capture
int32_t wb_gemm_init();
int32_t wb_attn_verify(const void *q, const void *k_cache, const void *v_cache, const void *block_table, const void *seq_ids,
                       const void *positions, const void *row_start, const void *row_count, const void *gate, void *out,
                       float q_scale, uint32_t bpr, uint32_t block_size, uint32_t q_heads, uint32_t kv_heads, uint32_t head_dim,
                       uint32_t n_spans, uint32_t max_count, uint32_t max_ctx, uint32_t seg_pages, void *scratch,
                       uint64_t scratch_bytes, uint32_t *status, bool deep, cudaStream_t st);  // status: optional, indexed by sequence id;
                       // deep: three page stages per warp (200 KB CTAs) instead of two; never changes a result
int32_t wb_attn_init(uint32_t head_dim);  // one-time shared-memory opt-in, outside any stream capture
int32_t wein_b200_argmax_partials(const void *x, const void *rows, void *part, uint32_t n, uint32_t s, uint32_t split, cudaStream_t st);

struct FilterArgs {
    const void *logits; const uint32_t *rows, *row_seq; uint32_t rows_per_seq;
    const float *temp, *top_p; const uint32_t *top_k; uint32_t n, s;
    uint32_t *out_ids; float *out_probs; uint32_t *out_n; uint32_t out_mul, out_off;
    uint32_t *sample_out; uint32_t sample_mul, sample_off; const uint64_t *seed, *round; uint32_t position;
};
int32_t wb_topk_filter_args(const FilterArgs &a, cudaStream_t st);

struct AcceptArgs {
    const uint64_t *am_part; uint32_t am_split;
    const uint32_t *p_ids, *q_ids, *p_n, *q_n; const float *p_probs, *q_probs;
    const float *temp; const uint64_t *seed, *round; const uint32_t *slot_of;
    const uint32_t *drafts; uint32_t draft_stride; const uint32_t *n_drafts; uint32_t B, k;
    uint32_t *accept_len, *out_tokens, *target;
};
int32_t wb_accept_args(const AcceptArgs &a, cudaStream_t st);

// fused glue (fused_glue.cu), all bit-exact against the unfused reference sequence
int32_t wb_qk_prep(const void *qgkv, uint32_t ld, const void *qn, const void *kn, const float *cosv, const float *sinv,
                   const uint32_t *rope_pos, const uint32_t *kv_pos, const uint32_t *seq_ids, const uint32_t *block_table,
                   uint32_t bpr, void *qh, void *gate, void *k_pool, void *v_pool, uint32_t tokens, uint32_t q_heads,
                   uint32_t kv_heads, uint32_t head_dim, uint32_t rot_dim, float eps, cudaStream_t st);
int32_t wb_mtp_cat(const uint32_t *tok, uint32_t tok_stride, const void *embed, const void *hid, const uint32_t *hid_rows,
                   const void *pre_e, const void *pre_h, void *cat, uint32_t rows, uint32_t hidden, float eps, cudaStream_t st);
int32_t wb_silu_mul_rows(const void *gu, uint32_t ld, void *out, uint32_t rows, uint32_t inter, cudaStream_t st);
int32_t wb_argmax_finish(const void *part, uint32_t split, uint32_t *out, uint32_t out_mul, uint32_t out_off, uint32_t s, cudaStream_t st);
int32_t wb_rms_norm_gated_rows(const void *x, const void *z, uint32_t z_tok_stride, const float *w, void *out, uint32_t tokens,
                               uint32_t heads, uint32_t hidden, float eps, cudaStream_t st);
int32_t wb_gdn_layer(const void *proj, uint32_t ld, const void *conv_w, void *conv_state, const void *a_log, const void *dt_bias,
                     const void *norm_w, void *state, uint32_t state_f32, void *out, const void *row_start, const void *row_count,
                     const void *in_row, const void *out_base, uint32_t n_rows, uint32_t k_heads, uint32_t v_heads, float l2_eps,
                     float rms_eps, void *log, void *kq_scratch, cudaStream_t st);  // log != null: no state snapshots, one update record per
                     // position; kq_scratch != null ([tokens, k_heads, 256] f32): large grids compute k-hat / q-hat once per k-head
int32_t wb_gdn_commit(void *const *states, const float *const *logs, uint32_t n_layers, uint32_t state_f32, const void *row_start,
                      const void *row_count, const void *in_row, const void *out_base, const void *accept_len, uint32_t n_rows,
                      uint32_t v_heads, cudaStream_t st);  // replays records 0..accept_len on row in_row, stores row out_base + accept_len
