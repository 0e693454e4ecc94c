/*
 * wein_b200.h -- C-ABI of libwein_b200.so: hand-written sm_100a kernels for wein's MTP speculative-decoding
 * hot path (draft k tokens with the MTP head -> verify k+1 positions in one forward -> accept on the device).
 *
 * Conventions
 *  - Every pointer is a DEVICE pointer unless its name starts with `host_`.  bf16 tensors are raw 16-bit
 *    words; index tables are uint32; nothing here is a torch / framework type.
 *  - `stream` is a CUstream / cudaStream_t passed as void*.  Every entry is stream-ordered, allocation-free
 *    after engine creation and safe to record into a CUDA graph unless stated otherwise.
 *  - Return value: 0 = ok, < 0 = rejected before any launch (see the WEIN_B200_ERR_* codes);
 *    wein_b200_last_error() returns the message of the calling thread's last failure.  Kernels never trap;
 *    in-band error values are documented per entry.
 *  - "reference" below is the wein source tree; each entry names the interface it stands in for.
 */
#ifndef WEIN_B200_H
#define WEIN_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define WEIN_B200_OK 0
#define WEIN_B200_ERR_ARG (-1)
#define WEIN_B200_ERR_SHAPE (-2)
#define WEIN_B200_ERR_CUDA (-3)
#define WEIN_B200_ERR_CAPACITY (-4)

/* Device status word of a sequence slot: bits OR-ed in by kernels when a round meets an anomaly (the pattern of the reference's
 * in-band sampler error, kernels/src/lib.rs:8197-8202).  Kernels clamp and flag; they never trap and never touch memory
 * outside what the slot was admitted with.  Read with wein_b200_engine_status or in the last word of each read_round row. */
#define WEIN_B200_STATUS_POS_LIMIT 1u  /* the slot sat a round out: position + 1 would pass its position limit */
#define WEIN_B200_STATUS_K_CLAMPED 2u  /* fewer drafts than asked were verified: the chain would have passed the limit */
#define WEIN_B200_STATUS_CTX_BOUND 4u  /* ctx_bound was below position + chain length: attention ignored later segments */
#define WEIN_B200_STATUS_SAMPLER 8u    /* the sampler met an invalid parameter */

const char *wein_b200_last_error(void);
uint32_t wein_b200_abi_version(void);

/* ------------------------------------------------------------------------------------------------------
 * Operator level: one entry per Op trait of crates/wein-kernel/src/ops/mod.rs on the path, same argument
 * order (DevBuf -> pointer, &Stream -> stream).
 * ---------------------------------------------------------------------------------------------------- */

/* EmbedOp::run (ops/mod.rs:286-307): out[t,:] = w[ids[t],:] */
int32_t wein_b200_embed(const void *ids, const void *w, void *out, uint32_t hidden, uint32_t tokens, void *stream);

/* RmsNormZcOp::run (ops/mod.rs:376-515): out = x * rsqrt(mean(x^2)+eps) * (1+w); in place allowed */
int32_t wein_b200_rms_norm_zc(const void *x, const void *w, void *out, uint32_t rows, uint32_t hidden, float eps, void *stream);

/* AddNormZcOp::run (ops/mod.rs:376-515, kernel kernels/src/lib.rs:4674): sum_out = bf16(a+b); norm_out = norm_zc(sum_out) */
int32_t wein_b200_add_norm_zc(const void *a, const void *b, const void *w, void *sum_out, void *norm_out, uint32_t rows,
                              uint32_t hidden, float eps, void *stream);

/* RmsNormGatedOp::run (ops/mod.rs:1308-1327): norm(x) * w_f32 * silu(z), rows of `hidden` */
int32_t wein_b200_rms_norm_gated(const void *x, const void *z, const void *w, void *out, uint32_t rows, uint32_t hidden,
                                 float eps, void *stream);

/* RopePtOp::run (ops/mod.rs:657-702): partial rotary on the first rot_dim dims; cos/sin f32 tables [max_pos, rot_dim/2] */
int32_t wein_b200_rope_pt(const void *x, const void *cosv, const void *sinv, const void *pos, void *out, uint32_t rot_dim,
                          uint32_t head_dim, uint32_t heads, uint32_t tokens, void *stream);

/* AddOp / MulOp / SiluOp / SiluMulOp / SigmulOp (ops/mod.rs:286-372, :705-725) */
int32_t wein_b200_add(const void *a, const void *b, void *out, uint64_t n, void *stream);
int32_t wein_b200_mul(const void *a, const void *b, void *out, uint64_t n, void *stream);
int32_t wein_b200_silu(const void *x, void *out, uint64_t n, void *stream);
int32_t wein_b200_silu_mul(const void *g, const void *u, void *out, uint64_t n, void *stream);
int32_t wein_b200_sigmul(const void *x, const void *g, void *out, uint64_t n, void *stream);

/* KvScatterOp::run / run_f32 (ops/mod.rs:1588-1680) */
int32_t wein_b200_kv_scatter(const void *src_k, const void *src_v, const void *block_table, const void *seq_ids,
                             const void *positions, void *k_dst, void *v_dst, uint32_t bpr, uint32_t block_size,
                             uint32_t head_elems, uint32_t tokens, void *stream);
int32_t wein_b200_kv_scatter_f32(const void *src_k, const void *src_v, const void *block_table, const void *seq_ids,
                                 const void *positions, void *k_dst, void *v_dst, uint32_t bpr, uint32_t block_size,
                                 uint32_t head_elems, uint32_t tokens, void *stream);

/* Conv1dDwOp::run (ops/mod.rs:727-741) and ConvStateRollOp::run (ops/mod.rs:827-843, per-span `specs`) */
int32_t wein_b200_conv1d_dw(const void *x, const void *w, const void *state_in, void *out, const void *tok_row,
                            const void *tok_pos, uint32_t conv_dim, uint32_t kernel, uint32_t tokens, void *stream);
int32_t wein_b200_conv_state_roll(const void *x, void *state, const void *row_start, const void *row_count, const void *row_id,
                                  uint32_t conv_dim, uint32_t kernel, uint32_t n_rows, const void *specs, void *stream);
/* Both of the above in one launch for chain spans: span r reads state row in_row[r] and writes the window after its
 * token t to row out_base[r]+t (the reference contract is out_base = in_row + 1).  x rows are x_stride elements apart. */
int32_t wein_b200_conv_verify(const void *x, uint32_t x_stride, const void *w, void *state, void *out, const void *row_start,
                              const void *row_count, const void *in_row, const void *out_base, uint32_t conv_dim,
                              uint32_t kernel, uint32_t n_rows, void *stream);

/* DeltanetOp::run (ops/mod.rs:888-919), bf16 state pool [rows, v_heads, 128, 128]; k_dim = v_dim = 128 only
 * (WEIN_B200_ERR_SHAPE otherwise).  The l2-norm pre-kernel of the reference is folded in. */
int32_t wein_b200_deltanet(const void *q, const void *k, const void *v, const void *a, const void *b, const void *a_log,
                           const void *dt_bias, void *state, void *core_out, const void *row_start, const void *row_count,
                           const void *row_id, uint32_t n_rows, uint32_t k_heads, uint32_t v_heads, uint32_t k_dim,
                           uint32_t v_dim, uint32_t tokens, float l2_eps, const void *specs, uint32_t vsplit, void *stream);
/* The verify-shaped form: the state of each (span, head) is read once, advanced on chip over the span's tokens and
 * written once per position.  q/k/v/a/b are read in place with the given token strides (elements); span r reads row
 * in_row[r] and writes the state after token t to row out_base[r]+t (specs[r] != 0 or specs == NULL) or only the final
 * state to row out_base[r] (specs[r] == 0).  state_f32: pool element type (0 = bf16 rounded on every store, the
 * reference's pool; 1 = f32).  rows_per_warp: 0 (auto), 8, 16 or 32; it never changes a result bit. */
int32_t wein_b200_gdn_verify(const void *q, const void *k, const void *v, uint32_t q_stride, uint32_t k_stride, uint32_t v_stride,
                             const void *a, const void *b, uint32_t ab_stride, const void *a_log, const void *dt_bias,
                             void *state, uint32_t state_f32, void *core_out, const void *row_start, const void *row_count,
                             const void *in_row, const void *out_base, const void *specs, uint32_t n_rows, uint32_t k_heads,
                             uint32_t v_heads, uint32_t k_dim, uint32_t v_dim, float l2_eps, uint32_t rows_per_warp, void *stream);

/* The whole token mixer of a gated-DeltaNet layer for chain spans of <= 8 tokens in one launch: conv1d_dw + conv_state_roll +
 * dn_split_qkv + dn_qk_l2norm + deltanet + rms_norm_gated of the reference's layer (crates/wein-exec/src/qwen.rs:3971-4077), same
 * values bit for bit.  proj [tokens, ld] = raw qkv (2*k_heads*128 + v_heads*128) | z (v_heads*128) | a (v_heads) | b (v_heads);
 * out [tokens, v_heads*128] = gated-normalised core output.  Span r reads conv / recurrent state row in_row[r] and writes the
 * rows after its token t to out_base[r]+t in both pools. */
int32_t wein_b200_gdn_layer(const void *proj, uint32_t ld, const void *conv_w, void *conv_state, const void *a_log,
                            const void *dt_bias, const void *norm_w, void *state, uint32_t state_f32, void *out,
                            const void *row_start, const void *row_count, const void *in_row, const void *out_base,
                            uint32_t n_rows, uint32_t k_heads, uint32_t v_heads, float l2_eps, float rms_eps, void *stream);

/* Snapshot-lite pair.  No counterpart in the reference's operator set: the reference writes a full state row per verify
 * position (DeltanetOp::run with per-position rows, ops/mod.rs:886-1050) and names this scheme as the next step for its
 * speculative commit (crates/wein-exec/src/qwen.rs:5480-5624).
 * gdn_layer_lite: as gdn_layer, but the recurrent state pool is only READ (row in_row[r]); instead of state rows it writes one
 *   record per (token, v-head) to log [tokens, v_heads, 264] f32 (16-byte aligned): delta[128] | k-hat[128] | decay | pad.  Conv
 *   state rows and `out` are written exactly as by gdn_layer.
 * gdn_commit: for every span r and every head of n_layers layers, replays records 0..a (a = min(accept_len[r], row_count[r]-1))
 *   on state row in_row[r] and stores row out_base[r] + a: bit for bit the row gdn_layer would have written there.  `states`
 *   and `logs` are DEVICE arrays of n_layers device pointers (state pools / logs of the layers). */
int32_t wein_b200_gdn_layer_lite(const void *proj, uint32_t ld, const void *conv_w, void *conv_state, const void *a_log,
                                 const void *dt_bias, const void *norm_w, const void *state, uint32_t state_f32, void *out,
                                 const void *row_start, const void *row_count, const void *in_row, const void *out_base,
                                 uint32_t n_rows, uint32_t k_heads, uint32_t v_heads, float l2_eps, float rms_eps, void *log,
                                 void *stream);
/* gdn_layer / gdn_layer_lite in one entry: log may be null (state snapshots), kq_scratch may be null.  kq_scratch (f32,
 * 16-byte aligned, tokens x v_heads x 388 words, sized by the caller for every token row of the call) lets calls with at
 * least 296 (span, v-head) pairs -- and 16-byte aligned proj / state, ld a multiple of 8 -- run the large-grid kernel: a
 * launch of its own makes the per-token operands (conv + SiLU, l2 norms, k-hat / q-hat, gates) once per span, and persistent
 * CTAs stream the heads' states through shared memory one item ahead.  Results are identical; the scratch contents after
 * the call are unspecified. */
int32_t wein_b200_gdn_layer_ws(const void *proj, uint32_t ld, const void *conv_w, void *conv_state, const void *a_log,
                               const void *dt_bias, const void *norm_w, void *state, uint32_t state_f32, void *out,
                               const void *row_start, const void *row_count, const void *in_row, const void *out_base,
                               uint32_t n_rows, uint32_t k_heads, uint32_t v_heads, float l2_eps, float rms_eps, void *log,
                               void *kq_scratch, void *stream);
/* Copy waits of the large-grid layer kernel that ran into their time limit since the library was loaded (0 in a healthy
 * run; a non-zero count means a launch's results were abandoned, not that a kernel hung).  Synchronises the device. */
int32_t wein_b200_gdn_wait_timeouts(uint32_t *out);
int32_t wein_b200_gdn_commit(const void *states, const void *logs, uint32_t n_layers, uint32_t state_f32, const void *row_start,
                             const void *row_count, const void *in_row, const void *out_base, const void *accept_len,
                             uint32_t n_rows, uint32_t v_heads, void *stream);

/* PagedAttnOp::run (ops/mod.rs:1687-1704) plus the scratch buffer that the reference's op object owns privately
 * (wein_b200_attn_scratch_bytes(tokens, kv_heads, head_dim, 16) bytes).  16-token pages; head_dim 64 / 128 / 256. */
uint64_t wein_b200_attn_scratch_bytes(uint32_t n_spans, uint32_t kv_heads, uint32_t head_dim, uint32_t max_segs);
int32_t wein_b200_paged_attn(const void *q, const void *k_cache, const void *v_cache, const void *block_table, const void *seq_ids,
                             const void *positions, void *out, float q_scale, uint32_t bpr, uint32_t block_size, uint32_t q_heads,
                             uint32_t kv_heads, uint32_t head_dim, uint32_t tokens, void *scratch, uint64_t scratch_bytes, void *stream);
/* Verify attention (stands in for Qwen35Executor::attn_long on chain rows, crates/wein-exec/src/qwen.rs:1134-1422): span r =
 * rows row_start[r] .. +row_count[r] of one sequence at consecutive positions (<= 32 / group rows).  max_ctx bounds
 * position+1 over the call (sizes the grid only); seg_pages = pages per context segment (fixes the summation order: keep it
 * constant between runs that must agree bit for bit); gate (optional) applies out = sigmul(attn, gate).
 * scratch >= wein_b200_attn_scratch_bytes(n_spans, kv_heads, head_dim, ceil(ceil(max_ctx/16)/seg_pages)).
 * status (optional): u32 words indexed by sequence id; when max_ctx is below a row's position + 1 the row is reduced over the
 * segments the grid covers only (no slot that nobody wrote is read) and WEIN_B200_STATUS_CTX_BOUND is OR-ed into its word. */
int32_t wein_b200_attn_verify(const void *q, const void *k_cache, const void *v_cache, const void *block_table, const void *seq_ids,
                              const void *positions, const void *row_start, const void *row_count, const void *gate, void *out,
                              float q_scale, uint32_t bpr, uint32_t block_size, uint32_t q_heads, uint32_t kv_heads, uint32_t head_dim,
                              uint32_t n_spans, uint32_t max_count, uint32_t max_ctx, uint32_t seg_pages, void *scratch,
                              uint64_t scratch_bytes, void *status, void *stream);

/* GemmOp::run_wt (ops/mod.rs:3378-3449): C[m,n] = A[m,k] W[n,k]^T, bf16, f32 accumulate; k a multiple of 32, operands 16-byte
 * aligned.  Two hand-written weight-streaming kernels, no library call (the reference sends m > 1 to cuBLASLt,
 * cuda/cublaslt.rs:249-257): m <= 32 runs the register-streaming mma.sync kernel, larger m the tensor-memory kernel
 * (tcgen05.mma with the tokens as the M operand and a tile of 80 - 256 weight rows as N, tensor-map bulk copies, k split over a
 * thread-block cluster for narrow n).  In both
 * the result of a row does not depend on the other rows of the call; the two kernels do not agree with each other bit for bit,
 * so forwards that must agree across row counts use the _tc entries (the tensor-memory kernel at every m) throughout.
 * scratch is optional and may be null (reserved for a split-k mode of the m <= 32 kernel). */
uint64_t wein_b200_gemm_scratch_bytes(uint32_t n_max);
int32_t wein_b200_gemm_wt(const void *a, const void *w, void *c, uint32_t m, uint32_t n, uint32_t k, void *scratch,
                          uint64_t scratch_bytes, void *stream);
int32_t wein_b200_gemm_wt_tc(const void *a, const void *w, void *c, uint32_t m, uint32_t n, uint32_t k, void *stream);
/* Gate|up projection with the SwiGLU activation in the epilogue (GemmOp::run_wt x2 + SiluMulOp of the reference's MLP,
 * crates/wein-exec/src/qwen.rs:4090-4099): w_gate_up = [gate; up] of shape [2*inter, k]; out[m, inter] holds exactly the
 * values silu_mul produces from the two separately rounded projections of the same kernel. */
int32_t wein_b200_gemm_swiglu(const void *a, const void *w_gate_up, void *out, uint32_t m, uint32_t inter, uint32_t k,
                              void *scratch, uint64_t scratch_bytes, void *stream);
int32_t wein_b200_gemm_swiglu_tc(const void *a, const void *w_gate_up, void *out, uint32_t m, uint32_t inter, uint32_t k,
                                 void *stream);
/* How the tensor-memory kernel runs a product of m rows with an [n, k] weight matrix (swiglu != 0: [2n, k] = gate | up) on the
 * current device: out[5] = CTAs, k split (thread-block cluster size), pipeline stages, shared-memory bytes per CTA, weight rows
 * per tile.  The k split, which fixes the summation order, depends on (n, k) and the device only. */
int32_t wein_b200_gemm_plan(uint32_t m, uint32_t n, uint32_t k, uint32_t swiglu, uint32_t *out);
/* Barrier waits of the tensor-memory kernel that ran into their time limit since the library was loaded (0 in a healthy
 * run; a non-zero count means a result was abandoned, not that a kernel hung).  Synchronises the device. */
int32_t wein_b200_gemm_wait_timeouts(uint32_t *out);

/* Fused glue of the forward passes; each writes, bit for bit, what the operator chain it replaces writes.
 * qk_prep: row t of qgkv (stride ld) = [q_heads x (q | gate) x head_dim | k | v]; replaces the q / gate de-interleave
 *   (2 x EmbedOp), RmsNormZcOp on the q and k heads, 2 x RopePtOp and KvScatterOp of a full-attention layer
 *   (crates/wein-exec/src/qwen.rs:3888-3950): qh, gate [tokens, q_heads, head_dim]; K / V rows go to page slot
 *   block_table[seq_ids[t]][kv_pos[t] / 16] * 16 + kv_pos[t] % 16.  rope_pos indexes the cos / sin tables [*, rot_dim / 2] f32.
 * mtp_cat: cat[r] = [norm_zc(embed[tok[r]], pre_e) | norm_zc(hid[hid_rows ? hid_rows[r] : r], pre_h)], the input of the MTP
 *   head's fc (2 gathers, 2 x RmsNormZcOp and a row copy in the reference, qwen.rs:4451-4468).
 * silu_mul_rows: SiluMulOp over rows that hold gate | up side by side (row stride ld >= 2 * inter). */
int32_t wein_b200_qk_prep(const void *qgkv, uint32_t ld, const void *qn, const void *kn, const void *cosv, const void *sinv,
                          const void *rope_pos, const void *kv_pos, const void *seq_ids, const void *block_table, uint32_t bpr,
                          void *qh, void *gate, void *k_pool, void *v_pool, uint32_t tokens, uint32_t q_heads, uint32_t kv_heads,
                          uint32_t head_dim, uint32_t rot_dim, float eps, void *stream);
int32_t wein_b200_mtp_cat(const void *tok, const void *embed, const void *hid, const void *hid_rows, const void *pre_e,
                          const void *pre_h, void *cat, uint32_t rows, uint32_t hidden, float eps, void *stream);
int32_t wein_b200_silu_mul_rows(const void *gu, uint32_t ld, void *out, uint32_t rows, uint32_t inter, void *stream);

/* ArgmaxRowsOp::run (ops/mod.rs:1332-1367): total order (value desc, index asc); scratch = s*32 u64 words;
 * a row with no comparable element yields 0xFFFFFFFF, as the reference. */
int32_t wein_b200_argmax_rows(const void *x, const void *rows, void *scratch, void *out, uint32_t n, uint32_t s, void *stream);

/* No counterpart in the reference.  wein_b200_argmax_rows for callers that cannot allocate device memory (a plugin that only
 * receives one call's tensors; code inside a graph-capture region or under a memory pool it does not own): the slice maxima
 * live in a 64 KiB array built into the library (held by every GPU that loads it) instead of a caller buffer.  At most 256
 * rows per call (WEIN_B200_ERR_CAPACITY beyond).  The first call on each device looks the array's address up on the host:
 * make it outside any stream capture.  All calls on a device share the array: calls that may overlap on the GPU race.  The
 * looked-up address is kept per device ordinal (ordinals >= 64 are refused with WEIN_B200_ERR_CUDA) without a lock -- two
 * threads making the first call together store the same value -- and does not survive a cudaDeviceReset of that device. */
int32_t wein_b200_argmax_rows_noalloc(const void *x, const void *rows, void *out, uint32_t n, uint32_t s, void *stream);

/* SampleRowsOp::run (ops/mod.rs:1379-1393): temperature / top-k (<= 64) / top-p sampler with one PCG-XSH-RR state per slot in
 * `rng` (0 = derive from the row's seed), per-row parameters; temp <= 0 -> argmax; top_k == 0 -> 0xFFFFFFFF (in-band). */
int32_t wein_b200_sample_rows(const void *x, const void *rows, const void *slots, const void *temp, const void *top_k, const void *top_p,
                              const void *seed, void *rng, void *out, uint32_t n, uint32_t s, void *stream);

/* ------------------------------------------------------------------------------------------------------
 * Acceptance (stands in for Qwen35Executor::spec_finish, crates/wein-exec/src/qwen.rs:2419-2502, which runs on the
 * host after a sync and a readback in the reference).
 * ---------------------------------------------------------------------------------------------------- */

/* Greedy: argmax of the B*(k+1) verify rows rows[b*(k+1)+j] of `logits` [*, n], then accept while drafts[b][a] == target[b][a];
 * out_tokens[b] = accepted drafts followed by the bonus token target[b][a], padded with 0xFFFFFFFF.  n_drafts (optional)
 * gives per-sequence draft counts <= k.  scratch = B*(k+1)*32 u64 words.  target (optional) receives the argmax tokens. */
int32_t wein_b200_accept_greedy(const void *logits, const void *rows, const void *drafts, const void *n_drafts, uint32_t n,
                                uint32_t B, uint32_t k, void *scratch, void *accept_len, void *out_tokens, void *target, void *stream);

/* Temperature / top-k (<= 64) / top-p filter of one logits row into a compact distribution: out_ids / out_probs [s, 64],
 * out_n [s].  The filter follows SampleRowsOp (ops/mod.rs:1374-1441, reference.rs:787-877); probabilities are renormalised
 * over the kept entries.  Row r uses the parameters of sequence row_seq[r] (or r / rows_per_seq).  temp <= 0 yields the
 * one-hot argmax; top_k == 0 yields out_n = 0 and ids 0xFFFFFFFF (in-band error, as the reference sampler).  If sample_out
 * is given, a token is drawn from each row's distribution with Philox4x32-10 uniforms keyed by (seed, round, position). */
int32_t wein_b200_topk_filter(const void *logits, const void *rows, const void *row_seq, uint32_t rows_per_seq, const void *temp,
                              const void *top_k, const void *top_p, uint32_t n, uint32_t s, void *out_ids, void *out_probs,
                              void *out_n, void *sample_out, const void *seed, const void *round, uint32_t position, void *stream);

/* Rejection sampling over compact distributions: p_* of the B*(k+1) verify rows, q_* of the B*k draft rows ([B][k]).
 * Sequences with temp <= 0 follow the greedy rule on entry 0 of their rows.  No counterpart in the reference. */
int32_t wein_b200_accept_sampled(const void *drafts, const void *n_drafts, const void *p_ids, const void *p_probs, const void *p_n,
                                 const void *q_ids, const void *q_probs, const void *q_n, const void *temp, const void *seed,
                                 const void *round, uint32_t B, uint32_t k, void *accept_len, void *out_tokens, void *stream);

/* ------------------------------------------------------------------------------------------------------
 * Step level: the speculative step of Qwen35Executor (crates/wein-exec/src/qwen.rs:5225-5654: spec_draft_batch ->
 * forward_batch_mixed -> spec_finish) with every per-round decision on the device, so that one round is a single
 * CUDA-graph replay with no host synchronisation.
 * ---------------------------------------------------------------------------------------------------- */

#define WEIN_B200_MAX_LAYERS 64

typedef struct {
    /* Qwen35Config (crates/wein-model/src/config.rs:17-46) */
    uint32_t hidden, n_layers, q_heads, kv_heads, head_dim, rot_dim, inter, vocab;
    uint32_t lin_k_heads, lin_v_heads, lin_k_dim, lin_v_dim, conv_kernel;
    float rms_eps, l2_eps;
    double rope_theta;
    uint8_t layer_is_full[WEIN_B200_MAX_LAYERS];
    uint32_t has_mtp;
    /* capacity (CtxConfig of crates/wein-exec/src/ctx.rs) */
    uint32_t max_seqs;       /* sequence slots */
    uint32_t k_max;          /* most drafts per round (<= 7); chains and prefill chunks hold k_max+1 rows */
    uint32_t max_pos;        /* positions per sequence (block-table rows hold ceil(max_pos/16) pages) */
    uint32_t n_pages;        /* 16-token pages per KV pool */
    uint32_t state_f32;      /* recurrent state pool: 1 = f32, 0 = bf16 (the reference's pool) */
    uint32_t attn_seg_pages; /* pages per attention segment (0 = chosen from max_pos: 4 ... 128) */
    uint32_t state_snapshots;/* 0: rounds of >= 3 positions log their state updates and materialise the accepted row once;
                                1: every round writes one recurrent-state row per verify position (the reference's scheme) */
} wein_b200_model_cfg;

/* Weights stay caller-owned device memory for the life of the engine (bf16 unless noted; layouts as the safetensors
 * tensors the reference uploads, crates/wein-exec/src/qwen.rs:1483-1579).  When the projection matrices of a layer are
 * adjacent in memory in the order qkv|z|a|b, qg|k|v and wg|wu, the engine multiplies them in one launch each. */
typedef struct {
    const void *ln1, *ln2;            /* [hidden] */
    const void *wg, *wu, *wd;         /* [inter,hidden] x2, [hidden,inter] */
    /* full-attention layer */
    const void *qg, *k, *v;           /* [2*q_heads*head_dim, hidden] (per head q then gate), [kv_heads*head_dim, hidden] x2 */
    const void *qn, *kn, *o;          /* [head_dim] x2, [hidden, q_heads*head_dim] */
    /* gated-DeltaNet layer */
    const void *qkv, *z, *a, *b;      /* [2*kh*kd+vh*vd, hidden], [vh*vd, hidden], [vh, hidden] x2 */
    const void *conv;                 /* [conv_dim, conv_kernel] */
    const void *a_log;                /* f32 [vh] */
    const void *dt_bias;              /* [vh] */
    const void *norm;                 /* f32 [vd] */
    const void *out;                  /* [hidden, vh*vd] */
} wein_b200_layer_weights;

typedef struct {
    const void *embed;                /* [vocab, hidden], tied lm_head */
    const void *norm_f;               /* [hidden] */
    wein_b200_layer_weights layers[WEIN_B200_MAX_LAYERS];
    /* MTP head (crates/wein-exec/src/qwen.rs:1537-1579): pre-norms, fc [hidden, 2*hidden], one full-attention layer, norm */
    const void *mtp_pre_e, *mtp_pre_h, *mtp_fc, *mtp_norm;
    wein_b200_layer_weights mtp_layer;
} wein_b200_weights;

typedef struct wein_b200_engine wein_b200_engine;

/* Allocates pools (recurrent / conv state rows, KV pages), scratch and tables.  create, warm and the first call of a round
 * shape (which captures its CUDA graph) are the only entries that allocate; every forward of an engine whose largest forward
 * (max_seqs x (k_max+1) rows) exceeds 32 rows multiplies on the tensor-memory GEMM at every row count, smaller engines on
 * the m <= 32 kernel, so that plain, draft and verify forwards of one engine sum in one order. */
int32_t wein_b200_engine_create(const wein_b200_model_cfg *cfg, const wein_b200_weights *weights, wein_b200_engine **out);
void wein_b200_engine_destroy(wein_b200_engine *e);
uint64_t wein_b200_engine_device_bytes(const wein_b200_engine *e);

/* Admission of a sequence into a slot: zeroes its state rows, installs its block-table row (host_pages: n_pages page
 * ids) and its sampling parameters (SampleParams of crates/wein-engine/src/protocol.rs:50-76; temp <= 0 = greedy).  The slot's
 * position limit becomes min(max_pos, 16 * n_pages): no round reads or writes a position at or past it (see the status bits). */
int32_t wein_b200_engine_admit(wein_b200_engine *e, uint32_t slot, const uint32_t *host_pages, uint32_t n_pages, float temp,
                               uint32_t top_k, float top_p, uint64_t seed, void *stream);

/* Per-request draft length (Qwen35Executor::set_spec, crates/wein-exec/src/qwen.rs:2604-2647): later rounds verify
 * min(round k, k) drafts for this slot; 0 makes it a plain decode row inside a speculative round (the mixed batch of
 * qwen.rs:5295-5361).  Admission resets it to "whatever the round drafts".  Stream-ordered. */
int32_t wein_b200_engine_set_spec(wein_b200_engine *e, uint32_t slot, uint32_t k, void *stream);

/* A sequence that does not start at position 0 (a prefix-cache hit: the reference restores KV pages and a recurrent-state
 * snapshot from its radix cache, qwen.rs:3056-3100): after admit, the caller writes the first `position` tokens' K / V into
 * the slot's pages and the state after them into row 2 * (k_max + 1) * slot of every "lin_state:<i>" / "conv_state:<i>" pool
 * (wein_b200_engine_buffer), then names the position and the token to feed next.  The stashed hidden of the MTP head starts
 * at zero.  Stream-ordered. */
int32_t wein_b200_engine_resume(wein_b200_engine *e, uint32_t slot, uint32_t position, uint32_t pending_token, void *stream);

/* Prefill: feeds host_lens[i] prompt tokens of slot host_slots[i] (tokens concatenated in host_tokens) through the verify
 * forward in chunks of k_max+1 positions starting at the slot's current position, then emits each sequence's next token.
 * WEIN_B200_ERR_CAPACITY when a prompt does not fit below the slot's position limit.  Not graph-captured; synchronises. */
int32_t wein_b200_engine_prefill(wein_b200_engine *e, uint32_t n, const uint32_t *host_slots, const uint32_t *host_tokens,
                                 const uint32_t *host_lens, void *stream);

/* One round for the slots host_slots[0..n): draft k tokens with the MTP head (k = 0: plain decode step), verify the k+1
 * positions in one forward, accept on the device, commit (position, pending token, state row, hidden, token ring).
 * ctx_bound = an upper bound of (position + k + 1) over the batch; it sizes the attention grid (an understated bound is
 * flagged in the status word, never a memory error).  use_graph bit 0 replays a CUDA graph cached per (n, k, sampling mode,
 * ctx bucket), captured on first use or by wein_b200_engine_warm; bit 1 forces the upload of the slot table even when it
 * is unchanged.  No host synchronisation unless the slot table changes. */
int32_t wein_b200_engine_spec_step(wein_b200_engine *e, uint32_t n, const uint32_t *host_slots, uint32_t k, uint32_t ctx_bound,
                                   uint32_t use_graph, void *stream);

/* The draft phase alone (Qwen35Executor::spec_draft_batch, qwen.rs:2748-2853): k MTP forwards with the hidden chained on the
 * device.  drafts_out (optional, DEVICE, [n, k] u32) receives the drafts; they also stay in the engine, with their
 * distributions in sampled mode, for a following spec_verify with WEIN_B200_VERIFY_ENGINE_DRAFTS. */
int32_t wein_b200_engine_draft(wein_b200_engine *e, uint32_t n, const uint32_t *host_slots, uint32_t k, void *drafts_out,
                               uint32_t use_graph, void *stream);

/* Verify + accept + commit with the caller's drafts (Qwen35Executor::spec_verify / spec_commit_batch(&[(ReqId, Vec<u32>)]),
 * qwen.rs:2261-2303).  DEVICE arrays: drafts [n, k] u32; n_drafts [n] (optional, ragged chains: row b verifies
 * min(n_drafts[b], k, the slot's set_spec value) drafts); q_ids / q_probs [n, k, 64] and q_n [n, k] (optional, all three or
 * none): the distributions the drafts were drawn from, as compact lists in the layout of wein_b200_topk_filter -- without
 * them a sampled slot treats each draft as drawn from a point mass.  A draft id outside the vocabulary is rejected like any
 * wrong draft. */
#define WEIN_B200_VERIFY_GRAPH 1u          /* replay a CUDA graph (as use_graph of spec_step) */
#define WEIN_B200_VERIFY_FORCE_SLOTS 2u    /* upload the slot table even when unchanged */
#define WEIN_B200_VERIFY_DRY_RUN 4u        /* decide but commit nothing: slot state, token ring, counters and committed rows stay */
#define WEIN_B200_VERIFY_ENGINE_DRAFTS 8u  /* use the drafts (and distributions) a preceding wein_b200_engine_draft left */
int32_t wein_b200_engine_spec_verify(wein_b200_engine *e, uint32_t n, const uint32_t *host_slots, uint32_t k, const void *drafts,
                                     const void *n_drafts, const void *q_ids, const void *q_probs, const void *q_n,
                                     uint32_t ctx_bound, uint32_t flags, void *stream);

/* Captures and instantiates the graphs later calls with the same (n, k, sampling mode of the slots, ctx bucket) replay, so
 * that those calls allocate nothing (the reference warms its graphs at open_graph, qwen.rs:1994-2034).  what: bit 0
 * spec_step, bit 1 spec_verify, bit 2 spec_verify as a dry run, bit 3 engine_draft.  The slots must be admitted. */
int32_t wein_b200_engine_warm(wein_b200_engine *e, uint32_t n, const uint32_t *host_slots, uint32_t k, uint32_t ctx_bound,
                              uint32_t what, void *stream);

/* The readback of a round for the whole batch in one copy (the reference reads back its [B*P] argmax table once per step,
 * forward_batch_mixed, qwen.rs:3453-3703): host_out [n, 4 + k_max + 1] u32 = per batch row of the most recent round the
 * accept length a, the position, the tokens emitted since admission, the round's a + 1 tokens (other words 0xFFFFFFFF; no
 * token for a slot that sat the round out), then the slot's status word.  Synchronises the stream. */
int32_t wein_b200_engine_read_round(wein_b200_engine *e, uint32_t *host_out, uint32_t host_words, void *stream);

/* Synchronises the stream and reads a slot: the most recent min(cap, emitted) tokens (oldest first), the number of
 * tokens emitted since admission (host_n_tokens), the position, and the first three counters of
 * spec_stats() (crates/wein-exec/src/qwen.rs:4257-4259): rounds, drafts, accepted. */
int32_t wein_b200_engine_read(wein_b200_engine *e, uint32_t slot, uint32_t *host_tokens, uint32_t cap, uint32_t *host_n_tokens,
                              uint32_t *host_pos, uint64_t *host_stats3, void *stream);

/* All speculation counters of a slot since admission (spec_stats / spec_k_stats, qwen.rs:4257-4259, :2670):
 * host_stats[WEIN_B200_STATS_WORDS] = rounds, drafts, accepted, fallbacks (rounds cut or refused at the position limit),
 * draft-length switches, rounds by draft count [8], rounds by accept length [9], last draft count, spare.  Synchronises. */
#define WEIN_B200_STATS_WORDS 24
int32_t wein_b200_engine_stats(wein_b200_engine *e, uint32_t slot, uint64_t *host_stats, void *stream);

/* Status word of a slot (WEIN_B200_STATUS_*); clear != 0 resets it after the read.  Synchronises the stream. */
int32_t wein_b200_engine_status(wein_b200_engine *e, uint32_t slot, uint32_t *host_status, uint32_t clear, void *stream);

/* Phase timers (spec_timing_ms, qwen.rs:4277-4279): while on, rounds run without a graph record device events around the
 * draft phase, the verify forward and acceptance + commit; host_ms3 (optional) receives the totals in milliseconds. */
int32_t wein_b200_engine_timing(wein_b200_engine *e, uint32_t on, double *host_ms3);

/* Test / profiling access to engine-owned device buffers by name ("logits", "x", "accept_len", "state_row", "lin_state:<i>",
 * "k_pool:<i>", ...): returns the device pointer and its size in bytes, or NULL. */
void *wein_b200_engine_buffer(wein_b200_engine *e, const char *name, uint64_t *bytes);
/* Kernel launches recorded by the most recent round (eager) or captured in the graph it replayed. */
uint32_t wein_b200_engine_last_launches(const wein_b200_engine *e);

#ifdef __cplusplus
}
#endif
#endif /* WEIN_B200_H */
