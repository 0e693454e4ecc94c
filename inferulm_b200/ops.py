"""Operator-level mirror of the reference's Op traits over the C-ABI.

One function per trait of crates/wein-kernel/src/ops/mod.rs that lies on the
MTP draft -> verify -> accept path, same argument order and meaning; tensors
are torch CUDA tensors used only as device buffers (bf16 data travels as
int16 / bf16 storage, u32 tables as int32).  Every call forwards raw device
pointers, sizes and the current CUDA stream to libwein_b200.so.
"""
import ctypes as C

import torch

from .lib import check, load

U32, U64, F32, VP = C.c_uint32, C.c_uint64, C.c_float, C.c_void_p


def _ptr(t):
    if t is None:
        return VP(0)
    assert t.is_cuda and t.is_contiguous(), "operators take contiguous CUDA tensors"
    return VP(t.data_ptr())


def _stream():
    return VP(torch.cuda.current_stream().cuda_stream)


def embed(ids, w, out, hidden, tokens):
    check(load().wein_b200_embed(_ptr(ids), _ptr(w), _ptr(out), U32(hidden), U32(tokens), _stream()))


def rms_norm_zc(x, w, out, rows, hidden, eps):
    check(load().wein_b200_rms_norm_zc(_ptr(x), _ptr(w), _ptr(out), U32(rows), U32(hidden), F32(eps), _stream()))


def add_norm_zc(a, b, w, sum_out, norm_out, rows, hidden, eps):
    check(load().wein_b200_add_norm_zc(_ptr(a), _ptr(b), _ptr(w), _ptr(sum_out), _ptr(norm_out), U32(rows), U32(hidden),
                                       F32(eps), _stream()))


def rms_norm_gated(x, z, w, out, rows, hidden, eps):
    check(load().wein_b200_rms_norm_gated(_ptr(x), _ptr(z), _ptr(w), _ptr(out), U32(rows), U32(hidden), F32(eps), _stream()))


def rope_pt(x, cos, sin, pos, out, rot_dim, head_dim, heads, tokens):
    check(load().wein_b200_rope_pt(_ptr(x), _ptr(cos), _ptr(sin), _ptr(pos), _ptr(out), U32(rot_dim), U32(head_dim),
                                   U32(heads), U32(tokens), _stream()))


def add(a, b, out, n):
    check(load().wein_b200_add(_ptr(a), _ptr(b), _ptr(out), U64(n), _stream()))


def mul(a, b, out, n):
    check(load().wein_b200_mul(_ptr(a), _ptr(b), _ptr(out), U64(n), _stream()))


def silu(x, out, n):
    check(load().wein_b200_silu(_ptr(x), _ptr(out), U64(n), _stream()))


def silu_mul(g, u, out, n):
    check(load().wein_b200_silu_mul(_ptr(g), _ptr(u), _ptr(out), U64(n), _stream()))


def sigmul(x, g, out, n):
    check(load().wein_b200_sigmul(_ptr(x), _ptr(g), _ptr(out), U64(n), _stream()))


def kv_scatter(src_k, src_v, block_table, seq_ids, positions, k_dst, v_dst, bpr, block_size, head_elems, tokens, f32=False):
    fn = load().wein_b200_kv_scatter_f32 if f32 else load().wein_b200_kv_scatter
    check(fn(_ptr(src_k), _ptr(src_v), _ptr(block_table), _ptr(seq_ids), _ptr(positions), _ptr(k_dst), _ptr(v_dst),
             U32(bpr), U32(block_size), U32(head_elems), U32(tokens), _stream()))


def conv1d_dw(x, w, state_in, out, tok_row, tok_pos, conv_dim, kernel, tokens):
    check(load().wein_b200_conv1d_dw(_ptr(x), _ptr(w), _ptr(state_in), _ptr(out), _ptr(tok_row), _ptr(tok_pos),
                                     U32(conv_dim), U32(kernel), U32(tokens), _stream()))


def conv_state_roll(x, state, row_start, row_count, row_id, conv_dim, kernel, n_rows, specs):
    check(load().wein_b200_conv_state_roll(_ptr(x), _ptr(state), _ptr(row_start), _ptr(row_count), _ptr(row_id),
                                           U32(conv_dim), U32(kernel), U32(n_rows), _ptr(specs), _stream()))


def conv_verify(x, x_stride, w, state, out, row_start, row_count, in_row, out_base, conv_dim, kernel, n_rows):
    check(load().wein_b200_conv_verify(_ptr(x), U32(x_stride), _ptr(w), _ptr(state), _ptr(out), _ptr(row_start),
                                       _ptr(row_count), _ptr(in_row), _ptr(out_base), U32(conv_dim), U32(kernel),
                                       U32(n_rows), _stream()))


def deltanet(q, k, v, a, b, a_log, dt_bias, state, core_out, row_start, row_count, row_id, n_rows, k_heads, v_heads,
             k_dim, v_dim, tokens, l2_eps, specs, vsplit):
    check(load().wein_b200_deltanet(_ptr(q), _ptr(k), _ptr(v), _ptr(a), _ptr(b), _ptr(a_log), _ptr(dt_bias), _ptr(state),
                                    _ptr(core_out), _ptr(row_start), _ptr(row_count), _ptr(row_id), U32(n_rows),
                                    U32(k_heads), U32(v_heads), U32(k_dim), U32(v_dim), U32(tokens), F32(l2_eps),
                                    _ptr(specs), U32(vsplit), _stream()))


def gdn_verify(q, k, v, q_stride, k_stride, v_stride, a, b, ab_stride, a_log, dt_bias, state, state_f32, core_out,
               row_start, row_count, in_row, out_base, specs, n_rows, k_heads, v_heads, k_dim, v_dim, l2_eps,
               rows_per_warp=0):
    check(load().wein_b200_gdn_verify(_ptr(q), _ptr(k), _ptr(v), U32(q_stride), U32(k_stride), U32(v_stride), _ptr(a),
                                      _ptr(b), U32(ab_stride), _ptr(a_log), _ptr(dt_bias), _ptr(state), U32(state_f32),
                                      _ptr(core_out), _ptr(row_start), _ptr(row_count), _ptr(in_row), _ptr(out_base),
                                      _ptr(specs), U32(n_rows), U32(k_heads), U32(v_heads), U32(k_dim), U32(v_dim),
                                      F32(l2_eps), U32(rows_per_warp), _stream()))


ARGMAX_SPLIT = 32


def argmax_rows(x, rows, scratch, out, n, s):
    """scratch: at least s * ARGMAX_SPLIT int64 words."""
    check(load().wein_b200_argmax_rows(_ptr(x), _ptr(rows), _ptr(scratch), _ptr(out), U32(n), U32(s), _stream()))


def paged_attn(q, k_cache, v_cache, block_table, seq_ids, positions, out, q_scale, bpr, block_size, q_heads, kv_heads,
               head_dim, tokens, scratch):
    """PagedAttnOp::run plus the scratch buffer the reference's op object owns (attn_scratch_bytes(tokens, kv_heads,
    head_dim, 16))."""
    sb = scratch.numel() * scratch.element_size()
    check(load().wein_b200_paged_attn(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), _ptr(seq_ids),
                                      _ptr(positions), _ptr(out), F32(q_scale), U32(bpr), U32(block_size), U32(q_heads),
                                      U32(kv_heads), U32(head_dim), U32(tokens), _ptr(scratch), U64(sb), _stream()))


def attn_scratch_bytes(n_spans, kv_heads, head_dim, max_segs):
    fn = load().wein_b200_attn_scratch_bytes
    fn.restype = U64
    return int(fn(U32(n_spans), U32(kv_heads), U32(head_dim), U32(max_segs)))


def attn_verify(q, k_cache, v_cache, block_table, seq_ids, positions, row_start, row_count, gate, out, q_scale, bpr,
                block_size, q_heads, kv_heads, head_dim, n_spans, max_count, max_ctx, seg_pages, scratch, status=None):
    """status: optional int32 tensor indexed by sequence id; an understated max_ctx sets bit 4 (STATUS_CTX_BOUND) there."""
    sb = scratch.numel() * scratch.element_size()
    check(load().wein_b200_attn_verify(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), _ptr(seq_ids),
                                       _ptr(positions), _ptr(row_start), _ptr(row_count), _ptr(gate), _ptr(out),
                                       F32(q_scale), U32(bpr), U32(block_size), U32(q_heads), U32(kv_heads),
                                       U32(head_dim), U32(n_spans), U32(max_count), U32(max_ctx), U32(seg_pages),
                                       _ptr(scratch), U64(sb), _ptr(status), _stream()))


def gemm_scratch_bytes(n_max):
    fn = load().wein_b200_gemm_scratch_bytes
    fn.restype = U64
    return int(fn(U32(n_max)))


def gemm_wt(a, w, c, m, n, k, scratch=None, tc=False):
    """C[m,n] = A[m,k] W[n,k]^T.  tc: the tensor-memory kernel whatever m (otherwise m <= 32 runs the mma.sync kernel)."""
    if tc:
        check(load().wein_b200_gemm_wt_tc(_ptr(a), _ptr(w), _ptr(c), U32(m), U32(n), U32(k), _stream()))
        return
    sb = scratch.numel() * scratch.element_size() if scratch is not None else 0
    check(load().wein_b200_gemm_wt(_ptr(a), _ptr(w), _ptr(c), U32(m), U32(n), U32(k), _ptr(scratch), U64(sb), _stream()))


def gemm_plan(m, n, k, swiglu=False):
    """(CTAs, k split, stages, shared-memory bytes, weight rows per tile) the tensor-memory GEMM uses for this shape on the
    current device."""
    out = (C.c_uint32 * 5)()
    check(load().wein_b200_gemm_plan(U32(m), U32(n), U32(k), U32(int(swiglu)), out))
    return tuple(int(v) for v in out)


def gemm_wait_timeouts():
    """Barrier waits of the tensor-memory GEMM that ran into their time limit since the library was loaded (0 in a healthy run)."""
    v = C.c_uint32(0)
    check(load().wein_b200_gemm_wait_timeouts(C.byref(v)))
    return v.value


DIST_CAP = 64


def topk_filter(logits, rows, row_seq, rows_per_seq, temp, top_k, top_p, n, s, out_ids, out_probs, out_n, sample_out=None,
                seed=None, rnd=None, position=0):
    check(load().wein_b200_topk_filter(_ptr(logits), _ptr(rows), _ptr(row_seq), U32(rows_per_seq), _ptr(temp), _ptr(top_k),
                                       _ptr(top_p), U32(n), U32(s), _ptr(out_ids), _ptr(out_probs), _ptr(out_n),
                                       _ptr(sample_out), _ptr(seed), _ptr(rnd), U32(position), _stream()))


def accept_greedy(logits, rows, drafts, n_drafts, n, B, k, scratch, accept_len, out_tokens, target=None):
    check(load().wein_b200_accept_greedy(_ptr(logits), _ptr(rows), _ptr(drafts), _ptr(n_drafts), U32(n), U32(B), U32(k),
                                         _ptr(scratch), _ptr(accept_len), _ptr(out_tokens), _ptr(target), _stream()))


def accept_sampled(drafts, n_drafts, p_ids, p_probs, p_n, q_ids, q_probs, q_n, temp, seed, rnd, B, k, accept_len, out_tokens):
    check(load().wein_b200_accept_sampled(_ptr(drafts), _ptr(n_drafts), _ptr(p_ids), _ptr(p_probs), _ptr(p_n), _ptr(q_ids),
                                          _ptr(q_probs), _ptr(q_n), _ptr(temp), _ptr(seed), _ptr(rnd), U32(B), U32(k),
                                          _ptr(accept_len), _ptr(out_tokens), _stream()))


def gemm_swiglu(a, w_gate_up, out, m, inter, k, scratch=None, tc=False):
    """out[m, inter] = silu_mul(a @ gate^T, a @ up^T) with W = [gate; up] ([2*inter, k])."""
    if tc:
        check(load().wein_b200_gemm_swiglu_tc(_ptr(a), _ptr(w_gate_up), _ptr(out), U32(m), U32(inter), U32(k), _stream()))
        return
    sb = scratch.numel() * scratch.element_size() if scratch is not None else 0
    check(load().wein_b200_gemm_swiglu(_ptr(a), _ptr(w_gate_up), _ptr(out), U32(m), U32(inter), U32(k), _ptr(scratch), U64(sb), _stream()))


def gdn_layer_lite(proj, ld, conv_w, conv_state, a_log, dt_bias, norm_w, state, state_f32, out, row_start, row_count, in_row, out_base,
                   n_rows, k_heads, v_heads, l2_eps, rms_eps, log):
    """gdn_layer without state snapshots: one update record per (token, v-head) into log [tokens, v_heads, 264] f32."""
    check(load().wein_b200_gdn_layer_lite(_ptr(proj), U32(ld), _ptr(conv_w), _ptr(conv_state), _ptr(a_log), _ptr(dt_bias), _ptr(norm_w),
                                          _ptr(state), U32(state_f32), _ptr(out), _ptr(row_start), _ptr(row_count), _ptr(in_row),
                                          _ptr(out_base), U32(n_rows), U32(k_heads), U32(v_heads), F32(l2_eps), F32(rms_eps), _ptr(log),
                                          _stream()))


def gdn_layer_ws(proj, ld, conv_w, conv_state, a_log, dt_bias, norm_w, state, state_f32, out, row_start, row_count, in_row, out_base,
                 n_rows, k_heads, v_heads, l2_eps, rms_eps, log=None, kq_scratch=None):
    """General form of gdn_layer: optional update log, optional scratch of tokens x v_heads x 388 f32 words
    for the per-token operands (used from 296 (span, v-head) pairs on)."""
    check(load().wein_b200_gdn_layer_ws(_ptr(proj), U32(ld), _ptr(conv_w), _ptr(conv_state), _ptr(a_log), _ptr(dt_bias), _ptr(norm_w),
                                        _ptr(state), U32(state_f32), _ptr(out), _ptr(row_start), _ptr(row_count), _ptr(in_row),
                                        _ptr(out_base), U32(n_rows), U32(k_heads), U32(v_heads), F32(l2_eps), F32(rms_eps), _ptr(log),
                                        _ptr(kq_scratch), _stream()))


def gdn_wait_timeouts():
    """Copy waits of the large-grid DeltaNet layer kernel that ran into their time limit since the library was loaded (0 in a
    healthy run)."""
    v = C.c_uint32(0)
    check(load().wein_b200_gdn_wait_timeouts(C.byref(v)))
    return v.value


def ptr_table(tensors):
    """Device array of the tensors' device pointers (for entries that take an array of per-layer pointers)."""
    return torch.tensor([t.data_ptr() for t in tensors], dtype=torch.int64, device="cuda")


def gdn_commit(states, logs, state_f32, row_start, row_count, in_row, out_base, accept_len, n_rows, v_heads):
    """Replays records 0..accept_len[r] on row in_row[r] of every layer's pool and stores row out_base[r] + accept_len[r].
    states / logs: lists of device tensors (one per layer), or pointer tables made once with ptr_table()."""
    own = not torch.is_tensor(states)
    sp = ptr_table(states) if own else states
    lp = ptr_table(logs) if not torch.is_tensor(logs) else logs
    check(load().wein_b200_gdn_commit(_ptr(sp), _ptr(lp), U32(sp.numel()), U32(state_f32), _ptr(row_start), _ptr(row_count), _ptr(in_row),
                                      _ptr(out_base), _ptr(accept_len), U32(n_rows), U32(v_heads), _stream()))
    if own:
        torch.cuda.current_stream().synchronize()   # the pointer tables above are temporaries


def gdn_layer(proj, ld, conv_w, conv_state, a_log, dt_bias, norm_w, state, state_f32, out, row_start, row_count, in_row, out_base,
              n_rows, k_heads, v_heads, l2_eps, rms_eps):
    check(load().wein_b200_gdn_layer(_ptr(proj), U32(ld), _ptr(conv_w), _ptr(conv_state), _ptr(a_log), _ptr(dt_bias), _ptr(norm_w),
                                     _ptr(state), U32(state_f32), _ptr(out), _ptr(row_start), _ptr(row_count), _ptr(in_row),
                                     _ptr(out_base), U32(n_rows), U32(k_heads), U32(v_heads), F32(l2_eps), F32(rms_eps), _stream()))


ARGMAX_NOALLOC_MAX_ROWS = 256


def argmax_rows_noalloc(x, rows, out, n, s):
    """argmax_rows without a scratch argument: for callers that cannot allocate (at most ARGMAX_NOALLOC_MAX_ROWS rows)."""
    check(load().wein_b200_argmax_rows_noalloc(_ptr(x), _ptr(rows), _ptr(out), U32(n), U32(s), _stream()))


def sample_rows(x, rows, slots, temp, top_k, top_p, seed, rng, out, n, s):
    """SampleRowsOp::run: per-row temperature / top-k / top-p sampling with PCG state in `rng` (int64 tensor, advanced in place)."""
    check(load().wein_b200_sample_rows(_ptr(x), _ptr(rows), _ptr(slots), _ptr(temp), _ptr(top_k), _ptr(top_p), _ptr(seed), _ptr(rng),
                                       _ptr(out), U32(n), U32(s), _stream()))


def qk_prep(qgkv, ld, qn, kn, cos, sin, rope_pos, kv_pos, seq_ids, block_table, bpr, qh, gate, k_pool, v_pool, tokens, q_heads,
            kv_heads, head_dim, rot_dim, eps):
    """Fused q / gate split + q-norm + k-norm + partial rotary + KV page scatter of a full-attention layer."""
    check(load().wein_b200_qk_prep(_ptr(qgkv), U32(ld), _ptr(qn), _ptr(kn), _ptr(cos), _ptr(sin), _ptr(rope_pos), _ptr(kv_pos),
                                   _ptr(seq_ids), _ptr(block_table), U32(bpr), _ptr(qh), _ptr(gate), _ptr(k_pool), _ptr(v_pool),
                                   U32(tokens), U32(q_heads), U32(kv_heads), U32(head_dim), U32(rot_dim), F32(eps), _stream()))


def mtp_cat(tok, embed_w, hid, hid_rows, pre_e, pre_h, cat, rows, hidden, eps):
    """Input of the MTP head: [norm(embed[tok]) | norm(hidden)] per row."""
    check(load().wein_b200_mtp_cat(_ptr(tok), _ptr(embed_w), _ptr(hid), _ptr(hid_rows), _ptr(pre_e), _ptr(pre_h), _ptr(cat),
                                   U32(rows), U32(hidden), F32(eps), _stream()))


def silu_mul_rows(gu, ld, out, rows, inter):
    """SwiGLU activation over rows holding gate | up side by side."""
    check(load().wein_b200_silu_mul_rows(_ptr(gu), U32(ld), _ptr(out), U32(rows), U32(inter), _stream()))
