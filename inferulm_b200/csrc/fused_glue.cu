// Fusions of the glue operators around the verify / draft GEMMs.  Each kernel performs, per element, exactly
// the operation sequence (and bf16 roundings) of the reference operators it replaces, so its outputs are
// bit-identical to running them one after another.  Compiled with -fmad=false.
#include "common.cuh"
#include "internal.h"

// ---- full-attention layer: q/gate split + q-norm + k-norm + partial RoPE + KV page scatter ----------------
// Replaces, per layer, 2x embed gather (q / gate de-interleave), 2x rms_norm_zc (head_dim rows), 2x rope_pt and
// kv_scatter of the reference (crates/wein-exec/src/qwen.rs:3888-3950).  Input row t of `qgkv`:
// [q_heads x (q | gate) x head_dim | kv_heads x head_dim (k) | kv_heads x head_dim (v)].
// One block of head_dim threads per (token, unit): unit < q_heads: q head; < q_heads + kv_heads: k head; else v head.
__global__ void qk_prep_kernel(const bf16_t *qgkv, uint32_t ld, const bf16_t *qn, const bf16_t *kn,
                               const float *cosv, const float *sinv, const uint32_t *rope_pos,
                               const uint32_t *kv_pos, const uint32_t *seq_ids,
                               const uint32_t *block_table, uint32_t bpr, bf16_t *qh, bf16_t *gate,
                               bf16_t *k_pool, bf16_t *v_pool, uint32_t q_heads, uint32_t kv_heads, uint32_t rot_dim, float eps) {
    PDL_ENTRY();
    __shared__ float red[33];
    __shared__ bf16_t nrm[256];
    const uint32_t hd = blockDim.x, t = blockIdx.y, unit = blockIdx.x, i = threadIdx.x;
    const bf16_t *row = qgkv + (size_t)t * ld;
    const uint32_t he = kv_heads * hd;
    const bool is_q = unit < q_heads, is_k = !is_q && unit < q_heads + kv_heads;
    // a row whose cache position is 0xFFFFFFFF belongs to no live chain position: it writes no K / V and rotates by position 0
    const uint32_t kvp = kv_pos[t];
    const bool dead = kvp == 0xffffffffu;
    size_t slot = 0;
    if (!is_q) {
        if (dead) return;
        slot = (size_t)block_table[(size_t)seq_ids[t] * bpr + kvp / 16] * 16 + kvp % 16;
    }
    if (!is_q && !is_k) {  // v head: plain copy into the page
        uint32_t h = unit - q_heads - kv_heads;
        v_pool[slot * he + h * hd + i] = row[2 * q_heads * hd + he + h * hd + i];
        return;
    }
    const bf16_t *src;
    const bf16_t *w;
    if (is_q) { src = row + (size_t)unit * 2 * hd; w = qn; }
    else { src = row + 2 * q_heads * hd + (unit - q_heads) * hd; w = kn; }
    // every global operand is fetched before the first store (one round trip): element, norm weight, gate, rotary factors
    const uint32_t half = rot_dim / 2;
    const float v = bf2f(src[i]), wn = bf2f(w[i]);
    const bf16_t gv = is_q ? src[hd + i] : (bf16_t)0;
    float rc = 0.0f, rs = 0.0f;
    if (i < rot_dim) {
        uint32_t p = i < half ? i : i - half;
        const uint32_t rp = rope_pos[t];
        size_t ci = (size_t)(rp == 0xffffffffu ? 0u : rp) * half + p;
        rc = cosv[ci]; rs = sinv[ci];
    }
    if (is_q) gate[((size_t)t * q_heads + unit) * hd + i] = gv;
    // zero-centred RMSNorm over the head (reference.rs:418-430; one element per thread, block tree)
    float total = block_sum_tree(fmaf(v, v, 0.0f), red);
    float inv = 1.0f / sqrtf(total / (float)hd + eps);
    bf16_t nb = f2bf(v * inv * (1.0f + wn));
    nrm[i] = nb;
    __syncthreads();
    // partial RoPE on the first rot_dim dims (reference.rs:436-460), from the rounded norm output
    bf16_t o = nb;
    if (i < rot_dim) {
        uint32_t p = i < half ? i : i - half;
        float x1 = bf2f(nrm[p]), x2 = bf2f(nrm[p + half]);
        o = i < half ? f2bf(x1 * rc - x2 * rs) : f2bf(x2 * rc + x1 * rs);
    }
    if (is_q) qh[((size_t)t * q_heads + unit) * hd + i] = o;
    else k_pool[slot * he + (unit - q_heads) * hd + i] = o;
}

int32_t wb_qk_prep(const void *qgkv, uint32_t ld, const void *qn, const void *kn, const float *cosv, const float *sinv,
                   const uint32_t *rope_pos, const uint32_t *kv_pos, const uint32_t *seq_ids, const uint32_t *block_table,
                   uint32_t bpr, void *qh, void *gate, void *k_pool, void *v_pool, uint32_t tokens, uint32_t q_heads,
                   uint32_t kv_heads, uint32_t head_dim, uint32_t rot_dim, float eps, cudaStream_t st) {
    WB_CHECK_ARG(head_dim % 32 == 0 && head_dim <= 256 && rot_dim <= head_dim && rot_dim % 2 == 0, "qk_prep: head_dim %u / rot_dim %u not built", head_dim, rot_dim);
    if (tokens == 0) return WB_OK;
    dim3 grid(q_heads + 2 * kv_heads, tokens);
    WB_LAUNCH((qk_prep_kernel), grid, head_dim, 0, st, (const bf16_t *)qgkv, ld, (const bf16_t *)qn, (const bf16_t *)kn, cosv, sinv, rope_pos, kv_pos,
                                              seq_ids, block_table, bpr, (bf16_t *)qh, (bf16_t *)gate, (bf16_t *)k_pool, (bf16_t *)v_pool,
                                              q_heads, kv_heads, rot_dim, eps);
    WB_LAUNCH_CHECK();
    return WB_OK;
}

// ---- MTP head input: embed gather + the two pre-norms + concatenation ---------------------------------------
// cat[r] = [ norm_zc(embed[tok[r]], pre_e) | norm_zc(hid[hid_rows[r]], pre_h) ]  (crates/wein-exec/src/qwen.rs:4451-4468:
// 2 gathers, 2 rms_norm_zc and a batched row copy in the reference).  Block (row, half), 256 threads.
__global__ void mtp_cat_kernel(const uint32_t *tok, uint32_t tok_stride, const bf16_t *embed,
                               const bf16_t *hid, const uint32_t *hid_rows, const bf16_t *pre_e,
                               const bf16_t *pre_h, bf16_t *cat, uint32_t hidden, float eps) {
    PDL_ENTRY();
    __shared__ float red[33];
    const uint32_t r = blockIdx.x, half = blockIdx.y;
    const bf16_t *src = half == 0 ? embed + (size_t)tok[(size_t)r * tok_stride] * hidden
                                  : hid + (size_t)(hid_rows ? hid_rows[r] : r) * hidden;
    const bf16_t *w = half == 0 ? pre_e : pre_h;
    bf16_t *dst = cat + (size_t)r * 2 * hidden + (size_t)half * hidden;
    // elements and weights of this thread first (independent loads), the rest of a wider row in a plain loop
    constexpr int CACHE = 12;
    float vals[CACHE], wv[CACHE], acc = 0.0f;
#pragma unroll
    for (int it = 0; it < CACHE; it++) {
        uint32_t i = threadIdx.x + it * blockDim.x;
        vals[it] = i < hidden ? bf2f(src[i]) : 0.0f;
        wv[it] = i < hidden ? bf2f(w[i]) : 0.0f;
    }
#pragma unroll
    for (int it = 0; it < CACHE; it++)
        if (threadIdx.x + it * blockDim.x < hidden) acc = fmaf(vals[it], vals[it], acc);
    for (uint32_t i = threadIdx.x + CACHE * blockDim.x; i < hidden; i += blockDim.x) { float v = bf2f(src[i]); acc = fmaf(v, v, acc); }
    float total = block_sum_tree(acc, red);
    float inv = 1.0f / sqrtf(total / (float)hidden + eps);
#pragma unroll
    for (int it = 0; it < CACHE; it++) {
        uint32_t i = threadIdx.x + it * blockDim.x;
        if (i < hidden) dst[i] = f2bf(vals[it] * inv * (1.0f + wv[it]));
    }
    for (uint32_t i = threadIdx.x + CACHE * blockDim.x; i < hidden; i += blockDim.x) dst[i] = f2bf(bf2f(src[i]) * inv * (1.0f + bf2f(w[i])));
}
int32_t wb_mtp_cat(const uint32_t *tok, uint32_t tok_stride, const void *embed, const void *hid, const uint32_t *hid_rows,
                   const void *pre_e, const void *pre_h, void *cat, uint32_t rows, uint32_t hidden, float eps, cudaStream_t st) {
    WB_CHECK_ARG(hidden >= 256, "mtp_cat: hidden %u below 256 is not built", hidden);
    if (rows == 0) return WB_OK;
    dim3 grid(rows, 2);
    WB_LAUNCH((mtp_cat_kernel), grid, 256, 0, st, tok, tok_stride, (const bf16_t *)embed, (const bf16_t *)hid, hid_rows, (const bf16_t *)pre_e,
                                         (const bf16_t *)pre_h, (bf16_t *)cat, hidden, eps);
    WB_LAUNCH_CHECK();
    return WB_OK;
}

// ---- SwiGLU activation on the fused gate|up projection: out[r, i] = bf16(bf16(silu(g)) * u) -----------------
__global__ void silu_mul_rows_kernel(const bf16_t *gu, uint32_t ld, bf16_t *out, uint32_t inter) {
    PDL_ENTRY();
    const bf16_t *g = gu + (size_t)blockIdx.y * ld, *u = g + inter;
    uint32_t i = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
    if (i >= inter) return;
    uint32_t gv = *reinterpret_cast<const uint32_t *>(g + i), uv = *reinterpret_cast<const uint32_t *>(u + i);
    bf16_t r0 = f2bf(rbf(silu_ref(bf2f((bf16_t)(gv & 0xffff)))) * bf2f((bf16_t)(uv & 0xffff)));
    bf16_t r1 = f2bf(rbf(silu_ref(bf2f((bf16_t)(gv >> 16)))) * bf2f((bf16_t)(uv >> 16)));
    *reinterpret_cast<uint32_t *>(out + (size_t)blockIdx.y * inter + i) = (uint32_t)r0 | ((uint32_t)r1 << 16);
}
int32_t wb_silu_mul_rows(const void *gu, uint32_t ld, void *out, uint32_t rows, uint32_t inter, cudaStream_t st) {
    WB_CHECK_ARG(inter % 2 == 0 && ld % 2 == 0, "silu_mul_rows: odd width");
    if (rows == 0) return WB_OK;
    dim3 grid((inter / 2 + 255) / 256, rows);
    WB_LAUNCH((silu_mul_rows_kernel), grid, 256, 0, st, (const bf16_t *)gu, ld, (bf16_t *)out, inter);
    WB_LAUNCH_CHECK();
    return WB_OK;
}

// ---- argmax phase 2 with a strided destination (draft token j of batch row r lands at out[r*mul + off]) -----
__global__ void argmax_finish_kernel(const uint64_t *part, uint32_t split, uint32_t *out, uint32_t out_mul, uint32_t out_off) {
    PDL_ENTRY();
    uint32_t r = blockIdx.x;
    uint64_t k = 0ull;
    for (uint32_t i = threadIdx.x; i < split; i += 32) { uint64_t o = part[(size_t)r * split + i]; k = o > k ? o : k; }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) { uint64_t o = __shfl_xor_sync(0xffffffffu, k, off); k = o > k ? o : k; }
    if (threadIdx.x == 0) out[(size_t)r * out_mul + out_off] = k == 0ull ? 0xffffffffu : ~(uint32_t)k;
}
int32_t wb_argmax_finish(const void *part, uint32_t split, uint32_t *out, uint32_t out_mul, uint32_t out_off, uint32_t s, cudaStream_t st) {
    if (s == 0) return WB_OK;
    WB_LAUNCH((argmax_finish_kernel), s, 32, 0, st, (const uint64_t *)part, split, out, out_mul, out_off);
    WB_LAUNCH_CHECK();
    return WB_OK;
}

// ---- gated RMSNorm with the gate z read in place from the fused projection output --------------------------
// Row (t, h): x = core[t, h, :], z = z_base[t*z_tok_stride + h*hidden + :]  (reference.rs:699-713).
__global__ void rms_norm_gated_rows_kernel(const bf16_t *x, const bf16_t *z, uint32_t z_tok_stride,
                                           const float *w, bf16_t *out, uint32_t heads, uint32_t hidden, float eps) {
    PDL_ENTRY();
    __shared__ float red[33];
    const uint32_t t = blockIdx.y, h = blockIdx.x, i = threadIdx.x;
    size_t xb = ((size_t)t * heads + h) * hidden, zb = (size_t)t * z_tok_stride + (size_t)h * hidden;
    float v = bf2f(x[xb + i]);
    float total = block_sum_tree(fmaf(v, v, 0.0f), red);
    float inv = 1.0f / sqrtf(total / (float)hidden + eps);
    float xw = w[i] * rbf(v * inv);
    float zv = bf2f(z[zb + i]);
    out[xb + i] = f2bf(xw * (zv * (1.0f / (1.0f + expf_ref(-zv)))));
}
int32_t wb_rms_norm_gated_rows(const void *x, const void *z, uint32_t z_tok_stride, const float *w, void *out, uint32_t tokens,
                               uint32_t heads, uint32_t hidden, float eps, cudaStream_t st) {
    WB_CHECK_ARG(hidden % 32 == 0 && hidden >= 32 && hidden <= 256 && (hidden & (hidden - 1)) == 0, "rms_norm_gated_rows: hidden %u not built", hidden);
    if (tokens == 0) return WB_OK;
    dim3 grid(heads, tokens);
    WB_LAUNCH((rms_norm_gated_rows_kernel), grid, hidden, 0, st, (const bf16_t *)x, (const bf16_t *)z, z_tok_stride, w, (bf16_t *)out, heads, hidden, eps);
    WB_LAUNCH_CHECK();
    return WB_OK;
}


// ---- C-ABI of the fused forms, so that each one is checked on its own against the operator chain it replaces ----
extern "C" {
int32_t wein_b200_qk_prep(const void *qgkv, uint32_t ld, const void *qn, const void *kn, const void *cosv, const void *sinv,
                          const void *rope_pos, const void *kv_pos, const void *seq_ids, const void *block_table, uint32_t bpr,
                          void *qh, void *gate, void *k_pool, void *v_pool, uint32_t tokens, uint32_t q_heads, uint32_t kv_heads,
                          uint32_t head_dim, uint32_t rot_dim, float eps, void *stream) {
    WB_CHECK_ARG(qgkv && qn && kn && cosv && sinv && rope_pos && kv_pos && seq_ids && block_table && qh && gate && k_pool && v_pool,
                 "qk_prep: null pointer");
    WB_CHECK_ARG(ld >= 2 * q_heads * head_dim + 2 * kv_heads * head_dim, "qk_prep: row stride %u shorter than q|gate|k|v", ld);
    return wb_qk_prep(qgkv, ld, qn, kn, (const float *)cosv, (const float *)sinv, (const uint32_t *)rope_pos, (const uint32_t *)kv_pos,
                      (const uint32_t *)seq_ids, (const uint32_t *)block_table, bpr, qh, gate, k_pool, v_pool, tokens, q_heads, kv_heads,
                      head_dim, rot_dim, eps, (cudaStream_t)stream);
}
int32_t wein_b200_mtp_cat(const void *tok, const void *embed, const void *hid, const void *hid_rows, const void *pre_e,
                          const void *pre_h, void *cat, uint32_t rows, uint32_t hidden, float eps, void *stream) {
    WB_CHECK_ARG(tok && embed && hid && pre_e && pre_h && cat, "mtp_cat: null pointer");
    return wb_mtp_cat((const uint32_t *)tok, 1, embed, hid, (const uint32_t *)hid_rows, pre_e, pre_h, cat, rows, hidden, eps,
                      (cudaStream_t)stream);
}
int32_t wein_b200_silu_mul_rows(const void *gu, uint32_t ld, void *out, uint32_t rows, uint32_t inter, void *stream) {
    WB_CHECK_ARG(gu && out && ld >= 2 * inter, "silu_mul_rows: null pointer or row stride %u shorter than gate|up", ld);
    return wb_silu_mul_rows(gu, ld, out, rows, inter, (cudaStream_t)stream);
}
}  // extern "C"

