// Glue operators of the verify / draft forward, bit-exact against the
// reference's CPU kernels: embed gather, zero-centred RMSNorm (+ fused residual
// add), gated RMSNorm, partial RoPE, gate multiplies, SwiGLU activation, KV page
// scatter, causal depthwise conv + conv-state rows, row argmax.
// Each kernel cites the reference function whose arithmetic order it keeps.
// Compiled with -fmad=false: a*b+c is two roundings unless fmaf() is written.
#include "common.cuh"
#include "internal.h"

// ------------------------------------------------------------------ embed
// out[t, :] = w[ids[t], :]  (reference.rs:298-305).  One block per row.
__global__ void embed_kernel(const uint32_t *ids, const bf16_t *w, bf16_t *out,
                             uint32_t hidden) {
    PDL_ENTRY();
    size_t src = (size_t)ids[blockIdx.x] * hidden, dst = (size_t)blockIdx.x * hidden;
    if ((hidden & 7u) == 0 && ((((uintptr_t)w) | ((uintptr_t)out)) & 15u) == 0) {
        const uint4 *s = reinterpret_cast<const uint4 *>(w + src);
        uint4 *d = reinterpret_cast<uint4 *>(out + dst);
        for (uint32_t i = threadIdx.x; i < hidden / 8; i += blockDim.x) d[i] = s[i];
    } else {
        for (uint32_t i = threadIdx.x; i < hidden; i += blockDim.x) out[dst + i] = w[src + i];
    }
}

// ------------------------------------------------------------------ norms
// Row sum of squares in the reference's order (reference.rs:400-414): thread t
// owns elements t, t+bdim, ... (fused multiply-add chain), then the block tree.
// MODE 0: out = x*inv*(1+w)                      rms_norm_zc   (reference.rs:418-430)
// MODE 1: s = bf16(a+b) -> sum_out; norm of s    add_norm_zc   (kernels/src/lib.rs:4674-4755)
template <int MODE>
__global__ void rms_norm_zc_kernel(const bf16_t *a, const bf16_t *b, const bf16_t *w, bf16_t *sum_out,
                                   bf16_t *norm_out, uint32_t hidden, float eps) {
    PDL_ENTRY();
    constexpr int CACHE = 12;  // elements per thread kept in registers between the two passes (hidden <= 3072 at 256 threads)
    __shared__ float red[33];
    size_t base = (size_t)blockIdx.x * hidden;
    float vals[CACHE], wv[CACHE];
    float acc = 0.0f;
    // all loads first (independent, one round trip), then the arithmetic in element order
    bf16_t av[CACHE], bv[CACHE];
#pragma unroll
    for (int it = 0; it < CACHE; it++) {
        uint32_t i = threadIdx.x + it * blockDim.x;
        bool ok = i < hidden;
        av[it] = ok ? a[base + i] : (bf16_t)0;
        bv[it] = (ok && MODE == 1) ? b[base + i] : (bf16_t)0;
        wv[it] = ok ? bf2f(w[i]) : 0.0f;
    }
#pragma unroll
    for (int it = 0; it < CACHE; it++) {
        uint32_t i = threadIdx.x + it * blockDim.x;
        vals[it] = 0.0f;
        if (i < hidden) {
            float v;
            if (MODE == 1) {
                bf16_t s = f2bf(bf2f(av[it]) + bf2f(bv[it]));
                sum_out[base + i] = s;
                v = bf2f(s);
            } else {
                v = bf2f(av[it]);
            }
            vals[it] = v;
            acc = fmaf(v, v, acc);
        }
    }
    for (uint32_t i = threadIdx.x + CACHE * blockDim.x; i < hidden; i += blockDim.x) {
        float v;
        if (MODE == 1) {
            bf16_t s = f2bf(bf2f(a[base + i]) + bf2f(b[base + i]));
            sum_out[base + i] = s;
            v = bf2f(s);
        } else {
            v = bf2f(a[base + i]);
        }
        acc = fmaf(v, v, acc);
    }
    float total = block_sum_tree(acc, red);
    float inv = 1.0f / sqrtf(total / (float)hidden + eps);
#pragma unroll
    for (int it = 0; it < CACHE; it++) {
        uint32_t i = threadIdx.x + it * blockDim.x;
        if (i < hidden) norm_out[base + i] = f2bf(vals[it] * inv * (1.0f + wv[it]));
    }
    const bf16_t *src = MODE == 1 ? sum_out : a;
    for (uint32_t i = threadIdx.x + CACHE * blockDim.x; i < hidden; i += blockDim.x)
        norm_out[base + i] = f2bf(bf2f(src[base + i]) * inv * (1.0f + bf2f(w[i])));
}

// rms_norm_gated (reference.rs:699-713): xb = bf16(x*inv); xw = w*xb (kept
// f32); out = bf16(xw * (z*sigmoid(z))).
__global__ void rms_norm_gated_kernel(const bf16_t *x, const bf16_t *z,
                                      const float *w, bf16_t *out, uint32_t hidden, float eps) {
    PDL_ENTRY();
    __shared__ float red[33];
    size_t base = (size_t)blockIdx.x * hidden;
    float acc = 0.0f;
    for (uint32_t i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v = bf2f(x[base + i]);
        acc = fmaf(v, v, acc);
    }
    float total = block_sum_tree(acc, red);
    float inv = 1.0f / sqrtf(total / (float)hidden + eps);
    for (uint32_t i = threadIdx.x; i < hidden; i += blockDim.x) {
        float xb = rbf(bf2f(x[base + i]) * inv);
        float xw = w[i] * xb;
        float zv = bf2f(z[base + i]);
        out[base + i] = f2bf(xw * (zv * (1.0f / (1.0f + expf_ref(-zv)))));
    }
}

// ------------------------------------------------------------------- rope
// Partial rotary, rotate-half (reference.rs:436-460).  One thread per
// (token, head, pair); in place allowed.
__global__ void rope_pt_kernel(const bf16_t *x, const float *cosv, const float *sinv,
                               const uint32_t *pos, bf16_t *out, uint32_t rot_dim, uint32_t head_dim,
                               uint32_t heads, uint32_t tokens) {
    PDL_ENTRY();
    uint32_t half = rot_dim / 2;
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t total = (size_t)tokens * heads * half;
    if (idx >= total) return;
    uint32_t p = idx % half;
    size_t th = idx / half;
    uint32_t t = th / heads;
    size_t row = th * head_dim;
    float c = cosv[(size_t)pos[t] * half + p], s = sinv[(size_t)pos[t] * half + p];
    float x1 = bf2f(x[row + p]), x2 = bf2f(x[row + half + p]);
    out[row + p] = f2bf(x1 * c - x2 * s);
    out[row + half + p] = f2bf(x2 * c + x1 * s);
}
// copy of the non-rotated tail when out != x
__global__ void rope_tail_copy_kernel(const bf16_t *x, bf16_t *out, uint32_t rot_dim, uint32_t head_dim, size_t rows) {
    PDL_ENTRY();
    uint32_t tail = head_dim - rot_dim;
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * tail) return;
    size_t r = idx / tail;
    uint32_t e = rot_dim + idx % tail;
    out[r * head_dim + e] = x[r * head_dim + e];
}

// ------------------------------------------------------------ elementwise
// OP 0 add (reference.rs:308-313)   1 mul (:316-321)   2 silu (:141-148)
// OP 3 silu_mul (kernels/src/lib.rs:576-584)   4 sigmul (reference.rs:463-472)
template <int OP>
__global__ void eltwise_kernel(const bf16_t *a, const bf16_t *b, bf16_t *out, size_t n) {
    PDL_ENTRY();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float x = bf2f(a[i]);
    float y = OP == 2 ? 0.0f : bf2f(b[i]);
    bf16_t r;
    if (OP == 0) r = f2bf(x + y);
    else if (OP == 1) r = f2bf(x * y);
    else if (OP == 2) r = f2bf(silu_ref(x));
    else if (OP == 3) r = f2bf(rbf(silu_ref(x)) * y);
    else r = f2bf(x * rbf(sigmoid_ref(y)));  // sigmul: x * bf16(sigmoid(g))
    out[i] = r;
}

// -------------------------------------------------------------- kv scatter
// slot = block_table[seq*bpr + pos/bs]*bs + pos%bs (reference.rs:192-215).
// DST_F32 widens exactly (kernels/src/lib.rs:620).
template <bool DST_F32>
__global__ void kv_scatter_kernel(const bf16_t *src_k, const bf16_t *src_v,
                                  const uint32_t *block_table, const uint32_t *seq_ids,
                                  const uint32_t *positions, void *k_dst, void *v_dst, uint32_t bpr,
                                  uint32_t block_size, uint32_t head_elems, uint32_t tokens) {
    PDL_ENTRY();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)tokens * head_elems) return;
    uint32_t t = idx / head_elems, e = idx % head_elems;
    uint32_t pos = positions[t];
    size_t slot = (size_t)block_table[(size_t)seq_ids[t] * bpr + pos / block_size] * block_size + pos % block_size;
    if (DST_F32) {
        ((float *)k_dst)[slot * head_elems + e] = bf2f(src_k[idx]);
        ((float *)v_dst)[slot * head_elems + e] = bf2f(src_v[idx]);
    } else {
        ((bf16_t *)k_dst)[slot * head_elems + e] = src_k[idx];
        ((bf16_t *)v_dst)[slot * head_elems + e] = src_v[idx];
    }
}

// -------------------------------------------------------------------- conv
// Causal depthwise conv (taps k ascending, acc = v*w + acc as two roundings),
// rounded to bf16, then SiLU rounded again (reference.rs:476-506).
__global__ void conv1d_dw_kernel(const bf16_t *x, const bf16_t *w,
                                 const bf16_t *state_in, const uint32_t *tok_row,
                                 const uint32_t *tok_pos, bf16_t *out, uint32_t conv_dim,
                                 uint32_t kernel, uint32_t tokens) {
    PDL_ENTRY();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)tokens * conv_dim) return;
    uint32_t g = idx / conv_dim, c = idx % conv_dim;
    int st = (int)kernel - 1;
    int p = (int)tok_pos[g];
    size_t row = tok_row[g];
    float acc = 0.0f;
    for (int k = 0; k < (int)kernel; k++) {
        int i = p - st + k;
        float v = i < 0 ? bf2f(state_in[row * conv_dim * st + (size_t)c * st + (i + st)])
                        : bf2f(x[(size_t)((int)g - p + i) * conv_dim + c]);
        acc = v * bf2f(w[(size_t)c * kernel + k]) + acc;
    }
    float cv = rbf(acc);
    out[idx] = f2bf(silu_ref(cv));
}
// Conv-state rows (reference.rs:511-562).  One thread per (span, channel).
// spec == 1: the window after token t goes to row row_id+t+1 (row j = state
// after the first j tokens); spec == 0: the span's own row is rolled in place.
__global__ void conv_state_roll_kernel(const bf16_t *x, bf16_t *state, const uint32_t *row_start,
                                       const uint32_t *row_count, const uint32_t *row_id,
                                       const uint32_t *specs, uint32_t conv_dim, uint32_t kernel, uint32_t n_rows) {
    PDL_ENTRY();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)n_rows * conv_dim) return;
    uint32_t r = idx / conv_dim, c = idx % conv_dim;
    int st = (int)kernel - 1;
    int t0 = (int)row_start[r], cnt = (int)row_count[r];
    size_t rid = row_id[r];
    bf16_t old[8];
    for (int j = 0; j < st; j++) old[j] = state[rid * conv_dim * st + (size_t)c * st + j];
    if (specs[r] != 0) {
        for (int ti = 0; ti < cnt; ti++) {
            size_t wbase = (rid + ti + 1) * conv_dim * st + (size_t)c * st;
            for (int j = 0; j < st; j++) {
                int li = ti + 1 - st + j;
                state[wbase + j] = li < 0 ? old[li + st] : x[(size_t)(t0 + li) * conv_dim + c];
            }
        }
    } else {
        for (int j = 0; j < st; j++) {
            int i = cnt - st + j;
            state[rid * conv_dim * st + (size_t)c * st + j] = i < 0 ? old[i + st] : x[(size_t)(t0 + i) * conv_dim + c];
        }
    }
}
// Verify-shaped fusion of the two kernels above for chain spans: one thread per
// (span, channel) walks the span's tokens with the window in registers, writes
// conv+SiLU outputs and the per-position conv-state rows.  The window after
// token t is written to row out_base[r]+t; the span reads row in_row[r].
// Values are bit-identical to conv1d_dw followed by conv_state_roll.
__global__ void conv_verify_kernel(const bf16_t *x, uint32_t x_stride, const bf16_t *w,
                                   bf16_t *state, const uint32_t *row_start,
                                   const uint32_t *row_count, const uint32_t *in_row,
                                   const uint32_t *out_base, bf16_t *out, uint32_t conv_dim,
                                   uint32_t n_rows) {
    PDL_ENTRY();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)n_rows * conv_dim) return;
    uint32_t r = idx / conv_dim, c = idx % conv_dim;
    uint32_t t0 = row_start[r], cnt = row_count[r];
    const bf16_t *sp = state + ((size_t)in_row[r] * conv_dim + c) * 3;
    bf16_t w0 = sp[0], w1 = sp[1], w2 = sp[2];
    float k0 = bf2f(w[(size_t)c * 4 + 0]), k1 = bf2f(w[(size_t)c * 4 + 1]), k2 = bf2f(w[(size_t)c * 4 + 2]),
          k3 = bf2f(w[(size_t)c * 4 + 3]);
    size_t ob = out_base[r];
    for (uint32_t t = 0; t < cnt; t++) {
        bf16_t xv = x[(size_t)(t0 + t) * x_stride + c];
        float acc = 0.0f;
        acc = bf2f(w0) * k0 + acc;
        acc = bf2f(w1) * k1 + acc;
        acc = bf2f(w2) * k2 + acc;
        acc = bf2f(xv) * k3 + acc;
        out[(size_t)(t0 + t) * conv_dim + c] = f2bf(silu_ref(rbf(acc)));
        w0 = w1; w1 = w2; w2 = xv;
        bf16_t *dp = state + ((ob + t) * conv_dim + c) * 3;
        dp[0] = w0; dp[1] = w1; dp[2] = w2;
    }
}

// ------------------------------------------------------------------ argmax
// Total order (value desc, index asc) is an associative, commutative "max", so
// any scan order gives the reference's answer (reference.rs:717-733).  Keys
// pack (ordered value, ~index) into one u64 and the reduction is a plain max.
__device__ __forceinline__ uint64_t argmax_key(bf16_t h, uint32_t i) {
    float v = bf2f(h);
    // NaN never wins in the reference (every comparison false); -0.0 == +0.0
    if (v != v) return 0ull;
    uint32_t u = __float_as_uint(v == 0.0f ? 0.0f : v);
    uint32_t ord = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return ((uint64_t)ord << 32) | (uint32_t)(~i);
}
__device__ __forceinline__ uint64_t warp_max_u64(uint64_t k) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
        uint64_t o = __shfl_xor_sync(0xffffffffu, k, off);
        k = o > k ? o : k;
    }
    return k;
}
// phase 1: grid (split, s); each block scans one slice of one row
__global__ void argmax_p1_kernel(const bf16_t *x, const uint32_t *rows, uint64_t *part,
                                 uint32_t n, uint32_t split) {
    PDL_ENTRY();
    __shared__ uint64_t sm[32];
    uint32_t r = blockIdx.y, sl = blockIdx.x;
    const bf16_t *row = x + (size_t)rows[r] * n;
    uint32_t per = ((n + split - 1) / split + 7) & ~7u;
    uint32_t lo = sl * per, hi = min(n, lo + per);
    uint64_t best = 0ull;
    if ((((uintptr_t)row) & 15u) == 0) {
        for (uint32_t i = lo + threadIdx.x * 8; i < hi; i += blockDim.x * 8) {
            if (i + 8 <= hi) {
                uint4 v = *reinterpret_cast<const uint4 *>(row + i);
                uint32_t wv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    uint64_t k0 = argmax_key((bf16_t)(wv[j] & 0xffff), i + 2 * j);
                    uint64_t k1 = argmax_key((bf16_t)(wv[j] >> 16), i + 2 * j + 1);
                    best = k0 > best ? k0 : best;
                    best = k1 > best ? k1 : best;
                }
            } else {
                for (uint32_t j = i; j < hi; j++) { uint64_t k = argmax_key(row[j], j); best = k > best ? k : best; }
            }
        }
    } else {
        for (uint32_t i = lo + threadIdx.x; i < hi; i += blockDim.x) { uint64_t k = argmax_key(row[i], i); best = k > best ? k : best; }
    }
    best = warp_max_u64(best);
    if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x < 32) {
        uint64_t k = threadIdx.x < (blockDim.x >> 5) ? sm[threadIdx.x] : 0ull;
        k = warp_max_u64(k);
        if (threadIdx.x == 0) part[(size_t)r * split + sl] = k;
    }
}
// phase 2: one warp per row merges the slices
__global__ void argmax_p2_kernel(const uint64_t *part, uint32_t *out, uint32_t split) {
    PDL_ENTRY();
    uint32_t r = blockIdx.x;
    uint64_t k = 0ull;
    for (uint32_t i = threadIdx.x; i < split; i += 32) { uint64_t o = part[(size_t)r * split + i]; k = o > k ? o : k; }
    k = warp_max_u64(k);
    // no finite / infinite candidate at all (empty row or all NaN): the reference returns 0xffffffff
    if (threadIdx.x == 0) out[r] = k == 0ull ? 0xffffffffu : ~(uint32_t)k;
}

// ----------------------------------------------------------- host launchers
#define STREAM(s) ((cudaStream_t)(s))
static inline uint32_t norm_bdim(uint32_t hidden) {
    uint32_t m = hidden < 256 ? hidden : 256, p = 1;
    while (p < m) p <<= 1;
    return p;
}

extern "C" {

int32_t wein_b200_embed(const void *ids, const void *w, void *out, uint32_t hidden, uint32_t tokens, void *stream) {
    WB_CHECK_ARG(ids && w && out && hidden > 0, "embed: null pointer or zero width");
    if (tokens == 0) return WB_OK;
    WB_LAUNCH((embed_kernel), tokens, 256, 0, STREAM(stream), (const uint32_t *)ids, (const bf16_t *)w, (bf16_t *)out, hidden);
    WB_LAUNCH_CHECK();
    return WB_OK;
}

int32_t wein_b200_rms_norm_zc(const void *x, const void *w, void *out, uint32_t rows, uint32_t hidden, float eps, void *stream) {
    WB_CHECK_ARG(x && w && out && hidden > 0, "rms_norm_zc: null pointer or zero width");
    uint32_t bd = norm_bdim(hidden);
    if (bd < 32) { wb_set_error("rms_norm_zc: hidden %u below one warp is not built", hidden); return WB_ERR_SHAPE; }
    if (rows == 0) return WB_OK;
    WB_LAUNCH((rms_norm_zc_kernel<0>), rows, bd, 0, STREAM(stream), (const bf16_t *)x, nullptr, (const bf16_t *)w, nullptr, (bf16_t *)out, hidden, eps);
    WB_LAUNCH_CHECK();
    return WB_OK;
}

int32_t wein_b200_add_norm_zc(const void *a, const void *b, const void *w, void *sum_out, void *norm_out, uint32_t rows,
                              uint32_t hidden, float eps, void *stream) {
    WB_CHECK_ARG(a && b && w && sum_out && norm_out && hidden > 0, "add_norm_zc: null pointer or zero width");
    uint32_t bd = norm_bdim(hidden);
    if (bd < 32) { wb_set_error("add_norm_zc: hidden %u below one warp is not built", hidden); return WB_ERR_SHAPE; }
    if (rows == 0) return WB_OK;
    WB_LAUNCH((rms_norm_zc_kernel<1>), rows, bd, 0, STREAM(stream), (const bf16_t *)a, (const bf16_t *)b, (const bf16_t *)w, (bf16_t *)sum_out,
                                                          (bf16_t *)norm_out, hidden, eps);
    WB_LAUNCH_CHECK();
    return WB_OK;
}

int32_t wein_b200_rms_norm_gated(const void *x, const void *z, const void *w, void *out, uint32_t rows, uint32_t hidden,
                                 float eps, void *stream) {
    WB_CHECK_ARG(x && z && w && out && hidden > 0, "rms_norm_gated: null pointer or zero width");
    uint32_t bd = norm_bdim(hidden);
    if (bd < 32) { wb_set_error("rms_norm_gated: hidden %u below one warp is not built", hidden); return WB_ERR_SHAPE; }
    if (rows == 0) return WB_OK;
    WB_LAUNCH((rms_norm_gated_kernel), rows, bd, 0, STREAM(stream), (const bf16_t *)x, (const bf16_t *)z, (const float *)w, (bf16_t *)out, hidden, eps);
    WB_LAUNCH_CHECK();
    return WB_OK;
}

int32_t wein_b200_rope_pt(const void *x, const void *cosv, const void *sinv, const void *pos, void *out, uint32_t rot_dim,
                          uint32_t head_dim, uint32_t heads, uint32_t tokens, void *stream) {
    WB_CHECK_ARG(x && cosv && sinv && pos && out, "rope_pt: null pointer");
    WB_CHECK_ARG(rot_dim % 2 == 0 && rot_dim <= head_dim && rot_dim > 0, "rope_pt: rot_dim %u must be even and <= head_dim %u", rot_dim, head_dim);
    if (tokens == 0 || heads == 0) return WB_OK;
    size_t total = (size_t)tokens * heads * (rot_dim / 2);
    WB_LAUNCH((rope_pt_kernel), (unsigned)((total + 255) / 256), 256, 0, STREAM(stream), (const bf16_t *)x, (const float *)cosv, (const float *)sinv,
                                                                               (const uint32_t *)pos, (bf16_t *)out, rot_dim, head_dim, heads, tokens);
    WB_LAUNCH_CHECK();
    if (out != x && rot_dim < head_dim) {
        size_t rows = (size_t)tokens * heads, n = rows * (head_dim - rot_dim);
        WB_LAUNCH((rope_tail_copy_kernel), (unsigned)((n + 255) / 256), 256, 0, STREAM(stream), (const bf16_t *)x, (bf16_t *)out, rot_dim, head_dim, rows);
        WB_LAUNCH_CHECK();
    }
    return WB_OK;
}

#define ELTWISE_ENTRY(name, OP, needs_b)                                                                        \
    int32_t name(const void *a, const void *b, void *out, uint64_t n, void *stream) {                           \
        WB_CHECK_ARG(a && out && (!(needs_b) || b), #name ": null pointer");                                    \
        if (n == 0) return WB_OK;                                                                               \
        WB_LAUNCH((eltwise_kernel<OP>), (unsigned)((n + 255) / 256), 256, 0, STREAM(stream), (const bf16_t *)a, (const bf16_t *)b, (bf16_t *)out, (size_t)n); \
        WB_LAUNCH_CHECK();                                                                                      \
        return WB_OK;                                                                                           \
    }
ELTWISE_ENTRY(wein_b200_add, 0, 1)
ELTWISE_ENTRY(wein_b200_mul, 1, 1)
ELTWISE_ENTRY(wein_b200_silu_mul, 3, 1)
ELTWISE_ENTRY(wein_b200_sigmul, 4, 1)
int32_t wein_b200_silu(const void *x, void *out, uint64_t n, void *stream) {
    WB_CHECK_ARG(x && out, "silu: null pointer");
    if (n == 0) return WB_OK;
    WB_LAUNCH((eltwise_kernel<2>), (unsigned)((n + 255) / 256), 256, 0, STREAM(stream), (const bf16_t *)x, nullptr, (bf16_t *)out, (size_t)n);
    WB_LAUNCH_CHECK();
    return WB_OK;
}

static int32_t kv_scatter_impl(bool f32, const void *src_k, const void *src_v, const void *block_table, const void *seq_ids,
                               const void *positions, void *k_dst, void *v_dst, uint32_t bpr, uint32_t block_size,
                               uint32_t head_elems, uint32_t tokens, void *stream) {
    WB_CHECK_ARG(src_k && src_v && block_table && seq_ids && positions && k_dst && v_dst, "kv_scatter: null pointer");
    WB_CHECK_ARG(bpr > 0 && block_size > 0 && head_elems > 0, "kv_scatter: zero geometry");
    if (tokens == 0) return WB_OK;
    size_t n = (size_t)tokens * head_elems;
    unsigned grid = (unsigned)((n + 255) / 256);
    if (f32)
        WB_LAUNCH((kv_scatter_kernel<true>), grid, 256, 0, STREAM(stream), (const bf16_t *)src_k, (const bf16_t *)src_v, (const uint32_t *)block_table,
            (const uint32_t *)seq_ids, (const uint32_t *)positions, k_dst, v_dst, bpr, block_size, head_elems, tokens);
    else
        WB_LAUNCH((kv_scatter_kernel<false>), grid, 256, 0, STREAM(stream), (const bf16_t *)src_k, (const bf16_t *)src_v, (const uint32_t *)block_table,
            (const uint32_t *)seq_ids, (const uint32_t *)positions, k_dst, v_dst, bpr, block_size, head_elems, tokens);
    WB_LAUNCH_CHECK();
    return WB_OK;
}
int32_t wein_b200_kv_scatter(const void *src_k, const void *src_v, const void *block_table, const void *seq_ids,
                             const void *positions, void *k_dst, void *v_dst, uint32_t bpr, uint32_t block_size,
                             uint32_t head_elems, uint32_t tokens, void *stream) {
    return kv_scatter_impl(false, src_k, src_v, block_table, seq_ids, positions, k_dst, v_dst, bpr, block_size, head_elems, tokens, stream);
}
int32_t wein_b200_kv_scatter_f32(const void *src_k, const void *src_v, const void *block_table, const void *seq_ids,
                                 const void *positions, void *k_dst, void *v_dst, uint32_t bpr, uint32_t block_size,
                                 uint32_t head_elems, uint32_t tokens, void *stream) {
    return kv_scatter_impl(true, src_k, src_v, block_table, seq_ids, positions, k_dst, v_dst, bpr, block_size, head_elems, tokens, stream);
}

int32_t wein_b200_conv1d_dw(const void *x, const void *w, const void *state_in, void *out, const void *tok_row,
                            const void *tok_pos, uint32_t conv_dim, uint32_t kernel, uint32_t tokens, void *stream) {
    WB_CHECK_ARG(x && w && state_in && out && tok_row && tok_pos, "conv1d_dw: null pointer");
    WB_CHECK_ARG(kernel >= 2 && kernel <= 9 && conv_dim > 0, "conv1d_dw: kernel %u outside 2..9", kernel);
    if (tokens == 0) return WB_OK;
    size_t n = (size_t)tokens * conv_dim;
    WB_LAUNCH((conv1d_dw_kernel), (unsigned)((n + 255) / 256), 256, 0, STREAM(stream), (const bf16_t *)x, (const bf16_t *)w, (const bf16_t *)state_in,
        (const uint32_t *)tok_row, (const uint32_t *)tok_pos, (bf16_t *)out, conv_dim, kernel, tokens);
    WB_LAUNCH_CHECK();
    return WB_OK;
}

int32_t wein_b200_conv_state_roll(const void *x, void *state, const void *row_start, const void *row_count, const void *row_id,
                                  uint32_t conv_dim, uint32_t kernel, uint32_t n_rows, const void *specs, void *stream) {
    WB_CHECK_ARG(x && state && row_start && row_count && row_id && specs, "conv_state_roll: null pointer");
    WB_CHECK_ARG(kernel >= 2 && kernel <= 9 && conv_dim > 0, "conv_state_roll: kernel %u outside 2..9", kernel);
    if (n_rows == 0) return WB_OK;
    size_t n = (size_t)n_rows * conv_dim;
    WB_LAUNCH((conv_state_roll_kernel), (unsigned)((n + 255) / 256), 256, 0, STREAM(stream), (const bf16_t *)x, (bf16_t *)state, (const uint32_t *)row_start,
        (const uint32_t *)row_count, (const uint32_t *)row_id, (const uint32_t *)specs, conv_dim, kernel, n_rows);
    WB_LAUNCH_CHECK();
    return WB_OK;
}

int32_t wein_b200_conv_verify(const void *x, uint32_t x_stride, const void *w, void *state, void *out, const void *row_start,
                              const void *row_count, const void *in_row, const void *out_base, uint32_t conv_dim,
                              uint32_t kernel, uint32_t n_rows, void *stream) {
    WB_CHECK_ARG(x && w && state && out && row_start && row_count && in_row && out_base, "conv_verify: null pointer");
    if (kernel != 4) { wb_set_error("conv_verify: built for kernel width 4, got %u", kernel); return WB_ERR_SHAPE; }
    WB_CHECK_ARG(x_stride >= conv_dim && conv_dim > 0, "conv_verify: x_stride %u < conv_dim %u", x_stride, conv_dim);
    if (n_rows == 0) return WB_OK;
    size_t n = (size_t)n_rows * conv_dim;
    WB_LAUNCH((conv_verify_kernel), (unsigned)((n + 127) / 128), 128, 0, STREAM(stream), (const bf16_t *)x, x_stride, (const bf16_t *)w, (bf16_t *)state,
        (const uint32_t *)row_start, (const uint32_t *)row_count, (const uint32_t *)in_row, (const uint32_t *)out_base, (bf16_t *)out, conv_dim, n_rows);
    WB_LAUNCH_CHECK();
    return WB_OK;
}

}  // extern "C"

// phase 1 only (the accept kernel merges the slices itself)
int32_t wein_b200_argmax_partials(const void *x, const void *rows, void *part, uint32_t n, uint32_t s, uint32_t split, cudaStream_t st) {
    WB_CHECK_ARG(x && rows && part && split > 0, "argmax: null pointer");
    if (s == 0) return WB_OK;
    dim3 grid(split, s);
    WB_LAUNCH((argmax_p1_kernel), grid, 256, 0, st, (const bf16_t *)x, (const uint32_t *)rows, (uint64_t *)part, n, split);
    WB_LAUNCH_CHECK();
    return WB_OK;
}

extern "C" {

// scratch: s * 32 u64 words
int32_t wein_b200_argmax_rows(const void *x, const void *rows, void *scratch, void *out, uint32_t n, uint32_t s, void *stream) {
    WB_CHECK_ARG(x && rows && scratch && out, "argmax_rows: null pointer");
    if (s == 0) return WB_OK;
    const uint32_t split = 32;
    dim3 grid(split, s);
    WB_LAUNCH((argmax_p1_kernel), grid, 256, 0, STREAM(stream), (const bf16_t *)x, (const uint32_t *)rows, (uint64_t *)scratch, n, split);
    WB_LAUNCH_CHECK();
    WB_LAUNCH((argmax_p2_kernel), s, 32, 0, STREAM(stream), (const uint64_t *)scratch, (uint32_t *)out, split);
    WB_LAUNCH_CHECK();
    return WB_OK;
}

// ---------------------------------------------------------------------------------------------------------------------
// Row argmax for callers that cannot allocate device memory.
//
// Some hosts of this library have no way to hand over a scratch buffer: a plugin that is only given the tensors of one call,
// or code that runs where cudaMalloc is forbidden (inside a region being recorded into a CUDA graph, or under a memory pool the
// embedding process owns and does not expose).  For them the per-row slice maxima of the two-phase argmax live in a fixed array
// inside the library image instead of a caller buffer.  The array costs WEIN_B200_ARGMAX_NOALLOC_MAX_ROWS * 32 * 8 bytes = 64 KiB
// on every GPU that loads the library, for the life of the process.
//
// In host code `g_argmax_static` is only a handle for the symbol, not a device address, so its address is looked up once
// per device with cudaGetSymbolAddress (with that device current) and the looked-up pointer is what the kernels receive.
#define WEIN_B200_ARGMAX_NOALLOC_MAX_ROWS 256
static __device__ __align__(256) unsigned long long g_argmax_static[WEIN_B200_ARGMAX_NOALLOC_MAX_ROWS * 32];

// Same result as wein_b200_argmax_rows, without a scratch argument and without any allocation.
//  - at most WEIN_B200_ARGMAX_NOALLOC_MAX_ROWS (256) rows per call; more is rejected with WEIN_B200_ERR_CAPACITY;
//  - the first call on each device resolves the address of the built-in array (a host-side lookup, no allocation): make
//    that first call outside any stream capture;
//  - every call on a device uses the same array.  Nothing in it needs clearing (each call overwrites all the words it reads
//    back), but two calls whose kernels may run at the same time -- different streams, or different host threads -- would
//    overwrite each other's slice maxima: serialise them on one stream.
int32_t wein_b200_argmax_rows_noalloc(const void *x, const void *rows, void *out, uint32_t n, uint32_t s, void *stream) {
    WB_CHECK_ARG(x && rows && out, "argmax_rows_noalloc: null pointer");
    if (s > WEIN_B200_ARGMAX_NOALLOC_MAX_ROWS) {
        wb_set_error("argmax_rows_noalloc: %u rows exceed the built-in scratch of %d rows; use wein_b200_argmax_rows with a caller buffer",
                     s, WEIN_B200_ARGMAX_NOALLOC_MAX_ROWS);
        return WB_ERR_CAPACITY;
    }
    if (s == 0) return WB_OK;
    static void *scratch_of_device[64] = {nullptr};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { wb_set_error("argmax_rows_noalloc: no current CUDA device"); return WB_ERR_CUDA; }
    if (!scratch_of_device[dev]) {
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_argmax_static);
        if (e != cudaSuccess || !p) { wb_set_error("argmax_rows_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e)); return WB_ERR_CUDA; }
        scratch_of_device[dev] = p;
    }
    uint64_t *scratch = (uint64_t *)scratch_of_device[dev];
    const uint32_t split = 32;
    dim3 grid(split, s);
    WB_LAUNCH((argmax_p1_kernel), grid, 256, 0, STREAM(stream), (const bf16_t *)x, (const uint32_t *)rows, scratch, n, split);
    WB_LAUNCH_CHECK();
    WB_LAUNCH((argmax_p2_kernel), s, 32, 0, STREAM(stream), (const uint64_t *)scratch, (uint32_t *)out, split);
    WB_LAUNCH_CHECK();
    return WB_OK;
}

}  // extern "C"

