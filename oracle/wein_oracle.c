/*
 * wein_oracle.c -- CPU restatement of wein's reference kernels for the MTP
 * draft -> verify -> accept path.
 *
 * THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE.  Only the test-suite, the
 * smoke check and the CPU-baseline leg of the benchmark may load it; the CUDA
 * library never links or calls it.
 *
 * Every function restates, in plain scalar C, the arithmetic of one function of
 * the reference's crates/wein-kernel/src/reference.rs (cited per function) with
 * the same loop order and the same rounding points.  Compile with
 * -ffp-contract=off: a*b+c must stay two roundings unless fmaf() is written.
 * Pinned against the reference's golden files (paged_attn, silu, rope,
 * rms_norm, kv_scatter) and the published bf16-vs-f32 state drift figures.
 *
 * The speculative-sampling part at the end (Philox4x32-10, filtered
 * distributions, rejection sampling with residual resampling) has no
 * counterpart in the reference, whose speculative path is greedy-only
 * (crates/wein-exec/src/qwen.rs:2610-2615); it is the specification the CUDA
 * accept kernel is checked against: parity unpinned for sampled accept lengths.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

/* ---------------------------------------------------------------- scalars */

/* reference.rs:14-16 */
static inline float bf2f(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
/* reference.rs:19-23 (round to nearest even, no NaN special case) */
static inline uint16_t f2bf(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    uint32_t lsb = (u >> 16) & 1u;
    return (uint16_t)((u + 0x7fffu + lsb) >> 16);
}
static inline float rbf(float x) { return bf2f(f2bf(x)); }
static inline uint32_t fbits(float x) { uint32_t u; memcpy(&u, &x, 4); return u; }
static inline float bitsf(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

ORC_API float orc_bf16_to_f32(uint16_t h) { return bf2f(h); }
ORC_API uint16_t orc_f32_to_bf16(float x) { return f2bf(x); }

/* reference.rs:27-34 */
ORC_API float orc_splitmix_f32(uint64_t seed) {
    uint64_t z = seed + 0x9e3779b97f4a7c15ull;
    uint64_t x = z ^ (z >> 30);
    x *= 0xbf58476d1ce4e5b9ull;
    x *= 0x94d049bb133111ebull;
    uint32_t u = (uint32_t)(x >> 40);
    return bitsf((u & 0xffffffu) | 0x40000000u) - 3.0f;
}
/* tests' vec_bf16 helper (crates/wein-kernel/tests/spec_rows.rs:52-56) */
ORC_API void orc_vec_bf16(uint64_t seed_hi, int64_t n, float scale, uint16_t *out) {
    for (int64_t i = 0; i < n; i++) out[i] = f2bf(orc_splitmix_f32((uint64_t)i ^ seed_hi) * scale);
}

/* reference.rs:61-94 */
static float expf_ref(float x) {
    const float LOG2E = 1.4426950408889634f;
    const float A7 = 1.5252733804059838e-05f, A6 = 0.00015403530393381606f,
                A5 = 0.0013333558146428441f, A4 = 0.009618129107628477f,
                A3 = 0.055504108664821576f, A2 = 0.2402265069591007f,
                A1 = 0.6931471805599453f, A0 = 1.0f;
    float t = x * LOG2E;
    float kf = floorf(t);
    if (kf < -126.0f) return 0.0f;
    if (kf > 127.0f) return INFINITY;
    float f = t - kf;
    float p = A7;
    p = p * f + A6;
    p = p * f + A5;
    p = p * f + A4;
    p = p * f + A3;
    p = p * f + A2;
    p = p * f + A1;
    p = p * f + A0;
    int32_t pb = (int32_t)fbits(p);
    pb += ((int32_t)kf) << 23;
    return bitsf((uint32_t)pb);
}
ORC_API float orc_expf(float x) { return expf_ref(x); }

/* reference.rs:329-345 */
static float log2f_ref(float z) {
    const float SQRT2 = 1.4142135f, LN2 = 0.6931471805599453f;
    uint32_t bits = fbits(z);
    int32_t e = (int32_t)(bits >> 23) - 127;
    float m = bitsf((bits & 0x007fffffu) | 0x3f800000u);
    if (m > SQRT2) { m = m * 0.5f; e += 1; }
    float r = (m - 1.0f) / (m + 1.0f);
    float r2 = r * r;
    float atanh = r * (1.0f + r2 * (1.0f / 3.0f + r2 * (1.0f / 5.0f + r2 * (1.0f / 7.0f
                  + r2 * (1.0f / 9.0f + r2 * (1.0f / 11.0f))))));
    return (float)e + atanh * (2.0f / LN2);
}
/* reference.rs:348-355 */
static float softplus_ref(float x) {
    const float LN2 = 0.6931471805599453f;
    if (x > 20.0f) return x;
    return log2f_ref(1.0f + expf_ref(x)) * LN2;
}
ORC_API float orc_log2f(float z) { return log2f_ref(z); }
ORC_API float orc_softplus(float x) { return softplus_ref(x); }

static inline float sigmoid_ref(float x) { return 1.0f / (1.0f + expf_ref(0.0f - x)); }

/* ---------------------------------------------------------- elementwise */

/* reference.rs:141-148 */
ORC_API void orc_silu(const uint16_t *x, uint16_t *out, int64_t n) {
    for (int64_t i = 0; i < n; i++) {
        float v = bf2f(x[i]);
        out[i] = f2bf(v * (1.0f / (1.0f + expf_ref(-v))));
    }
}
/* reference.rs:308-313 */
ORC_API void orc_add(const uint16_t *a, const uint16_t *b, uint16_t *out, int64_t n) {
    for (int64_t i = 0; i < n; i++) out[i] = f2bf(bf2f(a[i]) + bf2f(b[i]));
}
/* reference.rs:316-321 */
ORC_API void orc_mul(const uint16_t *a, const uint16_t *b, uint16_t *out, int64_t n) {
    for (int64_t i = 0; i < n; i++) out[i] = f2bf(bf2f(a[i]) * bf2f(b[i]));
}
/* silu then mul with the bf16 rounding of the activation kept
 * (crates/wein-kernel/kernels/src/lib.rs:576-584) */
ORC_API void orc_silu_mul(const uint16_t *g, const uint16_t *u, uint16_t *out, int64_t n) {
    for (int64_t i = 0; i < n; i++) {
        float v = bf2f(g[i]);
        uint16_t act = f2bf(v * (1.0f / (1.0f + expf_ref(-v))));
        out[i] = f2bf(bf2f(act) * bf2f(u[i]));
    }
}
/* reference.rs:463-472 */
ORC_API void orc_sigmul(const uint16_t *x, const uint16_t *g, uint16_t *out, int64_t n) {
    for (int64_t i = 0; i < n; i++) {
        float v = bf2f(x[i]), s = bf2f(g[i]);
        uint16_t sig = f2bf(1.0f / (1.0f + expf_ref(-s)));
        out[i] = f2bf(v * bf2f(sig));
    }
}
/* reference.rs:298-305 */
ORC_API void orc_embed(const uint32_t *ids, const uint16_t *w, uint16_t *out, int64_t t, int64_t hidden) {
    for (int64_t i = 0; i < t; i++) memcpy(out + i * hidden, w + (int64_t)ids[i] * hidden, hidden * 2);
}

/* ---------------------------------------------------------------- norms */

/* reference.rs:39-55 */
ORC_API void orc_rms_norm(const uint16_t *x, const uint16_t *w, uint16_t *out, int64_t rows, int64_t hidden, float eps) {
    for (int64_t r = 0; r < rows; r++) {
        const uint16_t *xr = x + r * hidden;
        float acc = 0.0f;
        for (int64_t i = 0; i < hidden; i++) { float v = bf2f(xr[i]); acc = fmaf(v, v, acc); }
        float inv = 1.0f / sqrtf(acc / (float)hidden + eps);
        for (int64_t i = 0; i < hidden; i++) out[r * hidden + i] = f2bf(bf2f(xr[i]) * inv * bf2f(w[i]));
    }
}

/* reference.rs:360-393: the GPU block-reduction tree restated on scalars */
static float merge_parts(const float *s, int bdim) {
    if (bdim >= 32 && bdim % 32 == 0) {
        int nw = bdim / 32;
        float l2[32];
        for (int i = 0; i < 32; i++) l2[i] = 0.0f;
        for (int w = 0; w < nw; w++) {
            float l[32];
            memcpy(l, s + w * 32, sizeof l);
            for (int off = 16; off >= 1; off >>= 1)
                for (int i = 0; i < 32; i++)
                    if (i + off < 32) l[i] = l[i] + l[i + off];
            l2[w] = l[0];
        }
        for (int off = 16; off >= 1; off >>= 1)
            for (int i = 0; i < 32; i++)
                if (i + off < 32) l2[i] = l2[i] + l2[i + off];
        return l2[0];
    }
    float total = 0.0f;
    for (int u = 0; u < bdim; u++) total = s[u] + total;
    return total;
}
static int next_pow2(int v) { int p = 1; while (p < v) p <<= 1; return p; }
/* reference.rs:400-414 */
static float rms_block_sum(const uint16_t *x, int64_t hidden) {
    int bdim = next_pow2(hidden < 256 ? (int)hidden : 256);
    float s[256];
    for (int t = 0; t < bdim; t++) {
        float acc = 0.0f;
        for (int64_t i = t; i < hidden; i += bdim) { float v = bf2f(x[i]); acc = fmaf(v, v, acc); }
        s[t] = acc;
    }
    return merge_parts(s, bdim);
}
/* reference.rs:418-430 */
ORC_API void orc_rms_norm_zc(const uint16_t *x, const uint16_t *w, uint16_t *out, int64_t rows, int64_t hidden, float eps) {
    for (int64_t r = 0; r < rows; r++) {
        const uint16_t *xr = x + r * hidden;
        float acc = rms_block_sum(xr, hidden);
        float inv = 1.0f / sqrtf(acc / (float)hidden + eps);
        for (int64_t i = 0; i < hidden; i++)
            out[r * hidden + i] = f2bf(bf2f(xr[i]) * inv * (1.0f + bf2f(w[i])));
    }
}
/* residual add rounded to bf16, then the zero-centred norm of the rounded sum
 * (crates/wein-kernel/kernels/src/lib.rs:4674-4755) */
ORC_API void orc_add_norm_zc(const uint16_t *a, const uint16_t *b, const uint16_t *w, uint16_t *sum_out,
                             uint16_t *norm_out, int64_t rows, int64_t hidden, float eps) {
    orc_add(a, b, sum_out, rows * hidden);
    orc_rms_norm_zc(sum_out, w, norm_out, rows, hidden, eps);
}
/* reference.rs:699-713 */
ORC_API void orc_rms_norm_gated(const uint16_t *x, const uint16_t *z, const float *w, uint16_t *out,
                                int64_t rows, int64_t hidden, float eps) {
    for (int64_t r = 0; r < rows; r++) {
        const uint16_t *xr = x + r * hidden;
        float acc = rms_block_sum(xr, hidden);
        float inv = 1.0f / sqrtf(acc / (float)hidden + eps);
        for (int64_t i = 0; i < hidden; i++) {
            uint16_t xb = f2bf(bf2f(xr[i]) * inv);
            float xw = w[i] * bf2f(xb);
            float zv = bf2f(z[r * hidden + i]);
            out[r * hidden + i] = f2bf(xw * (zv * (1.0f / (1.0f + expf_ref(-zv)))));
        }
    }
}

/* ----------------------------------------------------------------- rope */

/* reference.rs:98-110 (f64 frequencies, stored f32) */
ORC_API void orc_rope_table(int64_t max_pos, int64_t rot_pairs, double base, float *cosv, float *sinv) {
    for (int64_t p = 0; p < rot_pairs; p++) {
        double inv_freq = pow(base, -((double)p) / (double)rot_pairs);
        for (int64_t t = 0; t < max_pos; t++) {
            double a = (double)t * inv_freq;
            cosv[t * rot_pairs + p] = (float)cos(a);
            sinv[t * rot_pairs + p] = (float)sin(a);
        }
    }
}
/* reference.rs:114-138 */
ORC_API void orc_rope(const uint16_t *q, const uint16_t *k, const float *cosv, const float *sinv,
                      const uint32_t *pos, int64_t tokens, int64_t rot_dim, uint16_t *oq, uint16_t *ok) {
    int64_t half = rot_dim / 2;
    for (int64_t t = 0; t < tokens; t++) {
        int64_t ti = pos[t];
        for (int64_t p = 0; p < half; p++) {
            float c = cosv[ti * half + p], s = sinv[ti * half + p];
            float x1 = bf2f(q[t * rot_dim + p]), x2 = bf2f(q[t * rot_dim + half + p]);
            oq[t * rot_dim + p] = f2bf(x1 * c - x2 * s);
            oq[t * rot_dim + half + p] = f2bf(x2 * c + x1 * s);
            x1 = bf2f(k[t * rot_dim + p]); x2 = bf2f(k[t * rot_dim + half + p]);
            ok[t * rot_dim + p] = f2bf(x1 * c - x2 * s);
            ok[t * rot_dim + half + p] = f2bf(x2 * c + x1 * s);
        }
    }
}
/* reference.rs:436-460 */
ORC_API void orc_rope_pt(const uint16_t *x, const float *cosv, const float *sinv, const uint32_t *pos,
                         int64_t tokens, int64_t rot_dim, int64_t head_dim, int64_t heads, uint16_t *out) {
    int64_t half = rot_dim / 2;
    memcpy(out, x, (size_t)(tokens * heads * head_dim) * 2);
    for (int64_t t = 0; t < tokens; t++) {
        int64_t ti = pos[t];
        for (int64_t h = 0; h < heads; h++) {
            int64_t row = t * heads * head_dim + h * head_dim;
            for (int64_t p = 0; p < half; p++) {
                float c = cosv[ti * half + p], s = sinv[ti * half + p];
                float x1 = bf2f(x[row + p]), x2 = bf2f(x[row + half + p]);
                out[row + p] = f2bf(x1 * c - x2 * s);
                out[row + half + p] = f2bf(x2 * c + x1 * s);
            }
        }
    }
}

/* ------------------------------------------------------ KV pages, attention */

/* reference.rs:192-215: writes only the addressed slots of a caller-owned pool */
ORC_API void orc_kv_scatter(const uint16_t *src_k, const uint16_t *src_v, const uint32_t *block_table,
                            const uint32_t *seq_ids, const uint32_t *positions, int64_t tokens,
                            int64_t bpr, int64_t block_size, int64_t head_elems, uint16_t *k_pool, uint16_t *v_pool) {
    for (int64_t t = 0; t < tokens; t++) {
        int64_t blk = positions[t] / block_size, off = positions[t] % block_size;
        int64_t slot = (int64_t)block_table[seq_ids[t] * bpr + blk] * block_size + off;
        memcpy(k_pool + slot * head_elems, src_k + t * head_elems, head_elems * 2);
        memcpy(v_pool + slot * head_elems, src_v + t * head_elems, head_elems * 2);
    }
}

/* reference.rs:220-279: two-pass exact softmax, j ascending */
static void paged_attn_row(const uint16_t *q, const uint16_t *k_cache, const uint16_t *v_cache,
                           const uint32_t *block_table, int64_t s, int64_t pos, float q_scale, int64_t bpr,
                           int64_t block_size, int64_t kv_heads, int64_t head_dim, int64_t kh,
                           const uint16_t *qrow, uint16_t *orow, float *sc, float *p) {
    (void)q;
    int64_t he = kv_heads * head_dim;
    float m = -INFINITY;
    for (int64_t j = 0; j <= pos; j++) {
        int64_t slot = (int64_t)block_table[s * bpr + j / block_size] * block_size + j % block_size;
        const uint16_t *kr = k_cache + slot * he + kh * head_dim;
        float dot = 0.0f;
        for (int64_t i = 0; i < head_dim; i++) dot = fmaf(bf2f(qrow[i]), bf2f(kr[i]), dot);
        sc[j] = dot * q_scale;
        m = sc[j] > m ? sc[j] : m;
    }
    float denom = 0.0f;
    for (int64_t j = 0; j <= pos; j++) { p[j] = expf_ref(sc[j] - m); denom = p[j] + denom; }
    for (int64_t e = 0; e < head_dim; e++) {
        float acc = 0.0f;
        for (int64_t j = 0; j <= pos; j++) {
            int64_t slot = (int64_t)block_table[s * bpr + j / block_size] * block_size + j % block_size;
            acc = fmaf(p[j], bf2f(v_cache[slot * he + kh * head_dim + e]), acc);
        }
        orow[e] = f2bf(acc / denom);
    }
}
ORC_API void orc_paged_attn(const uint16_t *q, const uint16_t *k_cache, const uint16_t *v_cache,
                            const uint32_t *block_table, const uint32_t *seq_ids, const uint32_t *positions,
                            uint16_t *out, float q_scale, int64_t bpr, int64_t block_size, int64_t q_heads,
                            int64_t kv_heads, int64_t head_dim, int64_t tokens, int threads) {
    int64_t maxpos = 0;
    for (int64_t t = 0; t < tokens; t++) if (positions[t] > maxpos) maxpos = positions[t];
    int64_t work = tokens * q_heads;
#pragma omp parallel num_threads(threads > 0 ? threads : 1)
    {
        float *sc = (float *)malloc((size_t)(maxpos + 1) * 4), *p = (float *)malloc((size_t)(maxpos + 1) * 4);
#pragma omp for schedule(dynamic, 1)
        for (int64_t w = 0; w < work; w++) {
            int64_t t = w / q_heads, qh = w % q_heads;
            int64_t kh = qh / (q_heads / kv_heads);
            paged_attn_row(q, k_cache, v_cache, block_table, seq_ids[t], positions[t], q_scale, bpr, block_size,
                           kv_heads, head_dim, kh, q + (t * q_heads + qh) * head_dim,
                           out + (t * q_heads + qh) * head_dim, sc, p);
        }
        free(sc); free(p);
    }
}

/* ------------------------------------------------- gated DeltaNet, conv */

/* reference.rs:476-506 */
ORC_API void orc_conv1d_dw(const uint16_t *x, const uint16_t *w, const uint16_t *state_in, const uint32_t *tok_row,
                           const uint32_t *tok_pos, int64_t tokens, int64_t conv_dim, int64_t kernel, uint16_t *out) {
    int64_t st = kernel - 1;
    for (int64_t g = 0; g < tokens; g++) {
        int64_t row = tok_row[g], p = tok_pos[g];
        for (int64_t c = 0; c < conv_dim; c++) {
            float acc = 0.0f;
            for (int64_t k = 0; k < kernel; k++) {
                int64_t idx = p - st + k;
                float v = idx < 0 ? bf2f(state_in[row * conv_dim * st + c * st + (idx + st)])
                                  : bf2f(x[(g - p + idx) * conv_dim + c]);
                acc = v * bf2f(w[c * kernel + k]) + acc;
            }
            float cv = rbf(acc);
            out[g * conv_dim + c] = f2bf(cv * (1.0f / (1.0f + expf_ref(-cv))));
        }
    }
}

/* reference.rs:511-562; state is updated in place (the reads of a span never
 * alias its writes: spec spans write rows row_id+1.., plain spans read each
 * slot before overwriting it) */
ORC_API void orc_conv_state_roll(const uint16_t *x, uint16_t *state, const uint32_t *row_start,
                                 const uint32_t *row_count, const uint32_t *row_id, const uint32_t *specs,
                                 int64_t n_rows, int64_t conv_dim, int64_t kernel) {
    int64_t st = kernel - 1;
    uint16_t tmp[16];
    for (int64_t r = 0; r < n_rows; r++) {
        int64_t t0 = row_start[r], cnt = row_count[r], rid = row_id[r];
        for (int64_t c = 0; c < conv_dim; c++) {
            const uint16_t *old = state + rid * conv_dim * st + c * st;
            if (specs[r] != 0) {
                for (int64_t ti = 0; ti < cnt; ti++) {
                    uint16_t *dst = state + (rid + ti + 1) * conv_dim * st + c * st;
                    for (int64_t j = 0; j < st; j++) {
                        int64_t li = ti + 1 - st + j;
                        dst[j] = li < 0 ? old[li + st] : x[(t0 + li) * conv_dim + c];
                    }
                }
            } else {
                for (int64_t j = 0; j < st; j++) {
                    int64_t idx = cnt - st + j;
                    tmp[j] = idx < 0 ? old[idx + st] : x[(t0 + idx) * conv_dim + c];
                }
                memcpy(state + rid * conv_dim * st + c * st, tmp, (size_t)st * 2);
            }
        }
    }
}

/* reference.rs:564-694.  state_f32 == 0: the pool is bf16 and every update is
 * rounded on store (the reference's pool).  state_f32 == 1: the pool is f32,
 * same reduction tree and fused multiply-adds, no rounding on store.
 * state_f32 == 2: f32 pool with separate multiply and add, the f32-state
 * recurrence of crates/wein-kernel/tests/ops_i1.rs:343-388 (used only to
 * reproduce that test's published drift figures).  One (span, v-head) unit: */
static void deltanet_unit(const uint16_t *q, const uint16_t *k, const uint16_t *v, const uint16_t *a,
                          const uint16_t *b, const float *a_log, const uint16_t *dt_bias, void *state,
                          int state_f32, int64_t st0, int64_t cnt, int64_t rid, int spec, int64_t h,
                          int64_t k_heads, int64_t v_heads, int64_t k_dim, int64_t v_dim, float l2_eps,
                          uint16_t *out, float *s) {
    int sep = state_f32 == 2; /* separate multiply and add, as the drift test's f32 recurrence */
    float kd_sqrt = sqrtf((float)k_dim);
    int64_t kh = h * k_heads / v_heads;
    float big_a = expf_ref(a_log[h]);
    float dtb = bf2f(dt_bias[h]);
    int e2 = (k_dim == 128 && v_dim == 128);
    int64_t rstride = v_heads * v_dim * k_dim;
    int64_t base0 = (rid * v_heads + h) * v_dim * k_dim;
    int64_t n = v_dim * k_dim;
    for (int64_t i = 0; i < cnt; i++) {
        int64_t sbase = spec == 0 ? base0 : base0 + i * rstride;
        if (state_f32) memcpy(s, (float *)state + sbase, (size_t)n * 4);
        else for (int64_t e = 0; e < n; e++) s[e] = bf2f(((uint16_t *)state)[sbase + e]);
        int64_t g = st0 + i;
        float decay = expf_ref(0.0f - big_a * softplus_ref(bf2f(a[g * v_heads + h]) + dtb));
        float beta = rbf(1.0f / (1.0f + expf_ref(0.0f - bf2f(b[g * v_heads + h]))));
        int64_t qb = (g * k_heads + kh) * k_dim;
        float sq = 0.0f, sk = 0.0f;
        for (int64_t j = 0; j < k_dim; j++) {
            float qv = bf2f(q[qb + j]), kv = bf2f(k[qb + j]);
            sq = qv * qv + sq;
            sk = kv * kv + sk;
        }
        float invq = 1.0f / sqrtf(sq + l2_eps);
        float invk = 1.0f / sqrtf(sk + l2_eps);
        for (int64_t vv = 0; vv < v_dim; vv++) {
            float *srow = s + vv * k_dim;
            for (int64_t j = 0; j < k_dim; j++) srow[j] *= decay;
            float kvm = 0.0f;
            if (e2) {
                for (int sl = 0; sl < 32; sl++) {
                    float p = 0.0f;
                    for (int u = 0; u < 4; u++) {
                        float kk = bf2f(k[qb + sl * 4 + u]) * invk;
                        p = sep ? srow[sl * 4 + u] * kk + p : fmaf(srow[sl * 4 + u], kk, p);
                    }
                    kvm = p + kvm;
                }
            } else {
                for (int64_t j = 0; j < k_dim; j++) kvm = fmaf(srow[j], bf2f(k[qb + j]) * invk, kvm);
            }
            float vin = bf2f(v[(g * v_heads + h) * v_dim + vv]);
            float delta = (vin - kvm) * beta;
            for (int64_t j = 0; j < k_dim; j++) {
                float kk = bf2f(k[qb + j]) * invk;
                srow[j] = sep ? kk * delta + srow[j] : state_f32 ? fmaf(kk, delta, srow[j]) : rbf(fmaf(kk, delta, srow[j]));
            }
            float o = 0.0f;
            if (e2) {
                for (int sl = 0; sl < 32; sl++) {
                    float p = 0.0f;
                    for (int u = 0; u < 4; u++) {
                        float qq = (bf2f(q[qb + sl * 4 + u]) * invq) / kd_sqrt;
                        p = sep ? srow[sl * 4 + u] * qq + p : fmaf(srow[sl * 4 + u], qq, p);
                    }
                    o = p + o;
                }
            } else {
                for (int64_t j = 0; j < k_dim; j++) o = fmaf(srow[j], (bf2f(q[qb + j]) * invq) / kd_sqrt, o);
            }
            out[(g * v_heads + h) * v_dim + vv] = f2bf(o);
        }
        int64_t wbase = spec == 0 ? sbase : sbase + rstride;
        if (state_f32) memcpy((float *)state + wbase, s, (size_t)n * 4);
        else for (int64_t e = 0; e < n; e++) ((uint16_t *)state)[wbase + e] = f2bf(s[e]);
    }
}
ORC_API void orc_deltanet(const uint16_t *q, const uint16_t *k, const uint16_t *v, const uint16_t *a,
                          const uint16_t *b, const float *a_log, const uint16_t *dt_bias, void *state,
                          int state_f32, uint16_t *out, const uint32_t *row_start, const uint32_t *row_count,
                          const uint32_t *row_id, const uint32_t *specs, int64_t n_rows, int64_t k_heads,
                          int64_t v_heads, int64_t k_dim, int64_t v_dim, float l2_eps, int threads) {
    int64_t work = n_rows * v_heads;
#pragma omp parallel num_threads(threads > 0 ? threads : 1)
    {
        float *s = (float *)malloc((size_t)(v_dim * k_dim) * 4);
#pragma omp for schedule(dynamic, 1)
        for (int64_t w = 0; w < work; w++) {
            int64_t r = w / v_heads, h = w % v_heads;
            deltanet_unit(q, k, v, a, b, a_log, dt_bias, state, state_f32, row_start[r], row_count[r], row_id[r],
                          specs[r] != 0, h, k_heads, v_heads, k_dim, v_dim, l2_eps, out, s);
        }
        free(s);
    }
}

/* ------------------------------------------------------ argmax, sampler */

/* reference.rs:717-733: total order (value desc, index asc) */
static uint32_t argmax_row(const uint16_t *x, int64_t n) {
    float bv = -INFINITY;
    uint32_t bi = 0xffffffffu;
    for (int64_t i = 0; i < n; i++) {
        float v = bf2f(x[i]);
        if (v > bv || (v == bv && (uint32_t)i < bi)) { bv = v; bi = (uint32_t)i; }
    }
    return bi;
}
ORC_API void orc_argmax_rows(const uint16_t *x, const uint32_t *rows, int64_t s, int64_t n, uint32_t *out, int threads) {
#pragma omp parallel for num_threads(threads > 0 ? threads : 1)
    for (int64_t r = 0; r < s; r++) out[r] = argmax_row(x + (int64_t)rows[r] * n, n);
}

/* reference.rs:756-775 */
ORC_API uint64_t orc_rng_seed(uint64_t seed) {
    uint64_t x = seed + 0x9e3779b97f4a7c15ull;
    x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
    x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
    return (x ^ (x >> 31)) | 1ull;
}
static uint32_t rng_next(uint64_t *st) {
    uint64_t old = *st;
    *st = old * 6364136223846793005ull + 1442695040888963407ull;
    uint32_t x = (uint32_t)(((old >> 18) ^ old) >> 27);
    uint32_t rot = (uint32_t)(old >> 59);
    return (x >> rot) | (x << ((32 - rot) & 31));
}
static float rng_f32(uint64_t *st) { return (float)(rng_next(st) >> 8) * (1.0f / 16777216.0f); }
ORC_API uint32_t orc_rng_next(uint64_t *st) { return rng_next(st); }

/* Steps 2-4 of reference.rs:787-877 shared by the plain sampler and the
 * speculative one: scale by 1/temp, take the top-k (k clamped to 64) in the
 * total order (value desc, index asc), softmax numerators e_j = expf(v_j - m)
 * accumulated in descending order, top-p cut on the running sum of e_j/denom.
 * Returns the number of selected entries (0 if none); *keep gets the cut. */
static int filter_row(const uint16_t *x, int64_t n, float temp, uint32_t top_k, float top_p,
                      float *sel_v, uint32_t *sel_i, float *e, float *denom_out, int *keep_out) {
    int k = (int)(top_k < 64 ? top_k : 64);
    float pp = (top_p > 0.0f && top_p < 1.0f) ? top_p : 1.0f;
    float inv_t = 1.0f / temp;
    int len = 0;
    for (int64_t i = 0; i < n; i++) {
        float v = bf2f(x[i]) * inv_t;
        uint32_t ii = (uint32_t)i;
        int pos = len;
        for (int j = 0; j < len; j++)
            if (v > sel_v[j] || (v == sel_v[j] && ii < sel_i[j])) { pos = j; break; }
        if (pos < k) {
            int last = len < k ? len : k - 1;
            for (int j = last; j > pos; j--) { sel_v[j] = sel_v[j - 1]; sel_i[j] = sel_i[j - 1]; }
            sel_v[pos] = v; sel_i[pos] = ii;
            if (len < k) len++;
        }
    }
    if (len == 0) return 0;
    float m = sel_v[0], denom = 0.0f;
    for (int j = 0; j < len; j++) { e[j] = expf_ref(sel_v[j] - m); denom = e[j] + denom; }
    float c = 0.0f;
    int keep = 1;
    for (int j = 0; j < len; j++) {
        c = e[j] / denom + c;
        keep = j + 1;
        if (c >= pp) break;
    }
    *denom_out = denom;
    *keep_out = keep;
    return len;
}

/* reference.rs:787-877 */
ORC_API void orc_sample_rows(const uint16_t *x, const uint32_t *rows, int64_t s, int64_t n, const float *temp,
                             const uint32_t *top_k, const float *top_p, const uint64_t *seed,
                             const uint32_t *slots, uint64_t *rng, uint32_t *out) {
    for (int64_t blk = 0; blk < s; blk++) {
        const uint16_t *xr = x + (int64_t)rows[blk] * n;
        float t = temp[blk];
        if (!(t > 0.0f)) { out[blk] = argmax_row(xr, n); continue; }
        if (top_k[blk] == 0) { out[blk] = 0xffffffffu; continue; }
        float sel_v[64], e[64], denom;
        uint32_t sel_i[64];
        int keep;
        int len = filter_row(xr, n, t, top_k[blk], top_p[blk], sel_v, sel_i, e, &denom, &keep);
        if (len == 0) { out[blk] = 0xffffffffu; continue; }
        uint64_t st = rng[slots[blk]];
        if (st == 0) st = orc_rng_seed(seed[blk]);
        float u = rng_f32(&st);
        rng[slots[blk]] = st;
        float acc = 0.0f;
        int pick = keep - 1;
        for (int j = 0; j < keep; j++) {
            acc = e[j] / denom + acc;
            if (u < acc) { pick = j; break; }
        }
        out[blk] = sel_i[pick];
    }
}

/* reference.rs:881-893 (f64 accumulate; tolerance reference for GEMM) */
ORC_API void orc_gemm_wt(const uint16_t *a, const uint16_t *w, double *c, int64_t m, int64_t n, int64_t k, int threads) {
#pragma omp parallel for num_threads(threads > 0 ? threads : 1) schedule(static)
    for (int64_t col = 0; col < n; col++)
        for (int64_t r = 0; r < m; r++) {
            double acc = 0.0;
            for (int64_t i = 0; i < k; i++) acc += (double)bf2f(a[r * k + i]) * (double)bf2f(w[col * k + i]);
            c[r * n + col] = acc;
        }
}
/* the CPU model mirror's GEMM: f64 accumulate, one rounding to bf16
 * (crates/wein-exec/src/qwen_ref.rs gemm_bf16) */
ORC_API void orc_gemm_wt_bf16(const uint16_t *a, const uint16_t *w, uint16_t *c, int64_t m, int64_t n, int64_t k, int threads) {
#pragma omp parallel for num_threads(threads > 0 ? threads : 1) schedule(static)
    for (int64_t col = 0; col < n; col++)
        for (int64_t r = 0; r < m; r++) {
            double acc = 0.0;
            for (int64_t i = 0; i < k; i++) acc += (double)bf2f(a[r * k + i]) * (double)bf2f(w[col * k + i]);
            c[r * n + col] = f2bf((float)acc);
        }
}

/* ------------------------------------------------ speculative acceptance */

/* Greedy longest-prefix acceptance of one chain
 * (crates/wein-exec/src/qwen.rs:2433-2460): target[j] is the argmax of verify
 * row j; accept while drafts[a] == target[a]; emitted = drafts[..a] followed
 * by the bonus token target[a].  Returns a. */
ORC_API int orc_accept_greedy(const uint32_t *drafts, int k, const uint32_t *target, uint32_t *emitted) {
    int a = 0;
    while (a < k && drafts[a] == target[a]) a++;
    for (int j = 0; j < a; j++) emitted[j] = drafts[j];
    emitted[a] = target[a];
    return a;
}

/* Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3",
 * SC'11): counter ctr[4], key key[2], ten rounds. */
ORC_API void orc_philox4x32(const uint32_t ctr[4], const uint32_t key[2], uint32_t out[4]) {
    uint32_t c0 = ctr[0], c1 = ctr[1], c2 = ctr[2], c3 = ctr[3], k0 = key[0], k1 = key[1];
    for (int r = 0; r < 10; r++) {
        uint64_t p0 = (uint64_t)0xD2511F53u * c0, p1 = (uint64_t)0xCD9E8D57u * c2;
        uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0;
        uint32_t n1 = (uint32_t)p1;
        uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
        uint32_t n3 = (uint32_t)p0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}
/* The uniforms of one (sequence, round, chain position): key = the sequence's
 * 64-bit seed, counter = (round lo, round hi, position, stream).  stream 0
 * serves the draft sampler, stream 1 the accept kernel.  Lane 0 = the draw
 * that picks a token from a distribution, lane 1 = the accept test. */
static void spec_uniforms(uint64_t seed, uint64_t round, uint32_t position, uint32_t stream, float u[4]) {
    uint32_t ctr[4] = {(uint32_t)round, (uint32_t)(round >> 32), position, stream};
    uint32_t key[2] = {(uint32_t)seed, (uint32_t)(seed >> 32)}, o[4];
    orc_philox4x32(ctr, key, o);
    for (int i = 0; i < 4; i++) u[i] = (float)(o[i] >> 8) * (1.0f / 16777216.0f);
}
ORC_API void orc_spec_uniforms(uint64_t seed, uint64_t round, uint32_t position, uint32_t stream, float *u) {
    spec_uniforms(seed, round, position, stream, u);
}

/* The filtered, renormalised distribution of one logits row: the `keep`
 * highest entries after temperature / top-k / top-p, probabilities
 * e_j / sum_{j<keep} e_j with the sum accumulated in descending order.
 * ids/probs hold 64 slots; returns keep (0 = invalid parameters). */
ORC_API int orc_filtered_dist(const uint16_t *x, int64_t n, float temp, uint32_t top_k, float top_p,
                              uint32_t *ids, float *probs) {
    if (!(temp > 0.0f) || top_k == 0) return 0;
    float sel_v[64], e[64], denom;
    uint32_t sel_i[64];
    int keep;
    int len = filter_row(x, n, temp, top_k, top_p, sel_v, sel_i, e, &denom, &keep);
    if (len == 0) return 0;
    float z = 0.0f;
    for (int j = 0; j < keep; j++) z = e[j] + z;
    for (int j = 0; j < keep; j++) { ids[j] = sel_i[j]; probs[j] = e[j] / z; }
    for (int j = keep; j < 64; j++) { ids[j] = 0xffffffffu; probs[j] = 0.0f; }
    return keep;
}
/* Inverse-CDF pick in descending order; the last entry absorbs rounding. */
static int pick_from(const float *probs, int n, float u) {
    float acc = 0.0f;
    for (int j = 0; j < n; j++) { acc = probs[j] + acc; if (u < acc) return j; }
    return n - 1;
}
ORC_API uint32_t orc_draft_sample(const uint32_t *ids, const float *probs, int n, uint64_t seed, uint64_t round,
                                  uint32_t position) {
    float u[4];
    spec_uniforms(seed, round, position, 0, u);
    return ids[pick_from(probs, n, u[0])];
}

/* Rejection sampling of one chain (Leviathan et al. 2023 / Chen et al. 2023):
 * p_ids/p_probs [k+1][64] are the filtered target distributions of the k+1
 * verify rows (p_n their sizes), q_ids/q_probs [k][64] those the drafts were
 * drawn from.  Draft j is accepted iff u * q(x_j) < p(x_j); at the first
 * rejection the token is redrawn from max(p - q, 0) renormalised (target
 * order); after k acceptances the bonus token is drawn from row k.
 * Returns the accept length a; emitted gets a+1 tokens. */
ORC_API int orc_accept_sampled(const uint32_t *drafts, int k, const uint32_t *p_ids, const float *p_probs,
                               const int *p_n, const uint32_t *q_ids, const float *q_probs, const int *q_n,
                               uint64_t seed, uint64_t round, uint32_t *emitted) {
    int a = 0;
    for (; a < k; a++) {
        const uint32_t *pi = p_ids + a * 64, *qi = q_ids + a * 64;
        const float *pp = p_probs + a * 64, *qp = q_probs + a * 64;
        float u[4];
        spec_uniforms(seed, round, (uint32_t)a, 1, u);
        float px = 0.0f, qx = 0.0f;
        for (int j = 0; j < p_n[a]; j++) if (pi[j] == drafts[a]) px = pp[j];
        for (int j = 0; j < q_n[a]; j++) if (qi[j] == drafts[a]) qx = qp[j];
        if (u[1] * qx < px) { emitted[a] = drafts[a]; continue; }
        float r[64], z = 0.0f;
        for (int j = 0; j < p_n[a]; j++) {
            float qj = 0.0f;
            for (int t = 0; t < q_n[a]; t++) if (qi[t] == pi[j]) qj = qp[t];
            float d = pp[j] - qj;
            r[j] = d > 0.0f ? d : 0.0f;
            z = r[j] + z;
        }
        if (!(z > 0.0f)) { emitted[a] = pi[0]; return a; }
        for (int j = 0; j < p_n[a]; j++) r[j] = r[j] / z;
        emitted[a] = pi[pick_from(r, p_n[a], u[0])];
        return a;
    }
    float u[4];
    spec_uniforms(seed, round, (uint32_t)k, 1, u);
    emitted[k] = p_ids[k * 64 + pick_from(p_probs + k * 64, p_n[k], u[0])];
    return k;
}
