// Gated-DeltaNet recurrence for chain (verify) spans and plain spans.
//
// Reference contract: `deltanet` of crates/wein-kernel/src/reference.rs:564-694
// (device twin crates/wein-kernel/kernels/src/lib.rs:5231-5411).  Per (span,
// v-head) the state S[v][k] (128x128) is loaded ONCE, kept in registers for all
// tokens of the span, and written once per chain position (one snapshot row per
// verify position) or once at the end (plain span).  The reference's chain path
// re-reads the previous row from HBM for every token.
//
// Work split: every v-row of S evolves independently given k-hat, q-hat, beta
// and decay, so a warp owns R rows; lane l holds the 4-wide k slice [4l, 4l+4)
// of each of its rows.  The reference's reduction tree for kvm and o -- a
// 4-term fused chain inside the slice, then a 32-term ascending fold over the
// slices -- is reproduced exactly: the per-slice partials go through a padded
// shared-memory transpose and lane r folds row r in slice order.  The state
// moves between HBM and registers in fully coalesced 512 B (f32) / 256 B (bf16)
// row segments; HBM traffic is (1 + positions) x 64 KiB per head in f32 mode.
//
// Bit parity with the reference holds in the bf16-pool mode (state rounded on
// every store, as the reference's pool); the f32-pool mode keeps the same tree
// without that rounding.  Compiled with -fmad=false.
#include "common.cuh"
#include "internal.h"

struct GdnParams {
    const bf16_t *q, *k, *v, *a, *b;   // per-token inputs
    uint32_t q_stride, k_stride, v_stride, ab_stride;  // elements between consecutive tokens
    const float *a_log;                // [v_heads]
    const bf16_t *dt_bias;             // [v_heads]
    void *state;                       // [rows, v_heads, 128, 128] bf16 or f32
    bf16_t *out;                       // [tokens, v_heads*128]
    const uint32_t *row_start, *row_count, *row_id, *specs, *out_base;
    uint32_t n_rows, k_heads, v_heads;
    float l2_eps;
};

template <bool F32>
struct StateIO;
template <>
struct StateIO<true> {
    static __device__ __forceinline__ void load(const void *p, size_t e, float s[4]) {
        float4 v = *reinterpret_cast<const float4 *>((const float *)p + e);
        s[0] = v.x; s[1] = v.y; s[2] = v.z; s[3] = v.w;
    }
    static __device__ __forceinline__ void store(void *p, size_t e, const float s[4]) {
        *reinterpret_cast<float4 *>((float *)p + e) = make_float4(s[0], s[1], s[2], s[3]);
    }
};
template <>
struct StateIO<false> {
    static __device__ __forceinline__ void load(const void *p, size_t e, float s[4]) {
        uint2 v = *reinterpret_cast<const uint2 *>((const bf16_t *)p + e);
        s[0] = __uint_as_float(v.x << 16); s[1] = __uint_as_float(v.x & 0xffff0000u);
        s[2] = __uint_as_float(v.y << 16); s[3] = __uint_as_float(v.y & 0xffff0000u);
    }
    static __device__ __forceinline__ void store(void *p, size_t e, const float s[4]) {
        uint2 v;  // values are already bf16-representable: narrowing is exact
        v.x = (__float_as_uint(s[0]) >> 16) | (__float_as_uint(s[1]) & 0xffff0000u);
        v.y = (__float_as_uint(s[2]) >> 16) | (__float_as_uint(s[3]) & 0xffff0000u);
        *reinterpret_cast<uint2 *>((bf16_t *)p + e) = v;
    }
};

template <int R, bool F32>
__global__ void __launch_bounds__(128) gdn_kernel(const GdnParams P) {
    PDL_ENTRY();
    constexpr int KD = 128, VD = 128, WARPS = 4;
    constexpr int SLABS = VD / (WARPS * R);
    __shared__ float T[WARPS][R][33];
    const unsigned full = 0xffffffffu;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    uint32_t unit = blockIdx.x / SLABS, slab = blockIdx.x % SLABS;
    uint32_t r = unit / P.v_heads, h = unit % P.v_heads;
    if (r >= P.n_rows) return;
    const uint32_t t0 = P.row_start[r], cnt = P.row_count[r];
    if (cnt == 0) return;
    const uint32_t spec = P.specs ? P.specs[r] : 1u;
    const size_t in_row = P.row_id[r];
    // snapshot i goes to row base+i (chain span); a plain span writes only its own row at the end
    const size_t base = P.out_base ? P.out_base[r] : (spec ? in_row + 1 : in_row);
    const uint32_t kh = h * P.k_heads / P.v_heads;
    const uint32_t row0 = slab * (WARPS * R) + w * R;
    const size_t head_elems = (size_t)VD * KD, row_elems = (size_t)P.v_heads * head_elems;

    // the one HBM read of the state: issue all loads first, latency is hidden behind the norms below
    float S[R][4];
    {
        size_t e0 = in_row * row_elems + (size_t)h * head_elems + (size_t)row0 * KD + lane * 4;
#pragma unroll
        for (int i = 0; i < R; i++) StateIO<F32>::load(P.state, e0 + (size_t)i * KD, S[i]);
    }
    const float big_a = expf_ref(P.a_log[h]);
    const float dtb = bf2f(P.dt_bias[h]);
    const float kd_sqrt = sqrtf((float)KD);

    for (uint32_t tb = 0; tb < cnt; tb += 16) {
        // l2 norms of q and k for up to 16 tokens: lane 2i sums q of token tb+i, lane 2i+1 sums k, j ascending,
        // s = x*x + s as two roundings (reference.rs:629-637)
        float inv_mine = 0.0f;
        {
            uint32_t ti = tb + (lane >> 1);
            if (ti < cnt) {
                const bf16_t *src = (lane & 1) ? P.k + (size_t)(t0 + ti) * P.k_stride + kh * KD
                                               : P.q + (size_t)(t0 + ti) * P.q_stride + kh * KD;
                float s = 0.0f;
                for (int j = 0; j < KD; j += 8) {
                    uint4 vv = *reinterpret_cast<const uint4 *>(src + j);
                    uint32_t wv[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        float x0 = __uint_as_float(wv[u] << 16), x1 = __uint_as_float(wv[u] & 0xffff0000u);
                        s = __fadd_rn(__fmul_rn(x0, x0), s);
                        s = __fadd_rn(__fmul_rn(x1, x1), s);
                    }
                }
                inv_mine = __fdiv_rn(1.0f, sqrtf(__fadd_rn(s, P.l2_eps)));
            }
        }
        uint32_t tend = min(cnt, tb + 16);
        for (uint32_t i = tb; i < tend; i++) {
            const size_t g = t0 + i;
            const float invq = __shfl_sync(full, inv_mine, (int)(2 * (i - tb)));
            const float invk = __shfl_sync(full, inv_mine, (int)(2 * (i - tb) + 1));
            // gates (reference.rs:624-626): decay = exp(-A * softplus(a + dt_bias)); beta = bf16(sigmoid(b))
            const float av = bf2f(P.a[g * P.ab_stride + h]), bv = bf2f(P.b[g * P.ab_stride + h]);
            const float decay = expf_ref(__fsub_rn(0.0f, __fmul_rn(big_a, softplus_ref(__fadd_rn(av, dtb)))));
            const float beta = rbf(sigmoid_ref(bv));
            float kk[4], qq[4];
            {
                uint2 kv = *reinterpret_cast<const uint2 *>(P.k + g * P.k_stride + kh * KD + lane * 4);
                uint2 qv = *reinterpret_cast<const uint2 *>(P.q + g * P.q_stride + kh * KD + lane * 4);
                kk[0] = __fmul_rn(__uint_as_float(kv.x << 16), invk); kk[1] = __fmul_rn(__uint_as_float(kv.x & 0xffff0000u), invk);
                kk[2] = __fmul_rn(__uint_as_float(kv.y << 16), invk); kk[3] = __fmul_rn(__uint_as_float(kv.y & 0xffff0000u), invk);
                qq[0] = __fdiv_rn(__fmul_rn(__uint_as_float(qv.x << 16), invq), kd_sqrt);
                qq[1] = __fdiv_rn(__fmul_rn(__uint_as_float(qv.x & 0xffff0000u), invq), kd_sqrt);
                qq[2] = __fdiv_rn(__fmul_rn(__uint_as_float(qv.y << 16), invq), kd_sqrt);
                qq[3] = __fdiv_rn(__fmul_rn(__uint_as_float(qv.y & 0xffff0000u), invq), kd_sqrt);
            }
            float vin = 0.0f;
            if (lane < R) vin = bf2f(P.v[g * P.v_stride + h * VD + row0 + lane]);
            // decay, then kvm partial of this lane's slice for each row
#pragma unroll
            for (int rr = 0; rr < R; rr++) {
                float p = 0.0f;
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    S[rr][u] = __fmul_rn(S[rr][u], decay);
                    p = fmaf(S[rr][u], kk[u], p);
                }
                T[w][rr][lane] = p;
            }
            __syncwarp();
            float delta = 0.0f;
            if (lane < R) {
                float kvm = 0.0f;
#pragma unroll 8
                for (int sl = 0; sl < 32; sl++) kvm = __fadd_rn(T[w][lane][sl], kvm);
                delta = __fmul_rn(__fsub_rn(vin, kvm), beta);
            }
            __syncwarp();
            // rank-1 update S += k-hat (x) delta (rounded to bf16 in the bf16 pool mode), then o partials
#pragma unroll
            for (int rr = 0; rr < R; rr++) {
                float d = __shfl_sync(full, delta, rr);
                float p = 0.0f;
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    float s = fmaf(kk[u], d, S[rr][u]);
                    if (!F32) s = rbf(s);
                    S[rr][u] = s;
                    p = fmaf(s, qq[u], p);
                }
                T[w][rr][lane] = p;
            }
            __syncwarp();
            if (lane < R) {
                float o = 0.0f;
#pragma unroll 8
                for (int sl = 0; sl < 32; sl++) o = __fadd_rn(T[w][lane][sl], o);
                P.out[g * ((size_t)P.v_heads * VD) + h * VD + row0 + lane] = f2bf(o);
            }
            __syncwarp();
            if (spec) {
                size_t e0 = (base + i) * row_elems + (size_t)h * head_elems + (size_t)row0 * KD + lane * 4;
#pragma unroll
                for (int rr = 0; rr < R; rr++) StateIO<F32>::store(P.state, e0 + (size_t)rr * KD, S[rr]);
            }
        }
    }
    if (!spec) {
        size_t e0 = base * row_elems + (size_t)h * head_elems + (size_t)row0 * KD + lane * 4;
#pragma unroll
        for (int rr = 0; rr < R; rr++) StateIO<F32>::store(P.state, e0 + (size_t)rr * KD, S[rr]);
    }
}

template <int R>
static void launch_gdn(const GdnParams &p, bool f32, cudaStream_t st) {
    unsigned grid = p.n_rows * p.v_heads * (128 / (4 * R));
    if (f32) WB_LAUNCH((gdn_kernel<R, true>), grid, 128, 0, st, p);
    else WB_LAUNCH((gdn_kernel<R, false>), grid, 128, 0, st, p);
}

static int32_t gdn_dispatch(GdnParams &p, uint32_t k_dim, uint32_t v_dim, bool f32, uint32_t rows_per_warp, cudaStream_t st) {
    if (k_dim != 128 || v_dim != 128) {
        wb_set_error("deltanet: built for k_dim = v_dim = 128, got %u x %u", k_dim, v_dim);
        return WB_ERR_SHAPE;
    }
    WB_CHECK_ARG(p.q && p.k && p.v && p.a && p.b && p.a_log && p.dt_bias && p.state && p.out && p.row_start && p.row_count && p.row_id,
                 "deltanet: null pointer");
    WB_CHECK_ARG(p.k_heads > 0 && p.v_heads > 0 && p.v_heads % p.k_heads == 0, "deltanet: v_heads %u must be a multiple of k_heads %u", p.v_heads, p.k_heads);
    WB_CHECK_ARG(((p.q_stride | p.k_stride) & 7u) == 0 && ((((uintptr_t)p.q) | ((uintptr_t)p.k)) & 15u) == 0,
                 "deltanet: q/k rows must be 16-byte aligned");
    if (p.n_rows == 0) return WB_OK;
    uint32_t R = rows_per_warp;
    if (R == 0) {  // enough warps to cover the SMs a few times over, else the fewest (less replicated gate / norm work)
        uint64_t units = (uint64_t)p.n_rows * p.v_heads;
        R = units * 4 >= 4096 ? 32 : (units * 8 >= 2048 ? 16 : 8);
    }
    if (R == 32) launch_gdn<32>(p, f32, st);
    else if (R == 16) launch_gdn<16>(p, f32, st);
    else if (R == 8) launch_gdn<8>(p, f32, st);
    else { wb_set_error("deltanet: rows_per_warp must be 0, 8, 16 or 32"); return WB_ERR_ARG; }
    WB_LAUNCH_CHECK();
    return WB_OK;
}

extern "C" {

// Same argument order as DeltanetOp::run (crates/wein-kernel/src/ops/mod.rs:888-919); the state pool is bf16.
int32_t wein_b200_deltanet(const void *q, const void *k, const void *v, const void *a, const void *b, const void *a_log,
                           const void *dt_bias, void *state, void *core_out, const void *row_start, const void *row_count,
                           const void *row_id, uint32_t n_rows, uint32_t k_heads, uint32_t v_heads, uint32_t k_dim,
                           uint32_t v_dim, uint32_t tokens, float l2_eps, const void *specs, uint32_t vsplit, void *stream) {
    (void)tokens;
    WB_CHECK_ARG(specs != nullptr, "deltanet: specs is required");
    GdnParams p{};
    p.q = (const bf16_t *)q; p.k = (const bf16_t *)k; p.v = (const bf16_t *)v; p.a = (const bf16_t *)a; p.b = (const bf16_t *)b;
    p.q_stride = p.k_stride = k_heads * k_dim; p.v_stride = v_heads * v_dim; p.ab_stride = v_heads;
    p.a_log = (const float *)a_log; p.dt_bias = (const bf16_t *)dt_bias; p.state = state; p.out = (bf16_t *)core_out;
    p.row_start = (const uint32_t *)row_start; p.row_count = (const uint32_t *)row_count; p.row_id = (const uint32_t *)row_id;
    p.specs = (const uint32_t *)specs; p.out_base = nullptr;
    p.n_rows = n_rows; p.k_heads = k_heads; p.v_heads = v_heads; p.l2_eps = l2_eps;
    // vsplit is the caller's upper bound on v-row splitting (1 = never split): 1 -> 32 rows per warp
    uint32_t R = vsplit <= 1 ? 32 : (vsplit <= 2 ? 16 : 8);
    return gdn_dispatch(p, k_dim, v_dim, false, R, (cudaStream_t)stream);
}

// Chain-shaped entry: explicit strides (q/k/v may live inside the conv output, a/b inside the projection
// output), explicit input row and snapshot base per span, bf16 or f32 state pool.
int32_t wein_b200_gdn_verify(const void *q, const void *k, const void *v, uint32_t q_stride, uint32_t k_stride, uint32_t v_stride,
                             const void *a, const void *b, uint32_t ab_stride, const void *a_log, const void *dt_bias,
                             void *state, uint32_t state_f32, void *core_out, const void *row_start, const void *row_count,
                             const void *in_row, const void *out_base, const void *specs, uint32_t n_rows, uint32_t k_heads,
                             uint32_t v_heads, uint32_t k_dim, uint32_t v_dim, float l2_eps, uint32_t rows_per_warp, void *stream) {
    GdnParams p{};
    p.q = (const bf16_t *)q; p.k = (const bf16_t *)k; p.v = (const bf16_t *)v; p.a = (const bf16_t *)a; p.b = (const bf16_t *)b;
    p.q_stride = q_stride; p.k_stride = k_stride; p.v_stride = v_stride; p.ab_stride = ab_stride;
    p.a_log = (const float *)a_log; p.dt_bias = (const bf16_t *)dt_bias; p.state = state; p.out = (bf16_t *)core_out;
    p.row_start = (const uint32_t *)row_start; p.row_count = (const uint32_t *)row_count; p.row_id = (const uint32_t *)in_row;
    p.specs = (const uint32_t *)specs; p.out_base = (const uint32_t *)out_base;
    p.n_rows = n_rows; p.k_heads = k_heads; p.v_heads = v_heads; p.l2_eps = l2_eps;
    WB_CHECK_ARG(out_base != nullptr, "gdn_verify: out_base is required");
    return gdn_dispatch(p, k_dim, v_dim, state_f32 != 0, rows_per_warp, (cudaStream_t)stream);
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------------------------
// Whole gated-DeltaNet token mixer of a layer in one launch: causal depthwise conv + SiLU on the k-head's q / k channels and
// the v-head's v channels (with the per-position conv-state rows), l2 norms, gates, the chain recurrence above, and the
// gated RMSNorm of the head's output.  Replaces conv1d_dw + conv_state_roll + dn_split_qkv + dn_qk_l2norm + deltanet +
// rms_norm_gated of the reference's layer (crates/wein-exec/src/qwen.rs:3971-4077) with bit-identical values: every
// intermediate keeps its bf16 rounding point.  One CTA = (span, v-head): 16 warps x 8 v-rows.  Spans hold <= 8 tokens.
struct GdnLayerParams {
    const bf16_t *proj;        // [tokens, ld]: raw qkv (conv_dim) | z (v_heads*128) | a (v_heads) | b (v_heads)
    uint32_t ld;
    const bf16_t *conv_w;      // [conv_dim, 4]
    bf16_t *conv_state;        // [rows, conv_dim, 3]
    const float *a_log;
    const bf16_t *dt_bias;
    const float *norm_w;       // [128]
    void *state;               // [rows, v_heads, 128, 128]
    bf16_t *out;               // [tokens, v_heads*128] gated-normalised core output
    const uint32_t *row_start, *row_count, *in_row, *out_base;
    uint32_t n_rows, k_heads, v_heads;
    float l2_eps, rms_eps;
    float *kq;                 // null: this kernel derives k-hat / q-hat itself.  Else [tokens, k_heads, 256] f32 from gdn_qk_kernel
    float *log;                // null: write a state snapshot per position.  Else [tokens, v_heads, GDN_LOG_W]: write only what a
                               // position did to the state (delta[128], k-hat[128], decay) and no state at all
};
#define GDN_LOG_W 264          // floats per (token, v-head) record: delta at 0, k-hat at 128, decay at 256; 1056 bytes, 16-byte aligned

// Measured and dropped: the 128 v-rows of a head split over a cluster of 4 CTAs of 128 threads (gated-norm leaders exchanged
// through distributed shared memory, bit-identical).  The recurrence gets faster, but every CTA repeats the q / k conv, l2
// norms and k-hat / q-hat with a quarter of the threads, and those phases are half of the kernel: 2.78 vs 2.71 ms per round
// at batch 1, 6.80 vs 6.33 ms at batch 32.
// MINB = CTAs per SM the register budget is planned for: 2 for large grids (bandwidth: more bytes in flight per SM),
// 1 for small ones (latency: no spills in the token loop)
template <bool F32, int MINB>
__global__ void __launch_bounds__(512, MINB) gdn_layer_kernel(const GdnLayerParams P) {
    PDL_ENTRY();
    constexpr int KD = 128, VD = 128, R = 8, WARPS = 16, MAXT = 8;
    __shared__ __align__(16) float T[WARPS][R][36];   // lane partials of kvm, then of o; row stride 36 words: float4 reads of 8 lanes hit disjoint banks
    __shared__ float d_s[128];                                          // delta of the head's 128 v-rows for the current token
    __shared__ __align__(16) bf16_t qc[MAXT][KD], kc[MAXT][KD], vc[MAXT][VD];
    __shared__ float o_s[MAXT][VD];
    __shared__ float inv_s[MAXT][2], gate_s[MAXT][2], red_s[4][4];
    __shared__ __align__(16) float kk_s[MAXT][KD], qq_s[MAXT][KD];
    const unsigned full = 0xffffffffu;
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const uint32_t r = blockIdx.x / P.v_heads, h = blockIdx.x % P.v_heads;
    const uint32_t t0 = P.row_start[r], cnt = min(P.row_count[r], (uint32_t)MAXT);
    if (cnt == 0) return;
    const size_t in_row = P.in_row[r], base = P.out_base[r];
    const uint32_t group = P.v_heads / P.k_heads, kh = h / group;
    const uint32_t keyd = P.k_heads * KD, vald = P.v_heads * VD, cd = 2 * keyd + vald;
    const uint32_t row0 = w * R;
    const size_t head_elems = (size_t)VD * KD, row_elems = (size_t)P.v_heads * head_elems;
    // the one HBM read of the state goes out first
    float S[R][4];
    {
        size_t e0 = in_row * row_elems + (size_t)h * head_elems + (size_t)row0 * KD + lane * 4;
#pragma unroll
        for (int i = 0; i < R; i++) StateIO<F32>::load(P.state, e0 + (size_t)i * KD, S[i]);
    }
    // operands of the closing gated norm (this thread's element of tokens grp and grp+4): fetched now, used last
    const int n_grp = tid >> 7, n_i = tid & 127;
    const float n_wv = P.norm_w[n_i];
    bf16_t n_z[2];
#pragma unroll
    for (int q2 = 0; q2 < 2; q2++) {
        uint32_t t = n_grp + 4 * q2;
        n_z[q2] = t < cnt ? P.proj[(size_t)(t0 + t) * P.ld + cd + h * VD + n_i] : (bf16_t)0;
    }
    // ---- conv + SiLU (reference.rs:476-506) and conv-state rows (reference.rs:511-562): one thread per channel
    if (P.kq && tid < 2 * KD) {
        // k-hat and q-hat of the span's tokens were made once per k-head by gdn_qk_kernel: stage them (256 floats per token)
        for (uint32_t t = 0; t < cnt; t++) {
            const float v = P.kq[((size_t)(t0 + t) * P.k_heads + kh) * 256 + tid];
            if (tid < KD) kk_s[t][tid] = v; else qq_s[t][tid - KD] = v;
        }
    } else if (tid < 3 * KD) {
        const uint32_t part = tid / KD, i = tid % KD;
        const uint32_t ch = part == 0 ? kh * KD + i : (part == 1 ? keyd + kh * KD + i : 2 * keyd + h * VD + i);
        const bool owns_state = part == 2 || (h % group) == 0;   // q / k channels are shared by the v-heads of a k-head
        const bf16_t *sp = P.conv_state + ((size_t)in_row * cd + ch) * 3;
        bf16_t w0 = sp[0], w1 = sp[1], w2 = sp[2];
        const float k0 = bf2f(P.conv_w[(size_t)ch * 4 + 0]), k1 = bf2f(P.conv_w[(size_t)ch * 4 + 1]),
                    k2 = bf2f(P.conv_w[(size_t)ch * 4 + 2]), k3 = bf2f(P.conv_w[(size_t)ch * 4 + 3]);
        bf16_t (*dst)[KD] = part == 0 ? qc : (part == 1 ? kc : vc);
        bf16_t xs[MAXT];   // all of the span's inputs first: independent loads, one round trip
#pragma unroll
        for (int t = 0; t < MAXT; t++) xs[t] = (uint32_t)t < cnt ? P.proj[(size_t)(t0 + t) * P.ld + ch] : (bf16_t)0;
#pragma unroll
        for (int t = 0; t < MAXT; t++) {
            if ((uint32_t)t >= cnt) break;
            bf16_t xv = xs[t];
            float acc = 0.0f;
            acc = __fadd_rn(__fmul_rn(bf2f(w0), k0), acc);
            acc = __fadd_rn(__fmul_rn(bf2f(w1), k1), acc);
            acc = __fadd_rn(__fmul_rn(bf2f(w2), k2), acc);
            acc = __fadd_rn(__fmul_rn(bf2f(xv), k3), acc);
            dst[t][i] = f2bf(silu_ref(rbf(acc)));
            w0 = w1; w1 = w2; w2 = xv;
            if (owns_state) {
                bf16_t *dp = P.conv_state + ((size_t)(base + t) * cd + ch) * 3;
                dp[0] = w0; dp[1] = w1; dp[2] = w2;
            }
        }
    } else if (tid < 3 * KD + MAXT) {
        // gates (reference.rs:624-626), one thread per token
        const uint32_t t = tid - 3 * KD;
        if (t < cnt) {
            const size_t g = t0 + t;
            const float av = bf2f(P.proj[g * P.ld + cd + vald + h]), bv = bf2f(P.proj[g * P.ld + cd + vald + P.v_heads + h]);
            const float big_a = expf_ref(P.a_log[h]);
            gate_s[t][0] = expf_ref(__fsub_rn(0.0f, __fmul_rn(big_a, softplus_ref(__fadd_rn(av, bf2f(P.dt_bias[h]))))));
            gate_s[t][1] = rbf(sigmoid_ref(bv));
        }
    }
    __syncthreads();
    if (!P.kq) {
    // ---- l2 norms of q and k (reference.rs:629-637): thread (t, which) sums 128 squares in order, two roundings per term
    if (tid < 2 * (int)cnt) {
        const bf16_t *src = (tid & 1) ? kc[tid >> 1] : qc[tid >> 1];
        float s = 0.0f;
        uint4 raw[KD / 8];   // the whole row first (16 vector loads), then the ordered sum
#pragma unroll
        for (int v8 = 0; v8 < KD / 8; v8++) raw[v8] = *reinterpret_cast<const uint4 *>(src + v8 * 8);
#pragma unroll
        for (int v8 = 0; v8 < KD / 8; v8++) {
            const uint32_t wv[4] = {raw[v8].x, raw[v8].y, raw[v8].z, raw[v8].w};
#pragma unroll
            for (int u = 0; u < 4; u++) {
                float x0 = __uint_as_float(wv[u] << 16), x1 = __uint_as_float(wv[u] & 0xffff0000u);
                s = __fadd_rn(__fmul_rn(x0, x0), s);
                s = __fadd_rn(__fmul_rn(x1, x1), s);
            }
        }
        inv_s[tid >> 1][tid & 1] = __fdiv_rn(1.0f, sqrtf(__fadd_rn(s, P.l2_eps)));
    }
    __syncthreads();
    // k-hat = k * invk and q-hat = (q * invq) / sqrt(128) for every token, in parallel (reference.rs:651, :675)
    {
        const float kd_sqrt = sqrtf((float)KD);
        for (uint32_t idx = tid; idx < cnt * KD; idx += 512) {
            uint32_t t = idx / KD, j = idx % KD;
            kk_s[t][j] = __fmul_rn(bf2f(kc[t][j]), inv_s[t][1]);
            qq_s[t][j] = __fdiv_rn(__fmul_rn(bf2f(qc[t][j]), inv_s[t][0]), kd_sqrt);
        }
    }
    __syncthreads();
    }   // !P.kq
    // The recurrence.  Warp w owns v-rows 8w .. 8w+7, lane l the k slice 4l .. 4l+3 of each.  A row's kvm and o are sums of 32
    // lane partials in ascending lane order (the reference's two-level tree, reference.rs:644-678): a chain of 32 dependent
    // additions that one thread must make.  The four warps of a group (32 rows) therefore hand their partials to ONE warp,
    // whose 32 lanes fold one row each: a quarter of the fold instructions of a per-warp fold on 8 lanes (the kernel is bound
    // by instruction issue at large grids); the other three wait at the group's barrier and leave the issue slots to the
    // SM's other groups.  The folding duty rotates over the group's warps.
    const int grp4 = w >> 2, wg = w & 3, grow = grp4 * 32 + lane;   // group, warp within it, the row this lane folds
    auto group_sync = [&]() {   // barrier of the group's 128 threads (hardware barriers 1..4; 0 is the CTA's)
        switch (grp4) {
            case 0: asm volatile("bar.sync 1, 128;" ::: "memory"); break;
            case 1: asm volatile("bar.sync 2, 128;" ::: "memory"); break;
            case 2: asm volatile("bar.sync 3, 128;" ::: "memory"); break;
            default: asm volatile("bar.sync 4, 128;" ::: "memory"); break;
        }
    };
    for (uint32_t i = 0; i < cnt; i++) {
        const float decay = gate_s[i][0], beta = gate_s[i][1];
        float kk[4], qq[4];
        {
            const float4 k4 = *reinterpret_cast<const float4 *>(&kk_s[i][lane * 4]), q4 = *reinterpret_cast<const float4 *>(&qq_s[i][lane * 4]);
            kk[0] = k4.x; kk[1] = k4.y; kk[2] = k4.z; kk[3] = k4.w;
            qq[0] = q4.x; qq[1] = q4.y; qq[2] = q4.z; qq[3] = q4.w;
        }
#pragma unroll
        for (int rr = 0; rr < R; rr++) {
            float p = 0.0f;
#pragma unroll
            for (int u = 0; u < 4; u++) {
                S[rr][u] = __fmul_rn(S[rr][u], decay);
                p = fmaf(S[rr][u], kk[u], p);
            }
            T[w][rr][lane] = p;
        }
        group_sync();
        if (wg == (int)((2 * i) & 3)) {
            float tv[32];   // all 32 slice partials of this lane's row first (8 vector loads in flight), then the ordered fold
            const float *src = &T[grp4 * 4 + (lane >> 3)][lane & 7][0];
#pragma unroll
            for (int v4 = 0; v4 < 8; v4++) {
                const float4 t4 = *reinterpret_cast<const float4 *>(src + v4 * 4);
                tv[v4 * 4] = t4.x; tv[v4 * 4 + 1] = t4.y; tv[v4 * 4 + 2] = t4.z; tv[v4 * 4 + 3] = t4.w;
            }
            float kvm = 0.0f;
#pragma unroll
            for (int sl = 0; sl < 32; sl++) kvm = __fadd_rn(tv[sl], kvm);
            const float delta = __fmul_rn(__fsub_rn(bf2f(vc[i][grow]), kvm), beta);
            d_s[grow] = delta;
            if (P.log) P.log[((size_t)(t0 + i) * P.v_heads + h) * GDN_LOG_W + grow] = delta;
        }
        group_sync();
#pragma unroll
        for (int rr = 0; rr < R; rr++) {
            const float d = d_s[row0 + rr];
            float p = 0.0f;
#pragma unroll
            for (int u = 0; u < 4; u++) {
                float s = fmaf(kk[u], d, S[rr][u]);
                if (!F32) s = rbf(s);
                S[rr][u] = s;
                p = fmaf(s, qq[u], p);
            }
            T[w][rr][lane] = p;
        }
        group_sync();
        if (wg == (int)((2 * i + 1) & 3)) {
            float tv[32];
            const float *src = &T[grp4 * 4 + (lane >> 3)][lane & 7][0];
#pragma unroll
            for (int v4 = 0; v4 < 8; v4++) {
                const float4 t4 = *reinterpret_cast<const float4 *>(src + v4 * 4);
                tv[v4 * 4] = t4.x; tv[v4 * 4 + 1] = t4.y; tv[v4 * 4 + 2] = t4.z; tv[v4 * 4 + 3] = t4.w;
            }
            float o = 0.0f;
#pragma unroll
            for (int sl = 0; sl < 32; sl++) o = __fadd_rn(tv[sl], o);
            o_s[i][grow] = rbf(o);   // the core output is stored as bf16 by the reference before the norm reads it
        }
        group_sync();   // the o partials have been consumed: the next token may overwrite them
        if (P.log) {
            if (w == 0) {
                float *lg = P.log + ((size_t)(t0 + i) * P.v_heads + h) * GDN_LOG_W;
                *reinterpret_cast<float4 *>(&lg[128 + lane * 4]) = make_float4(kk[0], kk[1], kk[2], kk[3]);
                if (lane == 0) lg[256] = decay;
            }
        } else {
            size_t e0 = (base + i) * row_elems + (size_t)h * head_elems + (size_t)row0 * KD + lane * 4;
#pragma unroll
            for (int rr = 0; rr < R; rr++) StateIO<F32>::store(P.state, e0 + (size_t)rr * KD, S[rr]);
        }
    }
    __syncthreads();
    // ---- gated RMSNorm over the head (reference.rs:699-713): warp-group g = tid / 128 takes tokens g, g+4
    {
        const int grp = tid >> 7, i = tid & 127, wl = (tid >> 5) & 3;
        for (uint32_t tb = 0; tb < cnt; tb += 4) {
            const uint32_t t = tb + grp;
            const bool live = t < cnt;
            float v = live ? o_s[t][i] : 0.0f;
            float s = fmaf(v, v, 0.0f);
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) {
                float o2 = __shfl_down_sync(full, s, off);
                if (lane + off < 32) s = __fadd_rn(s, o2);
            }
            if (lane == 0) red_s[grp][wl] = s;
            __syncthreads();
            // second level of the block tree over 4 warp leaders: (w0 + w2) + (w1 + w3)
            float total = __fadd_rn(__fadd_rn(red_s[grp][0], red_s[grp][2]), __fadd_rn(red_s[grp][1], red_s[grp][3]));
            __syncthreads();
            if (live) {
                float inv = 1.0f / sqrtf(total / (float)VD + P.rms_eps);
                float xw = n_wv * rbf(v * inv);
                float zv = bf2f(n_z[tb >> 2]);
                P.out[((size_t)(t0 + t) * P.v_heads + h) * VD + i] = f2bf(xw * (zv * (1.0f / (1.0f + expf_ref(-zv)))));
            }
        }
    }
}

// k-hat and q-hat once per (span, k-head) instead of once per v-head: conv + SiLU of the head's q and k channels with their
// conv-state rows, the two l2 norms and the scaling, for every token of the span.  Used in front of gdn_layer_kernel when
// the grid is large: there the layer kernel is bound by the instructions and serial chains of its CTAs, and this part is
// repeated by the v-heads that share a k-head.  Output kq [tokens, k_heads, 256] f32: k-hat then q-hat.  Same arithmetic.
__global__ void __launch_bounds__(256) gdn_qk_kernel(const GdnLayerParams P) {
    PDL_ENTRY();
    constexpr int KD = 128, VD = 128, MAXT = 8;
    __shared__ __align__(16) bf16_t qk[2][MAXT][KD];   // [0] q, [1] k
    __shared__ float inv_s[MAXT][2];
    const int tid = threadIdx.x;
    const uint32_t r = blockIdx.x / P.k_heads, kh = blockIdx.x % P.k_heads;
    const uint32_t t0 = P.row_start[r], cnt = min(P.row_count[r], (uint32_t)MAXT);
    if (cnt == 0) return;
    const size_t in_row = P.in_row[r], base = P.out_base[r];
    const uint32_t keyd = P.k_heads * KD, vald = P.v_heads * VD, cd = 2 * keyd + vald;
    {
        const uint32_t part = tid / KD, i = tid % KD;
        const uint32_t ch = part == 0 ? kh * KD + i : keyd + kh * KD + i;
        const bf16_t *sp = P.conv_state + ((size_t)in_row * cd + ch) * 3;
        bf16_t w0 = sp[0], w1 = sp[1], w2 = sp[2];
        const float k0 = bf2f(P.conv_w[(size_t)ch * 4 + 0]), k1 = bf2f(P.conv_w[(size_t)ch * 4 + 1]),
                    k2 = bf2f(P.conv_w[(size_t)ch * 4 + 2]), k3 = bf2f(P.conv_w[(size_t)ch * 4 + 3]);
        bf16_t xs[MAXT];
#pragma unroll
        for (int t = 0; t < MAXT; t++) xs[t] = (uint32_t)t < cnt ? P.proj[(size_t)(t0 + t) * P.ld + ch] : (bf16_t)0;
#pragma unroll
        for (int t = 0; t < MAXT; t++) {
            if ((uint32_t)t >= cnt) break;
            bf16_t xv = xs[t];
            float acc = 0.0f;
            acc = __fadd_rn(__fmul_rn(bf2f(w0), k0), acc);
            acc = __fadd_rn(__fmul_rn(bf2f(w1), k1), acc);
            acc = __fadd_rn(__fmul_rn(bf2f(w2), k2), acc);
            acc = __fadd_rn(__fmul_rn(bf2f(xv), k3), acc);
            qk[part][t][i] = f2bf(silu_ref(rbf(acc)));
            w0 = w1; w1 = w2; w2 = xv;
            bf16_t *dp = P.conv_state + ((size_t)(base + t) * cd + ch) * 3;
            dp[0] = w0; dp[1] = w1; dp[2] = w2;
        }
    }
    __syncthreads();
    if (tid < 2 * (int)cnt) {
        const bf16_t *src = qk[tid & 1][tid >> 1];
        float s = 0.0f;
        uint4 raw[KD / 8];
#pragma unroll
        for (int v8 = 0; v8 < KD / 8; v8++) raw[v8] = *reinterpret_cast<const uint4 *>(src + v8 * 8);
#pragma unroll
        for (int v8 = 0; v8 < KD / 8; v8++) {
            const uint32_t wv[4] = {raw[v8].x, raw[v8].y, raw[v8].z, raw[v8].w};
#pragma unroll
            for (int u = 0; u < 4; u++) {
                float x0 = __uint_as_float(wv[u] << 16), x1 = __uint_as_float(wv[u] & 0xffff0000u);
                s = __fadd_rn(__fmul_rn(x0, x0), s);
                s = __fadd_rn(__fmul_rn(x1, x1), s);
            }
        }
        inv_s[tid >> 1][tid & 1] = __fdiv_rn(1.0f, sqrtf(__fadd_rn(s, P.l2_eps)));
    }
    __syncthreads();
    const float kd_sqrt = sqrtf((float)KD);
    for (uint32_t idx = tid; idx < cnt * 256; idx += 256) {
        const uint32_t t = idx / 256, j = idx % 256;
        float v;
        if (j < (uint32_t)KD) v = __fmul_rn(bf2f(qk[1][t][j]), inv_s[t][1]);
        else v = __fdiv_rn(__fmul_rn(bf2f(qk[0][t][j - KD]), inv_s[t][0]), kd_sqrt);
        P.kq[((size_t)(t0 + t) * P.k_heads + kh) * 256 + j] = v;
    }
}

int32_t wb_gdn_layer(const void *proj, uint32_t ld, const void *conv_w, void *conv_state, const void *a_log, const void *dt_bias,
                     const void *norm_w, void *state, uint32_t state_f32, void *out, const void *row_start, const void *row_count,
                     const void *in_row, const void *out_base, uint32_t n_rows, uint32_t k_heads, uint32_t v_heads, float l2_eps,
                     float rms_eps, void *log, void *kq_scratch, cudaStream_t st) {
    WB_CHECK_ARG(proj && conv_w && conv_state && a_log && dt_bias && norm_w && state && out && row_start && row_count && in_row && out_base,
                 "gdn_layer: null pointer");
    WB_CHECK_ARG(k_heads > 0 && v_heads % k_heads == 0, "gdn_layer: v_heads %u must be a multiple of k_heads %u", v_heads, k_heads);
    if (n_rows == 0) return WB_OK;
    GdnLayerParams p{};
    p.proj = (const bf16_t *)proj; p.ld = ld; p.conv_w = (const bf16_t *)conv_w; p.conv_state = (bf16_t *)conv_state;
    p.a_log = (const float *)a_log; p.dt_bias = (const bf16_t *)dt_bias; p.norm_w = (const float *)norm_w; p.state = state;
    p.out = (bf16_t *)out; p.row_start = (const uint32_t *)row_start; p.row_count = (const uint32_t *)row_count;
    p.in_row = (const uint32_t *)in_row; p.out_base = (const uint32_t *)out_base;
    p.n_rows = n_rows; p.k_heads = k_heads; p.v_heads = v_heads; p.l2_eps = l2_eps; p.rms_eps = rms_eps; p.log = (float *)log;
    WB_CHECK_ARG(((uintptr_t)log & 15u) == 0, "gdn_layer: the update log must be 16-byte aligned");
    const bool big = (uint64_t)n_rows * v_heads >= 296;
    if (big && kq_scratch) {
        // large grid: k-hat / q-hat once per k-head in a launch of their own
        WB_CHECK_ARG(((uintptr_t)kq_scratch & 15u) == 0, "gdn_layer: the k-hat / q-hat scratch must be 16-byte aligned");
        p.kq = (float *)kq_scratch;
        WB_LAUNCH((gdn_qk_kernel), n_rows * k_heads, 256, 0, st, p);
        WB_LAUNCH_CHECK();
    }
    if (state_f32) {
        if (big) WB_LAUNCH((gdn_layer_kernel<true, 2>), n_rows * v_heads, 512, 0, st, p);
        else WB_LAUNCH((gdn_layer_kernel<true, 1>), n_rows * v_heads, 512, 0, st, p);
    } else {
        if (big) WB_LAUNCH((gdn_layer_kernel<false, 2>), n_rows * v_heads, 512, 0, st, p);
        else WB_LAUNCH((gdn_layer_kernel<false, 1>), n_rows * v_heads, 512, 0, st, p);
    }
    WB_LAUNCH_CHECK();
    return WB_OK;
}

// Chain spans of at most 8 tokens; 128x128 heads, conv width 4.  See the kernel comment for the layout of `proj`.
extern "C" int32_t wein_b200_gdn_layer(const void *proj, uint32_t ld, const void *conv_w, void *conv_state, const void *a_log,
                                       const void *dt_bias, const void *norm_w, void *state, uint32_t state_f32, void *out,
                                       const void *row_start, const void *row_count, const void *in_row, const void *out_base,
                                       uint32_t n_rows, uint32_t k_heads, uint32_t v_heads, float l2_eps, float rms_eps, void *stream) {
    return wb_gdn_layer(proj, ld, conv_w, conv_state, a_log, dt_bias, norm_w, state, state_f32, out, row_start, row_count, in_row, out_base,
                        n_rows, k_heads, v_heads, l2_eps, rms_eps, nullptr, nullptr, (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------------------------------------------------
// Snapshot-lite verification.  A state snapshot per position costs (1 + P) x 64 KiB (f32) of HBM traffic per head and
// layer, although only one of the P snapshots survives acceptance.  With a log the layer kernel above writes no state: per
// position it records what that position did to the state -- S <- decay * S, then S[r][c] <- fma(k-hat[c], delta[r], S[r][c])
// -- in 1 KiB, and once the accept length a is known gdn_commit_kernel replays records 0..a on the input state, element by
// element with the very operations of the layer kernel, and stores the one state that is kept: (1 + 1 + 1) x 64 KiB
// instead of (1 + P).  The stored row is out_base + a, i.e. the row the snapshot of position a would occupy, so the
// result is bit-identical to the snapshot path and nothing around it changes.
struct GdnCommitParams {
    void *const *states;        // [layers] state pools [rows, v_heads, 128, 128]
    const float *const *logs;   // [layers] logs [tokens, v_heads, GDN_LOG_W]
    const uint32_t *row_start, *row_count, *in_row, *out_base, *accept_len;
    uint32_t v_heads;
};

template <bool F32>
__global__ void __launch_bounds__(512) gdn_commit_kernel(const GdnCommitParams P) {
    PDL_ENTRY();
    constexpr int KD = 128, VD = 128, R = 8;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const uint32_t r = blockIdx.x / P.v_heads, h = blockIdx.x % P.v_heads, layer = blockIdx.y;
    const uint32_t cnt = P.row_count[r];
    if (cnt == 0) return;
    const uint32_t a = min(P.accept_len[r], cnt - 1), t0 = P.row_start[r];
    const size_t head_elems = (size_t)VD * KD, row_elems = (size_t)P.v_heads * head_elems;
    const uint32_t row0 = w * R;
    void *state = P.states[layer];
    const float *log = P.logs[layer];
    float S[R][4];
    {
        size_t e0 = (size_t)P.in_row[r] * row_elems + (size_t)h * head_elems + (size_t)row0 * KD + lane * 4;
#pragma unroll
        for (int i = 0; i < R; i++) StateIO<F32>::load(state, e0 + (size_t)i * KD, S[i]);
    }
    for (uint32_t i = 0; i <= a; i++) {
        const float *lg = log + ((size_t)(t0 + i) * P.v_heads + h) * GDN_LOG_W;
        const float decay = lg[256];
        const float4 k4 = *reinterpret_cast<const float4 *>(&lg[128 + lane * 4]);
        const float kk[4] = {k4.x, k4.y, k4.z, k4.w};
        float d[R];
#pragma unroll
        for (int rr = 0; rr < R; rr++) d[rr] = lg[row0 + rr];
#pragma unroll
        for (int rr = 0; rr < R; rr++)
#pragma unroll
            for (int u = 0; u < 4; u++) {
                float s = fmaf(kk[u], d[rr], __fmul_rn(S[rr][u], decay));
                if (!F32) s = rbf(s);
                S[rr][u] = s;
            }
    }
    size_t e1 = ((size_t)P.out_base[r] + a) * row_elems + (size_t)h * head_elems + (size_t)row0 * KD + lane * 4;
#pragma unroll
    for (int rr = 0; rr < R; rr++) StateIO<F32>::store(state, e1 + (size_t)rr * KD, S[rr]);
}

int32_t wb_gdn_commit(void *const *states, const float *const *logs, uint32_t n_layers, uint32_t state_f32, const void *row_start,
                      const void *row_count, const void *in_row, const void *out_base, const void *accept_len, uint32_t n_rows,
                      uint32_t v_heads, cudaStream_t st) {
    WB_CHECK_ARG(states && logs && row_start && row_count && in_row && out_base && accept_len, "gdn_commit: null pointer");
    if (n_rows == 0 || n_layers == 0) return WB_OK;
    GdnCommitParams p{};
    p.states = states; p.logs = logs; p.row_start = (const uint32_t *)row_start; p.row_count = (const uint32_t *)row_count;
    p.in_row = (const uint32_t *)in_row; p.out_base = (const uint32_t *)out_base; p.accept_len = (const uint32_t *)accept_len; p.v_heads = v_heads;
    dim3 grid(n_rows * v_heads, n_layers);
    if (state_f32) WB_LAUNCH((gdn_commit_kernel<true>), grid, 512, 0, st, p);
    else WB_LAUNCH((gdn_commit_kernel<false>), grid, 512, 0, st, p);
    WB_LAUNCH_CHECK();
    return WB_OK;
}

// The layer kernel in log mode: as wein_b200_gdn_layer, but the state pool is only read (row in_row) and `log`
// ([tokens, v_heads, 264] f32) receives one record per position and head.  No counterpart in the reference's operator set:
// it implements what the reference lists as its next step for the speculative commit.
extern "C" int32_t wein_b200_gdn_layer_lite(const void *proj, uint32_t ld, const void *conv_w, void *conv_state, const void *a_log,
                                            const void *dt_bias, const void *norm_w, const void *state, uint32_t state_f32, void *out,
                                            const void *row_start, const void *row_count, const void *in_row, const void *out_base,
                                            uint32_t n_rows, uint32_t k_heads, uint32_t v_heads, float l2_eps, float rms_eps, void *log,
                                            void *stream) {
    WB_CHECK_ARG(log != nullptr, "gdn_layer_lite: the update log is required");
    return wb_gdn_layer(proj, ld, conv_w, conv_state, a_log, dt_bias, norm_w, const_cast<void *>(state), state_f32, out, row_start, row_count,
                        in_row, out_base, n_rows, k_heads, v_heads, l2_eps, rms_eps, log, nullptr, (cudaStream_t)stream);
}

// The general form: optional update log (null = state snapshots) and optional scratch kq [tokens, k_heads, 256] f32
// (16-byte aligned, sized by the caller for all tokens of the call).  With the scratch and at least 296 (span, v-head)
// pairs, k-hat and q-hat are computed once per k-head by a launch of their own; results never depend on it.
extern "C" int32_t wein_b200_gdn_layer_ws(const void *proj, uint32_t ld, const void *conv_w, void *conv_state, const void *a_log,
                                          const void *dt_bias, const void *norm_w, void *state, uint32_t state_f32, void *out,
                                          const void *row_start, const void *row_count, const void *in_row, const void *out_base,
                                          uint32_t n_rows, uint32_t k_heads, uint32_t v_heads, float l2_eps, float rms_eps, void *log,
                                          void *kq_scratch, void *stream) {
    return wb_gdn_layer(proj, ld, conv_w, conv_state, a_log, dt_bias, norm_w, state, state_f32, out, row_start, row_count, in_row, out_base,
                        n_rows, k_heads, v_heads, l2_eps, rms_eps, log, kq_scratch, (cudaStream_t)stream);
}

// Replays the records 0..accept_len[r] of span r on state row in_row[r] and stores row out_base[r] + accept_len[r], for
// every head of `n_layers` layers in one launch.  `states` and `logs` are DEVICE arrays of n_layers device pointers.
extern "C" int32_t wein_b200_gdn_commit(const void *states, const void *logs, uint32_t n_layers, uint32_t state_f32, const void *row_start,
                                        const void *row_count, const void *in_row, const void *out_base, const void *accept_len,
                                        uint32_t n_rows, uint32_t v_heads, void *stream) {
    return wb_gdn_commit((void *const *)states, (const float *const *)logs, n_layers, state_f32, row_start, row_count, in_row, out_base,
                         accept_len, n_rows, v_heads, (cudaStream_t)stream);
}

