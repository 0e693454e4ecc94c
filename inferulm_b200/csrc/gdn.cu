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
#include <cuda.h>
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
    float *kq;                 // null: the layer kernel derives its per-token operands itself.  Else the scratch gdn_pre_kernel fills:
                               // per token and v-head a record of 388 floats = k-hat | q-hat | conv + SiLU of v (bf16) | z (bf16) | decay, beta, 0, 0
    float *log;                // null: write a state snapshot per position.  Else [tokens, v_heads, GDN_LOG_W]: write only what a
                               // position did to the state (delta[128], k-hat[128], decay) and no state at all
};
#define GDN_LOG_W 264          // floats per (token, v-head) record: delta at 0, k-hat at 128, decay at 256; 1056 bytes, 16-byte aligned

// Small grids (fewer CTAs than two per SM) and calls without a scratch: one CTA = (span, v-head) = 16 warps x 8 v-rows, lane l
// holds the 4-wide k slice [4l, 4l+4) of each of its warp's rows, and the whole prologue (conv, norms, gates) is made by the
// CTA's 512 threads.  The two ordered 32-term folds per token go through a shared-memory transpose; the four warps of a
// group hand their partials to ONE warp, whose 32 lanes fold one row each, the folding duty rotating over the group.
// MINB = CTAs per SM the register budget is planned for.
template <bool F32, int MINB>
__global__ void __launch_bounds__(512, MINB) gdn_layer_small_kernel(const GdnLayerParams P) {
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
    if (tid < 3 * KD) {
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
    {
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
    }
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


// Large grids.  Work item = (span, v-head); a CTA of 128 threads takes items blockIdx.x, blockIdx.x + gridDim.x, ... and a
// thread owns a 2 x 64 block of the head's state in registers for the whole span: v-rows 32w + 16j + g (j = 0, 1) x
// k-columns 64q .. 64q+63, with g = lane & 15 and q = lane >> 4.  A row's kvm and o are, in the reference, sums of 32 slice
// partials (4 fused terms each) folded in ascending slice order (reference.rs:644-678).  Here a thread makes the 16 slice
// partials of its half for each of its 2 rows, and the fold walks the row's two owners -- lanes 16 apart in ONE warp -- with
// one shuffle in between.  The token loop has no barrier and no shared-memory exchange; k-hat / q-hat are read from shared
// memory once per 2 rows, and the fold of a token's o runs beside the next token's first half (they are independent).
//
// Everything an item reads arrives by copies that complete on one mbarrier: the state as four tensor-map copies of 128 rows x
// 128 bytes under the 128-byte swizzle (the per-thread reads -- lanes one row apart -- are then free of bank conflicts),
// and per token ONE bulk copy of a 1552-byte record that gdn_pre_kernel made once per span: k-hat | q-hat, conv + SiLU of
// v, z, the gates (128 threads that hold a head's state are too few to make them quickly).  One thread issues them.  As
// soon as an item's state has moved into registers the copies of the CTA's NEXT item are issued, so they land while this
// item's tokens are processed: the HBM read of the state and every dependent load latency leave the critical path.  Every
// wait is bounded by a clock; a wait that gives up counts itself, and the CTA leaves after a delay.
//
// Measured and dropped: the small-grid kernel above on large grids -- 47.7 us per layer at 32 chains x 4 positions: bound by
// the chain of barriers and 32 dependent additions per fold, not by memory or issue slots; 4 x 32 blocks per thread (four fold
// passes of 8 additions: three quarters of them wasted); a whole row per thread (the broadcast reads of k-hat / q-hat then
// bound the loop); this kernel with one item per CTA and its own prologue (the serial load latencies and the prologue on
// 128 threads cost more than the recurrence); the state as one bulk copy per row into padded rows (128 copy instructions
// per item take 6,000 cycles to issue); the head split over a cluster of 4 CTAs.
template <bool F32> struct GdnStage {
    static constexpr uint32_t ROWB = F32 ? 512u : 256u;   // bytes of a state row of one head
    static constexpr uint32_t BOXES = ROWB / 128u;        // tensor-map boxes of 128 rows x 128 bytes
    static constexpr uint32_t BYTES = 128u * ROWB;
};
// per-token record of an item (scratch and shared memory): k-hat | q-hat (1024 B), conv + SiLU of v (256 B), z (256 B), decay | beta | 0 | 0
#define GDN_REC_VC 1024u
#define GDN_REC_Z 1280u
#define GDN_REC_GATE 1536u
#define GDN_REC_BYTES 1552u
#define GDN_OPS_BYTES (8u * GDN_REC_BYTES)
#define GDN_TAIL_BYTES (4096u + 256u)   // core outputs [8][128] f32, norm leaders / inverse norms
template <bool F32>
static constexpr uint32_t gdn_layer_smem() { return 1024u + GdnStage<F32>::BYTES + 2u * GDN_OPS_BYTES + GDN_TAIL_BYTES; }   // 1024: alignment slack
#define GDN_WAIT_CYCLES 2000000000ll   // about a second
__device__ unsigned int g_gdn_timeouts;   // bounded waits that gave up (that launch's results are then undefined, nothing hangs)

// floats of scratch per token: one record per v-head
__host__ __device__ __forceinline__ uint32_t gdn_pre_words(uint32_t v_heads) { return v_heads * (GDN_REC_BYTES / 4u); }

// This thread's half of state row r out of the staging area: box b holds bytes [128 b, 128 b + 128) of every row, 16-byte
// chunk c of row r at r * 128 + ((c ^ (r & 7)) << 4).
template <bool F32>
__device__ __forceinline__ void gdn_block_from(const unsigned char *stage, uint32_t r, uint32_t q, float (&S)[64]) {
    const uint32_t sw = r & 7;
    if (F32) {
#pragma unroll
        for (uint32_t cc = 0; cc < 16; cc++) {
            const float4 v = *reinterpret_cast<const float4 *>(stage + (2 * q + (cc >> 3)) * 16384 + r * 128 + (((cc & 7) ^ sw) << 4));
            S[4 * cc] = v.x; S[4 * cc + 1] = v.y; S[4 * cc + 2] = v.z; S[4 * cc + 3] = v.w;
        }
    } else {
#pragma unroll
        for (uint32_t c2 = 0; c2 < 8; c2++) {
            const uint4 raw = *reinterpret_cast<const uint4 *>(stage + q * 16384 + r * 128 + ((c2 ^ sw) << 4));
            const uint32_t wv[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int u = 0; u < 4; u++) {
                S[8 * c2 + 2 * u] = __uint_as_float(wv[u] << 16);
                S[8 * c2 + 2 * u + 1] = __uint_as_float(wv[u] & 0xffff0000u);
            }
        }
    }
}
__device__ __forceinline__ void gdn_bulk(void *dst_smem, const void *src, uint32_t bytes, uint32_t bar_a) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"((uint32_t)__cvta_generic_to_shared(dst_smem)), "l"(src), "r"(bytes), "r"(bar_a) : "memory");
}
__device__ __forceinline__ void gdn_tensor_2d(void *dst_smem, const CUtensorMap *tm, uint32_t x, uint32_t y, uint32_t bar_a) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"((uint32_t)__cvta_generic_to_shared(dst_smem)), "l"(tm), "r"(x), "r"(y), "r"(bar_a) : "memory");
}
struct GdnItem { uint32_t t0, cnt, h, in_row, base; };

template <bool F32>
__global__ void __launch_bounds__(128, 2) gdn_layer_kernel(const __grid_constant__ CUtensorMap tm_state, const GdnLayerParams P) {
    constexpr int KD = 128, VD = 128, MAXT = 8;
    constexpr uint32_t ROWB = GdnStage<F32>::ROWB;
    constexpr size_t EB = F32 ? 4 : 2;   // bytes per state word
    extern __shared__ unsigned char gsm_raw[];
    unsigned char *stage = reinterpret_cast<unsigned char *>(((uintptr_t)gsm_raw + 1023) & ~(uintptr_t)1023);   // swizzled boxes: 1024-byte aligned
    unsigned char *ops0 = stage + GdnStage<F32>::BYTES;
    float (*o_s)[VD] = reinterpret_cast<float (*)[VD]>(ops0 + 2 * GDN_OPS_BYTES);
    float (*red_s)[4] = reinterpret_cast<float (*)[4]>(ops0 + 2 * GDN_OPS_BYTES + 4096);   // [8][4]
    float *inv_s = reinterpret_cast<float *>(ops0 + 2 * GDN_OPS_BYTES + 4096 + 128);        // [8]
    __shared__ __align__(8) unsigned long long bar[2];
    __shared__ volatile uint32_t abort_s;
    const unsigned full = 0xffffffffu;
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const size_t head_elems = (size_t)VD * KD, row_elems = (size_t)P.v_heads * head_elems;
    const uint32_t W = gdn_pre_words(P.v_heads);
    const uint32_t n_items = P.n_rows * P.v_heads;
    const uint32_t g16 = lane & 15, q = lane >> 4;
    const uint32_t row_a = w * 32 + g16, row_b = row_a + 16;   // this thread's two v-rows
    const float n_wv = P.norm_w[tid];                          // a weight: no produced data
    pdl_trigger();
    if (tid == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_state) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"((uint32_t)__cvta_generic_to_shared(&bar[0])) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"((uint32_t)__cvta_generic_to_shared(&bar[1])) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        abort_s = 0;
    }
    pdl_wait();
    auto item_of = [&](uint32_t idx) {
        GdnItem it;
        it.cnt = 0; it.t0 = 0; it.h = 0; it.in_row = 0; it.base = 0;
        if (idx < n_items) {
            const uint32_t r = idx / P.v_heads;
            it.h = idx % P.v_heads;
            it.t0 = P.row_start[r];
            it.cnt = min(P.row_count[r], (uint32_t)MAXT);
            it.in_row = P.in_row[r];
            it.base = P.out_base[r];
        }
        return it;
    };
    // thread 0 announces the bytes of an item on its barrier and issues the item's copies
    auto issue = [&](const GdnItem &it, uint32_t b) {
        if (tid != 0 || !it.cnt) return;
        const uint32_t bar_a = (uint32_t)__cvta_generic_to_shared(&bar[b]);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_a), "r"(128u * ROWB + it.cnt * GDN_REC_BYTES) : "memory");
        const uint32_t y = (it.in_row * P.v_heads + it.h) * 128u;
#pragma unroll
        for (uint32_t bx = 0; bx < GdnStage<F32>::BOXES; bx++) gdn_tensor_2d(stage + bx * 16384, &tm_state, bx * (F32 ? 32u : 64u), y, bar_a);
        unsigned char *ob = ops0 + b * GDN_OPS_BYTES;
        for (uint32_t t = 0; t < it.cnt; t++)
            gdn_bulk(ob + t * GDN_REC_BYTES, P.kq + (size_t)(it.t0 + t) * W + it.h * (GDN_REC_BYTES / 4u), GDN_REC_BYTES, bar_a);
    };
    // ascending fold of a row's 32 slice partials: the owner of the upper half adds its 16 on top of the lower half's sum
    auto fold = [&](const float (&p)[2][16], float (&res)[2]) {
        float c[2] = {0.0f, 0.0f};
#pragma unroll
        for (int cc = 0; cc < 16; cc++)
#pragma unroll
            for (int j = 0; j < 2; j++) c[j] = __fadd_rn(p[j][cc], c[j]);
        float d[2];
#pragma unroll
        for (int j = 0; j < 2; j++) d[j] = __shfl_up_sync(full, c[j], 16);
#pragma unroll
        for (int cc = 0; cc < 16; cc++)
#pragma unroll
            for (int j = 0; j < 2; j++) d[j] = __fadd_rn(p[j][cc], d[j]);
#pragma unroll
        for (int j = 0; j < 2; j++) res[j] = d[j];   // complete in the lanes of the upper half (q == 1)
    };
    uint32_t idx = blockIdx.x, b = 0, ph0 = 0, ph1 = 0;
    GdnItem cur = item_of(idx), nxt = item_of(idx + gridDim.x);
    issue(cur, 0);     // (thread 0 initialised the barriers itself)
    __syncthreads();   // barriers initialised before anyone polls them
    for (; idx < n_items; idx += gridDim.x, b ^= 1) {
        GdnItem after;
        after.cnt = 0; after.t0 = 0; after.h = 0; after.in_row = 0; after.base = 0;
        const unsigned char *ob = ops0 + b * GDN_OPS_BYTES;
        float S[2][64];
        if (cur.cnt) {
            // ---- the item's copies have landed: this thread's blocks of the state move into registers
            const uint32_t bar_a = (uint32_t)__cvta_generic_to_shared(&bar[b]), parity = b ? ph1 : ph0;
            if (b) ph1 ^= 1; else ph0 ^= 1;
            const long long c0 = clock64();
            for (;;) {
                uint32_t ok;
                asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                             : "=r"(ok) : "r"(bar_a), "r"(parity) : "memory");
                if (ok || abort_s) break;
                if (clock64() - c0 > GDN_WAIT_CYCLES) { abort_s = 1; atomicAdd(&g_gdn_timeouts, 1u); break; }
            }
            gdn_block_from<F32>(stage, row_a, q, S[0]);
            gdn_block_from<F32>(stage, row_b, q, S[1]);
        }
        __syncthreads();   // the staging area and the other operand buffer are free
        if (abort_s) { __nanosleep(1000000); return; }   // a copy did not arrive: leave, after a delay that outlasts what is in flight
        issue(nxt, b ^ 1);
        if (cur.cnt) {
            const uint32_t cnt = cur.cnt, t0 = cur.t0, h = cur.h;
            // ---- the recurrence (reference.rs:639-690)
            float p2[2][16];
#pragma unroll
            for (int j = 0; j < 2; j++)
#pragma unroll
                for (int cc = 0; cc < 16; cc++) p2[j][cc] = 0.0f;
#pragma unroll 1
            for (uint32_t i = 0; i < cnt; i++) {
                const unsigned char *rec = ob + i * GDN_REC_BYTES;
                const float *kk_i = reinterpret_cast<const float *>(rec), *qq_i = kk_i + KD;
                const bf16_t *vc_i = reinterpret_cast<const bf16_t *>(rec + GDN_REC_VC);
                const float decay = reinterpret_cast<const float *>(rec + GDN_REC_GATE)[0];
                const float beta = reinterpret_cast<const float *>(rec + GDN_REC_GATE)[1];
                float p1[2][16], kvm[2], o_prev[2], delta[2];
#pragma unroll
                for (int cc = 0; cc < 16; cc++) {
                    const float4 k4 = *reinterpret_cast<const float4 *>(&kk_i[(16 * q + cc) * 4]);
                    const float kk[4] = {k4.x, k4.y, k4.z, k4.w};
#pragma unroll
                    for (int j = 0; j < 2; j++) {
                        float pj = 0.0f;
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            S[j][cc * 4 + u] = __fmul_rn(S[j][cc * 4 + u], decay);
                            pj = fmaf(S[j][cc * 4 + u], kk[u], pj);
                        }
                        p1[j][cc] = pj;
                    }
                }
                fold(p2, o_prev);   // o of the previous token: independent of the lines above, the scheduler runs them side by side
                if (i > 0 && q == 1) {
                    // the core output is stored as bf16 by the reference before the norm reads it
                    o_s[i - 1][row_a] = rbf(o_prev[0]);
                    o_s[i - 1][row_b] = rbf(o_prev[1]);
                }
                fold(p1, kvm);
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    const float d = __fmul_rn(__fsub_rn(bf2f(vc_i[j ? row_b : row_a]), kvm[j]), beta);
                    delta[j] = __shfl_sync(full, d, 16 + g16);
                }
#pragma unroll
                for (int cc = 0; cc < 16; cc++) {
                    const float4 k4 = *reinterpret_cast<const float4 *>(&kk_i[(16 * q + cc) * 4]), q4 = *reinterpret_cast<const float4 *>(&qq_i[(16 * q + cc) * 4]);
                    const float kk[4] = {k4.x, k4.y, k4.z, k4.w}, qq[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
                    for (int j = 0; j < 2; j++) {
                        float pj = 0.0f;
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            float sv = fmaf(kk[u], delta[j], S[j][cc * 4 + u]);
                            if (!F32) sv = rbf(sv);
                            S[j][cc * 4 + u] = sv;
                            pj = fmaf(sv, qq[u], pj);
                        }
                        p2[j][cc] = pj;
                    }
                }
                if (P.log) {
                    float *lg = P.log + ((size_t)(t0 + i) * P.v_heads + h) * GDN_LOG_W;
                    if (q == 1) { lg[row_a] = delta[0]; lg[row_b] = delta[1]; }
                    lg[128 + tid] = kk_i[tid];
                    if (tid == 0) lg[256] = decay;
                } else {
                    // snapshot of position i, 16 bytes per lane
                    unsigned char *st_out = (unsigned char *)P.state + (((size_t)cur.base + i) * row_elems + (size_t)h * head_elems) * EB;
#pragma unroll
                    for (int j = 0; j < 2; j++) {
                        unsigned char *rp = st_out + (size_t)(j ? row_b : row_a) * ROWB + q * (ROWB / 2);
                        if (F32) {
#pragma unroll
                            for (int cc = 0; cc < 16; cc++)
                                *reinterpret_cast<float4 *>(rp + cc * 16) = make_float4(S[j][4 * cc], S[j][4 * cc + 1], S[j][4 * cc + 2], S[j][4 * cc + 3]);
                        } else {   // values are already bf16-representable: narrowing is exact
#pragma unroll
                            for (int c2 = 0; c2 < 8; c2++) {
                                uint32_t wv[4];
#pragma unroll
                                for (int u = 0; u < 4; u++)
                                    wv[u] = (__float_as_uint(S[j][8 * c2 + 2 * u]) >> 16) | (__float_as_uint(S[j][8 * c2 + 2 * u + 1]) & 0xffff0000u);
                                *reinterpret_cast<uint4 *>(rp + c2 * 16) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
                            }
                        }
                    }
                }
            }
            after = item_of(idx + 2 * gridDim.x);   // tables of the item after next (the state registers are free now)
            {
                float o_last[2];
                fold(p2, o_last);
                if (q == 1) {
                    o_s[cnt - 1][row_a] = rbf(o_last[0]);
                    o_s[cnt - 1][row_b] = rbf(o_last[1]);
                }
            }
            __syncthreads();
            // ---- gated RMSNorm over the head (reference.rs:699-713), thread = row: every token's sum of squares by the block
            //      tree (lanes pairwise downwards, then the four warp leaders as (w0 + w2) + (w1 + w3)); thread t then makes
            //      token t's inverse norm once for all rows
            float ov[MAXT];
#pragma unroll
            for (int t = 0; t < MAXT; t++) {
                if ((uint32_t)t >= cnt) break;
                ov[t] = o_s[t][tid];
                float s2 = fmaf(ov[t], ov[t], 0.0f);
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) {
                    float o2 = __shfl_down_sync(full, s2, off);
                    if (lane + off < 32) s2 = __fadd_rn(s2, o2);
                }
                if (lane == 0) red_s[t][w] = s2;
            }
            __syncthreads();
            if ((uint32_t)tid < cnt) {
                const float total = __fadd_rn(__fadd_rn(red_s[tid][0], red_s[tid][2]), __fadd_rn(red_s[tid][1], red_s[tid][3]));
                inv_s[tid] = 1.0f / sqrtf(total / (float)VD + P.rms_eps);
            }
            __syncthreads();
#pragma unroll
            for (int t = 0; t < MAXT; t++) {
                if ((uint32_t)t >= cnt) break;
                const float xw = n_wv * rbf(ov[t] * inv_s[t]);
                const float zv = bf2f(reinterpret_cast<const bf16_t *>(ob + t * GDN_REC_BYTES + GDN_REC_Z)[tid]);
                P.out[((size_t)(t0 + t) * P.v_heads + h) * VD + tid] = f2bf(xw * (zv * (1.0f / (1.0f + expf_ref(-zv)))));
            }
        }
        if (!cur.cnt) after = item_of(idx + 2 * gridDim.x);
        cur = nxt;
        nxt = after;
    }
}

// Everything of a DeltaNet layer that is per token and not per state row, once per span instead of once per v-head CTA:
// unit < k_heads: conv + SiLU of that k-head's q and k channels with their conv-state rows, the two l2 norms and the
// scaling (k-hat, q-hat); unit >= k_heads: conv + SiLU and conv-state rows of two v-heads' channels, their z and their gates.
// Output: per token one 1552-byte record per v-head (k-hat | q-hat | conv of v | z | decay, beta), gdn_pre_words() floats.  Same arithmetic as the small-grid kernel's own prologue.
__global__ void __launch_bounds__(256) gdn_pre_kernel(const GdnLayerParams P) {
    PDL_ENTRY();
    constexpr int KD = 128, VD = 128, MAXT = 8;
    __shared__ __align__(16) bf16_t qk[2][MAXT][KD];   // [0] q, [1] k
    __shared__ float inv_s[MAXT][2];
    const int tid = threadIdx.x;
    const uint32_t units = P.k_heads + (P.v_heads + 1) / 2;
    const uint32_t r = blockIdx.x / units, unit = blockIdx.x % units;
    const uint32_t t0 = P.row_start[r], cnt = min(P.row_count[r], (uint32_t)MAXT);
    if (cnt == 0) return;
    const size_t in_row = P.in_row[r], base = P.out_base[r];
    const uint32_t keyd = P.k_heads * KD, vald = P.v_heads * VD, cd = 2 * keyd + vald;
    const uint32_t W = gdn_pre_words(P.v_heads), RW = GDN_REC_BYTES / 4u, group = P.v_heads / P.k_heads;
    const bool is_v = unit >= P.k_heads;
    const uint32_t part = tid / KD, i = tid % KD;
    const uint32_t kh = unit, h = 2 * (unit - P.k_heads) + part;
    if (is_v && h >= P.v_heads) return;
    {
        const uint32_t ch = is_v ? 2 * keyd + h * VD + i : (part == 0 ? kh * KD + i : keyd + kh * KD + i);
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
            const bf16_t y = f2bf(silu_ref(rbf(acc)));
            if (is_v) {
                float *rec = P.kq + (size_t)(t0 + t) * W + h * RW;
                reinterpret_cast<bf16_t *>(rec + GDN_REC_VC / 4u)[i] = y;
                reinterpret_cast<bf16_t *>(rec + GDN_REC_Z / 4u)[i] = P.proj[(size_t)(t0 + t) * P.ld + cd + h * VD + i];
            }
            else qk[part][t][i] = y;
            w0 = w1; w1 = w2; w2 = xv;
            bf16_t *dp = P.conv_state + ((size_t)(base + t) * cd + ch) * 3;
            dp[0] = w0; dp[1] = w1; dp[2] = w2;
        }
    }
    if (is_v) {
        if (i < cnt) {
            // gates (reference.rs:624-626), one thread per (token, head)
            const size_t g = t0 + i;
            const float av = bf2f(P.proj[g * P.ld + cd + vald + h]), bv = bf2f(P.proj[g * P.ld + cd + vald + P.v_heads + h]);
            const float big_a = expf_ref(P.a_log[h]);
            float *gp = P.kq + g * W + h * RW + GDN_REC_GATE / 4u;
            gp[0] = expf_ref(__fsub_rn(0.0f, __fmul_rn(big_a, softplus_ref(__fadd_rn(av, bf2f(P.dt_bias[h]))))));
            gp[1] = rbf(sigmoid_ref(bv));
        }
        return;
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
        for (uint32_t hh = kh * group; hh < (kh + 1) * group; hh++) P.kq[(size_t)(t0 + t) * W + hh * RW + j] = v;   // a copy per v-head of the group
    }
}

// The shared-memory opt-in is a per-device function attribute: one flag per device ordinal, set once (writing it twice from
// two threads stores the same value).
static bool g_gdn_ready[64];
static int g_gdn_sms[64];
static int32_t gdn_layer_prepare(int *sms) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { wb_set_error("gdn_layer: cudaGetDevice failed or device ordinal >= 64"); return WB_ERR_CUDA; }
    if (!g_gdn_ready[dev]) {
        int n = 0;
        cudaError_t e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gdn_layer_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gdn_layer_smem<true>());
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gdn_layer_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gdn_layer_smem<false>());
        if (e != cudaSuccess || n <= 0) { wb_set_error("gdn_layer: cannot reserve shared memory: %s", cudaGetErrorString(e)); return WB_ERR_CUDA; }
        g_gdn_sms[dev] = n;
        g_gdn_ready[dev] = true;
    }
    *sms = g_gdn_sms[dev];
    return WB_OK;
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
    const uint32_t items = n_rows * v_heads;
    // the persistent kernel needs a scratch, more work than two CTAs per SM of the small-grid kernel cover, and operands its
    // 16-byte bulk copies can address
    const bool large = kq_scratch && items >= 296 && (((uintptr_t)state | (uintptr_t)proj | (uintptr_t)kq_scratch) & 15u) == 0 && ld % 8 == 0;
    if (large) {
        int sms = 0;
        if (int32_t rc = gdn_layer_prepare(&sms)) return rc;
        p.kq = (float *)kq_scratch;
        WB_LAUNCH((gdn_pre_kernel), n_rows * (k_heads + (v_heads + 1) / 2), 256, 0, st, p);
        WB_LAUNCH_CHECK();
        // the state pool as rows of 128 words; its row count is not known here: the bound is nominal, the row indices come from
        // the caller's tables as for every other access to the pool
        alignas(64) CUtensorMap tm;
        if (int32_t rc = wb_tensor_map_2d(&tm, state_f32 != 0, state, 128, 0x7fffff00ull, state_f32 ? 512 : 256, state_f32 ? 32 : 64, 128)) return rc;
        const uint32_t grid = items < 2u * (uint32_t)sms ? items : 2u * (uint32_t)sms;
        if (state_f32) WB_LAUNCH((gdn_layer_kernel<true>), grid, 128, gdn_layer_smem<true>(), st, tm, p);
        else WB_LAUNCH((gdn_layer_kernel<false>), grid, 128, gdn_layer_smem<false>(), st, tm, p);
    } else if (state_f32) {
        // more items than SMs: the register budget that lets two CTAs share an SM (all of 256 items resident at once: 26.9 -> 25.2 us)
        if (items > 160) WB_LAUNCH((gdn_layer_small_kernel<true, 2>), items, 512, 0, st, p);
        else WB_LAUNCH((gdn_layer_small_kernel<true, 1>), items, 512, 0, st, p);
    } else {
        if (items > 160) WB_LAUNCH((gdn_layer_small_kernel<false, 2>), items, 512, 0, st, p);
        else WB_LAUNCH((gdn_layer_small_kernel<false, 1>), items, 512, 0, st, p);
    }
    WB_LAUNCH_CHECK();
    return WB_OK;
}

// Barrier waits of the large-grid layer kernel that gave up since the library was loaded (0 in a healthy run); synchronises.
extern "C" int32_t wein_b200_gdn_wait_timeouts(uint32_t *out) {
    unsigned int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_gdn_timeouts, sizeof v);
    if (e != cudaSuccess) { wb_set_error("gdn_wait_timeouts: %s", cudaGetErrorString(e)); return WB_ERR_CUDA; }
    if (out) *out = v;
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

