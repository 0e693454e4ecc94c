// Weight-streaming skinny GEMM: C[m,n] = A[m,k] * W[n,k]^T, bf16 in / f32 accumulate / bf16 out,
// for the m = batch x (draft k + 1) <= 32 rows of a verify or draft forward.
//
// Reference contract: GemmOp::run_wt (crates/wein-kernel/src/ops/mod.rs:3378-3449), a cuBLASLt call (or a
// GEMV when m == 1) whose result the reference accepts within |got - ref| <= max(2^-7 |ref|, 2^-11) of an
// f64 product (crates/wein-kernel/tests/gemm.rs:11).
//
// At these m the product is bound by streaming W from HBM once (arithmetic intensity <= 32 flop/B).  Design:
//  * one CTA = 16 consecutive weight rows x one k slice; its 8 warps split the slice 8 ways and meet in a
//    fixed-order shared-memory reduction;
//  * W goes HBM -> registers directly: lane (g, c) of a warp loads 16 contiguous bytes of rows g and g+8.
//    Those 8 bf16 feed two m16n8k16 MMAs as the A operand under a permutation of the k index that the
//    activation (B operand) loads mirror, so no shared-memory staging or ldmatrix is needed;
//  * loads are software-pipelined UNR k-blocks ahead so every lane keeps 2*UNR 16-byte loads in flight;
//  * tokens are the n = 8 dimension of the MMA: every output column is accumulated independently and in an
//    order fixed by (n, k) alone, so a token's result does not depend on which other rows share the batch
//    (batch-shape invariance: a verify row equals the same row of a plain decode step bit for bit);
//  * small n with large k (the 2560-wide output projections) additionally split k over CTAs; partials go
//    to a scratch buffer and the last CTA of a tile to arrive adds them in slice order (deterministic).
// Larger m falls through to cuBLASLt, as in the reference.
#include <cublasLt.h>
#include <mutex>
#include "common.cuh"
#include "internal.h"

__device__ __forceinline__ uint4 ld_stream(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void mma_bf16(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct WgemmParams {
    const bf16_t *A, *W;
    bf16_t *C;
    float *partial;       // [ksplit][n_tiles][MT*8*16] when ksplit > 1
    uint32_t *counters;   // [n_tiles], zero on entry, left zero
    uint32_t m, n, k, lda, ldc, ksplit, kslice;  // kslice: k elements per CTA slice (multiple of 32)
};

template <int MT>
__global__ void __launch_bounds__(256) wgemm_kernel(const WgemmParams P) {
    constexpr int WARPS = 8, UNR = 4;
    __shared__ float red[WARPS][MT][32][4];
    __shared__ uint32_t is_last;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, c = lane & 3;
    const uint32_t tile = blockIdx.x, ky = blockIdx.y, n0 = tile * 16;
    // k blocks (32 elements) of this CTA's slice, split contiguously over the warps
    const uint32_t kb0 = ky * (P.kslice / 32), kb1 = min(P.k / 32, kb0 + P.kslice / 32);
    const uint32_t nb = kb1 - kb0, per = (nb + WARPS - 1) / WARPS;
    const uint32_t b_lo = min(kb1, kb0 + warp * per), b_hi = min(kb1, b_lo + per);

    const uint32_t r0 = min(n0 + g, P.n - 1), r1 = min(n0 + g + 8, P.n - 1);  // clamp: rows past n are loaded but never stored
    const bf16_t *w0 = P.W + (size_t)r0 * P.k + c * 8, *w1 = P.W + (size_t)r1 * P.k + c * 8;
    const bf16_t *ap[MT];
    bool av[MT];
#pragma unroll
    for (int mt = 0; mt < MT; mt++) {
        uint32_t tok = mt * 8 + g;
        av[mt] = tok < P.m;
        ap[mt] = P.A + (size_t)(av[mt] ? tok : 0) * P.lda + c * 8;
    }
    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; mt++) acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.0f;

    uint4 wa[UNR], wb[UNR];
    auto issue = [&](uint32_t b) {
#pragma unroll
        for (int u = 0; u < UNR; u++) {
            uint32_t bb = min(b + u, b_hi - 1);  // tail blocks are re-read and masked below
            wa[u] = ld_stream(w0 + (size_t)bb * 32);
            wb[u] = ld_stream(w1 + (size_t)bb * 32);
        }
    };
    if (b_lo < b_hi) issue(b_lo);
    for (uint32_t b = b_lo; b < b_hi; b += UNR) {
        uint4 ca[UNR], cb[UNR];
#pragma unroll
        for (int u = 0; u < UNR; u++) { ca[u] = wa[u]; cb[u] = wb[u]; }
        uint4 xa[UNR][MT];
#pragma unroll
        for (int u = 0; u < UNR; u++) {
            uint32_t bb = min(b + u, b_hi - 1);
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
                xa[u][mt] = av[mt] ? __ldg(reinterpret_cast<const uint4 *>(ap[mt] + (size_t)bb * 32)) : make_uint4(0, 0, 0, 0);
        }
        if (b + UNR < b_hi) issue(b + UNR);
#pragma unroll
        for (int u = 0; u < UNR; u++) {
            if (b + u < b_hi) {
#pragma unroll
                for (int mt = 0; mt < MT; mt++) {
                    mma_bf16(acc[mt], ca[u].x, cb[u].x, ca[u].y, cb[u].y, xa[u][mt].x, xa[u][mt].y);
                    mma_bf16(acc[mt], ca[u].z, cb[u].z, ca[u].w, cb[u].w, xa[u][mt].z, xa[u][mt].w);
                }
            }
        }
    }
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int j = 0; j < 4; j++) red[warp][mt][lane][j] = acc[mt][j];
    __syncthreads();
    // fixed-order sum over the warps; element (mt, lane, j) is output (token mt*8 + 2c + (j&1), row g + 8*(j>>1))
    const uint32_t n_tiles = gridDim.x;
    for (int idx = threadIdx.x; idx < MT * 128; idx += 256) {
        int mt = idx >> 7, ln = (idx >> 2) & 31, j = idx & 3;
        float s = 0.0f;
#pragma unroll
        for (int w = 0; w < WARPS; w++) s += red[w][mt][ln][j];
        if (P.ksplit > 1) {
            P.partial[((size_t)ky * n_tiles + tile) * (MT * 128) + idx] = s;
        } else {
            uint32_t tok = mt * 8 + 2 * (ln & 3) + (j & 1), row = n0 + (ln >> 2) + 8 * (j >> 1);
            if (tok < P.m && row < P.n) P.C[(size_t)tok * P.ldc + row] = f2bf(s);
        }
    }
    if (P.ksplit > 1) {
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            uint32_t prev = atomicAdd(&P.counters[tile], 1u);
            is_last = (prev == P.ksplit - 1);
            if (is_last) P.counters[tile] = 0;  // every slice has arrived: safe to re-arm for the next launch
        }
        __syncthreads();
        if (is_last) {
            __threadfence();
            for (int idx = threadIdx.x; idx < MT * 128; idx += 256) {
                float s = 0.0f;
                for (uint32_t y = 0; y < P.ksplit; y++) s += __ldcg(&P.partial[((size_t)y * n_tiles + tile) * (MT * 128) + idx]);
                int mt = idx >> 7, ln = (idx >> 2) & 31, j = idx & 3;
                uint32_t tok = mt * 8 + 2 * (ln & 3) + (j & 1), row = n0 + (ln >> 2) + 8 * (j >> 1);
                if (tok < P.m && row < P.n) P.C[(size_t)tok * P.ldc + row] = f2bf(s);
            }
        }
    }
}

// How many ways to split k over CTAs: only when there are too few row tiles to fill the machine.
// Depends on (n, k) only -- never on m -- so a row's accumulation order is the same at every batch size.
static uint32_t pick_ksplit(uint32_t n, uint32_t k) {
    uint32_t tiles = (n + 15) / 16, kb = k / 32;
    uint32_t ks = 1;
    while (tiles * ks < 592 && ks < 8 && kb / (ks * 2) >= 32) ks *= 2;
    return ks;
}

extern "C" uint64_t wein_b200_gemm_scratch_bytes(uint32_t n_max) {
    // partials for the split-k shapes (n <= 592*16 rows at most 8 slices, 32 token columns) + tile counters
    uint64_t tiles = (n_max + 15) / 16;
    if (tiles > 592) tiles = 592;
    return 8ull * tiles * (4 * 128) * 4 + 4096 * 4;
}

static int32_t wgemm_launch(const void *a, const void *w, void *c, uint32_t m, uint32_t n, uint32_t k, uint32_t lda, uint32_t ldc,
                            void *scratch, uint64_t scratch_bytes, cudaStream_t st) {
    WgemmParams p{};
    p.A = (const bf16_t *)a; p.W = (const bf16_t *)w; p.C = (bf16_t *)c;
    p.m = m; p.n = n; p.k = k; p.lda = lda; p.ldc = ldc;
    uint32_t tiles = (n + 15) / 16;
    uint32_t ks = scratch ? pick_ksplit(n, k) : 1;
    int mt = (m + 7) / 8;
    if (ks > 1) {
        uint64_t need = (uint64_t)ks * tiles * (mt * 128) * 4 + 4096 * 4;
        if (tiles > 4096 || need > scratch_bytes) ks = 1;
    }
    p.ksplit = ks;
    uint32_t kb = k / 32;
    p.kslice = ((kb + ks - 1) / ks) * 32;
    p.counters = (uint32_t *)scratch;
    p.partial = scratch ? (float *)((char *)scratch + 4096 * 4) : nullptr;
    dim3 grid(tiles, ks);
    switch (mt) {
        case 1: wgemm_kernel<1><<<grid, 256, 0, st>>>(p); break;
        case 2: wgemm_kernel<2><<<grid, 256, 0, st>>>(p); break;
        case 3: wgemm_kernel<3><<<grid, 256, 0, st>>>(p); break;
        default: wgemm_kernel<4><<<grid, 256, 0, st>>>(p); break;
    }
    WB_LAUNCH_CHECK();
    return WB_OK;
}

// ---------------------------------------------------------------- cuBLASLt path (m > 32)
struct LtState {
    cublasLtHandle_t h = nullptr;
    void *ws = nullptr;
    size_t ws_bytes = 32u << 20;
    std::mutex mu;
};
static LtState g_lt;

static int32_t lt_init() {
    if (!g_lt.h) {
        if (cublasLtCreate(&g_lt.h) != CUBLAS_STATUS_SUCCESS) { wb_set_error("cublasLtCreate failed"); return WB_ERR_CUDA; }
        if (cudaMalloc(&g_lt.ws, g_lt.ws_bytes) != cudaSuccess) { wb_set_error("cuBLASLt workspace allocation failed"); return WB_ERR_CUDA; }
    }
    return WB_OK;
}
int32_t wb_gemm_warmup() {
    std::lock_guard<std::mutex> lk(g_lt.mu);
    return lt_init();
}

static int32_t lt_gemm(const void *a, const void *w, void *c, uint32_t m, uint32_t n, uint32_t k, uint32_t lda, uint32_t ldc, cudaStream_t st) {
    std::lock_guard<std::mutex> lk(g_lt.mu);
    if (lt_init() != WB_OK) return WB_ERR_CUDA;
    // column-major view: C^T [n x m] = W [n x k] * A^T [k x m]  ->  op(W) = T on the stored k x n, op(A) = N on k x m
    cublasLtMatmulDesc_t desc = nullptr;
    cublasLtMatrixLayout_t la = nullptr, lb = nullptr, lc = nullptr;
    cublasLtMatmulPreference_t pref = nullptr;
    cublasOperation_t ta = CUBLAS_OP_T, tb = CUBLAS_OP_N;
    int32_t rc = WB_ERR_CUDA;
    float alpha = 1.0f, beta = 0.0f;
    cublasLtMatmulHeuristicResult_t heur;
    int found = 0;
    if (cublasLtMatmulDescCreate(&desc, CUBLAS_COMPUTE_32F, CUDA_R_32F) != CUBLAS_STATUS_SUCCESS) goto done;
    cublasLtMatmulDescSetAttribute(desc, CUBLASLT_MATMUL_DESC_TRANSA, &ta, sizeof ta);
    cublasLtMatmulDescSetAttribute(desc, CUBLASLT_MATMUL_DESC_TRANSB, &tb, sizeof tb);
    if (cublasLtMatrixLayoutCreate(&la, CUDA_R_16BF, k, n, k) != CUBLAS_STATUS_SUCCESS) goto done;
    if (cublasLtMatrixLayoutCreate(&lb, CUDA_R_16BF, k, m, lda) != CUBLAS_STATUS_SUCCESS) goto done;
    if (cublasLtMatrixLayoutCreate(&lc, CUDA_R_16BF, n, m, ldc) != CUBLAS_STATUS_SUCCESS) goto done;
    if (cublasLtMatmulPreferenceCreate(&pref) != CUBLAS_STATUS_SUCCESS) goto done;
    cublasLtMatmulPreferenceSetAttribute(pref, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &g_lt.ws_bytes, sizeof g_lt.ws_bytes);
    if (cublasLtMatmulAlgoGetHeuristic(g_lt.h, desc, la, lb, lc, lc, pref, 1, &heur, &found) != CUBLAS_STATUS_SUCCESS || found == 0) {
        wb_set_error("cuBLASLt: no algorithm for m=%u n=%u k=%u", m, n, k);
        goto done;
    }
    if (cublasLtMatmul(g_lt.h, desc, &alpha, w, la, a, lb, &beta, c, lc, c, lc, &heur.algo, g_lt.ws, g_lt.ws_bytes, st) != CUBLAS_STATUS_SUCCESS) {
        wb_set_error("cublasLtMatmul failed for m=%u n=%u k=%u", m, n, k);
        goto done;
    }
    rc = WB_OK;
done:
    if (pref) cublasLtMatmulPreferenceDestroy(pref);
    if (lc) cublasLtMatrixLayoutDestroy(lc);
    if (lb) cublasLtMatrixLayoutDestroy(lb);
    if (la) cublasLtMatrixLayoutDestroy(la);
    if (desc) cublasLtMatmulDescDestroy(desc);
    if (rc != WB_OK && !*wein_b200_last_error_buf()) wb_set_error("cuBLASLt descriptor setup failed");
    return rc;
}

// Shared by the engine: strided rows (lda / ldc in elements) so a GEMM can write into a wider buffer.
int32_t wb_gemm_wt(const void *a, const void *w, void *c, uint32_t m, uint32_t n, uint32_t k, uint32_t lda, uint32_t ldc,
                   void *scratch, uint64_t scratch_bytes, cudaStream_t st) {
    WB_CHECK_ARG(a && w && c, "gemm_wt: null pointer");
    WB_CHECK_ARG(n > 0 && k > 0 && k % 32 == 0, "gemm_wt: k = %u must be a positive multiple of 32", k);
    WB_CHECK_ARG(lda >= k && ldc >= n && lda % 8 == 0, "gemm_wt: bad leading dimensions");
    WB_CHECK_ARG(((((uintptr_t)a) | ((uintptr_t)w)) & 15u) == 0, "gemm_wt: operands must be 16-byte aligned");
    if (m == 0) return WB_OK;
    if (m <= 32) return wgemm_launch(a, w, c, m, n, k, lda, ldc, scratch, scratch_bytes, st);
    return lt_gemm(a, w, c, m, n, k, lda, ldc, st);
}

extern "C" int32_t wein_b200_gemm_wt(const void *a, const void *w, void *c, uint32_t m, uint32_t n, uint32_t k, void *scratch,
                                     uint64_t scratch_bytes, void *stream) {
    return wb_gemm_wt(a, w, c, m, n, k, k, n, scratch, scratch_bytes, (cudaStream_t)stream);
}
