// Weight-streaming skinny GEMM: C[m,n] = A[m,k] * W[n,k]^T, bf16 in / f32 accumulate / bf16 out,
// for the m = batch x (draft k + 1) <= 32 rows of a verify or draft forward.
//
// Reference contract: GemmOp::run_wt (crates/wein-kernel/src/ops/mod.rs:3378-3449), a cuBLASLt call (or a
// GEMV when m == 1) whose result the reference accepts within |got - ref| <= max(2^-7 |ref|, 2^-11) of an
// f64 product (crates/wein-kernel/tests/gemm.rs:11).
//
// At these m the product is bound by streaming W from HBM once (arithmetic intensity <= 32 flop/B).  Design:
//  * a row tile is 16 consecutive weight rows; KW warps (1..8, chosen from (n, k) so that about two CTAs per SM are
//    resident) split the tile's k range and meet in a fixed-order shared-memory reduction; a CTA of 8 warps holds
//    8/KW tiles;
//  * W goes HBM -> registers directly: lane (g, c) of a warp loads 16 contiguous bytes of rows g and g+8.
//    Those 8 bf16 feed two m16n8k16 MMAs as the A operand under a permutation of the k index that the
//    activation (B operand) loads mirror, so no shared-memory staging or ldmatrix is needed;
//  * loads are software-pipelined UNR k-blocks ahead so every lane keeps 2*UNR 16-byte loads in flight;
//  * tokens are the n = 8 dimension of the MMA: every output column is accumulated independently and in an
//    order fixed by (n, k) alone, so a token's result does not depend on which other rows share the batch
//    (batch-shape invariance: a verify row equals the same row of a plain decode step bit for bit);
//  * small n with large k (the 2560-wide output projections) additionally split k over CTAs; partials go
//    to a scratch buffer and the last CTA of a tile to arrive adds them in slice order (deterministic).
// Larger m runs the tensor-memory kernel of gemm_umma.cu (the reference hands those shapes to cuBLASLt).
#include "common.cuh"
#include "internal.h"

__device__ __forceinline__ uint4 ld_stream(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
// Activations are produced by the predecessor kernel, and this kernel starts before that one ends (programmatic dependent
// launch): they must never go through the non-coherent path.  Coherent load, cached in L1 (re-read by the CTA's 8/KW tiles).
__device__ __forceinline__ uint4 ld_act(const void *p) {
    uint4 v;
    asm volatile("ld.global.ca.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void mma_bf16(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct WgemmParams {
    const bf16_t *A, *W;
    bf16_t *C;
    float *partial;       // [ksplit][ctas][8/KW tiles * MT*128] when ksplit > 1
    uint32_t *counters;   // [ctas], zero on entry, left zero
    uint32_t m, n, k, lda, ldc, ksplit, kslice;  // kslice: k elements per CTA slice (multiple of 32)
    uint32_t pf_row_bytes; // per weight row of a warp's slab: how far ahead of the register window the pre-wait L2 prefetch reaches
    uint32_t swiglu;      // 1: W = [gate; up] (n = 2*inter rows); tile rows 0-7 are gate rows, 8-15 the matching up rows, and
                          //    the epilogue writes bf16(bf16(silu(bf16 g)) * bf16 u) into C[m, inter]
};

// One CTA = 8 warps = 8/KW row tiles of 16 weight rows; the KW warps of a tile split the CTA's k slice contiguously.
// UNR = depth of the weight window (k-blocks in flight per lane), XD = depth of the activation window (XD divides UNR).
// Every variant is built for at least two resident CTAs per SM: CTAs are short-lived (a few microseconds), and with one per
// SM nothing streams while a CTA retires and its successor starts (measured at m = 24: 3.0 -> 3.8 TB/s from 1 -> 2 CTAs).
// Measured and dropped for m > 16: deeper weight windows with one CTA per SM (16 deep: 2.5 TB/s), several row tiles per warp
// sharing one activation fragment (no gain: activations are not the limit), an L1 evict_last hint on activations.
template <int MT, int KW, int UNR, int XD>
__global__ void __launch_bounds__(256, (MT == 1 && UNR <= 4) ? 3 : 2) wgemm_kernel(const WgemmParams P) {
    pdl_trigger();
    constexpr int WARPS = 8, TPC = WARPS / KW;  // tiles per CTA
    __shared__ float red[WARPS][MT][32][4];
    __shared__ uint32_t is_last;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, c = lane & 3;
    const int tic = warp / KW, kp = warp % KW;
    const uint32_t ky = blockIdx.y;
    const uint32_t half_n = P.n >> 1;
    const uint32_t n_tiles = P.swiglu ? (half_n + 7) / 8 : (P.n + 15) / 16;
    const uint32_t tile = blockIdx.x * TPC + tic;
    const bool tile_ok = tile < n_tiles;
    // weight rows of this lane: plain tile = rows n0+g, n0+g+8; SwiGLU tile = gate row j0+g and up row inter+j0+g
    uint32_t r0, r1;
    if (P.swiglu) { uint32_t j = min(tile * 8 + g, half_n - 1); r0 = j; r1 = half_n + j; }
    else { r0 = min(tile * 16 + g, P.n - 1); r1 = min(tile * 16 + g + 8, P.n - 1); }
    if (!tile_ok) { r0 = 0; r1 = 0; }
    const uint32_t kb0 = ky * (P.kslice / 32), kb1 = min(P.k / 32, kb0 + P.kslice / 32);
    const uint32_t nb = kb1 - kb0, per = (nb + KW - 1) / KW;
    const uint32_t b_lo = min(kb1, kb0 + kp * per), b_hi = tile_ok ? min(kb1, b_lo + per) : b_lo;

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

    // Rolling register window, UNR k-blocks deep: slot u holds block b+u; as soon as a slot's MMAs are issued its
    // registers are refilled with block b+u+UNR, so 2*UNR weight loads stay in flight per lane with UNR*8 registers.
    static_assert(UNR % XD == 0, "activation window must divide the weight window");
    uint4 wa[UNR], wb[UNR], xa[XD][MT];
#pragma unroll
    for (int u = 0; u < UNR; u++) {
        wa[u] = wb[u] = make_uint4(0, 0, 0, 0);
        if (b_lo + u < b_hi) { wa[u] = ld_stream(w0 + (size_t)(b_lo + u) * 32); wb[u] = ld_stream(w1 + (size_t)(b_lo + u) * 32); }
    }
    // Weights are never written by the stream: pull this warp's slab towards L2 while the predecessor kernel is still
    // running (one 128-byte line per lane and step: lane -> row lane/2 of the tile, line lane%2 + 2*step)
    {
        const uint32_t row = lane >> 1;
        uint32_t rr;
        if (P.swiglu) { uint32_t j = min(tile * 8 + (row & 7), half_n - 1); rr = (row < 8) ? j : half_n + j; }
        else rr = min(tile * 16 + row, P.n - 1);
        const char *base = reinterpret_cast<const char *>(P.W + (size_t)rr * P.k + (size_t)b_lo * 32);
        const uint32_t bytes = min((b_hi - b_lo) * 64, P.pf_row_bytes);
        if (tile_ok)
            for (uint32_t off = (lane & 1) * 128 + UNR * 64; off < bytes; off += 256)
                asm volatile("prefetch.global.L2 [%0];" ::"l"(base + off));
    }
    pdl_wait();
#pragma unroll
    for (int u = 0; u < XD; u++)
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
            xa[u][mt] = (av[mt] && b_lo + u < b_hi) ? ld_act(ap[mt] + (size_t)(b_lo + u) * 32) : make_uint4(0, 0, 0, 0);
    for (uint32_t b = b_lo; b < b_hi; b += UNR) {
#pragma unroll
        for (int u = 0; u < UNR; u++) {
            if (b + u < b_hi) {
#pragma unroll
                for (int mt = 0; mt < MT; mt++) {
                    mma_bf16(acc[mt], wa[u].x, wb[u].x, wa[u].y, wb[u].y, xa[u % XD][mt].x, xa[u % XD][mt].y);
                    mma_bf16(acc[mt], wa[u].z, wb[u].z, wa[u].w, wb[u].w, xa[u % XD][mt].z, xa[u % XD][mt].w);
                }
            }
            const uint32_t nb2 = b + u + UNR, nx2 = b + u + XD;
            if (nb2 < b_hi) {
                wa[u] = ld_stream(w0 + (size_t)nb2 * 32);
                wb[u] = ld_stream(w1 + (size_t)nb2 * 32);
                if constexpr (XD == UNR) {
#pragma unroll
                    for (int mt = 0; mt < MT; mt++)
                        if (av[mt]) xa[u][mt] = ld_act(ap[mt] + (size_t)nb2 * 32);
                }
            }
            if constexpr (XD != UNR) {
                if (nx2 < b_hi) {
#pragma unroll
                    for (int mt = 0; mt < MT; mt++)
                        if (av[mt]) xa[u % XD][mt] = ld_act(ap[mt] + (size_t)nx2 * 32);
                }
            }
        }
    }
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int j = 0; j < 4; j++) red[warp][mt][lane][j] = acc[mt][j];
    __syncthreads();
    // element (tile t, mt, lane, j) is output (token mt*8 + 2c + (j&1), tile row g + 8*(j>>1)); fixed-order sum over the tile's warps
    auto emit = [&](int idx, float s, float s_hi) {
        int t = idx / (MT * 128), rem = idx % (MT * 128);
        int mt = rem >> 7, ln = (rem >> 2) & 31, j = rem & 3;
        uint32_t tl = blockIdx.x * TPC + t, tok = mt * 8 + 2 * (ln & 3) + (j & 1);
        if (tl >= n_tiles || tok >= P.m) return;
        if (P.swiglu) {
            if (j >= 2) return;  // handled together with its gate element
            uint32_t col = tl * 8 + (ln >> 2);
            if (col >= half_n) return;
            float gv = rbf(s), uv = rbf(s_hi);
            P.C[(size_t)tok * P.ldc + col] = f2bf(__fmul_rn(rbf(silu_ref(gv)), uv));
        } else {
            uint32_t row = tl * 16 + (ln >> 2) + 8 * (j >> 1);
            if (row < P.n) P.C[(size_t)tok * P.ldc + row] = f2bf(s);
        }
    };
    constexpr int PER_CTA = TPC * MT * 128;
    for (int idx = threadIdx.x; idx < PER_CTA; idx += 256) {
        int t = idx / (MT * 128), rem = idx % (MT * 128);
        int mt = rem >> 7, ln = (rem >> 2) & 31, j = rem & 3;
        float s = 0.0f, s_hi = 0.0f;
#pragma unroll
        for (int w = 0; w < KW; w++) s += red[t * KW + w][mt][ln][j];
        if (P.ksplit > 1) {
            P.partial[((size_t)ky * gridDim.x + blockIdx.x) * PER_CTA + idx] = s;
        } else {
            if (P.swiglu && j < 2) {
#pragma unroll
                for (int w = 0; w < KW; w++) s_hi += red[t * KW + w][mt][ln][j + 2];
            }
            emit(idx, s, s_hi);
        }
    }
    if (P.ksplit > 1) {
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            uint32_t prev = atomicAdd(&P.counters[blockIdx.x], 1u);
            is_last = (prev == P.ksplit - 1);
            if (is_last) P.counters[blockIdx.x] = 0;  // every slice has arrived: safe to re-arm for the next launch
        }
        __syncthreads();
        if (is_last) {
            __threadfence();
            for (int idx = threadIdx.x; idx < PER_CTA; idx += 256) {
                float s = 0.0f, s_hi = 0.0f;
                for (uint32_t y = 0; y < P.ksplit; y++) s += __ldcg(&P.partial[((size_t)y * gridDim.x + blockIdx.x) * PER_CTA + idx]);
                if (P.swiglu && (idx & 3) < 2)
                    for (uint32_t y = 0; y < P.ksplit; y++) s_hi += __ldcg(&P.partial[((size_t)y * gridDim.x + blockIdx.x) * PER_CTA + idx + 2]);
                emit(idx, s, s_hi);
            }
        }
    }
}

// Decomposition of a product: KW warps per row tile inside a CTA, ksplit k slices over CTAs.  It depends on (n, k)
// only -- never on m -- so a row's accumulation order is the same at every batch size.
struct WgemmPlan { uint32_t kw, ksplit; };
// Reach of the pre-wait L2 prefetch per weight row (bytes from the start of the warp's slab; the register window covers
// the first UNR x 64).  Measured on the captured round: prefetching the whole slab floods the memory system while the small
// kernel in front of this GEMM (a residual norm of 40 KB) is on the critical path -- its interval grows from ~2.4 to 4.8 us.
// Whole slab 2.714 ms per round, nothing 2.705, 512 B 2.663, 640-768 B 2.612-2.622, 1024 B 2.66, 2048 B 2.68.  Loading fewer slots
// of the register window before the wait was worse (none 2.78, half 2.64).
constexpr uint32_t WG_PF_ROW_BYTES = 768;

static WgemmPlan plan_for(uint32_t n_tiles, uint32_t k, bool has_scratch) {
    // Measured on B200 (graph replay, weights rotated through 3 GB, m = 4): the fewest warps per tile that still give
    // about two CTAs per SM win (tiles 1152 -> kw 2: 5.4 TB/s; 640-772 -> kw 4: 5.3 TB/s; 160 -> kw 8: 4.2-4.3 TB/s); the
    // vocabulary projection (9496 tiles) prefers kw 4 (6.2 TB/s).  Splitting k over CTAs never won: off by default.
    uint32_t kb = k / 32, kw = 1, ks = 1;
    while (kw < 8 && (n_tiles * kw + 7) / 8 < 280 && kb / (kw * 2) >= 4) kw *= 2;
    if (n_tiles >= 4096 && kb >= 32) kw = 4;
    (void)has_scratch;
    return {kw, ks};
}

extern "C" uint64_t wein_b200_gemm_scratch_bytes(uint32_t n_max) {
    // split-k partials: at most 8 slices x 296 CTAs x (8 tiles x 4 token tiles x 128) floats, plus the CTA counters
    (void)n_max;
    return 8ull * 592 * (8 * 4 * 128) * 4 + 4096 * 4;
}

template <int MT, int KW>
static void wgemm_go(const WgemmParams &p, dim3 grid, uint32_t unr, cudaStream_t st) {
    if constexpr (MT == 1) {
        if (unr == 8) { WB_LAUNCH((wgemm_kernel<MT, KW, 8, 8>), grid, 256, 0, st, p); return; }
        if (unr == 6) { WB_LAUNCH((wgemm_kernel<MT, KW, 6, 6>), grid, 256, 0, st, p); return; }
    }
    if constexpr (MT == 4) {
        // 25..32 rows: a 6-deep weight window with activations fetched 2 blocks ahead is what fits 128 registers
        WB_LAUNCH((wgemm_kernel<MT, KW, 6, 2>), grid, 256, 0, st, p); return;
    }
    WB_LAUNCH((wgemm_kernel<MT, KW, 4, 4>), grid, 256, 0, st, p);
}
template <int MT>
static void wgemm_go_kw(const WgemmParams &p, dim3 grid, uint32_t kw, uint32_t unr, cudaStream_t st) {
    switch (kw) {
        case 1: wgemm_go<MT, 1>(p, grid, unr, st); break;
        case 2: wgemm_go<MT, 2>(p, grid, unr, st); break;
        case 4: wgemm_go<MT, 4>(p, grid, unr, st); break;
        default: wgemm_go<MT, 8>(p, grid, unr, st); break;
    }
}

static int32_t wgemm_launch(const void *a, const void *w, void *c, uint32_t m, uint32_t n, uint32_t k, uint32_t lda, uint32_t ldc,
                            void *scratch, uint64_t scratch_bytes, bool swiglu, cudaStream_t st) {
    WgemmParams p{};
    p.A = (const bf16_t *)a; p.W = (const bf16_t *)w; p.C = (bf16_t *)c;
    p.m = m; p.n = n; p.k = k; p.lda = lda; p.ldc = ldc; p.swiglu = swiglu ? 1 : 0; p.pf_row_bytes = WG_PF_ROW_BYTES;
    uint32_t tiles = swiglu ? (n / 2 + 7) / 8 : (n + 15) / 16;
    int mt = (m + 7) / 8;
    WgemmPlan pl = plan_for(tiles, k, scratch != nullptr);
    uint32_t tpc = 8 / pl.kw, ctas = (tiles + tpc - 1) / tpc;
    if (pl.ksplit > 1) {
        uint64_t need = (uint64_t)pl.ksplit * ctas * (tpc * mt * 128) * 4 + 4096 * 4;
        if (ctas > 4096 || need > scratch_bytes) pl.ksplit = 1;
    }
    p.ksplit = pl.ksplit;
    uint32_t kb = k / 32;
    p.kslice = ((kb + pl.ksplit - 1) / pl.ksplit) * 32;
    p.counters = (uint32_t *)scratch;
    p.partial = scratch ? (float *)((char *)scratch + 4096 * 4) : nullptr;
    dim3 grid(ctas, pl.ksplit);
    uint32_t unr = ctas * pl.ksplit <= 296 ? 8 : 4;
    switch (mt) {
        case 1: wgemm_go_kw<1>(p, grid, pl.kw, unr, st); break;
        case 2: wgemm_go_kw<2>(p, grid, pl.kw, unr, st); break;
        case 3: wgemm_go_kw<3>(p, grid, pl.kw, unr, st); break;
        default: wgemm_go_kw<4>(p, grid, pl.kw, unr, st); break;
    }
    WB_LAUNCH_CHECK();
    return WB_OK;
}

// Which kernel multiplies.  The skinny kernel and the tensor-memory kernel each keep a token's sum independent of the batch,
// but they do not agree with each other bit for bit, so a caller that compares forwards of different row counts (a verify
// forward against a plain decode step) must run all of them on one kernel: WB_GEMM_TC for every m when any of them exceeds
// 32 rows.  WB_GEMM_AUTO picks by m alone.
int32_t wb_gemm_init() { return wb_ugemm_init(); }

// Shared by the engine: strided rows (lda / ldc in elements) so a GEMM can write into a wider buffer.
int32_t wb_gemm_wt(const void *a, const void *w, void *c, uint32_t m, uint32_t n, uint32_t k, uint32_t lda, uint32_t ldc,
                   void *scratch, uint64_t scratch_bytes, uint32_t path, cudaStream_t st) {
    WB_CHECK_ARG(a && w && c, "gemm_wt: null pointer");
    WB_CHECK_ARG(n > 0 && k > 0 && k % 32 == 0, "gemm_wt: k = %u must be a positive multiple of 32", k);
    WB_CHECK_ARG(lda >= k && ldc >= n && lda % 8 == 0, "gemm_wt: bad leading dimensions");
    WB_CHECK_ARG(((((uintptr_t)a) | ((uintptr_t)w)) & 15u) == 0, "gemm_wt: operands must be 16-byte aligned");
    if (m == 0) return WB_OK;
    if (m <= 32 && path != WB_GEMM_TC) return wgemm_launch(a, w, c, m, n, k, lda, ldc, scratch, scratch_bytes, false, st);
    return wb_ugemm(a, w, c, m, n, k, lda, ldc, false, st);
}

// Fused gate|up projection + SwiGLU activation: W = [gate; up] of shape [2*inter, k]; out[m, inter] =
// bf16(bf16(silu(bf16(a.gate_j))) * bf16(a.up_j)) -- the values silu_mul produces from the separately rounded
// projections (kernels/src/lib.rs:576-584 of the reference), without materialising them.
int32_t wb_gemm_swiglu(const void *a, const void *w_gate_up, void *out, uint32_t m, uint32_t inter, uint32_t k, uint32_t lda,
                       uint32_t ldc, void *scratch, uint64_t scratch_bytes, uint32_t path, cudaStream_t st) {
    WB_CHECK_ARG(a && w_gate_up && out, "gemm_swiglu: null pointer");
    WB_CHECK_ARG(inter > 0 && k > 0 && k % 32 == 0, "gemm_swiglu: k = %u must be a positive multiple of 32", k);
    WB_CHECK_ARG(lda >= k && ldc >= inter && lda % 8 == 0, "gemm_swiglu: bad leading dimensions");
    WB_CHECK_ARG(((((uintptr_t)a) | ((uintptr_t)w_gate_up)) & 15u) == 0, "gemm_swiglu: operands must be 16-byte aligned");
    if (m == 0) return WB_OK;
    if (m <= 32 && path != WB_GEMM_TC) return wgemm_launch(a, w_gate_up, out, m, 2 * inter, k, lda, ldc, scratch, scratch_bytes, true, st);
    return wb_ugemm(a, w_gate_up, out, m, 2 * inter, k, lda, ldc, true, st);
}

extern "C" int32_t wein_b200_gemm_wt(const void *a, const void *w, void *c, uint32_t m, uint32_t n, uint32_t k, void *scratch,
                                     uint64_t scratch_bytes, void *stream) {
    return wb_gemm_wt(a, w, c, m, n, k, k, n, scratch, scratch_bytes, WB_GEMM_AUTO, (cudaStream_t)stream);
}
extern "C" int32_t wein_b200_gemm_wt_tc(const void *a, const void *w, void *c, uint32_t m, uint32_t n, uint32_t k, void *stream) {
    return wb_gemm_wt(a, w, c, m, n, k, k, n, nullptr, 0, WB_GEMM_TC, (cudaStream_t)stream);
}

extern "C" int32_t wein_b200_gemm_swiglu(const void *a, const void *w_gate_up, void *out, uint32_t m, uint32_t inter, uint32_t k,
                                         void *scratch, uint64_t scratch_bytes, void *stream) {
    return wb_gemm_swiglu(a, w_gate_up, out, m, inter, k, k, inter, scratch, scratch_bytes, WB_GEMM_AUTO, (cudaStream_t)stream);
}
extern "C" int32_t wein_b200_gemm_swiglu_tc(const void *a, const void *w_gate_up, void *out, uint32_t m, uint32_t inter, uint32_t k,
                                            void *stream) {
    return wb_gemm_swiglu(a, w_gate_up, out, m, inter, k, k, inter, nullptr, 0, WB_GEMM_TC, (cudaStream_t)stream);
}
