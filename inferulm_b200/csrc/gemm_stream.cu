// Weight-streaming skinny GEMM, TMA staged: C[m,n] = A[m,k] * W[n,k]^T for m <= 32 rows (bf16 in, f32 accumulate,
// bf16 out), optionally with the SwiGLU epilogue over W = [gate; up].
//
// Same contract as the register-streaming kernel in gemm.cu (GemmOp::run_wt of the reference,
// crates/wein-kernel/src/ops/mod.rs:3378-3449); what differs is how the weights travel.  A round of speculative decoding
// is a chain of ~300 short launches, each bound by streaming its weights from HBM once, so what decides the round time is
// whether HBM keeps streaming ACROSS launch boundaries.  Here every CTA owns a ring of 16 KB shared-memory stages that one
// producer thread fills with tensor-map bulk copies (cp.async.bulk.tensor, completion counted on an mbarrier):
//  * the copies are issued BEFORE the kernel waits for its predecessor (programmatic dependent launch): weights are
//    never written inside a round, so as soon as a CTA of the previous kernel retires, a CTA of this one becomes resident
//    and pulls up to ~100 KB of its weights while the predecessor (and a small kernel in between, e.g. a norm) finishes;
//  * after the wait, the critical path is one activation load, MMAs out of shared memory and a fixed-order reduction;
//  * a stage = 16 weight rows x 512 k (one row tile of the m16n8k16 MMA) = ONE copy instruction (row-by-row 1 KB bulk
//    copies measured 16 B/cycle/SM, instruction bound).  The weight matrix is described to the copy engine as the 3-d
//    tensor (64 k, n rows, k/64 chunks) -- 4-d (64, inter, 2, k/64) for [gate; up], which puts 8 gate rows and the
//    matching 8 up rows into one tile -- with the 128-byte swizzle: the stage holds [chunk][row][128 B] and the 16-byte
//    piece p of row r sits at piece p ^ (r & 7).  Lane (g, c) reads pieces 2c and 2c + 1 of rows g and g + 8, so the 8
//    lanes of a quarter warp touch 8 distinct pieces: conflict-free 16-byte fragment reads, no ldmatrix;
//  * the 8 consumer warps split a stage by 64-wide chunk (warp w takes chunk w), accumulate over the stages of a row
//    tile, and meet in a shared-memory reduction that adds the warps in index order.  The order of every sum is fixed
//    by (n, k) alone -- not by m, the grid or timing -- so a row's result is the same in every batch;
//  * CTA i takes row tiles i, i + G, i + 2G, ... with G = min(tiles, 2 x SMs).
// Every barrier wait is bounded by a clock; a wait that gives up raises a CTA-wide abort flag (all later waits return at
// once), counts itself in g_tg_timeouts, and the CTA leaves after a fixed delay that outlasts its copies in flight.
// Needs k % 64 == 0; other shapes stay on the register-streaming kernel.
#include <cuda.h>
#include "common.cuh"
#include "internal.h"
#include <map>
#include <mutex>
#include <tuple>

namespace {

constexpr int TG_KC = 512;               // k elements per stage
constexpr int TG_CHUNKS = TG_KC / 64;    // 128-byte chunks per row and stage (= consumer warps)
constexpr int TG_STAGE = 16 * TG_KC * 2; // 16384 bytes, stages are 1024-byte aligned (swizzle atom)
constexpr long long TG_WAIT_CYCLES = 2000000000ll;  // ~1 s

__device__ unsigned int g_tg_timeouts;

struct TgParams {
    const bf16_t *A, *W;
    bf16_t *C;
    uint32_t m, n, k, lda, ldc, swiglu, n_tiles, stages, stage_tx;   // stage_tx: bytes one copy delivers
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t a, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(a), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t a, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(a), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t a) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(a) : "memory"); }
__device__ __forceinline__ bool mbar_try(uint32_t a, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(a), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: false (and the CTA-wide abort flag raised) when the phase did not complete within the clock limit.
__device__ __forceinline__ bool mbar_wait(uint32_t a, uint32_t parity, volatile uint32_t *abort_flag) {
    if (mbar_try(a, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
        if (mbar_try(a, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > TG_WAIT_CYCLES) {
            *abort_flag = 1;
            atomicAdd(&g_tg_timeouts, 1u);
            return false;
        }
    }
}
__device__ __forceinline__ void tma_tile_3d(uint32_t dst, const CUtensorMap *tm, uint32_t c0, uint32_t c1, uint32_t c2, uint32_t mbar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(dst), "l"(tm), "r"(c0), "r"(c1), "r"(c2), "r"(mbar) : "memory");
}
__device__ __forceinline__ void tma_tile_4d(uint32_t dst, const CUtensorMap *tm, uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t mbar) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
                 ::"r"(dst), "l"(tm), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(mbar) : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
// Activations come from the predecessor kernel, whose lifetime overlaps this one's: coherent loads only.
__device__ __forceinline__ uint4 ld_act(const void *p) {
    uint4 v;
    asm volatile("ld.global.ca.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void mma_bf16(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// Dynamic shared memory (base rounded up to 1024 bytes): [stages x 16 KB ring][2 x 8 x MT x 128 floats of reduction]
// [full barriers][empty barriers][abort flag]
template <int MT>
__global__ void __launch_bounds__(288, 2) tgemm_kernel(const __grid_constant__ CUtensorMap tmap, const TgParams P) {
    pdl_trigger();
    extern __shared__ unsigned char tg_smem_raw[];
    const uint32_t S = P.stages;
    unsigned char *tg_smem = tg_smem_raw + ((1024u - (smem_u32(tg_smem_raw) & 1023u)) & 1023u);
    float *red = reinterpret_cast<float *>(tg_smem + (size_t)S * TG_STAGE);
    uint64_t *bars = reinterpret_cast<uint64_t *>(red + 2 * 8 * MT * 128);
    volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(bars + 2 * S);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t ring0 = smem_u32(tg_smem), full0 = smem_u32(bars), empty0 = full0 + S * 8;
    if (tid == 0) {
        for (uint32_t s = 0; s < S; s++) { mbar_init(full0 + s * 8, 1); mbar_init(empty0 + s * 8, 8); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const uint32_t G = gridDim.x;
    const uint32_t my_tiles = blockIdx.x < P.n_tiles ? (P.n_tiles - blockIdx.x + G - 1) / G : 0;
    const uint32_t nc = (P.k + TG_KC - 1) / TG_KC, U = my_tiles * nc, half_n = P.n >> 1, k_chunks = P.k / 64;

    if (warp == 8) {
        // ---- producer: one thread, one copy per stage.  Weights are constant during a round, so nothing here waits for the
        // predecessor kernel: the ring fills while that kernel is still running.
        if (lane == 0) {
            for (uint32_t u = 0; u < U; u++) {
                const uint32_t s = u % S;
                if (u >= S && !mbar_wait(empty0 + s * 8, ((u / S) - 1) & 1, abort_flag)) break;   // the consumers see the abort flag
                const uint32_t tile = blockIdx.x + (u / nc) * G, cch = u % nc;
                mbar_expect_tx(full0 + s * 8, P.stage_tx);
                if (P.swiglu) tma_tile_4d(ring0 + s * TG_STAGE, &tmap, 0, tile * 8, 0, cch * TG_CHUNKS, full0 + s * 8);
                else tma_tile_3d(ring0 + s * TG_STAGE, &tmap, 0, tile * 16, cch * TG_CHUNKS, full0 + s * 8);
            }
        }
    } else {
        // ---- consumers: 8 warps, warp w takes the 64-wide chunk w of every stage; lane (g, c) pieces 2c and 2c + 1
        pdl_wait();
        const int g = lane >> 2, c = lane & 3;
        const bf16_t *ap[MT];
        bool av[MT];
#pragma unroll
        for (int mt = 0; mt < MT; mt++) {
            const uint32_t tok = mt * 8 + g;
            av[mt] = tok < P.m;
            ap[mt] = P.A + (size_t)(av[mt] ? tok : 0) * P.lda + warp * 64 + c * 16;
        }
        float acc[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; mt++) acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.0f;
        // Activations: with ~226 KB of the SM's memory configured as shared, L1 keeps next to nothing, so every activation
        // load is an L2 round trip (~700 cycles), about the time a stage lasts.  They are therefore fetched LA stages ahead
        // into a rotating register window (slot l holds stage u0 + l; refilled with stage u0 + l + LA once used).
        constexpr int LA = MT == 1 ? 6 : (MT == 2 ? 4 : 2);
        uint4 xq[LA][2][MT];
        auto load_acts = [&](uint32_t cch, uint4 (&x)[2][MT]) {
            const bool valid = cch * TG_CHUNKS + warp < k_chunks;
#pragma unroll
            for (int h = 0; h < 2; h++)
#pragma unroll
                for (int mt = 0; mt < MT; mt++)
                    x[h][mt] = (valid && av[mt]) ? ld_act(ap[mt] + (size_t)cch * TG_KC + h * 8) : make_uint4(0, 0, 0, 0);
        };
#pragma unroll
        for (int l = 0; l < LA; l++)
            if ((uint32_t)l < U) load_acts((uint32_t)l % nc, xq[l]);
        // this lane's two pieces of rows g and g + 8 inside a stage (both rows swizzle by g)
        const uint32_t frag0 = (warp * 16 + g) * 128 + (((2 * c) ^ g) << 4), frag1 = (warp * 16 + g) * 128 + (((2 * c + 1) ^ g) << 4);
        for (uint32_t u0 = 0; u0 < U; u0 += LA) {
#pragma unroll
          for (int l = 0; l < LA; l++) {
            const uint32_t u = u0 + l;
            if (u >= U) break;
            const uint32_t s = u % S, cch = u % nc;
            mbar_wait(full0 + s * 8, (u / S) & 1, abort_flag);   // on a timeout the result is garbage and flagged; no early exit
            if (cch * TG_CHUNKS + warp < k_chunks) {
                const uint32_t base = ring0 + s * TG_STAGE;
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const uint32_t fa = base + (h ? frag1 : frag0);
                    const uint4 wa = lds128(fa), wb = lds128(fa + 8 * 128);
#pragma unroll
                    for (int mt = 0; mt < MT; mt++) {
                        mma_bf16(acc[mt], wa.x, wb.x, wa.y, wb.y, xq[l][h][mt].x, xq[l][h][mt].y);
                        mma_bf16(acc[mt], wa.z, wb.z, wa.w, wb.w, xq[l][h][mt].z, xq[l][h][mt].w);
                    }
                }
            }
            if (u + LA < U) load_acts((u + LA) % nc, xq[l]);
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + s * 8);
            if (cch == nc - 1) {
                // row tile complete: element (mt, lane, j) is output (token mt*8 + 2c + (j&1), tile row g + 8*(j>>1))
                const uint32_t ti = u / nc, tile = blockIdx.x + ti * G;
                float *rb = red + (size_t)(ti & 1) * 8 * MT * 128;
#pragma unroll
                for (int mt = 0; mt < MT; mt++) {
                    *reinterpret_cast<float4 *>(&rb[((warp * MT + mt) * 32 + lane) * 4]) = make_float4(acc[mt][0], acc[mt][1], acc[mt][2], acc[mt][3]);
                    acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.0f;
                }
                consumer_sync();   // the buffer of tile ti-1 is free again once every warp has passed this barrier
                for (int idx = tid; idx < MT * 128; idx += 256) {
                    const int mt = idx >> 7, ln = (idx >> 2) & 31, j = idx & 3;
                    const uint32_t tok = mt * 8 + 2 * (ln & 3) + (j & 1);
                    if (tok >= P.m) continue;
                    float sum = 0.0f;
#pragma unroll
                    for (int w = 0; w < 8; w++) sum += rb[((w * MT + mt) * 32 + ln) * 4 + j];
                    if (P.swiglu) {
                        if (j >= 2) continue;   // the up-projection element is folded in with its gate element
                        float hi = 0.0f;
#pragma unroll
                        for (int w = 0; w < 8; w++) hi += rb[((w * MT + mt) * 32 + ln) * 4 + j + 2];
                        const uint32_t col = tile * 8 + (ln >> 2);
                        if (col < half_n) P.C[(size_t)tok * P.ldc + col] = f2bf(__fmul_rn(rbf(silu_ref(rbf(sum))), rbf(hi)));
                    } else {
                        const uint32_t row = tile * 16 + (ln >> 2) + 8 * (j >> 1);
                        if (row < P.n) P.C[(size_t)tok * P.ldc + row] = f2bf(sum);
                    }
                }
            }
          }
        }
    }
    if (*abort_flag)
        for (int i = 0; i < 1000; i++) __nanosleep(1000);   // let this CTA's copies in flight land before its shared memory is released
}

// Shared memory of a CTA: two CTAs per SM (227 KB), less the alignment slack, the reduction buffers and the barriers
static size_t tg_tail_bytes(int mt) { return (size_t)2 * 8 * mt * 128 * 4 + 256; }
static uint32_t tg_stages(int mt) { return (uint32_t)((115000u - 1024u - tg_tail_bytes(mt)) / TG_STAGE); }
static size_t tg_smem_bytes(int mt) { return 1024 + (size_t)tg_stages(mt) * TG_STAGE + tg_tail_bytes(mt); }

typedef CUresult (*tg_encode_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                 const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static tg_encode_fn g_tg_encode = nullptr;
static int g_tg_sms[64];
static std::mutex g_tg_mu;
// descriptors of the weight matrices seen so far: a descriptor holds address and shape only, never data, so it stays valid
static std::map<std::tuple<const void *, uint32_t, uint32_t, bool>, CUtensorMap> g_tg_maps;

static int32_t tg_init(int *sms) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { wb_set_error("gemm: cudaGetDevice failed"); return WB_ERR_CUDA; }
    std::lock_guard<std::mutex> lk(g_tg_mu);
    if (!g_tg_encode) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qr) != cudaSuccess || !fn || qr != cudaDriverEntryPointSuccess) {
            wb_set_error("gemm: the driver does not export cuTensorMapEncodeTiled");
            return WB_ERR_CUDA;
        }
        g_tg_encode = (tg_encode_fn)fn;
    }
    if (!g_tg_sms[dev]) {
        int n = 0;
        cudaError_t e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(tgemm_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tg_smem_bytes(1));
        if (e == cudaSuccess) e = cudaFuncSetAttribute(tgemm_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tg_smem_bytes(2));
        if (e == cudaSuccess) e = cudaFuncSetAttribute(tgemm_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tg_smem_bytes(3));
        if (e == cudaSuccess) e = cudaFuncSetAttribute(tgemm_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tg_smem_bytes(4));
        if (e != cudaSuccess || n <= 0) { wb_set_error("gemm: shared-memory opt-in failed: %s", cudaGetErrorString(e)); return WB_ERR_CUDA; }
        g_tg_sms[dev] = n;
    }
    *sms = g_tg_sms[dev];
    return WB_OK;
}

// The weight matrix as the copy engine sees it.  Plain: (64 k, n rows, k/64 chunks), box (64, 16, q).  [gate; up]:
// (64 k, inter rows, 2 halves, k/64 chunks), box (64, 8, 2, q).  Both land in shared memory as [q chunks][16 rows][128 B].
static int32_t tg_map_for(const void *w, uint32_t n, uint32_t k, bool swiglu, uint32_t box_q, CUtensorMap *out) {
    std::lock_guard<std::mutex> lk(g_tg_mu);
    const auto key = std::make_tuple(w, n, k, swiglu);
    auto it = g_tg_maps.find(key);
    if (it != g_tg_maps.end()) { *out = it->second; return WB_OK; }
    CUtensorMap tm;
    CUresult r;
    const cuuint32_t ones[4] = {1, 1, 1, 1};
    if (swiglu) {
        const uint64_t inter = n / 2;
        const cuuint64_t dims[4] = {64, inter, 2, k / 64};
        const cuuint64_t strides[3] = {(cuuint64_t)k * 2, inter * k * 2, 128};
        const cuuint32_t box[4] = {64, 8, 2, box_q};
        r = g_tg_encode(&tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void *>(w), dims, strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else {
        const cuuint64_t dims[3] = {64, n, k / 64};
        const cuuint64_t strides[2] = {(cuuint64_t)k * 2, 128};
        const cuuint32_t box[3] = {64, 16, box_q};
        r = g_tg_encode(&tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(w), dims, strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    if (r != CUDA_SUCCESS) { wb_set_error("gemm: cuTensorMapEncodeTiled failed (%d) for n=%u k=%u", (int)r, n, k); return WB_ERR_CUDA; }
    if (g_tg_maps.size() >= 8192) g_tg_maps.clear();
    g_tg_maps[key] = tm;
    *out = tm;
    return WB_OK;
}

}  // namespace

int32_t wb_tgemm_init() { int sms; return tg_init(&sms); }

bool wb_tgemm_supports(uint32_t n, uint32_t k, bool swiglu) { return k % 64 == 0 && k >= 64 && (!swiglu || n % 2 == 0); }

// Launch of the staged kernel; arguments as wb_gemm_wt / wb_gemm_swiglu (n = 2 * inter with swiglu), already validated.
int32_t wb_tgemm(const void *a, const void *w, void *c, uint32_t m, uint32_t n, uint32_t k, uint32_t lda, uint32_t ldc, bool swiglu,
                 cudaStream_t st) {
    int sms = 0;
    if (int32_t rc = tg_init(&sms)) return rc;
    TgParams p{};
    p.A = (const bf16_t *)a; p.W = (const bf16_t *)w; p.C = (bf16_t *)c;
    p.m = m; p.n = n; p.k = k; p.lda = lda; p.ldc = ldc; p.swiglu = swiglu ? 1 : 0;
    p.n_tiles = swiglu ? (n / 2 + 7) / 8 : (n + 15) / 16;
    const int mt = (m + 7) / 8;
    p.stages = tg_stages(mt);
    const uint32_t box_q = k / 64 < (uint32_t)TG_CHUNKS ? k / 64 : (uint32_t)TG_CHUNKS;
    p.stage_tx = box_q * 16 * 128;
    CUtensorMap tm;
    if (int32_t rc = tg_map_for(w, n, k, swiglu, box_q, &tm)) return rc;
    const uint32_t slots = 2 * sms;
    const uint32_t grid = p.n_tiles < slots ? p.n_tiles : slots;
    const size_t smem = tg_smem_bytes(mt);
    switch (mt) {
        case 1: WB_LAUNCH((tgemm_kernel<1>), grid, 288, smem, st, tm, p); break;
        case 2: WB_LAUNCH((tgemm_kernel<2>), grid, 288, smem, st, tm, p); break;
        case 3: WB_LAUNCH((tgemm_kernel<3>), grid, 288, smem, st, tm, p); break;
        default: WB_LAUNCH((tgemm_kernel<4>), grid, 288, smem, st, tm, p); break;
    }
    WB_LAUNCH_CHECK();
    return WB_OK;
}

// Number of barrier waits that gave up since the library was loaded (0 in a healthy run); synchronises the device.
extern "C" int32_t wein_b200_gemm_stream_timeouts(uint32_t *out) {
    unsigned int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_tg_timeouts, sizeof v);
    if (e != cudaSuccess) { wb_set_error("gemm_stream_timeouts: %s", cudaGetErrorString(e)); return WB_ERR_CUDA; }
    if (out) *out = v;
    return WB_OK;
}

WB_TRACE_SETTER(gemm_stream)   // diagnostic builds only (see common.cuh); expands to nothing otherwise
