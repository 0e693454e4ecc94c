// Weight-streaming GEMM on the 5th-generation tensor cores: C[m,n] = A[m,k] * W[n,k]^T (bf16 in, f32 accumulate in
// tensor memory, bf16 out) for forwards of more than 32 rows -- batch x (draft k + 1) = 33 ... 256 -- and for every
// smaller product of an engine whose largest forward exceeds 32 rows, so that one kernel (one summation order) serves
// the plain, draft and verify forwards of that engine.
//
// Reference contract: GemmOp::run_wt (crates/wein-kernel/src/ops/mod.rs:3378-3449), which hands these shapes to cuBLASLt
// (crates/wein-kernel/src/cuda/cublaslt.rs:249-257) and accepts |got - ref| <= max(2^-7 |ref|, 2^-11) against an f64 product
// (crates/wein-kernel/tests/gemm.rs:11).  The reference's own hand-written attempt (kernels/src/lib.rs:8655) lost on
// activation re-reads (ops/mod.rs:3392-3397); the shape of this kernel follows from that traffic algebra.
//
// The product is bound by streaming W from HBM once (at most 256 flop per weight byte, the ridge is ~270).  Design:
//  * the WEIGHTS are the M operand of the MMA: a CTA owns MT (1 or 2) tiles of 128 weight rows and a slice of k; the
//    tokens are the N operand (m rounded up to 16).  D[128 x N] f32 lives in tensor memory (MT x N columns), so no
//    register holds an accumulator during the main loop;
//  * a stage = 64 k of the MT weight tiles (16 KB each) + 64 k of all tokens (N x 128 B), brought in by tensor-map bulk
//    copies (cp.async.bulk.tensor, 128-byte swizzle, no multicast) that complete on an mbarrier; 3-7 stages per CTA keep
//    100-200 KB in flight per SM.  With MT = 2 the token stage is read once for 256 weight rows, which halves the
//    L2 -> SM activation traffic that decides the rate at m = 128 (it equals the weight traffic with MT = 1);
//  * weights are never written inside a round, so the producer thread issues the weight copies of the first stages
//    BEFORE the kernel waits for its predecessor (programmatic dependent launch); token copies, the tensor-memory
//    allocation and everything else come after the wait.  Allocating tensor memory before the wait could deadlock: a
//    CTA that holds columns while it waits for the predecessor grid can starve a predecessor CTA of columns;
//  * one thread issues tcgen05.mma (kind::f16, M = 128, K = 16: four per stage and tile); tcgen05.commit frees the
//    stage for the producer and finally signals the epilogue warps;
//  * narrow outputs (n = 2560) have only 20 tiles, so k is split over the CTAs of a thread-block cluster (up to 8): each
//    CTA sends its f32 partial of token-column slice j to CTA j of the cluster through distributed shared memory, and CTA j
//    adds the partials of its slice in rank order.  The split depends on (n, k) only: the order of every sum is fixed by
//    the weight shape, never by m, so a token's result does not depend on the batch it is computed in;
//  * the epilogue reads the accumulators with tcgen05.ld (lane = weight row), rounds to bf16 and writes C, or applies
//    SwiGLU across the two tiles of a CTA (tile 0 = 128 gate rows, tile 1 = the matching up rows).
// Every mbarrier wait is bounded by a clock; a wait that gives up raises a CTA-wide abort flag, is counted in a device
// counter, the CTA still joins its cluster barriers, frees its tensor memory and leaves after its copies have landed.
#include <cuda.h>
#include "common.cuh"
#include "internal.h"
#include <mutex>

namespace {

constexpr int UG_BK = 64;                      // k elements per stage (one 128-byte swizzle row)
constexpr int UG_WTILE = 128 * UG_BK * 2;      // bytes of one weight tile per stage
constexpr int UG_THREADS = 192;                // warp 0 producer, warp 1 MMA + tensor-memory owner, warps 2-5 epilogue
constexpr long long UG_WAIT_CYCLES = 2000000000ll;   // ~1 s
constexpr int UG_SMEM_MAX = 225 * 1024;

__device__ unsigned int g_ug_timeouts;

struct UgParams {
    bf16_t *C;
    uint32_t m, n, k, ldc;          // n = weight rows of the product (2 * inter with swiglu)
    uint32_t npad;                  // m rounded up to 16: N of the MMA, rows of the token box
    uint32_t nkb;                   // k blocks of 64 in the whole product
    uint32_t ksplit;                // cluster size: CTAs that share the k range of a tile group
    uint32_t stages;                // ring depth
    uint32_t swiglu, half_n;        // swiglu: tile 0 = gate rows r0.., tile 1 = up rows (half_n + r0..); output [m, half_n]
    uint32_t tmem_cols;             // power of two >= MT * npad
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t a, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(a), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t a, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(a), "r"(bytes) : "memory");
}
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
        if (clock64() - t0 > UG_WAIT_CYCLES) {
            *abort_flag = 1;
            atomicAdd(&g_ug_timeouts, 1u);
            return false;
        }
    }
}
__device__ __forceinline__ void tma_2d(uint32_t dst, const CUtensorMap *tm, uint32_t c0, uint32_t c1, uint32_t mbar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(tm), "r"(c0), "r"(c1), "r"(mbar) : "memory");
}
// Shared-memory matrix descriptor of a K-major tile of 128-byte rows under the 128-byte swizzle: 8-row groups are 1024
// bytes apart (stride byte offset), the leading offset is unused for swizzled K-major tiles, descriptor version 1.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3ffffu) >> 4);          // start address, 16-byte units
    d |= (uint64_t)1 << 16;                            // leading byte offset (ignored under a swizzle)
    d |= (uint64_t)(1024u >> 4) << 32;                 // stride byte offset
    d |= (uint64_t)1 << 46;                            // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                            // SWIZZLE_128B
    return d;
}
// Instruction descriptor: bf16 x bf16 -> f32, both operands K-major, M = 128, N = npad.
__device__ __forceinline__ uint32_t umma_idesc(uint32_t n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t mbar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                   "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                 : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
// Store into the shared memory of CTA `rank` of the cluster, at the address that `local_saddr` has in this CTA
__device__ __forceinline__ void st_remote_f32(uint32_t local_saddr, uint32_t rank, float v) {
    uint32_t ra;
    asm("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(local_saddr), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(ra), "f"(v) : "memory");
}

// Dynamic shared memory (base rounded up to 1024 bytes): [stages x (MT weight tiles | token tile)] ; the f32 partials of a
// k-split CTA alias the ring once the main loop is over.  Barriers, the abort flag and the tensor-memory address are static.
template <int MT>
__global__ void __launch_bounds__(UG_THREADS, 1)
ugemm_kernel(const __grid_constant__ CUtensorMap tm_w0, const __grid_constant__ CUtensorMap tm_w1,
             const __grid_constant__ CUtensorMap tm_x, const UgParams P) {
    pdl_trigger();
    extern __shared__ unsigned char ug_smem_raw[];
    __shared__ uint64_t bar_full[8], bar_empty[8], bar_accum;
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile uint32_t abort_s;
    unsigned char *ring = ug_smem_raw + ((1024u - (smem_u32(ug_smem_raw) & 1023u)) & 1023u);
    const uint32_t ring0 = smem_u32(ring);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t S = P.stages, x_bytes = P.npad * 128u, stage_bytes = MT * UG_WTILE + x_bytes;
    const uint32_t rank = P.ksplit > 1 ? cluster_rank() : 0u;
    const uint32_t group = blockIdx.x / P.ksplit;            // which tile group of MT x 128 weight rows
    // weight rows of the two tiles: consecutive 128-row tiles, or gate rows and the matching up rows
    const uint32_t r0 = P.swiglu ? group * 128u : group * (MT * 128u);
    const uint32_t r1 = P.swiglu ? r0 : r0 + 128u;            // swiglu: same coordinate in the second map (the up half)
    // k blocks of this CTA: nkb split into ksplit contiguous parts, the first `rem` parts one block longer
    const uint32_t per = P.nkb / P.ksplit, rem = P.nkb % P.ksplit;
    const uint32_t kb_lo = rank * per + min(rank, rem), my_kb = per + (rank < rem ? 1u : 0u);

    if (tid == 0) {
        for (uint32_t s = 0; s < S; s++) { mbar_init(smem_u32(&bar_full[s]), 1); mbar_init(smem_u32(&bar_empty[s]), 1); }
        mbar_init(smem_u32(&bar_accum), 1);
        abort_s = 0;
        tmem_base_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    const uint32_t pre = min(S, my_kb);
    if (warp == 0 && lane == 0) {
        // ---- producer, part 1: weight copies of the first stages while the predecessor kernel is still running
        for (uint32_t i = 0; i < pre; i++) {
            const uint32_t fb = smem_u32(&bar_full[i]), dst = ring0 + i * stage_bytes;
            mbar_expect_tx(fb, stage_bytes);
            tma_2d(dst, &tm_w0, (kb_lo + i) * UG_BK, r0, fb);
            if (MT == 2) tma_2d(dst + UG_WTILE, &tm_w1, (kb_lo + i) * UG_BK, r1, fb);
        }
    }
    pdl_wait();   // the tokens are the predecessor's output; tensor memory may only be claimed once that grid is gone
    if (warp == 0 && lane == 0) {
        for (uint32_t i = 0; i < pre; i++)
            tma_2d(ring0 + i * stage_bytes + MT * UG_WTILE, &tm_x, (kb_lo + i) * UG_BK, 0, smem_u32(&bar_full[i]));
    }
    __syncwarp();
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(P.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        tc_fence_before();
    }
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;

    if (warp == 0) {
        // ---- producer, part 2: the remaining stages, each as soon as the MMAs that read its slot have completed
        if (lane == 0) {
            for (uint32_t i = pre; i < my_kb; i++) {
                const uint32_t s = i % S;
                if (!mbar_wait(smem_u32(&bar_empty[s]), ((i / S) - 1) & 1, &abort_s)) break;
                const uint32_t fb = smem_u32(&bar_full[s]), dst = ring0 + s * stage_bytes;
                mbar_expect_tx(fb, stage_bytes);
                tma_2d(dst, &tm_w0, (kb_lo + i) * UG_BK, r0, fb);
                if (MT == 2) tma_2d(dst + UG_WTILE, &tm_w1, (kb_lo + i) * UG_BK, r1, fb);
                tma_2d(dst + MT * UG_WTILE, &tm_x, (kb_lo + i) * UG_BK, 0, fb);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---- MMA issue: one thread; D (+)= W_tile[128 x 16] * X[npad x 16]^T, four k-steps per stage and tile
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(P.npad);
            bool ok = true;
            for (uint32_t i = 0; i < my_kb && ok; i++) {
                const uint32_t s = i % S;
                ok = mbar_wait(smem_u32(&bar_full[s]), (i / S) & 1, &abort_s);
                if (!ok) break;
                tc_fence_after();
                const uint32_t base = ring0 + s * stage_bytes;
                const uint64_t db = umma_desc(base + MT * UG_WTILE);
#pragma unroll
                for (int kk = 0; kk < UG_BK / 16; kk++) {
#pragma unroll
                    for (int t = 0; t < MT; t++)
                        umma_bf16(tmem_base + t * P.npad, umma_desc(base + t * UG_WTILE) + 2 * kk, db + 2 * kk, idesc, (i | kk) != 0 ? 1u : 0u);
                }
                umma_commit(smem_u32(&bar_empty[s]));   // the slot is free once these MMAs have read it
            }
            umma_commit(smem_u32(&bar_accum));           // all MMAs of this CTA complete: the accumulators are final
        }
        __syncwarp();
    }

    // ---- epilogue: warps 2-5; warp w may touch the 32 tensor-memory lanes of quadrant w % 4
    const uint32_t q = warp & 3, row = q * 32 + lane;           // row of the tile this thread owns (warps 2..5)
    const uint32_t tq = tmem_base + ((q * 32u) << 16);
    bool go = false;    // warp-uniform: the tensor-memory loads below are warp-wide instructions
    if (warp >= 2) {
        const bool accum_ok = my_kb == 0 || mbar_wait(smem_u32(&bar_accum), 0, &abort_s);
        go = __all_sync(0xffffffffu, accum_ok && !abort_s) != 0;
        tc_fence_after();
    }
    // one finished element: round, optionally SwiGLU across the two tiles, store (a warp writes 64 contiguous bytes per token)
    auto emit = [&](uint32_t tok, float a0, float a1) {
        if (P.swiglu) {
            const uint32_t col = r0 + row;
            if (col < P.half_n) P.C[(size_t)tok * P.ldc + col] = f2bf(__fmul_rn(rbf(silu_ref(rbf(a0))), rbf(a1)));
        } else {
            if (r0 + row < P.n) P.C[(size_t)tok * P.ldc + r0 + row] = f2bf(a0);
            if (MT == 2 && r1 + row < P.n) P.C[(size_t)tok * P.ldc + r1 + row] = f2bf(a1);
        }
    };
    if (P.ksplit == 1) {
        if (go) {
            for (uint32_t c0 = 0; c0 < P.m; c0 += 16) {
                uint32_t v0[16], v1[16];
                tmem_ld16(tq + c0, v0);
                if (MT == 2) tmem_ld16(tq + P.npad + c0, v1);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; j++)
                    if (c0 + j < P.m) emit(c0 + j, __uint_as_float(v0[j]), MT == 2 ? __uint_as_float(v1[j]) : 0.0f);
            }
        }
        tc_fence_before();
        __syncthreads();
    } else {
        // k split over the cluster: token column c belongs to CTA c / cs.  Once every CTA of the cluster has left its main
        // loop (its ring is idle: every copy has landed and every MMA has read it), each CTA sends the columns of its f32
        // partial straight from tensor memory into the owner's ring, [source rank][tile][column of the slice][128 rows];
        // after a second barrier the owner adds the partials of a column in rank order from its own shared memory.
        const uint32_t cs = (P.m + P.ksplit - 1) / P.ksplit;
        float *recv = reinterpret_cast<float *>(ring);
        tc_fence_before();
        cluster_sync_all();
        if (go) {
            for (uint32_t c0 = 0; c0 < P.m; c0 += 16) {
                uint32_t v0[16], v1[16];
                if (my_kb) {
                    tmem_ld16(tq + c0, v0);
                    if (MT == 2) tmem_ld16(tq + P.npad + c0, v1);
                    tmem_ld_wait();
                }
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    const uint32_t c = c0 + j;
                    if (c >= P.m) break;
                    const uint32_t owner = c / cs, slot = c - owner * cs;
                    const uint32_t a0 = smem_u32(&recv[(((size_t)rank * MT + 0) * cs + slot) * 128 + row]);
                    st_remote_f32(a0, owner, my_kb ? __uint_as_float(v0[j]) : 0.0f);
                    if (MT == 2) st_remote_f32(a0 + cs * 128 * 4, owner, my_kb ? __uint_as_float(v1[j]) : 0.0f);
                }
            }
        }
        cluster_sync_all();   // release / acquire: the partials sent above are visible to their owners
        const uint32_t c_lo = min(P.m, rank * cs), c_hi = min(P.m, c_lo + cs);
        if (warp >= 2 && !abort_s) {   // (a peer that gave up sends nothing: the result is flagged by the timeout counter, not trusted)
            for (uint32_t c = c_lo; c < c_hi; c++) {
                float acc0 = 0.0f, acc1 = 0.0f;
                for (uint32_t rk = 0; rk < P.ksplit; rk++) {
                    acc0 += recv[(((size_t)rk * MT + 0) * cs + (c - c_lo)) * 128 + row];
                    if (MT == 2) acc1 += recv[(((size_t)rk * MT + 1) * cs + (c - c_lo)) * 128 + row];
                }
                emit(c, acc0, acc1);
            }
        }
        tc_fence_before();
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(P.tmem_cols) : "memory");
    }
    if (abort_s)
        for (int i = 0; i < 1000; i++) __nanosleep(1000);   // let this CTA's copies in flight land before its shared memory is released
}

typedef CUresult (*ug_encode_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                 const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
std::once_flag g_ug_once;
ug_encode_fn g_ug_encode = nullptr;   // resolved once, immutable afterwards

// (k, rows) bf16 matrix with row stride ld elements, boxes of 64 k x box_rows rows, 128-byte swizzle, zero fill outside
bool ug_map(CUtensorMap *tm, const void *base, uint64_t rows, uint64_t k, uint64_t ld, uint32_t box_rows) {
    const cuuint64_t dims[2] = {k, rows};
    const cuuint64_t strides[1] = {ld * 2};
    const cuuint32_t box[2] = {UG_BK, box_rows};
    const cuuint32_t ones[2] = {1, 1};
    return g_ug_encode(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
                       CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int MT>
cudaError_t ug_launch(const CUtensorMap &w0, const CUtensorMap &w1, const CUtensorMap &x, const UgParams &p, uint32_t ctas, size_t smem,
                      cudaStream_t st) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas); cfg.blockDim = dim3(UG_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute at[2];
    int na = 0;
    at[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[na].val.programmaticStreamSerializationAllowed = 1;
    na++;
    if (p.ksplit > 1) {
        at[na].id = cudaLaunchAttributeClusterDimension;
        at[na].val.clusterDim.x = p.ksplit; at[na].val.clusterDim.y = 1; at[na].val.clusterDim.z = 1;
        na++;
    }
    cfg.attrs = at; cfg.numAttrs = na;
    return cudaLaunchKernelEx(&cfg, ugemm_kernel<MT>, w0, w1, x, p);
}

}  // namespace

// Decomposition of a product, from the weight shape alone (never from m): tiles per CTA and the k split.
struct UgPlan { uint32_t mt, ksplit; };
static UgPlan ug_plan(uint32_t n, uint32_t k, bool swiglu, int sms) {
    const uint32_t nkb = (k + UG_BK - 1) / UG_BK;
    UgPlan best{swiglu ? 2u : 1u, 1u};
    double best_eff = -1.0;
    for (uint32_t mt = swiglu ? 2 : 1; mt <= 2; mt++) {
        const uint32_t rows = swiglu ? n / 2 : n;
        const uint32_t groups = swiglu ? (rows + 127) / 128 : (rows + mt * 128 - 1) / (mt * 128);
        for (uint32_t s = 1; s <= 8; s++) {
            if (s > 1 && nkb / s < 6) break;
            const uint32_t ctas = groups * s, waves = (ctas + sms - 1) / sms;
            // useful share of the machine over the product's waves; two tiles per CTA halve the token traffic (small bonus);
            // every extra k slice costs a partial exchange (small penalty)
            double eff = (double)ctas / ((double)waves * sms);
            if (!swiglu && mt == 2 && groups * 2 * 128 > rows + 128) eff *= (double)((rows + 127) / 128) / (double)(groups * 2);   // an empty half tile
            eff += (mt == 2 ? 0.02 : 0.0) - 0.004 * (s - 1);
            if (eff > best_eff) { best_eff = eff; best = {mt, s}; }
        }
    }
    return best;
}

static int g_ug_sms[64];   // SM count per device ordinal (0 = not looked up yet; written once, the same value by any thread)

int32_t wb_ugemm_init() {
    std::call_once(g_ug_once, [] {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qr) == cudaSuccess && fn && qr == cudaDriverEntryPointSuccess)
            g_ug_encode = (ug_encode_fn)fn;
    });
    if (!g_ug_encode) { wb_set_error("gemm: the driver does not export cuTensorMapEncodeTiled"); return WB_ERR_CUDA; }
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { wb_set_error("gemm: cudaGetDevice failed or device ordinal >= 64"); return WB_ERR_CUDA; }
    if (!g_ug_sms[dev]) {
        int n = 0;
        cudaError_t e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(ugemm_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, UG_SMEM_MAX);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(ugemm_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, UG_SMEM_MAX);
        if (e != cudaSuccess || n <= 0) { wb_set_error("gemm: shared-memory opt-in failed: %s", cudaGetErrorString(e)); return WB_ERR_CUDA; }
        g_ug_sms[dev] = n;
    }
    return WB_OK;
}

// C[m,n] = A W^T (swiglu: W = [gate; up] of n = 2 * inter rows, C[m, inter]); arguments validated by the callers in gemm.cu.
// m beyond 256 is processed in chunks of 256 token rows.
int32_t wb_ugemm(const void *a, const void *w, void *c, uint32_t m, uint32_t n, uint32_t k, uint32_t lda, uint32_t ldc, bool swiglu,
                 cudaStream_t st) {
    if (int32_t rc = wb_ugemm_init()) return rc;
    int dev = 0;
    cudaGetDevice(&dev);
    const int sms = g_ug_sms[dev];
    for (uint32_t m0 = 0; m0 < m; m0 += 256) {
        const uint32_t mc = m - m0 < 256 ? m - m0 : 256;
        UgParams p{};
        p.C = (bf16_t *)c + (size_t)m0 * ldc;
        p.m = mc; p.n = n; p.k = k; p.ldc = ldc;
        p.npad = (mc + 15) / 16 * 16;
        p.nkb = (k + UG_BK - 1) / UG_BK;
        p.swiglu = swiglu ? 1 : 0; p.half_n = n / 2;
        UgPlan pl = ug_plan(n, k, swiglu, sms);
        // shared memory: at least 3 stages, and the k-split partials must fit in the ring
        auto stage_bytes = [&](uint32_t mt) { return (size_t)mt * UG_WTILE + (size_t)p.npad * 128; };
        auto fits = [&](uint32_t mt, uint32_t ks) {
            const size_t ring = (UG_SMEM_MAX - 1024) / stage_bytes(mt) * stage_bytes(mt);
            const size_t cs = (mc + ks - 1) / ks;
            return (UG_SMEM_MAX - 1024) / stage_bytes(mt) >= 3 && (ks == 1 || (size_t)ks * mt * cs * 128 * 4 <= ring) && mt * p.npad <= 512;
        };
        if (!fits(pl.mt, pl.ksplit)) {
            if (swiglu || !fits(1, pl.ksplit)) { wb_set_error("gemm: m = %u rows do not fit the tensor-core kernel's shared memory", mc); return WB_ERR_SHAPE; }
            pl.mt = 1;   // tiles per CTA never change a result bit
        }
        p.ksplit = pl.ksplit;
        uint32_t stages = (uint32_t)((UG_SMEM_MAX - 1024) / stage_bytes(pl.mt));
        if (stages > 8) stages = 8;
        p.stages = stages;
        const size_t smem = 1024 + (size_t)stages * stage_bytes(pl.mt);
        uint32_t cols = 32;
        while (cols < pl.mt * p.npad) cols *= 2;
        p.tmem_cols = cols;
        const uint32_t rows = swiglu ? n / 2 : n;
        const uint32_t groups = swiglu ? (rows + 127) / 128 : (rows + pl.mt * 128 - 1) / (pl.mt * 128);
        CUtensorMap tw0, tw1, tx;
        bool ok = ug_map(&tw0, w, rows, k, k, 128) &&
                  ug_map(&tw1, swiglu ? (const bf16_t *)w + (size_t)rows * k : (const bf16_t *)w, rows, k, k, 128) &&
                  ug_map(&tx, (const bf16_t *)a + (size_t)m0 * lda, mc, k, lda, p.npad);
        if (!ok) { wb_set_error("gemm: cuTensorMapEncodeTiled failed for m=%u n=%u k=%u", mc, n, k); return WB_ERR_CUDA; }
        cudaError_t e = pl.mt == 2 ? ug_launch<2>(tw0, tw1, tx, p, groups * pl.ksplit, smem, st) : ug_launch<1>(tw0, tw1, tx, p, groups * pl.ksplit, smem, st);
        if (e != cudaSuccess) { wb_set_error("gemm: launch failed for m=%u n=%u k=%u: %s", mc, n, k, cudaGetErrorString(e)); return WB_ERR_CUDA; }
    }
    return WB_OK;
}

bool wb_ugemm_supports(uint32_t n, uint32_t k, uint32_t lda, bool swiglu) { return k % 8 == 0 && lda % 8 == 0 && k >= 8 && (!swiglu || n % 2 == 0); }

// Number of barrier waits of the tensor-core GEMM that gave up since the library was loaded (0 in a healthy run); synchronises.
extern "C" int32_t wein_b200_gemm_wait_timeouts(uint32_t *out) {
    unsigned int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_ug_timeouts, sizeof v);
    if (e != cudaSuccess) { wb_set_error("gemm_wait_timeouts: %s", cudaGetErrorString(e)); return WB_ERR_CUDA; }
    if (out) *out = v;
    return WB_OK;
}
