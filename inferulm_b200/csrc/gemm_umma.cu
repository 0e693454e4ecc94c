// Weight-streaming GEMM on the 5th-generation tensor cores: C[m,n] = A[m,k] * W[n,k]^T (bf16 in, f32 accumulate in
// tensor memory, bf16 out) for forwards of more than 32 rows -- batch x (draft k + 1) = 33 ... 256 -- and for every
// smaller product of an engine whose largest forward exceeds 32 rows, so that one kernel (one summation order) serves
// the plain, draft and verify forwards of that engine.
//
// Reference contract: GemmOp::run_wt (crates/wein-kernel/src/ops/mod.rs:3378-3449), which hands these shapes to cuBLASLt
// (crates/wein-kernel/src/cuda/cublaslt.rs:249-257) and accepts |got - ref| <= max(2^-7 |ref|, 2^-11) against an f64 product
// (crates/wein-kernel/tests/gemm.rs:11).  The reference's own hand-written attempt (kernels/src/lib.rs:8655) lost on
// activation re-reads (ops/mod.rs:3392-3397).
//
// The product is bound by streaming W from HBM once (at most 256 flop per weight byte, the ridge is ~270).  Design:
//  * the TOKENS are the M operand of the MMA (128 rows; only the rows up to m, rounded up to 8, are copied and kept in shared
//    memory -- a token's result is row-local, so what the MMA reads past them only lands in accumulator rows nobody reads;
//    a second block of 128 for m > 128) and a tile of NT WEIGHT rows (a multiple of 16 up to 256) is the N operand: D[128 tokens x NT] f32 lives in tensor memory.
//    Measured on B200: the thread that issues tcgen05.mma spends ~115 cycles per instruction whatever N is (16 or 128),
//    plus ~100 per stage on barriers, so what bounds an SM's streaming rate is weight bytes per instruction: 8 KB at
//    N = 256 against 4 KB with the weights as the M operand (which capped an SM at ~40 GB/s, below its share of HBM);
//  * a stage = 64 k of the weight tile (NT x 128 B) + 64 k of the token block(s) (16 KB each), brought in by tensor-map
//    bulk copies (cp.async.bulk.tensor, 128-byte swizzle, each CTA fetching its own tiles) that complete on an mbarrier; a CTA takes the whole
//    SM's shared memory for its stages;
//  * weights are never written inside a round, so the producer thread issues the weight copies of the first stages
//    and claims its tensor memory BEFORE the kernel waits for its predecessor (programmatic dependent launch); only the
//    token copies and the MMAs come after the wait;
//  * one thread issues the MMAs (kind::f16, M = 128, K = 16: four per stage and token block); tcgen05.commit frees the
//    stage for the producer and finally signals the epilogue warps;
//  * the epilogue is row-local and runs on all eight warps: thread = token (tensor-memory lane), columns = consecutive weight
//    rows, so a thread reads 16 columns with tcgen05.ld, rounds them to bf16 (or applies SwiGLU to a gate column and its up
//    column, which sit in the same lane; the activation comes from a table of all 65,536 bf16 inputs) and writes 32
//    contiguous bytes of its C row: no transposition, no shared memory;
//  * outputs with few tiles (n = 2560) split k over the CTAs of a thread-block cluster (up to 8, as many as the device
//    keeps resident at once): each CTA sends column slice j of its f32 partial to CTA j of the cluster through
//    distributed shared memory (16-byte remote stores), and CTA j adds the partials of its slice in rank order.  The split
//    depends on (n, k) and the device only: the order of every sum is fixed by the weight shape, never by m, so a token's
//    result does not depend on the batch it is computed in.
// Every mbarrier wait is bounded by a clock; a wait that gives up raises a CTA-wide abort flag, is counted in a device
// counter, the CTA still joins its cluster barriers, frees its tensor memory and leaves after its copies have landed.
#include <cuda.h>
#include "common.cuh"
#include "internal.h"
#include <math.h>
#include <mutex>

namespace {

constexpr int UG_BK = 64;                      // k elements per stage (one 128-byte swizzle row)
constexpr int UG_XTILE = 128 * UG_BK * 2;      // bytes of one block of 128 token rows per stage
constexpr int UG_NS = 2;                       // independent pipelines (producer + MMA issuer + accumulator) per CTA
constexpr int UG_THREADS = (2 * UG_NS + 4) * 32;   // per stream a producer warp and an MMA warp, then four epilogue warps
constexpr long long UG_WAIT_CYCLES = 2000000000ll;   // ~1 s
constexpr int UG_SMEM_MAX = 225 * 1024;        // one CTA per SM
constexpr int UG_SMEM_SOLO = 120 * 1024;       // a request of at least this much keeps a second CTA of the kernel off the SM
constexpr int UG_MAX_STAGES = 6;               // per stream

__device__ unsigned int g_ug_timeouts;

// bf16(silu(x)) for every bf16 x, filled once per device by the exact expression of the SwiGLU operator (silu_ref on the value,
// rounded to bf16: kernels/src/lib.rs:576-584 of the reference).  The SwiGLU epilogue looks the activation up instead of
// evaluating ~80 instructions per element; the table IS the function on its 65,536 possible inputs, so nothing changes.
__device__ bf16_t g_silu_lut[65536];
__global__ void silu_lut_kernel() {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < 65536u) g_silu_lut[i] = f2bf(silu_ref(bf2f((bf16_t)i)));
}

struct UgParams {
    bf16_t *C;
    uint32_t m, n, k, ldc;          // n = weight rows of the product (2 * inter with swiglu)
    uint32_t nt;                    // weight rows per tile: N of the MMA (a multiple of 16, 128 with swiglu or a k split; swiglu: nt/2 gate rows + nt/2 up rows)
    uint32_t passes;                // token blocks of 128 rows: 1 (m <= 128) or 2
    uint32_t x_bytes;               // bytes of the token rows a stage holds: passes == 2: 2 x 16 KB, else m rounded up to 8 rows x 128 B
    uint32_t nkb;                   // k blocks of 64 in the whole product
    uint32_t ksplit;                // cluster size: CTAs that share the k range of a tile
    uint32_t cw;                    // k split: output columns of a tile owned by each CTA of the cluster (a multiple of 8)
    uint32_t stages;                // ring depth of each stream
    uint32_t swiglu, half_n;        // swiglu: output [m, half_n], tile columns [0, nt/2) gate, [nt/2, nt) the matching up rows
    uint32_t acc_stride;            // tensor-memory columns between the streams' accumulators: power of two >= passes * nt
    uint32_t tmem_cols;             // UG_NS * acc_stride
    uint32_t vec_ok;                // C rows may be written in 16-byte pieces (C 16-byte aligned, ldc a multiple of 8)
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
// Instruction descriptor: bf16 x bf16 -> f32, both operands K-major, M = 128, N = n.
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
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]),
                   "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
                   "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                 : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
// 16-byte store into the shared memory of CTA `rank` of the cluster, at the address that `local_saddr` has in this CTA
__device__ __forceinline__ void st_remote_f32x4(uint32_t local_saddr, uint32_t rank, float a, float b, float c, float d) {
    uint32_t ra;
    asm("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(local_saddr), "r"(rank));
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(ra), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) { return (uint32_t)f2bf(lo) | ((uint32_t)f2bf(hi) << 16); }

// Dynamic shared memory (base rounded up to 1024 bytes): [UG_NS streams x stages x (weight tile | token block(s))]; once the main
// loop is over the idle ring holds, in a k-split CTA, the f32 partials it owns: [source rank][token][cw (x2 with swiglu)].
// Barriers, the abort flag and the tensor-memory address are static.
//
// Warps: 0 / 2 = producers and 1 / 3 = MMA issuers of streams 0 / 1, 4-7 = epilogue.  Measured on B200: the thread that issues
// tcgen05.mma needs ~800 cycles per k block (barrier wait ~200, four MMAs and the commit ~600) whatever the tile size and
// wherever the data comes from, which caps ONE issuing thread at ~40 GB/s of weights for a 128-row tile -- below an SM's share
// of HBM.  So a CTA runs UG_NS = 2 independent pipelines: stream j takes k blocks j, j + 2, ... through its own stages and
// barriers into its own accumulator; the epilogue adds accumulator 1 to accumulator 0.  Which block goes to which stream is
// fixed by the block index, so the order of every sum is still fixed by (n, k) alone.
__global__ void __launch_bounds__(UG_THREADS, 1)
ugemm_kernel(const __grid_constant__ CUtensorMap tm_w0, const __grid_constant__ CUtensorMap tm_w1,
             const __grid_constant__ CUtensorMap tm_x, const UgParams P) {
    pdl_trigger();
    if (threadIdx.x < 3) {   // the copy engine reads a 128-byte descriptor before its first copy: fetch the three of them now
        const CUtensorMap *tm = threadIdx.x == 0 ? &tm_w0 : (threadIdx.x == 1 ? &tm_w1 : &tm_x);
        asm volatile("prefetch.tensormap [%0];" ::"l"(tm) : "memory");
    }
    extern __shared__ unsigned char ug_smem_raw[];
    __shared__ uint64_t bar_full[UG_NS][UG_MAX_STAGES], bar_empty[UG_NS][UG_MAX_STAGES], bar_accum[UG_NS];
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile uint32_t abort_s;
    unsigned char *ring = ug_smem_raw + ((1024u - (smem_u32(ug_smem_raw) & 1023u)) & 1023u);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t S = P.stages, NT = P.nt, w_bytes = NT * 128u, stage_bytes = w_bytes + P.x_bytes;   // S: stages per stream
    const uint32_t rank = P.ksplit > 1 ? cluster_rank() : 0u;
    const uint32_t tile = blockIdx.x / P.ksplit;
    const uint32_t ocols = P.swiglu ? NT / 2 : NT;          // output columns of a tile
    const uint32_t r0 = tile * ocols;                        // first weight row of the tile (swiglu: in both halves), = first output column
    // k blocks of this CTA: nkb split into ksplit contiguous parts, the first `rem` parts one block longer
    const uint32_t per = P.nkb / P.ksplit, rem = P.nkb % P.ksplit;
    const uint32_t kb_lo = rank * per + min(rank, rem), my_kb = per + (rank < rem ? 1u : 0u);
    const uint32_t acc_cols = P.acc_stride;                  // tensor-memory columns between the streams' accumulators

    if (tid == 0) {
        for (uint32_t j = 0; j < UG_NS; j++) {
            for (uint32_t s = 0; s < S; s++) { mbar_init(smem_u32(&bar_full[j][s]), 1); mbar_init(smem_u32(&bar_empty[j][s]), 1); }
            mbar_init(smem_u32(&bar_accum[j]), 1);
        }
        abort_s = 0;
        tmem_base_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    auto load_w = [&](uint32_t dst, uint32_t kb, uint32_t fb) {
        tma_2d(dst, &tm_w0, kb * UG_BK, r0, fb);
        if (P.swiglu) tma_2d(dst + (NT / 2) * 128, &tm_w1, kb * UG_BK, r0, fb);
    };
    auto load_x = [&](uint32_t dst, uint32_t kb, uint32_t fb) {
        tma_2d(dst, &tm_x, kb * UG_BK, 0, fb);
        if (P.passes == 2) tma_2d(dst + UG_XTILE, &tm_x, kb * UG_BK, 128, fb);
    };
    // role of this warp: stream j = warp / 2 for warps 0..3 (even: producer, odd: MMA issuer)
    const uint32_t strm = (uint32_t)warp >> 1;
    const bool is_prod = warp < 2 * UG_NS && (warp & 1) == 0, is_mma = warp < 2 * UG_NS && (warp & 1) == 1;
    const uint32_t sring = smem_u32(ring) + strm * S * stage_bytes;                      // this stream's stages
    const uint32_t my_n = my_kb > strm ? (my_kb - strm + UG_NS - 1) / UG_NS : 0u;        // k blocks of this stream: kb_lo + strm + UG_NS * i
    const uint32_t pre = min(S, my_n);
    if (is_prod && lane == 0) {
        // ---- producer, part 1: weight copies of the first stages while the predecessor kernel is still running
        for (uint32_t i = 0; i < pre; i++) {
            const uint32_t fb = smem_u32(&bar_full[strm][i]);
            mbar_expect_tx(fb, stage_bytes);
            load_w(sring + i * stage_bytes, kb_lo + strm + UG_NS * i, fb);
        }
    }
    // Tensor memory is claimed before the wait for the predecessor grid.  That is safe only because no two CTAs that use
    // tensor memory can share an SM: every launch of this kernel takes more than half of an SM's shared memory (the host
    // pads the request), and nothing else in the library allocates tensor memory.  (A CTA that held columns while waiting
    // for a predecessor CTA on the same SM that still needed columns would deadlock.)
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(P.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        tc_fence_before();
    }
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;
    pdl_wait();   // the tokens are the predecessor's output
    if (is_prod && lane == 0) {
        for (uint32_t i = 0; i < pre; i++) load_x(sring + i * stage_bytes + w_bytes, kb_lo + strm + UG_NS * i, smem_u32(&bar_full[strm][i]));
    }
    __syncwarp();

    if (is_prod) {
        // ---- producer, part 2: the remaining stages, each as soon as the MMAs that read its slot have completed
        if (lane == 0) {
            for (uint32_t i = pre; i < my_n; i++) {
                const uint32_t s = i % S;
                if (!mbar_wait(smem_u32(&bar_empty[strm][s]), ((i / S) - 1) & 1, &abort_s)) break;
                const uint32_t fb = smem_u32(&bar_full[strm][s]), dst = sring + s * stage_bytes;
                mbar_expect_tx(fb, stage_bytes);
                load_w(dst, kb_lo + strm + UG_NS * i, fb);
                load_x(dst + w_bytes, kb_lo + strm + UG_NS * i, fb);
            }
        }
        __syncwarp();
    } else if (is_mma) {
        // ---- MMA issue: one thread per stream; D_j[128 tokens x NT] (+)= X[128 x 16] * W_tile[NT x 16]^T, four k-steps per stage
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(NT), td = tmem_base + strm * acc_cols;
            for (uint32_t i = 0; i < my_n; i++) {
                const uint32_t s = i % S;
                if (!mbar_wait(smem_u32(&bar_full[strm][s]), (i / S) & 1, &abort_s)) break;
                tc_fence_after();
                const uint32_t base = sring + s * stage_bytes;
                const uint64_t dw = umma_desc(base), dx = umma_desc(base + w_bytes);
#pragma unroll
                for (int kk = 0; kk < UG_BK / 16; kk++) {
                    umma_bf16(td, dx + 2 * kk, dw + 2 * kk, idesc, (i | kk) != 0 ? 1u : 0u);
                    if (P.passes == 2) umma_bf16(td + NT, dx + (UG_XTILE >> 4) + 2 * kk, dw + 2 * kk, idesc, (i | kk) != 0 ? 1u : 0u);
                }
                umma_commit(smem_u32(&bar_empty[strm][s]));   // the slot is free once these MMAs have read it
            }
            umma_commit(smem_u32(&bar_accum[strm]));           // all MMAs of this stream complete: its accumulators are final
        }
        __syncwarp();
    }

    // ---- epilogue: all eight warps (the producers and MMA issuers are done); warp w may touch the 32 tensor-memory lanes
    // (= tokens) of quadrant w % 4, so warps w and w + 4 share a quadrant and take one half of the tile's output columns each
    const uint32_t q = warp & 3, half = (uint32_t)warp >> 2;
    const uint32_t tq = tmem_base + ((q * 32u) << 16);
    const uint32_t n_acc = my_kb < UG_NS ? my_kb : UG_NS;     // streams that got at least one k block
    bool go = false;    // warp-uniform: the tensor-memory loads below are warp-wide instructions
    {
        bool accum_ok = true;
        for (uint32_t j = 0; j < n_acc; j++) accum_ok = accum_ok && mbar_wait(smem_u32(&bar_accum[j]), 0, &abort_s);
        go = __all_sync(0xffffffffu, accum_ok && !abort_s) != 0;
        tc_fence_after();
    }
    // 16 accumulator columns of this thread's token from each stream that ran: issue, then (after tmem_ld_wait) add stream 1 to
    // stream 0 (which k block went to which stream is fixed by the block index: a fixed order)
    auto acc_issue = [&](uint32_t col, uint32_t (&v)[16], uint32_t (&w)[16]) {
        if (n_acc >= 1) tmem_ld16(tq + col, v);
        if (n_acc == 2) tmem_ld16(tq + acc_cols + col, w);
    };
    auto acc_sum = [&](uint32_t (&v)[16], const uint32_t (&w)[16]) {
#pragma unroll
        for (int e = 0; e < 16; e++) {
            const float a = n_acc >= 1 ? __uint_as_float(v[e]) : 0.0f;
            v[e] = __float_as_uint(n_acc == 2 ? a + __uint_as_float(w[e]) : a);
        }
    };
    const uint32_t n_out = P.swiglu ? P.half_n : P.n;
    // eight finished output values of one token, columns col0 .. col0+7 of the tile
    auto store8 = [&](uint32_t tok, uint32_t col0, const float (&o)[8]) {
        const uint32_t gc = r0 + col0;
        if (gc >= n_out) return;
        bf16_t *dst = P.C + (size_t)tok * P.ldc + gc;
        if (P.vec_ok && gc + 8 <= n_out) *reinterpret_cast<uint4 *>(dst) = make_uint4(pack2(o[0], o[1]), pack2(o[2], o[3]), pack2(o[4], o[5]), pack2(o[6], o[7]));
        else for (uint32_t e = 0; e < 8 && gc + e < n_out; e++) dst[e] = f2bf(o[e]);
    };
    if (P.ksplit == 1) {
        if (go) {
            // the two warps of a lane quadrant split the tile's columns at a multiple of 32 (ocols is a multiple of 16; with
            // swiglu, where the halves must be equal, of 32)
            const uint32_t split = P.swiglu ? ocols / 2 : (ocols + 63) / 64 * 32;
            const uint32_t c_lo = half ? split : 0u, c_hi = half ? ocols : split;
            for (uint32_t p = 0; p < P.passes; p++) {
                if (p * 128 + q * 32 >= P.m) break;                 // no token of this warp's quadrant in this block (warp-uniform)
                const uint32_t tok = p * 128 + q * 32 + lane;
                if (!P.swiglu) {
                    // plain rows: 32 columns per step (one load per stream, one wait), 64 contiguous bytes of the C row; a tile
                    // whose width is an odd multiple of 16 ends with a 16-column step
                    for (uint32_t c0 = c_lo; c0 < c_hi; c0 += 32) {
                        if (c_hi - c0 < 32) {
                            uint32_t v[16], w[16];
                            acc_issue(p * NT + c0, v, w);
                            tmem_ld_wait();
                            acc_sum(v, w);
                            if (tok < P.m) {
#pragma unroll
                                for (int h = 0; h < 2; h++) {
                                    float o[8];
#pragma unroll
                                    for (int e = 0; e < 8; e++) o[e] = __uint_as_float(v[h * 8 + e]);
                                    store8(tok, c0 + h * 8, o);
                                }
                            }
                            break;
                        }
                        uint32_t v[32], w[32];
                        if (n_acc >= 1) tmem_ld32(tq + p * NT + c0, v);
                        if (n_acc == 2) tmem_ld32(tq + acc_cols + p * NT + c0, w);
                        tmem_ld_wait();
                        if (tok < P.m) {
#pragma unroll
                            for (int h = 0; h < 4; h++) {
                                float o[8];
#pragma unroll
                                for (int e = 0; e < 8; e++) {
                                    const float a = n_acc >= 1 ? __uint_as_float(v[h * 8 + e]) : 0.0f;
                                    o[e] = n_acc == 2 ? a + __uint_as_float(w[h * 8 + e]) : a;
                                }
                                store8(tok, c0 + h * 8, o);
                            }
                        }
                    }
                    continue;
                }
                for (uint32_t c0 = c_lo; c0 < c_hi; c0 += 16) {
                    uint32_t g[16], g1[16], u[16], u1[16];
                    acc_issue(p * NT + c0, g, g1);
                    if (P.swiglu) acc_issue(p * NT + NT / 2 + c0, u, u1);
                    tmem_ld_wait();
                    acc_sum(g, g1);
                    if (P.swiglu) acc_sum(u, u1);
                    if (tok < P.m) {
#pragma unroll
                        for (int h = 0; h < 2; h++) {
                            float o[8];
#pragma unroll
                            for (int e = 0; e < 8; e++) {
                                const float a = __uint_as_float(g[h * 8 + e]);
                                // SiluMulOp: bf16(bf16(silu(bf16 gate)) * bf16 up), the activation from the table of all bf16 inputs
                                o[e] = P.swiglu ? __fmul_rn(bf2f(g_silu_lut[f2bf(a)]), rbf(__uint_as_float(u[h * 8 + e]))) : a;
                            }
                            store8(tok, c0 + h * 8, o);
                        }
                    }
                }
            }
        }
    } else {
        // k split over the cluster: output column c of the tile belongs to CTA c / cw.  Once every CTA of the cluster has left its
        // main loop (its ring is idle: every copy has landed and every MMA has read it), each CTA sends the columns of its f32
        // partial straight from tensor memory into the owner's ring, [source rank][4-column piece][token] (gate | up: 2 cw
        // columns): a warp's 32 tokens of one piece are 512 contiguous bytes of the owner's memory.  After a second barrier
        // the owner adds the partials of its columns in rank order from its own shared memory.
        const uint32_t cw = P.cw, roww = P.swiglu ? 2 * cw : cw;   // floats per staged token row
        float *stg = reinterpret_cast<float *>(ring);
        tc_fence_before();
        cluster_sync_all();
        if (go) {
            const uint32_t c_lo = half * (NT / 2), c_hi = c_lo + NT / 2;
            for (uint32_t p = 0; p < P.passes; p++) {
                if (p * 128 + q * 32 >= P.m) break;
                const uint32_t tok = p * 128 + q * 32 + lane;
                for (uint32_t c0 = c_lo; c0 < c_hi; c0 += 16) {
                    uint32_t v[16], v1[16];
                    acc_issue(p * NT + c0, v, v1);
                    tmem_ld_wait();
                    acc_sum(v, v1);
                    if (tok < P.m) {
#pragma unroll
                        for (int h = 0; h < 4; h++) {
                            const uint32_t col = c0 + h * 4;                            // tile column of this 4-wide piece
                            const uint32_t oc = P.swiglu && col >= NT / 2 ? col - NT / 2 : col;   // the output column it feeds
                            const uint32_t owner = oc / cw, off = oc - owner * cw + (P.swiglu && col >= NT / 2 ? cw : 0u);
                            const uint32_t a = smem_u32(&stg[(((size_t)rank * (roww / 4) + off / 4) * P.m + tok) * 4]);
                            st_remote_f32x4(a, owner, __uint_as_float(v[h * 4]), __uint_as_float(v[h * 4 + 1]), __uint_as_float(v[h * 4 + 2]), __uint_as_float(v[h * 4 + 3]));
                        }
                    }
                }
            }
        }
        tc_fence_before();
        cluster_sync_all();   // release / acquire: the partials sent above are visible to their owners
        const uint32_t oc_lo = min(ocols, rank * cw), oc_hi = min(ocols, oc_lo + cw);
        if (!abort_s && oc_hi > oc_lo) {   // (a peer that gave up sends nothing: the timeout counter flags the result)
            const uint32_t chunks = (oc_hi - oc_lo + 7) / 8;
            for (uint32_t it = tid; it < P.m * chunks; it += UG_THREADS) {
                const uint32_t ch = it / P.m, tok = it - ch * P.m;   // consecutive threads: consecutive tokens of one piece
                float a[8] = {0, 0, 0, 0, 0, 0, 0, 0}, b[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                for (uint32_t rk = 0; rk < P.ksplit; rk++) {
                    const float *src = &stg[(((size_t)rk * (roww / 4) + ch * 2) * P.m + tok) * 4];   // pieces 2 ch and 2 ch + 1
                    const float4 x0 = *reinterpret_cast<const float4 *>(src), x1 = *reinterpret_cast<const float4 *>(src + (size_t)P.m * 4);
                    a[0] += x0.x; a[1] += x0.y; a[2] += x0.z; a[3] += x0.w; a[4] += x1.x; a[5] += x1.y; a[6] += x1.z; a[7] += x1.w;
                    if (P.swiglu) {
                        const float *up = src + (size_t)(cw / 4) * P.m * 4;
                        const float4 y0 = *reinterpret_cast<const float4 *>(up), y1 = *reinterpret_cast<const float4 *>(up + (size_t)P.m * 4);
                        b[0] += y0.x; b[1] += y0.y; b[2] += y0.z; b[3] += y0.w; b[4] += y1.x; b[5] += y1.y; b[6] += y1.z; b[7] += y1.w;
                    }
                }
                float o[8];
#pragma unroll
                for (int e = 0; e < 8; e++) o[e] = P.swiglu ? __fmul_rn(bf2f(g_silu_lut[f2bf(a[e])]), rbf(b[e])) : a[e];
                store8(tok, oc_lo + ch * 8, o);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
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

void ug_launch_cfg(cudaLaunchConfig_t *cfg, cudaLaunchAttribute *at, uint32_t ctas, uint32_t ksplit, size_t smem, cudaStream_t st) {
    *cfg = cudaLaunchConfig_t{};
    cfg->gridDim = dim3(ctas); cfg->blockDim = dim3(UG_THREADS); cfg->dynamicSmemBytes = smem; cfg->stream = st;
    int na = 0;
    at[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[na].val.programmaticStreamSerializationAllowed = 1;
    na++;
    if (ksplit > 1) {
        at[na].id = cudaLaunchAttributeClusterDimension;
        at[na].val.clusterDim.x = ksplit; at[na].val.clusterDim.y = 1; at[na].val.clusterDim.z = 1;
        na++;
    }
    cfg->attrs = at; cfg->numAttrs = na;
}

}  // namespace

// Per device: SM count and how many clusters of each size the device keeps resident at once (CTAs of the full shared-memory size).
struct UgDevice { int sms = 0; int max_clusters[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0}; };   // sms != 0: the device is set up (opt-ins made, activation table filled)
static UgDevice g_ug_dev[64];   // written once per device ordinal by wb_ugemm_init (the same values by any thread)

// The k split of a product, from the weight shape and the device alone (never from m, so a row's summation order is the same
// in every batch).  Cost of a split s, in k blocks: rounds of CTAs x (blocks per CTA + a CTA's fixed cost); one round holds
// as many CTAs as the device has SMs (two CTAs of an SM share its bandwidth, the second one only hides fixed costs) and, with
// a split, as many clusters as the device keeps resident.  Measured fixed costs: ~8 blocks per CTA, ~6 more for the
// cluster's exchange.
static uint32_t ug_ksplit(uint32_t tiles, uint32_t nkb, const UgDevice &d) {
    uint32_t best = 1;
    double best_cost = 1e30;
    for (uint32_t s = 1; s <= 8; s++) {
        if (s > 1 && (nkb / s < 6 || d.max_clusters[s] <= 0)) continue;
        const double cap = s == 1 ? (double)d.sms : (double)((uint32_t)d.max_clusters[s] * s < (uint32_t)d.sms ? d.max_clusters[s] * s : d.sms);
        const double rounds = ceil((double)tiles * s / cap);
        const double cost = rounds * ((double)((nkb + s - 1) / s) + (s == 1 ? 8.0 : 14.0));
        if (cost < best_cost - 1e-9) { best_cost = cost; best = s; }
    }
    return best;
}

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
    if (!g_ug_dev[dev].sms) {
        UgDevice d;
        cudaError_t e = cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(ugemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, UG_SMEM_MAX);
        if (e != cudaSuccess || d.sms <= 0) { wb_set_error("gemm: shared-memory opt-in failed: %s", cudaGetErrorString(e)); return WB_ERR_CUDA; }
        silu_lut_kernel<<<256, 256>>>();   // the activation table of this device, before anything can read it
        e = cudaGetLastError();
        if (e == cudaSuccess) e = cudaDeviceSynchronize();
        if (e != cudaSuccess) { wb_set_error("gemm: filling the activation table failed: %s", cudaGetErrorString(e)); return WB_ERR_CUDA; }
        for (uint32_t s = 2; s <= 8; s++) {
            cudaLaunchConfig_t cfg;
            cudaLaunchAttribute at[2];
            ug_launch_cfg(&cfg, at, s * 8, s, UG_SMEM_MAX, nullptr);
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, ugemm_kernel, &cfg) == cudaSuccess) d.max_clusters[s] = n;
            else cudaGetLastError();
        }
        g_ug_dev[dev] = d;
    }
    return WB_OK;
}

// A 2-d tensor map for other kernels of the library: `rows` rows of `inner` elements (4-byte when f32, else 2-byte), rows
// row_bytes apart, boxes of box_inner x box_rows elements (box_inner elements = 128 bytes), 128-byte swizzle.  `tm` points
// at a CUtensorMap (128 bytes, 64-byte aligned).
int32_t wb_tensor_map_2d(void *tm, bool f32, const void *base, uint64_t inner, uint64_t rows, uint64_t row_bytes, uint32_t box_inner, uint32_t box_rows) {
    if (int32_t rc = wb_ugemm_init()) return rc;
    const cuuint64_t dims[2] = {inner, rows};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {box_inner, box_rows};
    const cuuint32_t ones[2] = {1, 1};
    CUresult r = g_ug_encode((CUtensorMap *)tm, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims,
                             strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { wb_set_error("cuTensorMapEncodeTiled failed (%d)", (int)r); return WB_ERR_CUDA; }
    return WB_OK;
}


// Launch geometry of one chunk of mc <= 256 token rows.
struct UgGeom { uint32_t nt, tiles, nkb, ksplit, cw, passes, x_rows, x_bytes, stages, acc_stride, tmem_cols; size_t smem; };
static bool ug_geometry(uint32_t mc, uint32_t n, uint32_t k, bool swiglu, const UgDevice &d, UgGeom *g) {
    const uint32_t out_cols = swiglu ? n / 2 : n;
    g->nkb = (k + UG_BK - 1) / UG_BK;
    g->passes = mc > 128 ? 2 : 1;
    g->x_rows = g->passes == 2 ? 128 : (mc + 7) / 8 * 8;          // rows of the token box
    g->x_bytes = g->passes * g->x_rows * 128;
    // Weight rows per tile: 256 (8 KB of weights per MMA) when that still gives every SM a CTA, else 128.  The choice groups
    // output columns and never changes a sum; the k split is taken for 128-row tiles so that it does not depend on it.
    const uint32_t tiles128 = swiglu ? (out_cols + 63) / 64 : (out_cols + 127) / 128;
    g->ksplit = ug_ksplit(tiles128, g->nkb, d);
    const uint32_t tiles256 = (tiles128 + 1) / 2;
    g->nt = ((uint64_t)tiles256 * g->ksplit >= (uint64_t)d.sms && UG_NS * g->passes * 256 <= 512) ? 256 : 128;
    g->tiles = g->nt == 256 ? tiles256 : tiles128;
    if (!swiglu && g->ksplit == 1) {
        // A plain product without k split may take any tile width that is a multiple of 16: the width with the least
        // waves x (rows of a tile + the fixed cost of a CTA, about 5 us of streaming = 215 KB of weight rows), so that 12,352
        // rows are 129 tiles of 96 rather than 97 of 128 on 148 SMs, and 151,936 rows 731 of 208 (5 waves) rather than 594
        // of 256 (5 waves with 2 CTAs in the last).  At least 80 rows keep the two MMA threads ahead of an SM's share of HBM.
        const uint32_t fixed = 215u * 1024u / (k * 2u) + 1u, max_nt = UG_NS * g->passes * 256 <= 512 ? 256u : 128u;
        uint64_t best = ~0ull;
        for (uint32_t nt = 80; nt <= max_nt; nt += 16) {
            const uint64_t tiles = (out_cols + nt - 1) / nt, waves = (tiles + d.sms - 1) / d.sms, cost = waves * (nt + fixed);
            if (cost < best || (cost == best && nt == 128)) { best = cost; g->nt = nt; g->tiles = (uint32_t)tiles; }
        }
    }
    const uint32_t ocols = swiglu ? g->nt / 2 : g->nt;
    g->cw = ((ocols + g->ksplit - 1) / g->ksplit + 7) / 8 * 8;
    // Shared memory: one CTA per SM with as many stages as fit (measured: CTAs of half an SM with fewer stages each were slower
    // in every shape, 24 against 20 us for the gate|up product at 40 rows); in a k-split CTA the ring must hold the partials it
    // owns.
    const size_t stage = (size_t)g->nt * 128 + g->x_bytes;
    const size_t tail = UG_XTILE;   // the MMA reads 128 token rows from a stage that may hold fewer: keep that read inside the allocation
    const size_t staging = g->ksplit > 1 ? (size_t)g->ksplit * mc * (swiglu ? 2 : 1) * g->cw * 4 : 0;
    const size_t budget = UG_SMEM_MAX;
    uint32_t stages = (uint32_t)((budget - 1024 - tail) / (UG_NS * stage));   // per stream
    if (stages > UG_MAX_STAGES) stages = UG_MAX_STAGES;
    if (stages < 1 || UG_NS * stages * stage < staging || UG_NS * g->passes * g->nt > 512) return false;
    g->stages = stages;
    g->smem = 1024 + (size_t)UG_NS * stages * stage + tail;
    if (g->smem < (size_t)UG_SMEM_SOLO) g->smem = UG_SMEM_SOLO;   // never two of these CTAs on one SM (see the tensor-memory claim in the kernel)
    uint32_t cols = 32;
    while (cols < g->passes * g->nt) cols *= 2;
    g->acc_stride = cols;
    g->tmem_cols = UG_NS * cols;
    return true;
}

// C[m,n] = A W^T (swiglu: W = [gate; up] of n = 2 * inter rows, C[m, inter]); arguments validated by the callers in gemm.cu.
// m beyond 256 is processed in chunks of 256 token rows.
int32_t wb_ugemm(const void *a, const void *w, void *c, uint32_t m, uint32_t n, uint32_t k, uint32_t lda, uint32_t ldc, bool swiglu,
                 cudaStream_t st) {
    if (int32_t rc = wb_ugemm_init()) return rc;
    int dev = 0;
    cudaGetDevice(&dev);
    const UgDevice &d = g_ug_dev[dev];
    const uint32_t rows = swiglu ? n / 2 : n;                                   // rows of each weight map
    CUtensorMap tw0, tw1, tx;
    bool ok = true;
    for (uint32_t m0 = 0; ok && m0 < m; m0 += 256) {
        const uint32_t mc = m - m0 < 256 ? m - m0 : 256;
        UgGeom g;
        if (!ug_geometry(mc, n, k, swiglu, d, &g)) { wb_set_error("gemm: m = %u rows do not fit the tensor-memory kernel's shared memory", mc); return WB_ERR_SHAPE; }
        UgParams p{};
        p.C = (bf16_t *)c + (size_t)m0 * ldc;
        p.m = mc; p.n = n; p.k = k; p.ldc = ldc;
        p.acc_stride = g.acc_stride; p.nt = g.nt; p.passes = g.passes; p.x_bytes = g.x_bytes; p.nkb = g.nkb; p.ksplit = g.ksplit; p.cw = g.cw; p.stages = g.stages; p.tmem_cols = g.tmem_cols;
        p.swiglu = swiglu ? 1 : 0; p.half_n = n / 2;
        p.vec_ok = (ldc % 8 == 0 && ((uintptr_t)p.C & 15u) == 0) ? 1 : 0;
        const uint32_t wbox = swiglu ? g.nt / 2 : g.nt;
        ok = ug_map(&tw0, w, rows, k, k, wbox) && ug_map(&tw1, swiglu ? (const bf16_t *)w + (size_t)rows * k : (const bf16_t *)w, rows, k, k, wbox) &&
             ug_map(&tx, (const bf16_t *)a + (size_t)m0 * lda, mc, k, lda, g.x_rows);
        if (!ok) break;
        cudaLaunchConfig_t cfg;
        cudaLaunchAttribute at[2];
        ug_launch_cfg(&cfg, at, g.tiles * g.ksplit, g.ksplit, g.smem, st);
        cudaError_t e = cudaLaunchKernelEx(&cfg, ugemm_kernel, tw0, tw1, tx, p);
        if (e != cudaSuccess) { wb_set_error("gemm: launch failed for m=%u n=%u k=%u: %s", mc, n, k, cudaGetErrorString(e)); return WB_ERR_CUDA; }
    }
    if (!ok) { wb_set_error("gemm: cuTensorMapEncodeTiled failed for m=%u n=%u k=%u", m, n, k); return WB_ERR_CUDA; }
    return WB_OK;
}

// How the tensor-memory kernel would run a product on the current device: out[0] = CTAs, out[1] = k split (cluster size),
// out[2] = pipeline stages, out[3] = shared memory per CTA in bytes, out[4] = weight rows per tile.  The k split depends on (n, k) and the device, never on m.
extern "C" int32_t wein_b200_gemm_plan(uint32_t m, uint32_t n, uint32_t k, uint32_t swiglu, uint32_t *out) {
    WB_CHECK_ARG(out && m >= 1 && n >= 1 && k >= 8, "gemm_plan: bad argument");
    if (int32_t rc = wb_ugemm_init()) return rc;
    int dev = 0;
    cudaGetDevice(&dev);
    UgGeom g;
    if (!ug_geometry(m < 256 ? m : 256, swiglu ? 2 * n : n, k, swiglu != 0, g_ug_dev[dev], &g)) { wb_set_error("gemm_plan: shape does not fit"); return WB_ERR_SHAPE; }
    out[0] = g.tiles * g.ksplit; out[1] = g.ksplit; out[2] = g.stages; out[3] = (uint32_t)g.smem; out[4] = g.nt;
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
