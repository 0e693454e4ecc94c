// Shared device helpers of the wein-b200 kernels.
//
// Numeric discipline (mirrors crates/wein-kernel/src/reference.rs:7-11 of the
// reference): bf16 -> f32 is an exact shift; f32 -> bf16 is round-to-nearest-even
// by the reference's integer formula; multiply / add / divide / sqrt are the
// correctly rounded IEEE operations and a fused multiply-add appears only where
// the reference writes mul_add.  Files that include this header for bit-parity
// kernels are compiled with -fmad=false so the compiler never contracts a*b+c.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define WB_OK 0
#define WB_ERR_ARG (-1)      // invalid argument, rejected before any launch
#define WB_ERR_SHAPE (-2)    // shape outside what the kernels are built for
#define WB_ERR_CUDA (-3)     // a CUDA runtime call failed (see wein_b200_last_error)
#define WB_ERR_CAPACITY (-4) // caller-provided scratch too small

// Bits of a device status word (one per sequence slot of an engine; OR-ed in by kernels, never cleared by them)
#define WB_STATUS_POS_LIMIT 1u   // the round was refused for this slot: position + 1 would pass the slot's position limit
#define WB_STATUS_K_CLAMPED 2u   // fewer drafts than asked were verified because the chain would have passed the position limit
#define WB_STATUS_CTX_BOUND 4u   // the caller's context bound was below position + chain length: attention ignored later segments
#define WB_STATUS_SAMPLER 8u     // the sampler met an invalid parameter (top_k = 0 with temperature > 0)

typedef uint16_t bf16_t;

__host__ __device__ __forceinline__ float bf2f(bf16_t h) {
#ifdef __CUDA_ARCH__
    return __uint_as_float(((uint32_t)h) << 16);
#else
    union { uint32_t u; float f; } c; c.u = ((uint32_t)h) << 16; return c.f;
#endif
}
// reference.rs:19-23
__host__ __device__ __forceinline__ bf16_t f2bf(float x) {
#ifdef __CUDA_ARCH__
    uint32_t u = __float_as_uint(x);
#else
    union { uint32_t u; float f; } c; c.f = x; uint32_t u = c.u;
#endif
    uint32_t lsb = (u >> 16) & 1u;
    return (bf16_t)((u + 0x7fffu + lsb) >> 16);
}
__device__ __forceinline__ float rbf(float x) { return bf2f(f2bf(x)); }

// exp by floor + degree-7 Horner of 2^f, no MUFU (reference.rs:61-94).
// Written with explicit non-fused operations so it is exact under any -fmad.
__device__ __forceinline__ float expf_ref(float x) {
    const float LOG2E = 1.4426950408889634f;
    float t = __fmul_rn(x, LOG2E);
    float kf = floorf(t);
    if (kf < -126.0f) return 0.0f;
    if (kf > 127.0f) return __int_as_float(0x7f800000);
    float f = __fsub_rn(t, kf);
    float p = 1.5252733804059838e-05f;
    p = __fadd_rn(__fmul_rn(p, f), 0.00015403530393381606f);
    p = __fadd_rn(__fmul_rn(p, f), 0.0013333558146428441f);
    p = __fadd_rn(__fmul_rn(p, f), 0.009618129107628477f);
    p = __fadd_rn(__fmul_rn(p, f), 0.055504108664821576f);
    p = __fadd_rn(__fmul_rn(p, f), 0.2402265069591007f);
    p = __fadd_rn(__fmul_rn(p, f), 0.6931471805599453f);
    p = __fadd_rn(__fmul_rn(p, f), 1.0f);
    return __int_as_float(__float_as_int(p) + (((int)kf) << 23));
}
// reference.rs:329-345
__device__ __forceinline__ float log2f_ref(float z) {
    const float SQRT2 = 1.4142135f, LN2 = 0.6931471805599453f;
    uint32_t bits = __float_as_uint(z);
    int e = (int)(bits >> 23) - 127;
    float m = __uint_as_float((bits & 0x007fffffu) | 0x3f800000u);
    if (m > SQRT2) { m = __fmul_rn(m, 0.5f); e += 1; }
    float r = __fdiv_rn(__fsub_rn(m, 1.0f), __fadd_rn(m, 1.0f));
    float r2 = __fmul_rn(r, r);
    float s = 1.0f / 11.0f;
    s = __fadd_rn(1.0f / 9.0f, __fmul_rn(r2, s));
    s = __fadd_rn(1.0f / 7.0f, __fmul_rn(r2, s));
    s = __fadd_rn(1.0f / 5.0f, __fmul_rn(r2, s));
    s = __fadd_rn(1.0f / 3.0f, __fmul_rn(r2, s));
    s = __fadd_rn(1.0f, __fmul_rn(r2, s));
    float at = __fmul_rn(r, s);
    return __fadd_rn((float)e, __fmul_rn(at, 2.0f / LN2));
}
// reference.rs:348-355
__device__ __forceinline__ float softplus_ref(float x) {
    const float LN2 = 0.6931471805599453f;
    if (x > 20.0f) return x;
    return __fmul_rn(log2f_ref(__fadd_rn(1.0f, expf_ref(x))), LN2);
}
// 1 / (1 + exp(-x)) with a correctly rounded division
__device__ __forceinline__ float sigmoid_ref(float x) {
    return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf_ref(__fsub_rn(0.0f, x))));
}
// x * sigmoid(x), the reference's silu expression (reference.rs:141-148)
__device__ __forceinline__ float silu_ref(float v) {
    return __fmul_rn(v, __fdiv_rn(1.0f, __fadd_rn(1.0f, expf_ref(-v))));
}

// Sum over a block in the reference's fixed tree (reference.rs:360-393): a
// shfl.down tree inside each warp, then the same tree over the warp leaders.
// blockDim.x must be a multiple of 32 (<= 1024); every thread gets the total.
__device__ __forceinline__ float block_sum_tree(float v, float *smem /* >= 33 floats */) {
    const unsigned full = 0xffffffffu;
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
        float o = __shfl_down_sync(full, v, off);
        if (lane + off < 32) v = __fadd_rn(v, o);
    }
    __syncthreads();  // protects smem reuse across calls
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float w = lane < nw ? smem[lane] : 0.0f;
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
            float o = __shfl_down_sync(full, w, off);
            if (lane + off < 32) w = __fadd_rn(w, o);
        }
        if (lane == 0) smem[32] = w;
    }
    __syncthreads();
    return smem[32];
}

// Programmatic dependent launch (sm_90+): a kernel launched with the programmatic-serialization attribute may start
// while its predecessor in the stream is still running.  Every kernel of this library begins with PDL_ENTRY(): it lets
// its own successor start early, then waits until the predecessor grid has completed and its writes are visible.  Work
// that touches no produced data (weight prefetch) may be placed between the two.  Without the attribute both are no-ops.
// Because a kernel's lifetime now overlaps its producer's, data written by earlier kernels must never be read through the
// non-coherent path: no __ldg and no `const __restrict__` on such pointers (only weights use ld.global.nc).
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
#define PDL_ENTRY() do { pdl_trigger(); pdl_wait(); } while (0)

// Host-side launch helper: every kernel goes through cudaLaunchKernelEx with the programmatic-serialization attribute.
template <typename... KArgs, typename... Args>
static inline cudaError_t wb_launch_k(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}
#define WB_LAUNCH(kern, grid, block, smem, st, ...) wb_launch_k(kern, grid, block, smem, st, __VA_ARGS__)

// Host-side error plumbing (defined in capi.cu)
void wb_set_error(const char *fmt, ...);
const char *wein_b200_last_error_buf();
#define WB_CHECK_ARG(cond, ...)                          \
    do {                                                 \
        if (!(cond)) { wb_set_error(__VA_ARGS__); return WB_ERR_ARG; } \
    } while (0)
#define WB_LAUNCH_CHECK()                                               \
    do {                                                                \
        cudaError_t e__ = cudaGetLastError();                           \
        if (e__ != cudaSuccess) { wb_set_error("%s:%d launch failed: %s", __FILE__, __LINE__, cudaGetErrorString(e__)); return WB_ERR_CUDA; } \
    } while (0)
