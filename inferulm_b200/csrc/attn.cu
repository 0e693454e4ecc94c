// Paged GQA attention for verify chains: the k+1 query positions of a chain times the q heads of one GQA
// group (<= 32 query rows) share every 16-token bf16 KV page they read.
//
// Reference contract: PagedAttnOp::run (crates/wein-kernel/src/ops/mod.rs:1687-1704) -- causal, row (seq, pos)
// sees keys 0..=pos, kv head = q head / group -- with the numerics of reference.rs:220-279 as the oracle under
// the reference's online-softmax tolerance (rel2 <= 3e-3, peak <= 1.5e-2, crates/wein-kernel/tests/ops_m0.rs:968-977).
// The reference has no verify-shaped kernel: chain rows go through its generic long-context kernel, which
// re-reads the KV pages per row group and keeps its working set in global scratch.
//
// One CTA = (chain m-tile, kv head, context segment).  A page of one kv head is 16 rows of 512 B (stride = kv_heads*512 B in
// the pool); each warp streams its own pages with 16-byte cp.async into an XOR-swizzled, double-buffered
// shared-memory tile (zero-filled past the end of the sequence), so KV crosses HBM once per chain.  QK^T and
// PV run on m16n8k16 bf16 MMAs fed by ldmatrix; softmax is the online (running max / running sum) form in
// f32 with the probabilities rounded to bf16 for the PV product.
//
// Batch-shape invariance: the context is cut into fixed segments of `seg_pages` pages.  One CTA reduces one
// segment for one m-tile of 16 query rows: warp w takes pages w, w+4, ... of the segment in order, the four
// warps merge in a fixed order through shared memory and the segment's partial (max, sum, unnormalised O)
// goes to scratch; a second kernel merges the segments in index order (and can apply the layer's output
// gate, out = bf16(bf16(attn) * bf16(sigmoid(gate)))).  The arithmetic a query row sees depends only on its
// own position and seg_pages -- not on the chain length, the batch, or the grid -- so row (seq, pos) of a
// k+1-row verify chain equals the same row of a plain one-token step bit for bit.
#include "common.cuh"
#include "internal.h"

#define ATT_PAGE 16
// Per-warp page pipeline depth NS (a template parameter: it never changes a result).  Two stages (136 KB per CTA at head_dim 256)
// for callers whose GEMMs run on the register-streaming kernel: that kernel wants the SM's memory as L1, and with 200 KB
// attention CTAs in between the SM is re-split around every attention launch (measured at batch 1: 2.71 -> 3.6 ms per round).
// Three stages for callers whose GEMMs take the whole shared memory anyway (the tensor-memory kernel): two page pairs in
// flight per warp instead of one.

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) { return (uint32_t)f2bf(lo) | ((uint32_t)f2bf(hi) << 16); }

struct AttnParams {
    const bf16_t *q, *k_cache, *v_cache, *gate;
    const uint32_t *block_table, *seq_ids, *positions, *row_start, *row_count;  // row_start/row_count null: every row is its own span
    bf16_t *out;
    float *part_o, *part_ml;  // [span][kvh][seg][32][HD] and [...][32][2]
    float scale_log2;
    uint32_t bpr, q_heads, kv_heads, n_spans, seg_pages, max_segs, n_mtiles;
    uint32_t *status;         // optional, indexed by sequence id: WB_STATUS_CTX_BOUND is OR-ed in when the caller's context bound
                              // was too small for a row (the row is then reduced over the segments the grid covers only)
};

// byte offset of 16-byte chunk `ch` of row `r` in a [rows][HD] bf16 tile, XOR-swizzled over the row's low 3 bits
template <int HD>
__device__ __forceinline__ uint32_t tile_off(uint32_t r, uint32_t ch) { return r * (HD * 2) + ((ch ^ (r & 7)) << 4); }

// MT = m-tiles of 16 query rows a CTA reduces: with 17-32 rows per (chain, kv head) the two tiles sit in ONE CTA of 8 warps,
// warps w and w + 4 work on the same pages -- each fetches half of a page, a 64-thread named barrier joins the pair -- so
// the KV pages cross HBM and L2 once per chain, not once per tile (two tiles in two CTAs: 325 us against 213 us for 16 rows
// at 8 x 32K context, 1.4x the DRAM bytes).
template <int HD, int NS, int MT>
__global__ void __launch_bounds__(128 * MT) attn_verify_kernel(const AttnParams P) {
    PDL_ENTRY();
    constexpr int KS = HD / 16, ND = HD / 8, CH = HD / 8;       // k-steps of QK^T, d n-tiles of PV, 16-byte chunks per row
    constexpr int KL = 4;                                        // the four warps take the segment's pages round-robin
    constexpr int PAGE_BYTES = ATT_PAGE * HD * 2;
    extern __shared__ __align__(128) unsigned char smem[];
    // layout: Q tile [16 * MT][HD] | per page lane: NS stages x (K page, V page) ; merge area aliases the stages
    unsigned char *q_s = smem;
    unsigned char *stage = smem + 16 * MT * HD * 2;
    __shared__ int qpos_s[16 * MT];
    __shared__ float ml_s[4 * MT][16][2];

    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, g = lane >> 2, c = lane & 3;
    const uint32_t seg = blockIdx.x, kvh = blockIdx.y, span = blockIdx.z / P.n_mtiles, mt = (blockIdx.z % P.n_mtiles) * MT;   // first m-tile of this CTA
    const uint32_t group = P.q_heads / P.kv_heads;
    const uint32_t t0 = P.row_start ? P.row_start[span] : span;
    const uint32_t cnt = P.row_count ? P.row_count[span] : 1u;
    if (cnt == 0) return;
    const uint32_t R = cnt * group;
    if (mt * 16 >= R) return;
    const uint32_t seq = P.seq_ids[t0];
    const uint32_t he = P.kv_heads * HD;
    uint32_t L = 0;  // keys any row of the chain may see
    for (uint32_t p = 0; p < cnt; p++) L = max(L, P.positions[t0 + p] + 1);
    const uint32_t pages = min((L + ATT_PAGE - 1) / ATT_PAGE, P.bpr);   // never past the block-table row
    const uint32_t pg0 = seg * P.seg_pages, pg1 = min(pages, pg0 + P.seg_pages);
    if (pg0 >= pages) return;  // the combine kernel only reads the segments below ceil(pages / seg_pages)

    // stage Q (rows p*group + gq; padding rows zero, their position -1 masks every key)
    for (uint32_t i = threadIdx.x; i < 16 * MT * CH; i += 128 * MT) {
        uint32_t r = i / CH, ch = i % CH;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (mt * 16 + r < R) {
            uint32_t p = (mt * 16 + r) / group, gq = (mt * 16 + r) % group;
            v = *reinterpret_cast<const uint4 *>(P.q + ((size_t)(t0 + p) * P.q_heads + kvh * group + gq) * HD + ch * 8);
        }
        *reinterpret_cast<uint4 *>(q_s + tile_off<HD>(r, ch)) = v;
    }
    if (threadIdx.x < 16 * MT) qpos_s[threadIdx.x] = mt * 16 + threadIdx.x < R ? (int)P.positions[t0 + (mt * 16 + threadIdx.x) / group] : -1;
    __syncthreads();

    const int mi = w >> 2, kl = w & 3;   // m-tile of this warp within the CTA, page lane
    unsigned char *my_stage = stage + (size_t)kl * NS * 2 * PAGE_BYTES;
    // the MT warps of a page lane meet at hardware barrier 1 + kl (barrier 0 is the CTA's)
    auto lane_sync = [&]() {
        if (MT == 1) __syncwarp();
        else asm volatile("bar.sync %0, %1;" ::"r"(1 + kl), "r"(32 * MT) : "memory");
    };
    const uint32_t q_base = smem_u32(q_s), st_base = smem_u32(my_stage);
    const uint32_t *bt = P.block_table + (size_t)seq * P.bpr;

    auto load_page = [&](uint32_t pg, int buf) {
        uint32_t slot0 = bt[pg] * ATT_PAGE;
        uint32_t kdst = st_base + buf * 2 * PAGE_BYTES, vdst = kdst + PAGE_BYTES;
#pragma unroll 4
        for (uint32_t i = lane + 32 * mi; i < ATT_PAGE * CH; i += 32 * MT) {
            uint32_t key = i / CH, ch = i % CH;
            size_t src = (size_t)(slot0 + key) * he + kvh * HD + ch * 8;
            uint32_t nbytes = (pg * ATT_PAGE + key) < L ? 16u : 0u;  // zero-fill rows past the sequence end
            cp_async16(kdst + tile_off<HD>(key, ch), P.k_cache + src, nbytes);
            cp_async16(vdst + tile_off<HD>(key, ch), P.v_cache + src, nbytes);
        }
    };

    float o[ND][4];
#pragma unroll
    for (int i = 0; i < ND; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    const int pos_lo = qpos_s[mi * 16 + g], pos_hi = qpos_s[mi * 16 + g + 8];
    const bool live = (mt + mi) * 16 < R;   // a short chain leaves the second tile's warps with copies only

    uint32_t pg = pg0 + kl;
    int buf = 0;
#pragma unroll
    for (int s0 = 0; s0 < NS - 1; s0++) {
        if (pg + s0 * KL < pg1) load_page(pg + s0 * KL, s0);
        cp_async_commit();
    }
    for (; pg < pg1; pg += KL) {
        if (pg + (NS - 1) * KL < pg1) load_page(pg + (NS - 1) * KL, (buf + NS - 1) % NS);
        cp_async_commit();
        cp_async_wait<NS - 1>();
        lane_sync();
        const uint32_t k_s = st_base + buf * 2 * PAGE_BYTES, v_s = k_s + PAGE_BYTES;
        if (live) {
        // S = Q K^T for 16 keys
        float s[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
#pragma unroll
        for (int ks = 0; ks < KS; ks++) {
            uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
            ldsm_x4(q_base + tile_off<HD>(mi * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4)), a0, a1, a2, a3);
            ldsm_x4(k_s + tile_off<HD>((lane >> 4) * 8 + (lane & 7), ks * 2 + ((lane >> 3) & 1)), b0, b1, b2, b3);
            mma16816(s[0], a0, a1, a2, a3, b0, b1);
            mma16816(s[1], a0, a1, a2, a3, b2, b3);
        }
        // causal mask + online softmax (rows g and g+8 of the m-tile)
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < 2; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                int j = (int)(pg * ATT_PAGE) + nt * 8 + 2 * c + (e & 1);
                bool ok = j <= ((e >> 1) ? pos_hi : pos_lo);
                s[nt][e] = ok ? s[nt][e] : -INFINITY;
                mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
            }
        float alpha[2], moff[2];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            float m_new = fmaxf(m_run[h], mx[h]);
            moff[h] = m_new == -INFINITY ? 0.0f : m_new * P.scale_log2;
            alpha[h] = m_run[h] == -INFINITY ? 0.0f : exp2f(m_run[h] * P.scale_log2 - moff[h]);
            m_run[h] = m_new;
            l_run[h] *= alpha[h];
        }
        uint32_t pa[4];
        {
            float p[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; nt++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    p[nt][e] = exp2f(s[nt][e] * P.scale_log2 - moff[e >> 1]);
                    l_run[e >> 1] += p[nt][e];
                }
            pa[0] = pack_bf16(p[0][0], p[0][1]); pa[1] = pack_bf16(p[0][2], p[0][3]);
            pa[2] = pack_bf16(p[1][0], p[1][1]); pa[3] = pack_bf16(p[1][2], p[1][3]);
        }
#pragma unroll
        for (int i = 0; i < ND; i++) { o[i][0] *= alpha[0]; o[i][1] *= alpha[0]; o[i][2] *= alpha[1]; o[i][3] *= alpha[1]; }
        // O += P V
#pragma unroll
        for (int nd = 0; nd < ND / 2; nd++) {
            uint32_t b0, b1, b2, b3;
            ldsm_x4_t(v_s + tile_off<HD>(((lane >> 3) & 1) * 8 + (lane & 7), nd * 2 + (lane >> 4)), b0, b1, b2, b3);
            mma16816(o[2 * nd], pa[0], pa[1], pa[2], pa[3], b0, b1);
            mma16816(o[2 * nd + 1], pa[0], pa[1], pa[2], pa[3], b2, b3);
        }
        }   // live
        lane_sync();   // the stage may be refilled
        buf = (buf + 1) % NS;
    }
    cp_async_wait<0>();
#pragma unroll
    for (int h = 0; h < 2; h++) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
    __syncthreads();  // every warp is done with its stages: the merge area may alias them
    float *om = reinterpret_cast<float *>(stage);  // [4 * MT warps][16 rows][HD + 4]
    constexpr int OST = HD + 4;
#pragma unroll
    for (int i = 0; i < ND; i++) {
        float *r0 = om + ((size_t)w * 16 + g) * OST + i * 8 + 2 * c, *r1 = r0 + 8 * OST;
        r0[0] = o[i][0]; r0[1] = o[i][1]; r1[0] = o[i][2]; r1[1] = o[i][3];
    }
    if (c == 0) {
        ml_s[w][g][0] = m_run[0]; ml_s[w][g][1] = l_run[0];
        ml_s[w][g + 8][0] = m_run[1]; ml_s[w][g + 8][1] = l_run[1];
    }
    __syncthreads();
    // merge the four warps of an m-tile in warp order and emit the segment's partial
    for (uint32_t i = threadIdx.x; i < 16 * MT * (HD / 4); i += 128 * MT) {
        uint32_t r32 = i / (HD / 4), d4 = (i % (HD / 4)) * 4;
        uint32_t row = mt * 16 + r32;
        if (row >= R) continue;
        const uint32_t rr = r32 % 16, w0 = (r32 / 16) * KL;   // row within its m-tile, first warp of that tile
        float M = -INFINITY;
#pragma unroll
        for (int wi = 0; wi < KL; wi++) M = fmaxf(M, ml_s[w0 + wi][rr][0]);
        float acc[4] = {0, 0, 0, 0}, Lsum = 0.0f;
#pragma unroll
        for (int wi = 0; wi < KL; wi++) {
            const uint32_t ww = w0 + wi;
            float mw = ml_s[ww][rr][0];
            float f = mw == -INFINITY ? 0.0f : exp2f((mw - M) * P.scale_log2);
            Lsum += f * ml_s[ww][rr][1];
            const float4 v = *reinterpret_cast<const float4 *>(om + ((size_t)ww * 16 + rr) * OST + d4);
            acc[0] += f * v.x; acc[1] += f * v.y; acc[2] += f * v.z; acc[3] += f * v.w;
        }
        size_t pi = (((size_t)span * P.kv_heads + kvh) * P.max_segs + seg) * 32 + row;
        *reinterpret_cast<float4 *>(P.part_o + pi * HD + d4) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        if (d4 == 0) { P.part_ml[pi * 2] = M; P.part_ml[pi * 2 + 1] = Lsum; }
    }
}

// Merge of the segments in index order: one block per (span, kv head, query row), one thread per 4 output dims.
template <int HD>
__global__ void attn_combine_kernel(const AttnParams P) {
    PDL_ENTRY();
    const uint32_t row = blockIdx.x, kvh = blockIdx.y, span = blockIdx.z;
    const uint32_t group = P.q_heads / P.kv_heads;
    const uint32_t t0 = P.row_start ? P.row_start[span] : span;
    const uint32_t cnt = P.row_count ? P.row_count[span] : 1u;
    if (row >= cnt * group) return;
    const uint32_t d4 = threadIdx.x * 4;
    uint32_t L = 0;
    for (uint32_t p = 0; p < cnt; p++) L = max(L, P.positions[t0 + p] + 1);
    uint32_t nseg = (min((L + ATT_PAGE - 1) / ATT_PAGE, P.bpr) + P.seg_pages - 1) / P.seg_pages;
    if (nseg > P.max_segs) {
        // the grid was sized from a context bound below this row's position: segments past it were never computed.  Merge
        // what exists (never read a slot nobody wrote) and tell the host.
        nseg = P.max_segs;
        if (P.status && threadIdx.x == 0 && row == 0 && kvh == 0) atomicOr(&P.status[P.seq_ids[t0]], WB_STATUS_CTX_BOUND);
    }
    size_t p0 = ((size_t)span * P.kv_heads + kvh) * P.max_segs * 32 + row;
    float M = -INFINITY;
    for (uint32_t s = 0; s < nseg; s++) M = fmaxf(M, P.part_ml[(p0 + (size_t)s * 32) * 2]);
    float acc[4] = {0, 0, 0, 0}, Lsum = 0.0f;
    for (uint32_t s = 0; s < nseg; s++) {
        size_t pi = p0 + (size_t)s * 32;
        float ms = P.part_ml[pi * 2];
        float f = ms == -INFINITY ? 0.0f : exp2f((ms - M) * P.scale_log2);
        Lsum += f * P.part_ml[pi * 2 + 1];
        const float4 v = *reinterpret_cast<const float4 *>(P.part_o + pi * HD + d4);
        acc[0] += f * v.x; acc[1] += f * v.y; acc[2] += f * v.z; acc[3] += f * v.w;
    }
    uint32_t p = row / group, gq = row % group;
    size_t oi = ((size_t)(t0 + p) * P.q_heads + kvh * group + gq) * HD + d4;
    float inv = 1.0f / Lsum;
    bf16_t r[4];
#pragma unroll
    for (int e = 0; e < 4; e++) {
        r[e] = f2bf(acc[e] * inv);
        if (P.gate) r[e] = f2bf(bf2f(r[e]) * rbf(sigmoid_ref(bf2f(P.gate[oi + e]))));
    }
    *reinterpret_cast<uint2 *>(P.out + oi) = make_uint2((uint32_t)r[0] | ((uint32_t)r[1] << 16), (uint32_t)r[2] | ((uint32_t)r[3] << 16));
}

template <int HD, int NS, int MT>
static size_t attn_smem_bytes() {
    size_t smem = 16 * MT * HD * 2 + 4 * NS * 2 * (size_t)ATT_PAGE * HD * 2;
    size_t merge = 16 * MT * HD * 2 + 4 * MT * 16 * (size_t)(HD + 4) * 4;
    return smem < merge ? merge : smem;
}
// The shared-memory opt-in is a per-device function attribute: one flag per device ordinal, set once (writing it twice from
// two threads stores the same value).
static bool g_attn_ready[12][64];
template <int HD, int NS, int MT>
static int32_t attn_prepare(int which) {
    which += 6 * (MT - 1);
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { wb_set_error("attn: cudaGetDevice failed or device ordinal >= 64"); return WB_ERR_CUDA; }
    if (g_attn_ready[which][dev]) return WB_OK;
    const size_t smem = attn_smem_bytes<HD, NS, MT>();
    cudaError_t e = cudaFuncSetAttribute(attn_verify_kernel<HD, NS, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { wb_set_error("attn: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e)); return WB_ERR_CUDA; }
    g_attn_ready[which][dev] = true;
    return WB_OK;
}

// tiles = m-tiles of 16 query rows of the longest chain (1 or 2): both sit in one CTA
template <int HD, int NS>
static int32_t attn_launch(const AttnParams &p, uint32_t tiles, int which, cudaStream_t st) {
    dim3 grid(p.max_segs, p.kv_heads, p.n_spans * p.n_mtiles);
    if (tiles == 1) {
        if (int32_t rc = attn_prepare<HD, NS, 1>(which)) return rc;
        WB_LAUNCH((attn_verify_kernel<HD, NS, 1>), grid, 128, (attn_smem_bytes<HD, NS, 1>()), st, p);
    } else {
        if (int32_t rc = attn_prepare<HD, NS, 2>(which)) return rc;
        WB_LAUNCH((attn_verify_kernel<HD, NS, 2>), grid, 256, (attn_smem_bytes<HD, NS, 2>()), st, p);
    }
    WB_LAUNCH_CHECK();
    dim3 g2(16 * tiles, p.kv_heads, p.n_spans);
    WB_LAUNCH((attn_combine_kernel<HD>), g2, HD / 4, 0, st, p);
    WB_LAUNCH_CHECK();
    return WB_OK;
}

template <int HD>
static int32_t attn_prepare_all(int which) {
    int32_t rc = attn_prepare<HD, 2, 1>(which);
    if (!rc) rc = attn_prepare<HD, 3, 1>(which + 3);
    if (!rc) rc = attn_prepare<HD, 2, 2>(which);
    if (!rc) rc = attn_prepare<HD, 3, 2>(which + 3);
    return rc;
}

int32_t wb_attn_init(uint32_t head_dim) {
    switch (head_dim) {
        case 256: return attn_prepare_all<256>(0);
        case 128: return attn_prepare_all<128>(1);
        case 64: return attn_prepare_all<64>(2);
        default: wb_set_error("attn: head_dim %u not built", head_dim); return WB_ERR_SHAPE;
    }
}

extern "C" uint64_t wein_b200_attn_scratch_bytes(uint32_t n_spans, uint32_t kv_heads, uint32_t head_dim, uint32_t max_segs) {
    return (uint64_t)n_spans * kv_heads * max_segs * 32 * (head_dim + 2) * 4;
}

// max_count: the longest chain of the call (host knowledge; chains are at most 32 / group rows).
// max_ctx: an upper bound of (position + 1) over the call's rows; it sizes the grid, never the arithmetic.
// seg_pages: pages per segment (>= 1); callers that compare runs bit for bit keep it fixed.
int32_t wb_attn_verify(const void *q, const void *k_cache, const void *v_cache, const void *block_table, const void *seq_ids,
                       const void *positions, const void *row_start, const void *row_count, const void *gate, void *out,
                       float q_scale, uint32_t bpr, uint32_t block_size, uint32_t q_heads, uint32_t kv_heads, uint32_t head_dim,
                       uint32_t n_spans, uint32_t max_count, uint32_t max_ctx, uint32_t seg_pages, void *scratch,
                       uint64_t scratch_bytes, uint32_t *status, bool deep, cudaStream_t st) {
    WB_CHECK_ARG(q && k_cache && v_cache && block_table && seq_ids && positions && out && scratch, "attn_verify: null pointer");
    if (block_size != ATT_PAGE) { wb_set_error("attn_verify: built for 16-token pages, got %u", block_size); return WB_ERR_SHAPE; }
    WB_CHECK_ARG(kv_heads > 0 && q_heads % kv_heads == 0, "attn_verify: q_heads %u not a multiple of kv_heads %u", q_heads, kv_heads);
    uint32_t group = q_heads / kv_heads;
    WB_CHECK_ARG(max_count >= 1 && max_count * group <= 32, "attn_verify: chain of %u rows x group %u exceeds 32 query rows", max_count, group);
    WB_CHECK_ARG(seg_pages >= 1 && max_ctx >= 1 && max_ctx <= bpr * ATT_PAGE, "attn_verify: max_ctx %u outside 1..bpr*16 or seg_pages = 0", max_ctx);
    if (n_spans == 0) return WB_OK;
    AttnParams p{};
    p.seg_pages = seg_pages;
    p.max_segs = ((max_ctx + ATT_PAGE - 1) / ATT_PAGE + seg_pages - 1) / seg_pages;
    const uint32_t tiles = (max_count * group + 15) / 16;   // 1 or 2, both reduced by one CTA
    p.n_mtiles = 1;
    uint64_t need = wein_b200_attn_scratch_bytes(n_spans, kv_heads, head_dim, p.max_segs);
    if (need > scratch_bytes) { wb_set_error("attn_verify: scratch of %llu bytes needed, %llu given", (unsigned long long)need, (unsigned long long)scratch_bytes); return WB_ERR_CAPACITY; }
    p.q = (const bf16_t *)q; p.k_cache = (const bf16_t *)k_cache; p.v_cache = (const bf16_t *)v_cache; p.gate = (const bf16_t *)gate;
    p.block_table = (const uint32_t *)block_table; p.seq_ids = (const uint32_t *)seq_ids; p.positions = (const uint32_t *)positions;
    p.row_start = (const uint32_t *)row_start; p.row_count = (const uint32_t *)row_count; p.out = (bf16_t *)out;
    p.part_o = (float *)scratch;
    p.part_ml = (float *)scratch + (size_t)n_spans * kv_heads * p.max_segs * 32 * head_dim;
    p.scale_log2 = q_scale * 1.4426950408889634f;
    p.bpr = bpr; p.q_heads = q_heads; p.kv_heads = kv_heads; p.n_spans = n_spans; p.status = status;
    switch (head_dim) {
        case 256: return deep ? attn_launch<256, 3>(p, tiles, 3, st) : attn_launch<256, 2>(p, tiles, 0, st);
        case 128: return deep ? attn_launch<128, 3>(p, tiles, 4, st) : attn_launch<128, 2>(p, tiles, 1, st);
        case 64: return deep ? attn_launch<64, 3>(p, tiles, 5, st) : attn_launch<64, 2>(p, tiles, 2, st);
        default: wb_set_error("attn_verify: head_dim %u not built (64, 128, 256)", head_dim); return WB_ERR_SHAPE;
    }
}

extern "C" {

// Argument order of PagedAttnOp::run plus the scratch the reference's op object owns privately; every row is
// treated as its own chain of length 1 and the context bound is the block table's capacity.
int32_t wein_b200_paged_attn(const void *q, const void *k_cache, const void *v_cache, const void *block_table, const void *seq_ids,
                             const void *positions, void *out, float q_scale, uint32_t bpr, uint32_t block_size, uint32_t q_heads,
                             uint32_t kv_heads, uint32_t head_dim, uint32_t tokens, void *scratch, uint64_t scratch_bytes, void *stream) {
    uint32_t seg = (bpr + 15) / 16;  // at most 16 segments per row
    return wb_attn_verify(q, k_cache, v_cache, block_table, seq_ids, positions, nullptr, nullptr, nullptr, out, q_scale, bpr, block_size,
                          q_heads, kv_heads, head_dim, tokens, 1, bpr * ATT_PAGE, seg, scratch, scratch_bytes, nullptr, false, (cudaStream_t)stream);
}

int32_t wein_b200_attn_verify(const void *q, const void *k_cache, const void *v_cache, const void *block_table, const void *seq_ids,
                              const void *positions, const void *row_start, const void *row_count, const void *gate, void *out,
                              float q_scale, uint32_t bpr, uint32_t block_size, uint32_t q_heads, uint32_t kv_heads, uint32_t head_dim,
                              uint32_t n_spans, uint32_t max_count, uint32_t max_ctx, uint32_t seg_pages, void *scratch,
                              uint64_t scratch_bytes, void *status, void *stream) {
    WB_CHECK_ARG(row_start && row_count, "attn_verify: span tables are required");
    return wb_attn_verify(q, k_cache, v_cache, block_table, seq_ids, positions, row_start, row_count, gate, out, q_scale, bpr, block_size,
                          q_heads, kv_heads, head_dim, n_spans, max_count, max_ctx, seg_pages, scratch, scratch_bytes, (uint32_t *)status, false, (cudaStream_t)stream);
}

}  // extern "C"

