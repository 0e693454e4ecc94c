// Device-side acceptance for MTP speculative decoding.
//
// Greedy: the reference accepts on the host after a device argmax, a stream sync and a readback
// (crates/wein-exec/src/qwen.rs:3676-3702 and :2433-2460): accept while drafts[a] == target[a], then emit the
// bonus token target[a].  Here the same rule runs on the device, so the step needs no host round trip.
// Token ids and accept lengths are bit-identical to the reference rule given identical logits (the argmax
// keeps the reference's total order: value descending, index ascending).
//
// Sampled: the reference has no speculative sampling (its chains are forced greedy, qwen.rs:2610-2615).  The
// kernels below follow the filter of the reference's plain sampler (reference.rs:787-877: scale by 1/temp,
// top-k <= 64 in the total order, softmax numerators by the reference exp, top-p cut on the running sum) to
// turn a logits row into a compact distribution of at most 64 (id, probability) pairs, and then apply
// standard rejection sampling (accept draft x iff u*q(x) < p(x); on the first rejection redraw from
// max(p-q, 0) renormalised; after k acceptances draw the bonus token from the last row) with Philox4x32-10
// uniforms keyed by (seed, round, position), so a replayed CUDA graph needs no RNG state on the host.
// Every floating-point step is written in the oracle's order: results are bit-identical to oracle/.
// Compiled with -fmad=false.
#include "common.cuh"
#include "internal.h"

#define DIST_CAP 64

// ---------------------------------------------------------------- Philox4x32-10
__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1, uint32_t out[4]) {
#pragma unroll
    for (int r = 0; r < 10; r++) {
        uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
        uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
        uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
        c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}
// uniforms of (sequence seed, round, chain position, stream): lane 0 picks from a distribution, lane 1 is the accept test
__device__ __forceinline__ void spec_uniforms(uint64_t seed, uint64_t round, uint32_t position, uint32_t stream, float u[4]) {
    uint32_t o[4];
    philox4x32_10((uint32_t)round, (uint32_t)(round >> 32), position, stream, (uint32_t)seed, (uint32_t)(seed >> 32), o);
#pragma unroll
    for (int i = 0; i < 4; i++) u[i] = __fmul_rn((float)(o[i] >> 8), 1.0f / 16777216.0f);
}
__device__ __forceinline__ int pick_from(const float *probs, int n, float u) {
    float acc = 0.0f;
    for (int j = 0; j < n; j++) { acc = __fadd_rn(probs[j], acc); if (u < acc) return j; }
    return n - 1;
}

// ---------------------------------------------------------------- top-k / top-p filter
// 16-bit key whose unsigned order is the bf16 value order; -0 folds onto +0 (they compare equal in the reference)
__device__ __forceinline__ uint32_t ord_key(uint32_t h) {
    h &= 0xffffu;
    if (h == 0x8000u) h = 0;
    return (h & 0x8000u) ? (~h & 0xffffu) : (h | 0x8000u);
}
__device__ __forceinline__ bf16_t key_to_bf16(uint32_t key) { return (bf16_t)((key & 0x8000u) ? (key & 0x7fffu) : (~key & 0xffffu)); }

struct FilterParams {
    const bf16_t *x;           // [*, n] logits
    const uint32_t *rows;      // [s] logits row of each output row (null: identity)
    const uint32_t *row_seq;   // [s] sequence (parameter slot) of each row (null: row / rows_per_seq)
    uint32_t rows_per_seq;
    const float *temp, *top_p; // per sequence
    const uint32_t *top_k;
    uint32_t n, s;
    uint32_t *out_ids;         // [s, 64]
    float *out_probs;          // [s, 64]
    uint32_t *out_n;           // [s]
    uint32_t out_mul, out_off; // row r writes distribution slot r*out_mul + out_off
    // optional: draw a token from each row's distribution (draft sampling); row r writes sample_out[r*sample_mul + sample_off]
    uint32_t *sample_out;      // or null
    uint32_t sample_mul, sample_off;
    const uint64_t *seed, *round;  // per sequence
    uint32_t position;
    // optional: the reference's plain sampler (SampleRowsOp, reference.rs:787-877): PCG-XSH-RR state per slot in `pcg_rng`
    // (0 = not yet seeded: derived from pcg_seed[row]), one uniform per row, pick over e_j/denom (not renormalised)
    uint64_t *pcg_rng;
    const uint32_t *pcg_slots;
    const uint64_t *pcg_seed;
    uint32_t *pcg_out;         // [s]; the compact-distribution outputs may then be null
};

// Applies fn(key, index) to every element of the row, 8 elements per 16-byte load when aligned; a thread issues four loads
// before it consumes them (a row is read by one CTA: what bounds a pass is load latency, not bandwidth).
template <typename F>
__device__ __forceinline__ void scan_row(const bf16_t *row, uint32_t n, F fn) {
    if ((((uintptr_t)row) & 15u) == 0) {
        const uint32_t nv = n / 8, step = blockDim.x;
        auto eat = [&](const uint4 &q, uint32_t v) {
            const uint32_t wv[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int j = 0; j < 4; j++) { fn(ord_key(wv[j]), v * 8 + 2 * j); fn(ord_key(wv[j] >> 16), v * 8 + 2 * j + 1); }
        };
        uint32_t v = threadIdx.x;
        for (; v + 3 * step < nv; v += 4 * step) {
            const uint4 q0 = *reinterpret_cast<const uint4 *>(row + (size_t)v * 8);
            const uint4 q1 = *reinterpret_cast<const uint4 *>(row + (size_t)(v + step) * 8);
            const uint4 q2 = *reinterpret_cast<const uint4 *>(row + (size_t)(v + 2 * step) * 8);
            const uint4 q3 = *reinterpret_cast<const uint4 *>(row + (size_t)(v + 3 * step) * 8);
            eat(q0, v); eat(q1, v + step); eat(q2, v + 2 * step); eat(q3, v + 3 * step);
        }
        for (; v < nv; v += step) eat(*reinterpret_cast<const uint4 *>(row + (size_t)v * 8), v);
        for (uint32_t i = nv * 8 + threadIdx.x; i < n; i += blockDim.x) fn(ord_key(row[i]), i);
    } else {
        for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) fn(ord_key(row[i]), i);
    }
}

// One CTA of 1024 threads per row.
__global__ void __launch_bounds__(1024) topk_filter_kernel(const FilterParams P) {
    PDL_ENTRY();
    __shared__ __align__(16) uint32_t lm[1024];
    __shared__ uint32_t hist[256];
    __shared__ uint32_t warp_cnt[32];
    __shared__ uint32_t sv_idx[1024]; // survivors of the bound (their keys reuse lm)
    __shared__ uint32_t sh[9];        // 8: number of survivors; 0: bound key, 1: bin hi, 2: k left inside bin, 3: tau, 4: need, 5: count_eq, 6: list length, 7: ties emitted
    __shared__ uint32_t cand_key[DIST_CAP], cand_idx[DIST_CAP];
    __shared__ uint32_t srt_idx[DIST_CAP];
    __shared__ float srt_v[DIST_CAP], e_s[DIST_CAP], pn[DIST_CAP], shf[2];
    const uint32_t r = blockIdx.x, tid = threadIdx.x;
    const uint32_t seq = P.row_seq ? P.row_seq[r] : r / P.rows_per_seq;
    const bf16_t *row = P.x + (size_t)(P.rows ? P.rows[r] : r) * P.n;
    const float temp = P.temp[seq];
    const bool greedy = !(temp > 0.0f);
    uint32_t k = greedy ? 1u : min(P.top_k[seq], (uint32_t)DIST_CAP);
    const size_t oslot = (size_t)r * P.out_mul + P.out_off, sslot = (size_t)r * P.sample_mul + P.sample_off;
    uint32_t *ids = P.out_ids ? P.out_ids + oslot * DIST_CAP : nullptr;
    float *probs = P.out_probs ? P.out_probs + oslot * DIST_CAP : nullptr;
    if (k == 0 || P.n == 0) {  // top_k = 0 (whole vocabulary) is not supported on the device: in-band error, as the reference
        if (tid < DIST_CAP && ids) { ids[tid] = 0xffffffffu; probs[tid] = 0.0f; }
        if (tid == 0) {
            if (P.out_n) P.out_n[oslot] = 0;
            if (P.sample_out) P.sample_out[sslot] = 0xffffffffu;
            if (P.pcg_out) P.pcg_out[r] = 0xffffffffu;
        }
        return;
    }
    if (k > P.n) k = P.n;
    // pass 1: a lower bound of the k-th largest key = the k-th largest of the per-thread maxima
    uint32_t best = 0;
    scan_row(row, P.n, [&](uint32_t key, uint32_t) { best = max(best, key); });
    if (tid < 256) hist[tid] = 0;
    if (tid < 9) sh[tid] = 0;
    __syncthreads();
    // the k-th largest of the 1024 per-thread maxima by a two-level radix select (high byte, then low byte, of the 16-bit key)
    atomicAdd(&hist[best >> 8], 1u);
    __syncthreads();
    if (tid == 0) {
        uint32_t above = 0;
        int b = 255;
        for (; b > 0; b--) { if (above + hist[b] >= k) break; above += hist[b]; }
        sh[1] = (uint32_t)b; sh[2] = k - above;
    }
    __syncthreads();
    {
        const uint32_t mhi = sh[1];
        if (tid < 256) hist[tid] = 0;
        __syncthreads();
        if ((best >> 8) == mhi) atomicAdd(&hist[best & 255u], 1u);
        __syncthreads();
        if (tid == 0) {
            const uint32_t kin0 = sh[2];
            uint32_t above = 0;
            int b = 255;
            for (; b > 0; b--) { if (above + hist[b] >= kin0) break; above += hist[b]; }
            sh[0] = (mhi << 8) | (uint32_t)b;
        }
        __syncthreads();
    }
    const uint32_t bound = sh[0];
    const float inv_t = greedy ? 1.0f : __fdiv_rn(1.0f, temp);
    // pass 2: the survivors of the bound.  At most k threads hold a maximum >= bound, so barring heavy ties there are
    // barely more than k of them: list them (key, index) and rank the list by (value descending, index ascending) --
    // ranks 0..k-1 are the answer, ties at the threshold resolved towards the lowest index, already in output order.
    scan_row(row, P.n, [&](uint32_t key, uint32_t i) {
        if (key >= bound) { uint32_t slot = atomicAdd(&sh[8], 1u); if (slot < 1024u) { lm[slot] = key; sv_idx[slot] = i; } }
    });
    __syncthreads();
    const uint32_t n_surv = sh[8];
    if (n_surv <= 1024u) {
        if (tid < n_surv) {
            const uint32_t mk = lm[tid], mi = sv_idx[tid];
            uint32_t rank = 0;
            for (uint32_t u = 0; u < n_surv; u++) { const uint32_t ok = lm[u]; rank += (ok > mk) || (ok == mk && sv_idx[u] < mi); }
            if (rank < k) { srt_idx[rank] = mi; srt_v[rank] = __fmul_rn(bf2f(key_to_bf16(mk)), inv_t); }
        }
    } else {
    // more than 1024 elements at or above the bound (massive ties): exact selection by two histogram passes
    // pass 2b: histogram of the high byte over the survivors; find the byte holding the k-th largest
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    scan_row(row, P.n, [&](uint32_t key, uint32_t) { if (key >= bound) atomicAdd(&hist[key >> 8], 1u); });
    __syncthreads();
    if (tid == 0) {
        uint32_t above = 0;
        int b = 255;
        for (; b > 0; b--) { if (above + hist[b] >= k) break; above += hist[b]; }
        sh[1] = (uint32_t)b; sh[2] = k - above;
    }
    __syncthreads();
    const uint32_t bhi = sh[1], kin = sh[2];
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    // pass 3: low byte inside that bin -> the exact threshold key tau
    scan_row(row, P.n, [&](uint32_t key, uint32_t) { if ((key >> 8) == bhi && key >= bound) atomicAdd(&hist[key & 255u], 1u); });
    __syncthreads();
    if (tid == 0) {
        uint32_t above = 0;
        int b = 255;
        for (; b > 0; b--) { if (above + hist[b] >= kin) break; above += hist[b]; }
        sh[3] = (bhi << 8) | (uint32_t)b;
        sh[4] = kin - above;   // ties at tau still to take (lowest indices first)
        sh[5] = hist[b];       // ties at tau in the row
    }
    __syncthreads();
    const uint32_t tau = sh[3], need = sh[4], count_eq = sh[5];
    const bool all_ties = count_eq == need;
    // pass 4: everything above tau, plus the ties when all of them are wanted
    scan_row(row, P.n, [&](uint32_t key, uint32_t i) {
        if (key > tau || (all_ties && key == tau)) { uint32_t slot = atomicAdd(&sh[6], 1u); if (slot < DIST_CAP) { cand_key[slot] = key; cand_idx[slot] = i; } }
    });
    __syncthreads();
    if (!all_ties) {
        // ordered scan for the `need` lowest-index ties, 1024 consecutive indices per round
        const uint32_t lane = tid & 31, wid = tid >> 5;
        for (uint32_t base = 0; base < P.n; base += 1024) {
            uint32_t i = base + tid;
            bool hit = i < P.n && ord_key(row[i]) == tau;
            uint32_t bal = __ballot_sync(0xffffffffu, hit);
            if (lane == 0) warp_cnt[wid] = __popc(bal);
            __syncthreads();
            uint32_t before = sh[7];
            for (uint32_t w2 = 0; w2 < wid; w2++) before += warp_cnt[w2];
            uint32_t my = before + __popc(bal & ((1u << lane) - 1u));
            if (hit && my < need) { uint32_t slot = (k - need) + my; cand_key[slot] = tau; cand_idx[slot] = i; }
            __syncthreads();
            if (tid == 0) { uint32_t tot = 0; for (int w2 = 0; w2 < 32; w2++) tot += warp_cnt[w2]; sh[7] += tot; }
            __syncthreads();
            if (sh[7] >= need) break;
        }
    }
    __syncthreads();
    // sort the k candidates: value descending, index ascending
    if (tid < k) {
        uint32_t mk = cand_key[tid], mi = cand_idx[tid], rank = 0;
        for (uint32_t u = 0; u < k; u++) rank += (cand_key[u] > mk) || (cand_key[u] == mk && cand_idx[u] < mi);
        srt_idx[rank] = mi;
        srt_v[rank] = __fmul_rn(bf2f(key_to_bf16(mk)), inv_t);
    }
    }   // end of the massive-ties path
    __syncthreads();
    if (tid < k) e_s[tid] = expf_ref(__fsub_rn(srt_v[tid], srt_v[0]));
    __syncthreads();
    // top-p (reference.rs:845-856): the ordered sums stay with thread 0, the divisions run one per thread
    if (tid == 0) {
        float denom = 0.0f;
        for (uint32_t j = 0; j < k; j++) denom = __fadd_rn(e_s[j], denom);
        shf[0] = denom;
    }
    __syncthreads();
    if (tid < k) pn[tid] = __fdiv_rn(e_s[tid], shf[0]);
    __syncthreads();
    if (tid == 0) {
        uint32_t keep = 1;
        if (!greedy) {
            float pp = P.top_p[seq];
            pp = (pp > 0.0f && pp < 1.0f) ? pp : 1.0f;
            float cacc = 0.0f;
            for (uint32_t j = 0; j < k; j++) {
                cacc = __fadd_rn(pn[j], cacc);
                keep = j + 1;
                if (cacc >= pp) break;
            }
            if (P.pcg_out) {   // reference.rs:857-874, PCG of reference.rs:756-775
                uint64_t st = P.pcg_rng[P.pcg_slots[r]];
                if (st == 0) {
                    uint64_t x = P.pcg_seed[r] + 0x9e3779b97f4a7c15ull;
                    x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
                    x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
                    st = (x ^ (x >> 31)) | 1ull;
                }
                const uint64_t old = st;
                st = old * 6364136223846793005ull + 1442695040888963407ull;
                const uint32_t xs = (uint32_t)(((old >> 18) ^ old) >> 27), rot = (uint32_t)(old >> 59);
                const uint32_t rnd = (xs >> rot) | (xs << ((32 - rot) & 31));
                P.pcg_rng[P.pcg_slots[r]] = st;
                const float u = __fmul_rn((float)(rnd >> 8), 1.0f / 16777216.0f);
                float acc = 0.0f;
                uint32_t pick = keep - 1;
                for (uint32_t j = 0; j < keep; j++) {
                    acc = __fadd_rn(pn[j], acc);
                    if (u < acc) { pick = j; break; }
                }
                P.pcg_out[r] = srt_idx[pick];
            }
        } else if (P.pcg_out) {
            P.pcg_out[r] = srt_idx[0];   // temp <= 0: argmax, the RNG is not advanced (reference.rs:798-801)
        }
        float z = 0.0f;
        for (uint32_t j = 0; j < keep; j++) z = __fadd_rn(e_s[j], z);
        shf[1] = z;
        sh[6] = keep;
    }
    __syncthreads();
    if (tid < sh[6]) e_s[tid] = __fdiv_rn(e_s[tid], shf[1]);
    __syncthreads();
    if (tid == 0) {
        const uint32_t keep = sh[6];
        if (P.out_n) P.out_n[oslot] = keep;
        if (P.sample_out) {
            uint32_t tok = srt_idx[0];
            if (!greedy) {
                float u[4];
                spec_uniforms(P.seed[seq], P.round[seq], P.position, 0, u);
                tok = srt_idx[pick_from(e_s, (int)keep, u[0])];
            }
            P.sample_out[sslot] = tok;
        }
    }
    __syncthreads();
    if (tid < DIST_CAP && ids) {
        bool live = tid < sh[6];
        ids[tid] = live ? srt_idx[tid] : 0xffffffffu;
        probs[tid] = live ? e_s[tid] : 0.0f;
    }
}

// ---------------------------------------------------------------- acceptance
struct AcceptParams {
    // greedy inputs: per verify row argmax partials [rows][split] (keys of the argmax kernel) -- or null
    const uint64_t *am_part;
    uint32_t am_split;
    // sampled inputs: compact distributions of the verify rows [B*(k+1)] and of the draft rows [B*k] (draft row = b*k + j)
    const uint32_t *p_ids, *q_ids, *p_n, *q_n;
    const float *p_probs, *q_probs;
    const float *temp;              // per sequence; null or <= 0: greedy rule
    const uint64_t *seed, *round;   // per sequence
    const uint32_t *slot_of;        // [B] index of batch row b into temp / seed / round (null: b)
    uint32_t draft_stride;          // elements between the draft rows of consecutive sequences (>= k)
    const uint32_t *drafts;         // [B, draft_stride]
    const uint32_t *n_drafts;       // [B] or null (= k)
    uint32_t B, k;
    uint32_t *accept_len;           // [B]
    uint32_t *out_tokens;           // [B, k+1] emitted tokens, 0xffffffff beyond accept_len + 1
    uint32_t *target;               // [B, k+1] greedy targets (optional)
};

__device__ __forceinline__ uint32_t argmax_from_parts(const uint64_t *part, uint32_t split, int lane) {
    uint64_t best = 0ull;
    for (uint32_t i = lane; i < split; i += 32) { uint64_t o = part[i]; best = o > best ? o : best; }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) { uint64_t o = __shfl_xor_sync(0xffffffffu, best, off); best = o > best ? o : best; }
    return best == 0ull ? 0xffffffffu : ~(uint32_t)best;
}

// One warp per sequence.
__global__ void __launch_bounds__(32) accept_kernel(const AcceptParams P) {
    PDL_ENTRY();
    __shared__ float r_s[DIST_CAP];
    const uint32_t b = blockIdx.x, lane = threadIdx.x;
    const uint32_t k = P.k, rows = k + 1;
    const uint32_t nd = P.n_drafts ? min(P.n_drafts[b], k) : k;
    uint32_t *out = P.out_tokens + (size_t)b * rows;
    const uint32_t ps = P.slot_of ? P.slot_of[b] : b;
    const bool greedy = !P.temp || !(P.temp[ps] > 0.0f);
    if (greedy) {
        // target token of each row: from the argmax partials, or entry 0 of the row's compact distribution
        uint32_t a = 0;
        bool open = true;
        uint32_t emitted = 0xffffffffu;
        for (uint32_t j = 0; j <= nd; j++) {
            uint32_t t = P.am_part ? argmax_from_parts(P.am_part + ((size_t)b * rows + j) * P.am_split, P.am_split, lane)
                                   : P.p_ids[((size_t)b * rows + j) * DIST_CAP];
            if (P.target && lane == 0) P.target[(size_t)b * rows + j] = t;
            if (open) {
                if (j < nd && P.drafts[(size_t)b * P.draft_stride + j] == t) { a = j + 1; if (lane == 0) out[j] = t; }
                else { open = false; emitted = t; if (lane == 0) out[j] = t; }
            }
        }
        (void)emitted;
        if (lane == 0) {
            for (uint32_t j = a + 1; j < rows; j++) out[j] = 0xffffffffu;
            P.accept_len[b] = a;
        }
        return;
    }
    const uint64_t seed = P.seed[ps], round = P.round[ps];
    uint32_t a = 0;
    for (; a < nd; a++) {
        const uint32_t *pi = P.p_ids + ((size_t)b * rows + a) * DIST_CAP, *qi = P.q_ids + ((size_t)b * P.draft_stride + a) * DIST_CAP;
        const float *pp = P.p_probs + ((size_t)b * rows + a) * DIST_CAP, *qp = P.q_probs + ((size_t)b * P.draft_stride + a) * DIST_CAP;
        const uint32_t pn = P.p_n[(size_t)b * rows + a], qn = P.q_n[(size_t)b * P.draft_stride + a];
        const uint32_t x = P.drafts[(size_t)b * P.draft_stride + a];
        float u[4];
        spec_uniforms(seed, round, a, 1, u);
        // p(x), q(x): at most one match per list
        float px = 0.0f, qx = 0.0f;
        for (uint32_t j = lane; j < DIST_CAP; j += 32) {
            if (j < pn && pi[j] == x) px = pp[j];
            if (j < qn && qi[j] == x) qx = qp[j];
        }
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) { px += __shfl_xor_sync(0xffffffffu, px, off); qx += __shfl_xor_sync(0xffffffffu, qx, off); }
        if (__fmul_rn(u[1], qx) < px) { if (lane == 0) out[a] = x; continue; }
        // rejected: residual max(p - q, 0) in target order
        for (uint32_t j = lane; j < DIST_CAP; j += 32) {
            float rj = 0.0f;
            if (j < pn) {
                float qj = 0.0f;
                uint32_t id = pi[j];
                for (uint32_t t = 0; t < qn; t++) if (qi[t] == id) qj = qp[t];
                float d = __fsub_rn(pp[j], qj);
                rj = d > 0.0f ? d : 0.0f;
            }
            r_s[j] = rj;
        }
        __syncwarp();
        if (lane == 0) {
            float z = 0.0f;
            for (uint32_t j = 0; j < pn; j++) z = __fadd_rn(r_s[j], z);
            uint32_t tok;
            if (!(z > 0.0f)) tok = pi[0];
            else {
                for (uint32_t j = 0; j < pn; j++) r_s[j] = __fdiv_rn(r_s[j], z);
                tok = pi[pick_from(r_s, (int)pn, u[0])];
            }
            out[a] = tok;
            for (uint32_t j = a + 1; j < rows; j++) out[j] = 0xffffffffu;
            P.accept_len[b] = a;
        }
        return;
    }
    if (lane == 0) {
        float u[4];
        spec_uniforms(seed, round, nd, 1, u);
        const uint32_t *pi = P.p_ids + ((size_t)b * rows + nd) * DIST_CAP;
        const float *pp = P.p_probs + ((size_t)b * rows + nd) * DIST_CAP;
        out[nd] = pi[pick_from(pp, (int)P.p_n[(size_t)b * rows + nd], u[0])];
        for (uint32_t j = nd + 1; j < rows; j++) out[j] = 0xffffffffu;
        P.accept_len[b] = nd;
    }
}


int32_t wb_topk_filter(const FilterParams &p, cudaStream_t st) {
    WB_CHECK_ARG(p.x && p.temp && p.top_k && p.top_p && ((p.out_ids && p.out_probs && p.out_n) || p.pcg_out), "topk_filter: null pointer");
    WB_CHECK_ARG(!p.pcg_out || (p.pcg_rng && p.pcg_slots && p.pcg_seed), "sample_rows: rng, slots and seed are required");
    WB_CHECK_ARG(p.row_seq || p.rows_per_seq > 0, "topk_filter: rows_per_seq must be positive");
    WB_CHECK_ARG(!p.sample_out || (p.seed && p.round), "topk_filter: sampling needs seed and round");
    if (p.s == 0) return WB_OK;
    WB_LAUNCH((topk_filter_kernel), p.s, 1024, 0, st, p);
    WB_LAUNCH_CHECK();
    return WB_OK;
}
int32_t wb_accept(const AcceptParams &p, cudaStream_t st) {
    WB_CHECK_ARG((p.drafts || p.k == 0) && p.accept_len && p.out_tokens, "accept: null pointer");
    WB_CHECK_ARG(p.am_part || p.p_ids, "accept: needs argmax partials or target distributions");
    WB_CHECK_ARG(!p.temp || (p.p_ids && p.p_probs && p.p_n && (p.k == 0 || (p.q_ids && p.q_probs && p.q_n)) && p.seed && p.round),
                 "accept: sampled mode needs both distributions, seeds and rounds");
    WB_CHECK_ARG(p.k <= 15 && p.draft_stride >= p.k, "accept: k = %u outside 0..15 or draft stride too small", p.k);
    if (p.B == 0) return WB_OK;
    WB_LAUNCH((accept_kernel), p.B, 32, 0, st, p);
    WB_LAUNCH_CHECK();
    return WB_OK;
}

int32_t wb_topk_filter_args(const FilterArgs &a, cudaStream_t st) {
    FilterParams p{};
    p.x = (const bf16_t *)a.logits; p.rows = a.rows; p.row_seq = a.row_seq; p.rows_per_seq = a.rows_per_seq;
    p.temp = a.temp; p.top_k = a.top_k; p.top_p = a.top_p; p.n = a.n; p.s = a.s;
    p.out_ids = a.out_ids; p.out_probs = a.out_probs; p.out_n = a.out_n; p.out_mul = a.out_mul; p.out_off = a.out_off;
    p.sample_out = a.sample_out; p.sample_mul = a.sample_mul; p.sample_off = a.sample_off; p.seed = a.seed; p.round = a.round;
    p.position = a.position;
    return wb_topk_filter(p, st);
}
int32_t wb_accept_args(const AcceptArgs &a, cudaStream_t st) {
    AcceptParams p{};
    p.am_part = a.am_part; p.am_split = a.am_split; p.p_ids = a.p_ids; p.q_ids = a.q_ids; p.p_n = a.p_n; p.q_n = a.q_n;
    p.p_probs = a.p_probs; p.q_probs = a.q_probs; p.temp = a.temp; p.seed = a.seed; p.round = a.round; p.slot_of = a.slot_of;
    p.drafts = a.drafts; p.draft_stride = a.draft_stride; p.n_drafts = a.n_drafts; p.B = a.B; p.k = a.k;
    p.accept_len = a.accept_len; p.out_tokens = a.out_tokens; p.target = a.target;
    return wb_accept(p, st);
}

extern "C" {

int32_t wein_b200_topk_filter(const void *logits, const void *rows, const void *row_seq, uint32_t rows_per_seq, const void *temp,
                              const void *top_k, const void *top_p, uint32_t n, uint32_t s, void *out_ids, void *out_probs,
                              void *out_n, void *sample_out, const void *seed, const void *round, uint32_t position, void *stream) {
    FilterParams p{};
    p.x = (const bf16_t *)logits; p.rows = (const uint32_t *)rows; p.row_seq = (const uint32_t *)row_seq; p.rows_per_seq = rows_per_seq;
    p.temp = (const float *)temp; p.top_k = (const uint32_t *)top_k; p.top_p = (const float *)top_p; p.n = n; p.s = s;
    p.out_ids = (uint32_t *)out_ids; p.out_probs = (float *)out_probs; p.out_n = (uint32_t *)out_n;
    p.sample_out = (uint32_t *)sample_out; p.seed = (const uint64_t *)seed; p.round = (const uint64_t *)round; p.position = position;
    p.out_mul = 1; p.out_off = 0; p.sample_mul = 1; p.sample_off = 0;
    return wb_topk_filter(p, (cudaStream_t)stream);
}

// SampleRowsOp::run (crates/wein-kernel/src/ops/mod.rs:1379-1393): x [*, n] bf16, rows [s] sampled row ids, slots [s] RNG slot
// of each row, temp / top_k / top_p / seed [s] per row, rng [slots] u64 PCG states (0 = derive from the seed), out [s]
// (0xFFFFFFFF = top_k 0 with temp > 0).  Bit-identical to the reference sampler for rows whose top-k lies within the
// reference kernel's per-lane ladder (always, for distinct-enough logits; reference.rs:783-786).
int32_t wein_b200_sample_rows(const void *x, const void *rows, const void *slots, const void *temp, const void *top_k, const void *top_p,
                              const void *seed, void *rng, void *out, uint32_t n, uint32_t s, void *stream) {
    WB_CHECK_ARG(rows && slots && seed && rng && out, "sample_rows: null pointer");
    FilterParams p{};
    p.x = (const bf16_t *)x; p.rows = (const uint32_t *)rows; p.rows_per_seq = 1;
    p.temp = (const float *)temp; p.top_k = (const uint32_t *)top_k; p.top_p = (const float *)top_p; p.n = n; p.s = s;
    p.out_mul = 1; p.sample_mul = 1;
    p.pcg_rng = (uint64_t *)rng; p.pcg_slots = (const uint32_t *)slots; p.pcg_seed = (const uint64_t *)seed; p.pcg_out = (uint32_t *)out;
    return wb_topk_filter(p, (cudaStream_t)stream);
}

// Greedy acceptance straight from logits: argmax of the B*(k+1) verify rows (row b*(k+1)+j of `rows`), then the
// longest-prefix rule.  scratch: B*(k+1)*32 u64 words.
int32_t wein_b200_accept_greedy(const void *logits, const void *rows, const void *drafts, const void *n_drafts, uint32_t n,
                                uint32_t B, uint32_t k, void *scratch, void *accept_len, void *out_tokens, void *target, void *stream) {
    WB_CHECK_ARG(logits && rows && scratch, "accept_greedy: null pointer");
    const uint32_t T = B * (k + 1), split = T >= 64 ? 8u : (T >= 16 ? 16u : 32u);
    int32_t rc = wein_b200_argmax_partials(logits, rows, scratch, n, T, split, (cudaStream_t)stream);
    if (rc != WB_OK) return rc;
    AcceptParams p{};
    p.am_part = (const uint64_t *)scratch; p.am_split = split;
    p.drafts = (const uint32_t *)drafts; p.n_drafts = (const uint32_t *)n_drafts; p.B = B; p.k = k; p.draft_stride = k;
    p.accept_len = (uint32_t *)accept_len; p.out_tokens = (uint32_t *)out_tokens; p.target = (uint32_t *)target;
    return wb_accept(p, (cudaStream_t)stream);
}

// Rejection-sampling acceptance from compact distributions (rows with temp <= 0 use the greedy rule on entry 0).
int32_t wein_b200_accept_sampled(const void *drafts, const void *n_drafts, const void *p_ids, const void *p_probs, const void *p_n,
                                 const void *q_ids, const void *q_probs, const void *q_n, const void *temp, const void *seed,
                                 const void *round, uint32_t B, uint32_t k, void *accept_len, void *out_tokens, void *stream) {
    WB_CHECK_ARG(temp != nullptr, "accept_sampled: temp is required");
    AcceptParams p{};
    p.p_ids = (const uint32_t *)p_ids; p.p_probs = (const float *)p_probs; p.p_n = (const uint32_t *)p_n;
    p.q_ids = (const uint32_t *)q_ids; p.q_probs = (const float *)q_probs; p.q_n = (const uint32_t *)q_n;
    p.temp = (const float *)temp; p.seed = (const uint64_t *)seed; p.round = (const uint64_t *)round;
    p.drafts = (const uint32_t *)drafts; p.n_drafts = (const uint32_t *)n_drafts; p.B = B; p.k = k; p.draft_stride = k;
    p.accept_len = (uint32_t *)accept_len; p.out_tokens = (uint32_t *)out_tokens;
    return wb_accept(p, (cudaStream_t)stream);
}

}  // extern "C"

