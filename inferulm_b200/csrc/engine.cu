// Step-level host side: the speculative step of wein's executor re-stated for device-resident control.
//
// Reference: Qwen35Executor::step and its helpers (crates/wein-exec/src/qwen.rs): spec_draft_batch (:2748-2853, k MTP
// forwards, each ending in a stream sync and a readback), forward_batch_mixed / run_forward (:3453-3703, :3843-4153, one
// verify forward over all chain rows), spec_finish (:2419-2502, host-side acceptance, zero-copy state-row swap,
// hidden stash).  The reference never graph-captures this step (:2235-2237) because acceptance is decided on the host.
//
// Here every per-round decision lives on the device: small kernels build the round's row / span tables from the
// per-slot state (position, pending token, state row), the draft tokens stay in a device buffer, acceptance and
// commit are kernels.  A round is therefore a fixed launch sequence -- k draft forwards, one verify forward, accept,
// commit -- which is captured once per (batch, k, mode, context bucket) and replayed as one CUDA graph.
//
// State rows.  The reference claims k+2 contiguous rows per chain and commits by re-pointing state_row to head+1+a.
// Each slot here owns two banks of k_max+1 rows; a round reads the slot's current row and writes its snapshots into
// the other bank, then commits by setting state_row = bank base + a.  No state bytes are ever copied.
#include <math.h>
#include <stdio.h>
#include <string.h>
#include <map>
#include <string>
#include <tuple>
#include <vector>
#include "../../include/wein_b200.h"
#include "common.cuh"
#include "internal.h"

extern "C" {
int32_t wein_b200_embed(const void *, const void *, void *, uint32_t, uint32_t, void *);
int32_t wein_b200_rms_norm_zc(const void *, const void *, void *, uint32_t, uint32_t, float, void *);
int32_t wein_b200_add_norm_zc(const void *, const void *, const void *, void *, void *, uint32_t, uint32_t, float, void *);
}

#define CUDA_TRY(x)                                                                                        \
    do {                                                                                                   \
        cudaError_t e__ = (x);                                                                             \
        if (e__ != cudaSuccess) { wb_set_error("%s:%d %s: %s", __FILE__, __LINE__, #x, cudaGetErrorString(e__)); return WB_ERR_CUDA; } \
    } while (0)
#define TRY(x)                       \
    do {                             \
        int32_t rc__ = (x);          \
        if (rc__ != WB_OK) return rc__; \
    } while (0)

#define RING_CAP 8192u
#define STATS_WORDS 24u   // per slot: rounds, drafts, accepted, fallbacks, k switches, rounds by draft count [8], rounds by accept length [9], last draft count, spare
#define DEAD_ROW 0xffffffffu   // position of a batch row that belongs to no live chain position this round

struct wein_b200_engine {
    wein_b200_model_cfg cfg;
    wein_b200_weights w;
    uint32_t H, II, V, P, T_max, bpr, keyd, vald, cd, lpn, fpn, n_lin, n_full, rows_per_slot, seg_pages;
    std::vector<void *> allocs;
    uint64_t bytes = 0;
    std::vector<void *> lin_state, conv_state, k_pool, v_pool;  // k/v pools: full layers then the MTP layer
    std::vector<float *> lin_log;      // per DeltaNet layer: update records of a round's positions (snapshot-lite verification)
    float *gdn_kq = nullptr;           // per-token operands of a DeltaNet layer (k-hat, q-hat, conv of v, gates): T x v_heads x 388 floats
    void **d_state_ptrs = nullptr;     // device copies of lin_state / lin_log for the one-launch commit
    float **d_log_ptrs = nullptr;
    // per-slot device state
    uint32_t *d_pos, *d_pending, *d_state_row, *d_bank, *d_out_count, *d_top_k, *d_ring, *d_block_table;
    uint32_t *d_limit, *d_status, *d_kreq;   // per slot: position limit (admitted pages), status bits, draft length asked for
    uint64_t *d_round, *d_seed, *d_stats;
    float *d_temp, *d_top_p;
    bf16_t *d_hid;
    // per-step tables
    uint32_t *d_slots, *d_tok, *d_pos_rows, *d_seq_rows, *d_row_start, *d_row_count, *d_in_row, *d_out_base, *d_lg_rows, *d_iota, *d_ones;
    uint32_t *d_cnt_in, *d_tok_in, *d_last_in, *d_first_tok, *d_lg_of;
    uint32_t *d_drafts, *d_accept_len, *d_out_tokens, *d_target;
    uint32_t *d_nd, *d_nd_in;           // per batch row: drafts verified this round; the caller's draft counts (spec_verify)
    uint32_t *d_mtp_tok, *d_mtp_rope, *d_mtp_kvpos;
    // activations
    bf16_t *x, *n1, *h2, *n2, *o, *proj, *qkvc, *core, *normed, *qh, *gate, *attn, *gu, *m, *d, *logits, *lg_in, *cat;
    float *cosv, *sinv;
    void *gemm_scratch, *attn_scratch, *am_part;
    uint64_t gemm_scratch_bytes, attn_scratch_bytes;
    uint32_t *p_ids, *q_ids, *p_n, *q_n;
    float *p_probs, *q_probs;
    // host mirrors
    std::vector<float> h_temp;
    std::vector<uint32_t> h_limit;      // host mirror of d_limit
    uint32_t gemm_path = WB_GEMM_AUTO;  // WB_GEMM_TC when a forward of this engine can exceed 32 rows (one kernel for every row count)
    bool snapshots = false;             // true: a state snapshot per verify position in every round (no update records)
    bool timing = false;                // eager rounds record phase events (draft / forward / finish)
    cudaEvent_t ev[4] = {nullptr, nullptr, nullptr, nullptr};
    bool ev_pending = false;
    double ms_phase[3] = {0.0, 0.0, 0.0};
    std::vector<uint32_t> h_slots_cached;
    uint32_t *h_stage = nullptr;  // pinned
    size_t h_stage_words = 0;
    std::map<std::tuple<uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t>, std::pair<cudaGraphExec_t, uint32_t>> graphs;
    uint32_t launches = 0, last_launches = 0;
    uint32_t last_n = 0, last_P = 0;     // shape of the most recent round (for read_round)
    uint32_t *d_pack = nullptr, *h_pack = nullptr;   // per-round readback, device and pinned host: [max_seqs, 3 + P]
    std::map<std::string, std::pair<void *, uint64_t>> named;
};
typedef wein_b200_engine Engine;

template <typename T>
static int32_t dalloc(Engine *e, T **p, size_t n, const char *name, bool zero = true) {
    size_t bytes = n * sizeof(T);
    if (bytes == 0) bytes = 16;
    void *q = nullptr;
    cudaError_t er = cudaMalloc(&q, bytes);
    if (er != cudaSuccess) { wb_set_error("engine: cudaMalloc of %zu bytes for %s failed: %s", bytes, name, cudaGetErrorString(er)); return WB_ERR_CUDA; }
    if (zero) cudaMemset(q, 0, bytes);
    e->allocs.push_back(q);
    e->bytes += bytes;
    e->named[name] = {q, bytes};
    *p = (T *)q;
    return WB_OK;
}

// ------------------------------------------------------------------------------------------------ table kernels
struct SlotState {
    uint32_t *pos, *pending, *state_row, *bank, *out_count, *ring, *limit, *status, *kreq;
    uint64_t *round, *stats;
    bf16_t *hid;
};

// Block-wide copy of one hidden row, 16 bytes per thread and step (rows are 16-byte aligned: hidden is a multiple of 32)
__device__ __forceinline__ void copy_row(bf16_t *dst, const bf16_t *src, uint32_t H) {
    const uint4 *s = reinterpret_cast<const uint4 *>(src);
    uint4 *d = reinterpret_cast<uint4 *>(dst);
    for (uint32_t i = threadIdx.x; i < H / 8; i += blockDim.x) d[i] = s[i];
}

// Rows of a speculative round: batch row b = slot slots[b] owns rows b*P .. b*P+P-1; its chain takes the first nd+1 of them
// (the pending token, then drafts 0..nd-1), the others are dead rows (token 0, position DEAD_ROW: they are multiplied like
// any row, write no KV and belong to no span).  nd = min(round k, the slot's own draft length, the caller's count) and is cut
// further so that the chain stays below the slot's position limit (the reference cuts k to max_pos - (start + 1) and falls
// back to a plain step, qwen.rs:2771-2777); a slot already at its limit sits the round out (span of 0 rows) and gets
// WB_STATUS_POS_LIMIT: nothing is read or written past the pages it was admitted with.
__global__ void verify_prep_kernel(const uint32_t *slots, SlotState S, const uint32_t *drafts, uint32_t k_max, const uint32_t *nd_in,
                                   uint32_t n, uint32_t P, uint32_t vocab, uint32_t rows_per_slot, uint32_t bankrows, uint32_t *tok,
                                   uint32_t *pos_rows, uint32_t *seq_rows, uint32_t *row_start, uint32_t *row_count, uint32_t *in_row,
                                   uint32_t *out_base, uint32_t *lg_rows, uint32_t *nd_out) {
    PDL_ENTRY();
    uint32_t b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n) return;
    const uint32_t slot = slots[b], p0 = S.pos[slot], lim = S.limit[slot];
    uint32_t nd = min(P - 1, S.kreq[slot]);
    if (nd_in) nd = min(nd, nd_in[b]);
    uint32_t cnt;
    if (p0 + 1 > lim) { cnt = 0; nd = 0; atomicOr(&S.status[slot], WB_STATUS_POS_LIMIT); }
    else {
        if (p0 + nd + 1 > lim) { nd = lim - p0 - 1; atomicOr(&S.status[slot], WB_STATUS_K_CLAMPED); }
        cnt = nd + 1;
    }
    for (uint32_t j = 0; j < P; j++) {
        const uint32_t r = b * P + j;
        uint32_t t = 0;
        if (j < cnt) t = j == 0 ? S.pending[slot] : drafts[b * k_max + j - 1];
        tok[r] = t < vocab ? t : 0;    // a draft outside the vocabulary can never be accepted; the forward must not index with it
        pos_rows[r] = j < cnt ? p0 + j : DEAD_ROW;
        seq_rows[r] = slot;
        lg_rows[r] = r;
    }
    row_start[b] = b * P;
    row_count[b] = cnt;
    in_row[b] = S.state_row[slot];
    out_base[b] = slot * rows_per_slot + (S.bank[slot] ^ 1u) * bankrows;
    nd_out[b] = nd;
}

// Commit of a round (spec_finish, qwen.rs:2433-2460): emitted tokens to the slot's ring, position += a+1, pending =
// bonus token, state_row = snapshot a of this round's bank, hidden of chain row a stashed for the next draft; the counters
// of spec_stats() / spec_k_stats() (qwen.rs:4257-4259, :2670).  A slot that sat the round out keeps everything.
__global__ void commit_kernel(const uint32_t *slots, SlotState S, const uint32_t *accept_len, const uint32_t *row_count,
                              const uint32_t *nd_row, const uint32_t *out_tokens, const uint32_t *out_base, const bf16_t *x,
                              uint32_t P, uint32_t k, uint32_t H) {
    PDL_ENTRY();
    const uint32_t b = blockIdx.x, slot = slots[b];
    uint64_t *st = S.stats + (size_t)slot * STATS_WORDS;
    if (row_count[b] == 0) {
        if (threadIdx.x == 0) st[3] += 1;
        return;
    }
    const uint32_t nd = nd_row[b], a = min(accept_len[b], nd);
    copy_row(S.hid + (size_t)slot * H, x + (size_t)(b * P + a) * H, H);
    if (threadIdx.x == 0) {
        uint32_t oc = S.out_count[slot];
        for (uint32_t j = 0; j <= a; j++) S.ring[(size_t)slot * RING_CAP + ((oc + j) % RING_CAP)] = out_tokens[b * P + j];
        S.out_count[slot] = oc + a + 1;
        S.pending[slot] = out_tokens[b * P + a];
        S.pos[slot] += a + 1;
        S.state_row[slot] = out_base[b] + a;
        S.bank[slot] ^= 1u;
        S.round[slot] += 1;
        if (st[0] != 0 && st[22] != nd) st[4] += 1;                 // the chain length changed against the slot's previous round
        st[0] += 1; st[1] += nd; st[2] += a;
        if (nd < min(k, S.kreq[slot])) st[3] += 1;                  // fewer drafts than asked: cut at the position limit
        st[5 + min(nd, 7u)] += 1;
        st[13 + min(a, 8u)] += 1;
        st[22] = nd;
    }
}

// What the host reads back after a round, packed for one copy: per batch row [accept length, position, tokens emitted since
// admission, the round's a+1 tokens (padded to k_max+1 words; none for a slot that sat the round out), the slot's status word].  Stands in for the reference's per-step readback of its u32 [B*P]
// argmax table (forward_batch_mixed, qwen.rs:3453-3703).
__global__ void round_pack_kernel(const uint32_t *slots, SlotState S, const uint32_t *accept_len, const uint32_t *row_count,
                                  const uint32_t *out_tokens, uint32_t n, uint32_t P, uint32_t P_stride, uint32_t *out) {
    PDL_ENTRY();
    uint32_t b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n) return;
    const uint32_t slot = slots[b], live = row_count[b] != 0, a = live ? min(accept_len[b], P - 1) : 0u;
    uint32_t *o = out + (size_t)b * (4 + P_stride);
    o[0] = a; o[1] = S.pos[slot]; o[2] = S.out_count[slot];
    for (uint32_t j = 0; j < P_stride; j++) o[3 + j] = (live && j <= a && j < P) ? out_tokens[b * P + j] : 0xffffffffu;
    o[3 + P_stride] = S.status[slot];
}

// Prefill chunk tables: span b holds cnt[b] prompt tokens of slot slots[b] (tokens concatenated in tok_in).
__global__ void prefill_prep_kernel(const uint32_t *slots, SlotState S, const uint32_t *cnt,
                                    const uint32_t *tok_in, const uint32_t *last, uint32_t n, uint32_t rows_per_slot,
                                    uint32_t bankrows, uint32_t *tok, uint32_t *pos_rows, uint32_t *seq_rows, uint32_t *row_start,
                                    uint32_t *row_count, uint32_t *in_row, uint32_t *out_base, uint32_t *lg_rows, uint32_t *lg_of) {
    PDL_ENTRY();
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    uint32_t r = 0, nl = 0;
    for (uint32_t b = 0; b < n; b++) {
        uint32_t slot = slots[b], c = cnt[b], p0 = S.pos[slot];
        row_start[b] = r;
        row_count[b] = c;
        in_row[b] = S.state_row[slot];
        out_base[b] = slot * rows_per_slot + (S.bank[slot] ^ 1u) * bankrows;
        for (uint32_t j = 0; j < c; j++, r++) { tok[r] = tok_in[r]; pos_rows[r] = p0 + j; seq_rows[r] = slot; }
        lg_of[b] = 0xffffffffu;
        if (c > 0 && last[b]) { lg_rows[nl] = r - 1; lg_of[b] = nl; nl++; }
    }
}
__global__ void prefill_commit_kernel(const uint32_t *slots, SlotState S, const uint32_t *cnt,
                                      const uint32_t *row_start, const uint32_t *out_base,
                                      const uint32_t *lg_of, const uint32_t *first_tok, const bf16_t *x,
                                      uint32_t H) {
    PDL_ENTRY();
    uint32_t b = blockIdx.x, slot = slots[b], c = cnt[b];
    if (c == 0) return;
    copy_row(S.hid + (size_t)slot * H, x + (size_t)(row_start[b] + c - 1) * H, H);
    if (threadIdx.x == 0) {
        S.pos[slot] += c;
        S.state_row[slot] = out_base[b] + c - 1;
        S.bank[slot] ^= 1u;
        if (lg_of[b] != 0xffffffffu) {
            uint32_t t = first_tok[lg_of[b]];
            S.pending[slot] = t;
            uint32_t oc = S.out_count[slot];
            S.ring[(size_t)slot * RING_CAP + (oc % RING_CAP)] = t;
            S.out_count[slot] = oc + 1;
            S.round[slot] += 1;
        }
    }
}
// Inputs of draft step i: token = pending (i = 0) or the previous draft; rotary position absolute, KV slot chain-local.
__global__ void mtp_prep_kernel(const uint32_t *slots, SlotState S, const uint32_t *drafts, uint32_t k_max,
                                uint32_t n, uint32_t i, uint32_t vocab, uint32_t max_pos, uint32_t *tok, uint32_t *rope_pos, uint32_t *kv_pos) {
    PDL_ENTRY();
    uint32_t b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n) return;
    uint32_t slot = slots[b];
    const uint32_t t = i == 0 ? S.pending[slot] : drafts[b * k_max + i - 1];
    tok[b] = t < vocab ? t : 0;
    rope_pos[b] = min(S.pos[slot] + i, max_pos - 1);   // a draft past the position limit is dropped by the verify tables anyway
    kv_pos[b] = i;
}
// Caller-supplied drafts of a verify-only round (spec_verify): drafts [n, k], optional per-row counts, optional draft
// distributions as compact lists [n, k, 64]; without lists a draft counts as drawn from a point mass (q = 1 on the draft).
__global__ void import_drafts_kernel(const uint32_t *src, const uint32_t *src_nd, const uint32_t *src_q_ids, const float *src_q_probs,
                                     const uint32_t *src_q_n, uint32_t n, uint32_t k, uint32_t k_max, uint32_t *drafts, uint32_t *nd_in,
                                     uint32_t *q_ids, float *q_probs, uint32_t *q_n) {
    PDL_ENTRY();
    const uint32_t b = blockIdx.x, j = blockIdx.y, i = threadIdx.x;   // 64 threads
    const uint32_t d = src[b * k + j];
    const size_t di = (size_t)b * k_max + j, si = (size_t)b * k + j;
    if (i == 0) {
        drafts[di] = d;
        if (j == 0) nd_in[b] = src_nd ? min(src_nd[b], k) : k;
        q_n[di] = src_q_ids ? min(src_q_n[si], 64u) : 1u;
    }
    if (src_q_ids) { q_ids[di * 64 + i] = src_q_ids[si * 64 + i]; q_probs[di * 64 + i] = src_q_probs[si * 64 + i]; }
    else { q_ids[di * 64 + i] = i == 0 ? d : 0xffffffffu; q_probs[di * 64 + i] = i == 0 ? 1.0f : 0.0f; }
}
__global__ void resume_kernel(SlotState S, uint32_t slot, uint32_t position, uint32_t pending) { PDL_ENTRY(); S.pos[slot] = position; S.pending[slot] = pending; }
__global__ void set_kreq_kernel(uint32_t *kreq, uint32_t slot, uint32_t k) { PDL_ENTRY(); kreq[slot] = k; }
__global__ void clear_status_kernel(uint32_t *status, uint32_t slot) { PDL_ENTRY(); status[slot] = 0; }
__global__ void slot_init_kernel(SlotState S, uint32_t slot, uint32_t row0, uint32_t limit, float *temp, uint32_t *top_k, float *top_p,
                                 uint64_t *seed, float t, uint32_t k, float p, uint64_t sd) {
    PDL_ENTRY();
    S.pos[slot] = 0; S.pending[slot] = 0; S.state_row[slot] = row0; S.bank[slot] = 0; S.out_count[slot] = 0; S.round[slot] = 0;
    S.limit[slot] = limit; S.status[slot] = 0; S.kreq[slot] = 0xffffffffu;
    for (uint32_t i = 0; i < STATS_WORDS; i++) S.stats[(size_t)slot * STATS_WORDS + i] = 0;
    temp[slot] = t; top_k[slot] = k; top_p[slot] = p; seed[slot] = sd;
}

static SlotState slot_state(Engine *e) {
    SlotState s;
    s.pos = e->d_pos; s.pending = e->d_pending; s.state_row = e->d_state_row; s.bank = e->d_bank; s.out_count = e->d_out_count;
    s.ring = e->d_ring; s.round = e->d_round; s.stats = e->d_stats; s.hid = e->d_hid;
    s.limit = e->d_limit; s.status = e->d_status; s.kreq = e->d_kreq;
    return s;
}

// ------------------------------------------------------------------------------------------------ create / destroy
static bool adjacent(const void *a, const void *b, size_t a_elems) { return a && b && (const char *)b == (const char *)a + a_elems * 2; }

extern "C" int32_t wein_b200_engine_create(const wein_b200_model_cfg *cfg, const wein_b200_weights *weights, wein_b200_engine **out) {
    WB_CHECK_ARG(cfg && weights && out, "engine_create: null argument");
    WB_CHECK_ARG(cfg->n_layers >= 1 && cfg->n_layers <= WEIN_B200_MAX_LAYERS, "engine_create: n_layers %u outside 1..%d", cfg->n_layers, WEIN_B200_MAX_LAYERS);
    WB_CHECK_ARG(cfg->k_max <= 7 && cfg->max_seqs >= 1, "engine_create: k_max %u > 7 or no slots", cfg->k_max);
    WB_CHECK_ARG(cfg->hidden % 32 == 0 && cfg->inter % 32 == 0 && cfg->hidden >= 256, "engine_create: hidden / inter must be multiples of 32");
    WB_CHECK_ARG(cfg->lin_k_dim == 128 && cfg->lin_v_dim == 128 && cfg->conv_kernel == 4, "engine_create: DeltaNet heads must be 128x128 with conv width 4");
    WB_CHECK_ARG(cfg->q_heads % cfg->kv_heads == 0 && (cfg->q_heads / cfg->kv_heads) * (cfg->k_max + 1) <= 32,
                 "engine_create: (k_max+1) x GQA group exceeds 32 query rows");
    WB_CHECK_ARG(cfg->max_pos >= cfg->k_max + 2, "engine_create: max_pos %u leaves no room for one round", cfg->max_pos);
    Engine *e = new Engine();
    e->cfg = *cfg; e->w = *weights;
    e->H = cfg->hidden; e->II = cfg->inter; e->V = cfg->vocab; e->P = cfg->k_max + 1; e->T_max = cfg->max_seqs * e->P;
    e->bpr = (cfg->max_pos + 15) / 16;
    e->keyd = cfg->lin_k_heads * cfg->lin_k_dim; e->vald = cfg->lin_v_heads * cfg->lin_v_dim; e->cd = 2 * e->keyd + e->vald;
    e->lpn = e->cd + e->vald + 2 * cfg->lin_v_heads;
    e->fpn = 2 * cfg->q_heads * cfg->head_dim + 2 * cfg->kv_heads * cfg->head_dim;
    e->rows_per_slot = 2 * e->P;
    // One GEMM kernel per engine: the skinny kernel and the tensor-memory kernel each keep a row's bits independent of the
    // batch, but differ from each other, and greedy speculation is output-preserving only if the plain, draft and verify
    // forwards of a sequence sum in one order.  An engine whose largest forward fits 32 rows runs the skinny kernel
    // everywhere; any larger engine runs the tensor-memory kernel for every row count.
    e->gemm_path = e->T_max > 32 ? WB_GEMM_TC : WB_GEMM_AUTO;
    e->snapshots = cfg->state_snapshots != 0;
    // Pages per attention segment: fixed per engine, because it fixes the summation order (two engines agree bit for bit only
    // with the same value: pin cfg.attn_seg_pages to compare engines of different capacity).  A CTA reduces one segment of
    // one (chain, kv head): short segments cost a launch, a Q stage and a merge per 128 KB of KV, long ones leave SMs idle.
    // Aim at ~3 CTAs per SM when every slot is at the longest context (measured, 32 chains x 2K tokens: 16 pages 105 us,
    // 64 pages 78 us; 8 chains x 32K tokens: 128 pages 214 us, 256 pages 199 us = 5.4 TB/s).
    e->seg_pages = cfg->attn_seg_pages;
    if (!e->seg_pages) {
        int dev = 0, sms = 148;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        cudaGetLastError();
        const uint32_t pairs = cfg->max_seqs * cfg->kv_heads;
        uint32_t segs = (3u * (uint32_t)sms + pairs - 1) / pairs;
        if (segs < 1) segs = 1;
        const uint32_t want = (e->bpr + segs - 1) / segs;
        e->seg_pages = 4;
        while (e->seg_pages < want && e->seg_pages < 128) e->seg_pages *= 2;   // 256 pages: faster alone, slower in a round (1.7 waves)
        if (want >= 32) {
            // longer contexts: a segment CTA fills an SM (one CTA per SM at these shared-memory sizes), so what counts is that the
            // grid is a whole number of waves: the segment length (a multiple of 8 pages) with the least waves x (pages + the
            // fixed cost of a CTA, about 6 pages' worth).  8 chains x 32K tokens: 56 pages = 37 segments x 32 = 8 full waves on 148 SMs.
            uint64_t best = ~0ull;
            for (uint32_t sp = 32; sp <= 256; sp += 8) {
                const uint64_t ctas = (uint64_t)((e->bpr + sp - 1) / sp) * pairs, waves = (ctas + sms - 1) / sms, cost = waves * (sp + 6);
                if (cost <= best) { best = cost; e->seg_pages = sp; }
            }
        }
    }
    for (uint32_t l = 0; l < cfg->n_layers; l++) (cfg->layer_is_full[l] ? e->n_full : e->n_lin)++;
    *out = e;
    const uint32_t S = cfg->max_seqs, T = e->T_max, H = e->H;
    TRY(wb_gemm_init());
    TRY(wb_attn_init(cfg->head_dim));
    // pools
    size_t st_elem = cfg->state_f32 ? 4 : 2;
    size_t lin_row = (size_t)cfg->lin_v_heads * 128 * 128, conv_row = (size_t)e->cd * 3;
    for (uint32_t i = 0; i < e->n_lin; i++) {
        char *p; bf16_t *c;
        TRY(dalloc(e, &p, (size_t)S * e->rows_per_slot * lin_row * st_elem, ("lin_state:" + std::to_string(i)).c_str(), false));
        TRY(dalloc(e, &c, (size_t)S * e->rows_per_slot * conv_row, ("conv_state:" + std::to_string(i)).c_str(), false));
        e->lin_state.push_back(p); e->conv_state.push_back(c);
    }
    if (e->n_lin) TRY(dalloc(e, &e->gdn_kq, (size_t)T * ((size_t)cfg->lin_v_heads * 388), "gdn_kq", false));
    if (e->P >= 3 && e->n_lin && !e->snapshots) {
        // from three positions per round on, a round logs its state updates instead of writing a snapshot per position
        for (uint32_t i = 0; i < e->n_lin; i++) {
            float *lg;
            TRY(dalloc(e, &lg, (size_t)T * cfg->lin_v_heads * 264, ("lin_log:" + std::to_string(i)).c_str(), false));
            e->lin_log.push_back(lg);
        }
        TRY(dalloc(e, &e->d_state_ptrs, e->n_lin, "state_ptrs")); TRY(dalloc(e, &e->d_log_ptrs, e->n_lin, "log_ptrs"));
        CUDA_TRY(cudaMemcpy(e->d_state_ptrs, e->lin_state.data(), e->n_lin * sizeof(void *), cudaMemcpyHostToDevice));
        CUDA_TRY(cudaMemcpy(e->d_log_ptrs, e->lin_log.data(), e->n_lin * sizeof(float *), cudaMemcpyHostToDevice));
    }
    size_t he = (size_t)cfg->kv_heads * cfg->head_dim;
    for (uint32_t i = 0; i < e->n_full; i++) {
        bf16_t *k, *v;
        TRY(dalloc(e, &k, (size_t)cfg->n_pages * 16 * he, ("k_pool:" + std::to_string(i)).c_str(), false));
        TRY(dalloc(e, &v, (size_t)cfg->n_pages * 16 * he, ("v_pool:" + std::to_string(i)).c_str(), false));
        e->k_pool.push_back(k); e->v_pool.push_back(v);
    }
    if (cfg->has_mtp) {
        bf16_t *k, *v;
        TRY(dalloc(e, &k, (size_t)S * 16 * he, "k_pool:mtp"));
        TRY(dalloc(e, &v, (size_t)S * 16 * he, "v_pool:mtp"));
        e->k_pool.push_back(k); e->v_pool.push_back(v);
    }
    // slot state
    TRY(dalloc(e, &e->d_pos, S, "pos")); TRY(dalloc(e, &e->d_pending, S, "pending")); TRY(dalloc(e, &e->d_state_row, S, "state_row"));
    TRY(dalloc(e, &e->d_bank, S, "bank")); TRY(dalloc(e, &e->d_out_count, S, "out_count")); TRY(dalloc(e, &e->d_top_k, S, "top_k"));
    TRY(dalloc(e, &e->d_ring, (size_t)S * RING_CAP, "ring")); TRY(dalloc(e, &e->d_block_table, (size_t)S * e->bpr, "block_table"));
    TRY(dalloc(e, &e->d_round, S, "round")); TRY(dalloc(e, &e->d_seed, S, "seed")); TRY(dalloc(e, &e->d_stats, (size_t)S * STATS_WORDS, "stats"));
    TRY(dalloc(e, &e->d_temp, S, "temp")); TRY(dalloc(e, &e->d_top_p, S, "top_p")); TRY(dalloc(e, &e->d_hid, (size_t)S * H, "hid"));
    TRY(dalloc(e, &e->d_limit, S, "limit")); TRY(dalloc(e, &e->d_status, S, "status")); TRY(dalloc(e, &e->d_kreq, S, "kreq"));
    // step tables
    TRY(dalloc(e, &e->d_slots, S, "slots")); TRY(dalloc(e, &e->d_tok, T, "tok")); TRY(dalloc(e, &e->d_pos_rows, T, "pos_rows"));
    TRY(dalloc(e, &e->d_seq_rows, T, "seq_rows")); TRY(dalloc(e, &e->d_row_start, S, "row_start")); TRY(dalloc(e, &e->d_row_count, S, "row_count"));
    TRY(dalloc(e, &e->d_in_row, S, "in_row")); TRY(dalloc(e, &e->d_out_base, S, "out_base")); TRY(dalloc(e, &e->d_lg_rows, T, "lg_rows"));
    TRY(dalloc(e, &e->d_iota, T, "iota")); TRY(dalloc(e, &e->d_ones, T, "ones"));
    TRY(dalloc(e, &e->d_cnt_in, S, "cnt_in")); TRY(dalloc(e, &e->d_tok_in, T, "tok_in")); TRY(dalloc(e, &e->d_last_in, S, "last_in"));
    TRY(dalloc(e, &e->d_first_tok, S, "first_tok")); TRY(dalloc(e, &e->d_lg_of, S, "lg_of"));
    TRY(dalloc(e, &e->d_drafts, (size_t)S * (cfg->k_max ? cfg->k_max : 1), "drafts")); TRY(dalloc(e, &e->d_accept_len, S, "accept_len"));
    TRY(dalloc(e, &e->d_out_tokens, T, "out_tokens")); TRY(dalloc(e, &e->d_target, T, "target"));
    TRY(dalloc(e, &e->d_nd, S, "n_drafts")); TRY(dalloc(e, &e->d_nd_in, S, "n_drafts_in"));
    TRY(dalloc(e, &e->d_mtp_tok, S, "mtp_tok")); TRY(dalloc(e, &e->d_mtp_rope, S, "mtp_rope")); TRY(dalloc(e, &e->d_mtp_kvpos, S, "mtp_kvpos"));
    {
        std::vector<uint32_t> iota(T), ones(T, 1);
        for (uint32_t i = 0; i < T; i++) iota[i] = i;
        CUDA_TRY(cudaMemcpy(e->d_iota, iota.data(), T * 4, cudaMemcpyHostToDevice));
        CUDA_TRY(cudaMemcpy(e->d_ones, ones.data(), T * 4, cudaMemcpyHostToDevice));
    }
    // activations
    size_t qd = (size_t)cfg->q_heads * cfg->head_dim;
    TRY(dalloc(e, &e->x, (size_t)T * H, "x")); TRY(dalloc(e, &e->n1, (size_t)T * H, "n1")); TRY(dalloc(e, &e->h2, (size_t)T * H, "h2"));
    TRY(dalloc(e, &e->n2, (size_t)T * H, "n2")); TRY(dalloc(e, &e->o, (size_t)T * H, "o"));
    TRY(dalloc(e, &e->proj, (size_t)T * (e->lpn > e->fpn ? e->lpn : e->fpn), "proj")); TRY(dalloc(e, &e->qkvc, (size_t)T * e->cd, "qkvc"));
    TRY(dalloc(e, &e->core, (size_t)T * e->vald, "core")); TRY(dalloc(e, &e->normed, (size_t)T * e->vald, "normed"));
    TRY(dalloc(e, &e->qh, (size_t)T * qd, "qh")); TRY(dalloc(e, &e->gate, (size_t)T * qd, "gate")); TRY(dalloc(e, &e->attn, (size_t)T * qd, "attn"));
    TRY(dalloc(e, &e->gu, (size_t)T * 2 * e->II, "gu")); TRY(dalloc(e, &e->m, (size_t)T * e->II, "m")); TRY(dalloc(e, &e->d, (size_t)T * H, "d"));
    TRY(dalloc(e, &e->logits, (size_t)T * e->V, "logits")); TRY(dalloc(e, &e->lg_in, (size_t)T * H, "lg_in"));
    TRY(dalloc(e, &e->cat, (size_t)S * 2 * H, "cat"));
    // rope tables, rounded to bf16 as the reference executor does (qwen.rs:1581-1586)
    {
        uint32_t half = cfg->rot_dim / 2;
        std::vector<float> c((size_t)cfg->max_pos * half), s((size_t)cfg->max_pos * half);
        for (uint32_t p = 0; p < half; p++) {
            double inv_freq = pow(cfg->rope_theta, -((double)p) / (double)half);
            for (uint32_t t = 0; t < cfg->max_pos; t++) {
                double a = (double)t * inv_freq;
                c[(size_t)t * half + p] = bf2f(f2bf((float)cos(a)));
                s[(size_t)t * half + p] = bf2f(f2bf((float)sin(a)));
            }
        }
        TRY(dalloc(e, &e->cosv, c.size(), "cos")); TRY(dalloc(e, &e->sinv, s.size(), "sin"));
        CUDA_TRY(cudaMemcpy(e->cosv, c.data(), c.size() * 4, cudaMemcpyHostToDevice));
        CUDA_TRY(cudaMemcpy(e->sinv, s.data(), s.size() * 4, cudaMemcpyHostToDevice));
    }
    // kernel scratch
    e->gemm_scratch_bytes = wein_b200_gemm_scratch_bytes(e->V);
    char *gs; TRY(dalloc(e, &gs, e->gemm_scratch_bytes, "gemm_scratch")); e->gemm_scratch = gs;
    uint32_t max_segs = (e->bpr + e->seg_pages - 1) / e->seg_pages;
    e->attn_scratch_bytes = wein_b200_attn_scratch_bytes(S, cfg->kv_heads, cfg->head_dim, max_segs);
    char *as; TRY(dalloc(e, &as, e->attn_scratch_bytes, "attn_scratch", false)); e->attn_scratch = as;
    uint64_t *am; TRY(dalloc(e, &am, (size_t)T * 32, "am_part")); e->am_part = am;
    TRY(dalloc(e, &e->p_ids, (size_t)T * 64, "p_ids")); TRY(dalloc(e, &e->p_probs, (size_t)T * 64, "p_probs")); TRY(dalloc(e, &e->p_n, T, "p_n"));
    TRY(dalloc(e, &e->q_ids, (size_t)T * 64, "q_ids")); TRY(dalloc(e, &e->q_probs, (size_t)T * 64, "q_probs")); TRY(dalloc(e, &e->q_n, T, "q_n"));
    e->h_temp.assign(S, 0.0f);
    e->h_limit.assign(S, 0);
    TRY(dalloc(e, &e->d_pack, (size_t)S * (4 + e->P), "round_pack"));
    CUDA_TRY(cudaMallocHost((void **)&e->h_pack, (size_t)S * (4 + e->P) * 4));
    e->h_stage_words = (size_t)T + 5 * S + 16;
    CUDA_TRY(cudaMallocHost((void **)&e->h_stage, e->h_stage_words * 4));
    for (int i = 0; i < 4; i++) CUDA_TRY(cudaEventCreate(&e->ev[i]));
    CUDA_TRY(cudaDeviceSynchronize());
    return WB_OK;
}

extern "C" void wein_b200_engine_destroy(wein_b200_engine *e) {
    if (!e) return;
    cudaDeviceSynchronize();
    for (auto &g : e->graphs) cudaGraphExecDestroy(g.second.first);
    for (void *p : e->allocs) cudaFree(p);
    if (e->h_stage) cudaFreeHost(e->h_stage);
    if (e->h_pack) cudaFreeHost(e->h_pack);
    for (int i = 0; i < 4; i++) if (e->ev[i]) cudaEventDestroy(e->ev[i]);
    delete e;
}
extern "C" uint64_t wein_b200_engine_device_bytes(const wein_b200_engine *e) { return e ? e->bytes : 0; }
extern "C" uint32_t wein_b200_engine_last_launches(const wein_b200_engine *e) { return e ? e->last_launches : 0; }
extern "C" void *wein_b200_engine_buffer(wein_b200_engine *e, const char *name, uint64_t *bytes) {
    if (!e || !name) return nullptr;
    auto it = e->named.find(name);
    if (it == e->named.end()) return nullptr;
    if (bytes) *bytes = it->second.second;
    return it->second.first;
}

extern "C" int32_t wein_b200_engine_admit(wein_b200_engine *e, uint32_t slot, const uint32_t *host_pages, uint32_t n_pages, float temp,
                                          uint32_t top_k, float top_p, uint64_t seed, void *stream) {
    WB_CHECK_ARG(e && slot < e->cfg.max_seqs, "engine_admit: slot %u out of range", slot);
    WB_CHECK_ARG(host_pages && n_pages >= 1 && n_pages <= e->bpr, "engine_admit: %u pages outside 1..%u", n_pages, e->bpr);
    for (uint32_t i = 0; i < n_pages; i++) WB_CHECK_ARG(host_pages[i] < e->cfg.n_pages, "engine_admit: page id %u >= pool size %u", host_pages[i], e->cfg.n_pages);
    WB_CHECK_ARG(!(temp > 0.0f) || (top_k >= 1 && top_k <= 64), "engine_admit: sampling needs 1 <= top_k <= 64 (whole-vocabulary sampling is not built)");
    cudaStream_t st = (cudaStream_t)stream;
    uint32_t row0 = slot * e->rows_per_slot;
    size_t st_elem = e->cfg.state_f32 ? 4 : 2;
    size_t lin_row = (size_t)e->cfg.lin_v_heads * 128 * 128 * st_elem, conv_row = (size_t)e->cd * 3 * 2;
    for (uint32_t i = 0; i < e->n_lin; i++) {
        CUDA_TRY(cudaMemsetAsync((char *)e->lin_state[i] + (size_t)row0 * lin_row, 0, lin_row, st));
        CUDA_TRY(cudaMemsetAsync((char *)e->conv_state[i] + (size_t)row0 * conv_row, 0, conv_row, st));
    }
    CUDA_TRY(cudaMemcpyAsync(e->d_block_table + (size_t)slot * e->bpr, host_pages, (size_t)n_pages * 4, cudaMemcpyHostToDevice, st));
    // positions the slot may occupy: what its pages hold, never more than the engine's tables (rotary table, block-table row)
    const uint32_t limit = n_pages * 16 < e->cfg.max_pos ? n_pages * 16 : e->cfg.max_pos;
    WB_LAUNCH((slot_init_kernel), 1, 1, 0, st, slot_state(e), slot, row0, limit, e->d_temp, e->d_top_k, e->d_top_p, e->d_seed, temp, top_k, top_p, seed);
    WB_LAUNCH_CHECK();
    CUDA_TRY(cudaStreamSynchronize(st));  // host_pages may be pageable memory
    e->h_temp[slot] = temp;
    e->h_limit[slot] = limit;
    return WB_OK;
}

// Per-request draft length (Qwen35Executor::set_spec, qwen.rs:2604-2647): rounds verify min(round k, this value) drafts for the
// slot; 0 makes it a plain decode row inside a speculative round.  Admission resets it to "as many as the round drafts".
extern "C" int32_t wein_b200_engine_set_spec(wein_b200_engine *e, uint32_t slot, uint32_t k, void *stream) {
    WB_CHECK_ARG(e && slot < e->cfg.max_seqs, "engine_set_spec: slot out of range");
    WB_LAUNCH((set_kreq_kernel), 1, 1, 0, (cudaStream_t)stream, e->d_kreq, slot, k);
    WB_LAUNCH_CHECK();
    return WB_OK;
}

// A sequence that does not start at position 0: its first `position` tokens are already in the KV pages it was admitted with
// and its recurrent / conv state row (row 2 * (k_max + 1) * slot of every pool, see wein_b200_engine_buffer) holds the state
// after them -- what a prefix-cache hit restores in the reference (radix snapshots, qwen.rs:3056-3100).  The caller writes
// those buffers, then names the position and the token to feed next.  Call after admit, before the slot's first round.
extern "C" int32_t wein_b200_engine_resume(wein_b200_engine *e, uint32_t slot, uint32_t position, uint32_t pending_token, void *stream) {
    WB_CHECK_ARG(e && slot < e->cfg.max_seqs, "engine_resume: slot out of range");
    WB_CHECK_ARG(position + 1 <= e->h_limit[slot], "engine_resume: position %u leaves no room below the slot's limit %u", position, e->h_limit[slot]);
    WB_CHECK_ARG(pending_token < e->V, "engine_resume: token id %u outside the vocabulary", pending_token);
    WB_LAUNCH((resume_kernel), 1, 1, 0, (cudaStream_t)stream, slot_state(e), slot, position, pending_token);
    WB_LAUNCH_CHECK();
    return WB_OK;
}

// ------------------------------------------------------------------------------------------------ forward passes
static int32_t gemm(Engine *e, const void *a, const void *w, void *c, uint32_t m, uint32_t n, uint32_t k, uint32_t lda, uint32_t ldc, cudaStream_t st) {
    e->launches++;
    return wb_gemm_wt(a, w, c, m, n, k, lda, ldc, e->gemm_scratch, e->gemm_scratch_bytes, e->gemm_path, st);
}

// Full-attention block: projections -> fused q/k norm + rope + KV scatter -> paged verify attention (+ gate) -> o_proj.
static int32_t full_attn_block(Engine *e, const wein_b200_layer_weights &w, void *kp, void *vp, uint32_t T, uint32_t n_spans,
                               uint32_t max_count, uint32_t max_ctx, uint32_t seg_pages, const uint32_t *rope_pos, const uint32_t *kv_pos,
                               const uint32_t *seq_ids, const uint32_t *bt, uint32_t bpr, const uint32_t *row_start,
                               const uint32_t *row_count, uint32_t *status, cudaStream_t st) {
    const wein_b200_model_cfg &c = e->cfg;
    uint32_t H = e->H, qd = c.q_heads * c.head_dim, he = c.kv_heads * c.head_dim;
    if (adjacent(w.qg, w.k, (size_t)2 * qd * H) && adjacent(w.k, w.v, (size_t)he * H)) {
        TRY(gemm(e, e->n1, w.qg, e->proj, T, e->fpn, H, H, e->fpn, st));
    } else {
        TRY(gemm(e, e->n1, w.qg, e->proj, T, 2 * qd, H, H, e->fpn, st));
        TRY(gemm(e, e->n1, w.k, e->proj + 2 * qd, T, he, H, H, e->fpn, st));
        TRY(gemm(e, e->n1, w.v, e->proj + 2 * qd + he, T, he, H, H, e->fpn, st));
    }
    TRY(wb_qk_prep(e->proj, e->fpn, w.qn, w.kn, e->cosv, e->sinv, rope_pos, kv_pos, seq_ids, bt, bpr, e->qh, e->gate, kp, vp, T, c.q_heads,
                   c.kv_heads, c.head_dim, c.rot_dim, c.rms_eps, st));
    float q_scale = 1.0f / sqrtf((float)c.head_dim);
    TRY(wb_attn_verify(e->qh, kp, vp, bt, seq_ids, kv_pos, row_start, row_count, e->gate, e->attn, q_scale, bpr, 16, c.q_heads, c.kv_heads,
                       c.head_dim, n_spans, max_count, max_ctx, seg_pages, e->attn_scratch, e->attn_scratch_bytes, status, e->gemm_path == WB_GEMM_TC, st));
    e->launches += 3;
    TRY(gemm(e, e->attn, w.o, e->o, T, H, qd, qd, H, st));
    return WB_OK;
}

static int32_t mlp_block(Engine *e, const wein_b200_layer_weights &w, uint32_t T, cudaStream_t st) {
    uint32_t H = e->H, II = e->II;
    if (adjacent(w.wg, w.wu, (size_t)II * H)) {
        // gate|up projection with the SwiGLU activation in the epilogue: one launch, no [T, 2*inter] round trip
        e->launches++;
        TRY(wb_gemm_swiglu(e->n2, w.wg, e->m, T, II, H, H, II, e->gemm_scratch, e->gemm_scratch_bytes, e->gemm_path, st));
        TRY(gemm(e, e->m, w.wd, e->d, T, H, II, II, H, st));
        return WB_OK;
    }
    TRY(gemm(e, e->n2, w.wg, e->gu, T, II, H, H, 2 * II, st));
    TRY(gemm(e, e->n2, w.wu, e->gu + II, T, II, H, H, 2 * II, st));
    TRY(wb_silu_mul_rows(e->gu, 2 * II, e->m, T, II, st));
    e->launches++;
    TRY(gemm(e, e->m, w.wd, e->d, T, H, II, II, H, st));
    return WB_OK;
}

// The verify forward (run_forward, qwen.rs:3843-4153) over the T rows described by the step tables.  n_lg rows of
// lg_rows get logits (all T when lg_all).
static int32_t forward(Engine *e, uint32_t T, uint32_t n_spans, uint32_t max_count, uint32_t max_ctx, uint32_t n_lg, bool lg_all, bool lite, cudaStream_t st) {
    const wein_b200_model_cfg &c = e->cfg;
    uint32_t H = e->H;
    TRY(wein_b200_embed(e->d_tok, e->w.embed, e->x, H, T, st));
    TRY(wein_b200_rms_norm_zc(e->x, e->w.layers[0].ln1, e->n1, T, H, c.rms_eps, st));
    e->launches += 2;
    uint32_t li = 0, fi = 0;
    for (uint32_t l = 0; l < c.n_layers; l++) {
        const wein_b200_layer_weights &w = e->w.layers[l];
        if (c.layer_is_full[l]) {
            TRY(full_attn_block(e, w, e->k_pool[fi], e->v_pool[fi], T, n_spans, max_count, max_ctx, e->seg_pages, e->d_pos_rows, e->d_pos_rows,
                                e->d_seq_rows, e->d_block_table, e->bpr, e->d_row_start, e->d_row_count, e->d_status, st));
            fi++;
        } else {
            uint32_t vh = c.lin_v_heads;
            if (adjacent(w.qkv, w.z, (size_t)e->cd * H) && adjacent(w.z, w.a, (size_t)e->vald * H) && adjacent(w.a, w.b, (size_t)vh * H)) {
                TRY(gemm(e, e->n1, w.qkv, e->proj, T, e->lpn, H, H, e->lpn, st));
            } else {
                TRY(gemm(e, e->n1, w.qkv, e->proj, T, e->cd, H, H, e->lpn, st));
                TRY(gemm(e, e->n1, w.z, e->proj + e->cd, T, e->vald, H, H, e->lpn, st));
                TRY(gemm(e, e->n1, w.a, e->proj + e->cd + e->vald, T, vh, H, H, e->lpn, st));
                TRY(gemm(e, e->n1, w.b, e->proj + e->cd + e->vald + vh, T, vh, H, H, e->lpn, st));
            }
            // conv + SiLU + conv rows + l2 norms + gates + chain recurrence + gated norm: one launch per layer
            TRY(wb_gdn_layer(e->proj, e->lpn, w.conv, e->conv_state[li], w.a_log, w.dt_bias, w.norm, e->lin_state[li], c.state_f32, e->normed,
                             e->d_row_start, e->d_row_count, e->d_in_row, e->d_out_base, n_spans, c.lin_k_heads, vh, c.l2_eps, c.rms_eps,
                             lite ? e->lin_log[li] : nullptr, e->gdn_kq, st));
            e->launches += 1;
            TRY(gemm(e, e->normed, w.out, e->o, T, H, e->vald, e->vald, H, st));
            li++;
        }
        TRY(wein_b200_add_norm_zc(e->x, e->o, w.ln2, e->h2, e->n2, T, H, c.rms_eps, st));
        TRY(mlp_block(e, w, T, st));
        bool last = l + 1 == c.n_layers;
        TRY(wein_b200_add_norm_zc(e->h2, e->d, last ? e->w.norm_f : e->w.layers[l + 1].ln1, e->x, last ? e->n2 : e->n1, T, H, c.rms_eps, st));
        e->launches += 2;
    }
    if (n_lg == 0) return WB_OK;
    const bf16_t *src = e->n2;
    if (!lg_all) {
        TRY(wein_b200_embed(e->d_lg_rows, e->n2, e->lg_in, H, n_lg, st));
        e->launches++;
        src = e->lg_in;
    }
    TRY(gemm(e, src, e->w.embed, e->logits, n_lg, e->V, H, H, e->V, st));
    return WB_OK;
}

// Slices per logits row for the two-phase argmax: enough CTAs to cover the SMs several times, long enough slices to stream
static uint32_t am_split(uint32_t rows) { return rows >= 64 ? 8u : (rows >= 16 ? 16u : 32u); }

// Draft step i of the MTP head over n batch rows (run_mtp_forward, qwen.rs:4435-4522).
static int32_t mtp_forward(Engine *e, uint32_t n, uint32_t i, bool sampled, cudaStream_t st) {
    const wein_b200_model_cfg &c = e->cfg;
    uint32_t H = e->H, km = c.k_max;
    const wein_b200_layer_weights &w = e->w.mtp_layer;
    WB_LAUNCH((mtp_prep_kernel), (n + 127) / 128, 128, 0, st, e->d_slots, slot_state(e), e->d_drafts, km, n, i, e->V, c.max_pos, e->d_mtp_tok, e->d_mtp_rope,
                                          e->d_mtp_kvpos);
    WB_LAUNCH_CHECK();
    // hidden: the stashed target hidden of position pos-1 for the first draft, then the head's own normalised output
    TRY(wb_mtp_cat(e->d_mtp_tok, 1, e->w.embed, i == 0 ? e->d_hid : e->n2, i == 0 ? e->d_slots : nullptr, e->w.mtp_pre_e, e->w.mtp_pre_h, e->cat,
                   n, H, c.rms_eps, st));
    TRY(gemm(e, e->cat, e->w.mtp_fc, e->x, n, H, 2 * H, 2 * H, H, st));
    TRY(wein_b200_rms_norm_zc(e->x, w.ln1, e->n1, n, H, c.rms_eps, st));
    e->launches += 3;
    // each batch row is its own one-page chain: clean per round, chain-local KV slots, absolute rotary positions
    TRY(full_attn_block(e, w, e->k_pool[e->n_full], e->v_pool[e->n_full], n, n, 1, 16, 1, e->d_mtp_rope, e->d_mtp_kvpos, e->d_iota, e->d_iota, 1,
                        e->d_iota, e->d_ones, nullptr, st));
    TRY(wein_b200_add_norm_zc(e->x, e->o, w.ln2, e->h2, e->n2, n, H, c.rms_eps, st));
    TRY(mlp_block(e, w, n, st));
    TRY(wein_b200_add_norm_zc(e->h2, e->d, e->w.mtp_norm, e->x, e->n2, n, H, c.rms_eps, st));
    e->launches += 2;
    TRY(gemm(e, e->n2, e->w.embed, e->logits, n, e->V, H, H, e->V, st));
    if (!sampled) {
        const uint32_t split = am_split(n);
        TRY(wein_b200_argmax_partials(e->logits, e->d_iota, e->am_part, e->V, n, split, st));
        TRY(wb_argmax_finish(e->am_part, split, e->d_drafts, km, i, n, st));
        e->launches += 2;
    } else {
        FilterArgs f{};
        f.logits = e->logits; f.rows = nullptr; f.row_seq = e->d_slots; f.rows_per_seq = 1; f.temp = e->d_temp; f.top_k = e->d_top_k; f.top_p = e->d_top_p;
        f.n = e->V; f.s = n; f.out_ids = e->q_ids; f.out_probs = e->q_probs; f.out_n = e->q_n; f.out_mul = km; f.out_off = i;
        f.sample_out = e->d_drafts; f.sample_mul = km; f.sample_off = i; f.seed = e->d_seed; f.round = e->d_round; f.position = i;
        TRY(wb_topk_filter_args(f, st));
        e->launches++;
    }
    return WB_OK;
}

// The draft phase of a round (spec_draft_batch, qwen.rs:2748-2853): k MTP forwards, drafts and their distributions stay on the device.
static int32_t run_draft(Engine *e, uint32_t n, uint32_t k, bool sampled, cudaStream_t st) {
    for (uint32_t i = 0; i < k; i++) TRY(mtp_forward(e, n, i, sampled, st));
    e->launches += k;
    return WB_OK;
}

// Verify forward + acceptance + commit (forward_batch_mixed + spec_finish) over the drafts in the engine's draft buffer.
// caller_nd: per-row draft counts were imported (spec_verify); dry: decide but commit nothing.
static int32_t run_verify(Engine *e, uint32_t n, uint32_t k, bool sampled, uint32_t max_ctx, bool caller_nd, bool dry, cudaEvent_t after_forward,
                          cudaStream_t st) {
    const uint32_t P = k + 1, T = n * P, km = e->cfg.k_max ? e->cfg.k_max : 1;
    WB_LAUNCH((verify_prep_kernel), (n + 127) / 128, 128, 0, st, e->d_slots, slot_state(e), e->d_drafts, km, caller_nd ? e->d_nd_in : nullptr, n, P, e->V,
                                                      e->rows_per_slot, e->P, e->d_tok, e->d_pos_rows, e->d_seq_rows, e->d_row_start, e->d_row_count,
                                                      e->d_in_row, e->d_out_base, e->d_lg_rows, e->d_nd);
    WB_LAUNCH_CHECK();
    e->launches += 1;
    // three positions or more: log the state updates, materialise the accepted state once after acceptance (below)
    const bool lite = P >= 3 && !e->lin_log.empty();
    TRY(forward(e, T, n, P, max_ctx, T, true, lite, st));
    if (after_forward) cudaEventRecord(after_forward, st);
    AcceptArgs a{};
    a.drafts = e->d_drafts; a.draft_stride = km; a.n_drafts = e->d_nd; a.B = n; a.k = k; a.accept_len = e->d_accept_len; a.out_tokens = e->d_out_tokens;
    a.target = e->d_target;
    if (!sampled) {
        const uint32_t split = am_split(T);
        TRY(wein_b200_argmax_partials(e->logits, e->d_lg_rows, e->am_part, e->V, T, split, st));
        a.am_part = (const uint64_t *)e->am_part; a.am_split = split;
    } else {
        FilterArgs f{};
        f.logits = e->logits; f.rows = nullptr; f.row_seq = e->d_seq_rows; f.rows_per_seq = 1; f.temp = e->d_temp; f.top_k = e->d_top_k; f.top_p = e->d_top_p;
        f.n = e->V; f.s = T; f.out_ids = e->p_ids; f.out_probs = e->p_probs; f.out_n = e->p_n; f.out_mul = 1; f.out_off = 0;
        TRY(wb_topk_filter_args(f, st));
        a.p_ids = e->p_ids; a.p_probs = e->p_probs; a.p_n = e->p_n; a.q_ids = e->q_ids; a.q_probs = e->q_probs; a.q_n = e->q_n;
        a.temp = e->d_temp; a.seed = e->d_seed; a.round = e->d_round; a.slot_of = e->d_slots;
    }
    TRY(wb_accept_args(a, st));
    e->launches += 2;
    if (dry) return WB_OK;
    if (lite) {
        TRY(wb_gdn_commit(e->d_state_ptrs, e->d_log_ptrs, e->n_lin, e->cfg.state_f32, e->d_row_start, e->d_row_count, e->d_in_row, e->d_out_base,
                          e->d_accept_len, n, e->cfg.lin_v_heads, st));
        e->launches++;
    }
    WB_LAUNCH((commit_kernel), n, 128, 0, st, e->d_slots, slot_state(e), e->d_accept_len, e->d_row_count, e->d_nd, e->d_out_tokens, e->d_out_base, e->x, P, k, e->H);
    WB_LAUNCH_CHECK();
    e->launches += 1;
    return WB_OK;
}

static int32_t set_slots(Engine *e, uint32_t n, const uint32_t *host_slots, cudaStream_t st, bool force = false) {
    bool same = !force && e->h_slots_cached.size() == n;
    for (uint32_t i = 0; same && i < n; i++) same = e->h_slots_cached[i] == host_slots[i];
    if (same) return WB_OK;
    for (uint32_t i = 0; i < n; i++) {
        WB_CHECK_ARG(host_slots[i] < e->cfg.max_seqs, "slot %u out of range", host_slots[i]);
        for (uint32_t j = 0; j < i; j++) WB_CHECK_ARG(host_slots[j] != host_slots[i], "slot %u listed twice", host_slots[i]);
    }
    CUDA_TRY(cudaStreamSynchronize(st));  // the pinned staging words may still be in flight from an earlier call
    memcpy(e->h_stage, host_slots, (size_t)n * 4);
    CUDA_TRY(cudaMemcpyAsync(e->d_slots, e->h_stage, (size_t)n * 4, cudaMemcpyHostToDevice, st));
    e->h_slots_cached.assign(host_slots, host_slots + n);
    return WB_OK;
}

// What a call runs: the draft phase, the verify phase, or both (one round).
enum { PH_DRAFT = 1, PH_VERIFY = 2, PH_CALLER_ND = 4, PH_DRY = 8 };

static int32_t run_phases(Engine *e, uint32_t n, uint32_t k, bool sampled, uint32_t bucket, uint32_t phases, cudaStream_t st, bool timed) {
    const bool t = timed && e->timing;
    if (t) cudaEventRecord(e->ev[0], st);
    if (phases & PH_DRAFT) TRY(run_draft(e, n, k, sampled, st));
    if (t) cudaEventRecord(e->ev[1], st);
    if (phases & PH_VERIFY) TRY(run_verify(e, n, k, sampled, bucket, (phases & PH_CALLER_ND) != 0, (phases & PH_DRY) != 0, t ? e->ev[2] : nullptr, st));
    if (t) {
        if (!(phases & PH_VERIFY)) cudaEventRecord(e->ev[2], st);
        cudaEventRecord(e->ev[3], st);
        e->ev_pending = true;
    }
    return WB_OK;
}

// Folds the phase events of the last eager round into the totals (spec_timing_ms, qwen.rs:4277-4279); synchronises on them.
static void fold_timing(Engine *e) {
    if (!e->ev_pending) return;
    e->ev_pending = false;
    if (cudaEventSynchronize(e->ev[3]) != cudaSuccess) { cudaGetLastError(); return; }
    for (int i = 0; i < 3; i++) {
        float ms = 0.0f;
        if (cudaEventElapsedTime(&ms, e->ev[i], e->ev[i + 1]) == cudaSuccess) e->ms_phase[i] += ms;
        else cudaGetLastError();
    }
}

static uint32_t ctx_bucket(const Engine *e, uint32_t ctx_bound) {
    // the context bound only sizes the attention grid: round it up to a bucket so graphs are reused
    uint32_t bucket = 256;
    while (bucket < ctx_bound) bucket *= 2;
    if (bucket > e->bpr * 16) bucket = e->bpr * 16;
    return bucket;
}

// Captures (once) and returns the graph of the given phases; graph == nullptr only on error.
static int32_t get_graph(Engine *e, uint32_t n, uint32_t k, bool sampled, uint32_t bucket, uint32_t phases, cudaStream_t st,
                         std::pair<cudaGraphExec_t, uint32_t> **out) {
    auto key = std::make_tuple(phases, n, k, (uint32_t)sampled, bucket, 0u);
    auto it = e->graphs.find(key);
    if (it == e->graphs.end()) {
        cudaGraph_t g = nullptr;
        e->launches = 0;
        CUDA_TRY(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
        int32_t rc = run_phases(e, n, k, sampled, bucket, phases, st, false);
        cudaError_t ce = cudaStreamEndCapture(st, &g);
        if (rc != WB_OK) { if (g) cudaGraphDestroy(g); return rc; }
        if (ce != cudaSuccess) { wb_set_error("engine: stream capture failed: %s", cudaGetErrorString(ce)); return WB_ERR_CUDA; }
        cudaGraphExec_t ge = nullptr;
        ce = cudaGraphInstantiate(&ge, g, 0);
        cudaGraphDestroy(g);
        if (ce != cudaSuccess) { wb_set_error("engine: graph instantiation failed: %s", cudaGetErrorString(ce)); return WB_ERR_CUDA; }
        cudaGraphUpload(ge, st);   // so that the first replay does not allocate either
        cudaGetLastError();
        it = e->graphs.emplace(key, std::make_pair(ge, e->launches)).first;
    }
    *out = &it->second;
    return WB_OK;
}

static int32_t check_round_args(Engine *e, const char *who, uint32_t n, const uint32_t *host_slots, uint32_t k, uint32_t ctx_bound, bool graph, cudaStream_t st) {
    WB_CHECK_ARG(e && host_slots && n >= 1 && n <= e->cfg.max_seqs, "%s: batch of %u outside 1..max_seqs", who, n);
    WB_CHECK_ARG(k <= e->cfg.k_max, "%s: k = %u exceeds k_max = %u", who, k, e->cfg.k_max);
    WB_CHECK_ARG(ctx_bound >= 1 && ctx_bound <= e->cfg.max_pos, "%s: ctx_bound %u outside 1..max_pos", who, ctx_bound);
    WB_CHECK_ARG(!graph || st != nullptr, "%s: a CUDA graph cannot be captured on the default stream; pass a created stream", who);
    return WB_OK;
}

static bool any_sampled(const Engine *e, uint32_t n, const uint32_t *host_slots) {
    bool sampled = false;
    for (uint32_t i = 0; i < n; i++) sampled |= e->h_temp[host_slots[i]] > 0.0f;
    return sampled;
}

static int32_t launch_phases(Engine *e, uint32_t n, uint32_t k, bool sampled, uint32_t bucket, uint32_t phases, bool graph, cudaStream_t st) {
    if (!graph) {
        fold_timing(e);
        e->launches = 0;
        TRY(run_phases(e, n, k, sampled, bucket, phases, st, true));
        e->last_launches = e->launches;
        return WB_OK;
    }
    std::pair<cudaGraphExec_t, uint32_t> *g = nullptr;
    TRY(get_graph(e, n, k, sampled, bucket, phases, st, &g));
    e->last_launches = g->second;
    CUDA_TRY(cudaGraphLaunch(g->first, st));
    return WB_OK;
}

extern "C" int32_t wein_b200_engine_spec_step(wein_b200_engine *e, uint32_t n, const uint32_t *host_slots, uint32_t k, uint32_t ctx_bound,
                                              uint32_t use_graph, void *stream) {
    cudaStream_t st = (cudaStream_t)stream;
    TRY(check_round_args(e, "spec_step", n, host_slots, k, ctx_bound, (use_graph & 1u) != 0, st));
    WB_CHECK_ARG(k == 0 || e->cfg.has_mtp, "spec_step: drafting needs the MTP head");
    TRY(set_slots(e, n, host_slots, st, (use_graph & 2u) != 0));
    e->last_n = n; e->last_P = k + 1;
    return launch_phases(e, n, k, any_sampled(e, n, host_slots), ctx_bucket(e, ctx_bound), PH_DRAFT | PH_VERIFY, (use_graph & 1u) != 0, st);
}

// The draft phase alone (Qwen35Executor::spec_draft_batch, qwen.rs:2748): k MTP forwards for the listed slots; drafts_out
// (optional, device, [n, k]) receives the draft tokens, which also stay in the engine for a following spec_verify.
__global__ void export_drafts_kernel(const uint32_t *drafts, uint32_t k_max, uint32_t k, uint32_t *out) {
    PDL_ENTRY();
    if (threadIdx.x < k) out[blockIdx.x * k + threadIdx.x] = drafts[blockIdx.x * k_max + threadIdx.x];
}
extern "C" int32_t wein_b200_engine_draft(wein_b200_engine *e, uint32_t n, const uint32_t *host_slots, uint32_t k, void *drafts_out,
                                          uint32_t use_graph, void *stream) {
    cudaStream_t st = (cudaStream_t)stream;
    TRY(check_round_args(e, "engine_draft", n, host_slots, k, 1, (use_graph & 1u) != 0, st));
    WB_CHECK_ARG(k >= 1 && e->cfg.has_mtp, "engine_draft: needs k >= 1 and the MTP head");
    TRY(set_slots(e, n, host_slots, st, (use_graph & 2u) != 0));
    TRY(launch_phases(e, n, k, any_sampled(e, n, host_slots), 0, PH_DRAFT, (use_graph & 1u) != 0, st));
    if (drafts_out) {
        WB_LAUNCH((export_drafts_kernel), n, 32, 0, st, e->d_drafts, e->cfg.k_max, k, (uint32_t *)drafts_out);
        WB_LAUNCH_CHECK();
    }
    return WB_OK;
}

// Verify + accept + commit with the caller's drafts (Qwen35Executor::spec_verify / spec_commit_batch, qwen.rs:2261-2303).
extern "C" int32_t wein_b200_engine_spec_verify(wein_b200_engine *e, uint32_t n, const uint32_t *host_slots, uint32_t k, const void *drafts,
                                                const void *n_drafts, const void *q_ids, const void *q_probs, const void *q_n,
                                                uint32_t ctx_bound, uint32_t flags, void *stream) {
    cudaStream_t st = (cudaStream_t)stream;
    const bool graph = (flags & WEIN_B200_VERIFY_GRAPH) != 0, dry = (flags & WEIN_B200_VERIFY_DRY_RUN) != 0;
    TRY(check_round_args(e, "spec_verify", n, host_slots, k, ctx_bound, graph, st));
    WB_CHECK_ARG(k == 0 || drafts || (flags & WEIN_B200_VERIFY_ENGINE_DRAFTS), "spec_verify: drafts are required for k > 0");
    WB_CHECK_ARG((q_ids == nullptr) == (q_probs == nullptr) && (q_ids == nullptr) == (q_n == nullptr), "spec_verify: q_ids, q_probs and q_n go together");
    TRY(set_slots(e, n, host_slots, st, (flags & WEIN_B200_VERIFY_FORCE_SLOTS) != 0));
    e->last_n = n; e->last_P = k + 1;
    uint32_t phases = PH_VERIFY | (dry ? PH_DRY : 0u);
    if (k && !(flags & WEIN_B200_VERIFY_ENGINE_DRAFTS)) {
        // outside the graph: the caller's pointers may change from call to call
        WB_LAUNCH((import_drafts_kernel), dim3(n, k), 64, 0, st, (const uint32_t *)drafts, (const uint32_t *)n_drafts, (const uint32_t *)q_ids,
                                                   (const float *)q_probs, (const uint32_t *)q_n, n, k, e->cfg.k_max, e->d_drafts, e->d_nd_in,
                                                   e->q_ids, e->q_probs, e->q_n);
        WB_LAUNCH_CHECK();
        phases |= PH_CALLER_ND;
    }
    return launch_phases(e, n, k, any_sampled(e, n, host_slots), ctx_bucket(e, ctx_bound), phases, graph, st);
}

// Everything a later call with the same (n, k, sampling mode, context bucket) would otherwise do lazily: capture and
// instantiate its graphs (the reference warms its graphs at open_graph, qwen.rs:1994-2034).  `what` = bit 0: spec_step,
// bit 1: spec_verify, bit 2: spec_verify as a dry run, bit 3: engine_draft.  The slots named must be admitted.
extern "C" int32_t wein_b200_engine_warm(wein_b200_engine *e, uint32_t n, const uint32_t *host_slots, uint32_t k, uint32_t ctx_bound,
                                         uint32_t what, void *stream) {
    cudaStream_t st = (cudaStream_t)stream;
    TRY(check_round_args(e, "engine_warm", n, host_slots, k, ctx_bound, true, st));
    TRY(set_slots(e, n, host_slots, st));
    const bool sampled = any_sampled(e, n, host_slots);
    const uint32_t bucket = ctx_bucket(e, ctx_bound);
    std::pair<cudaGraphExec_t, uint32_t> *g = nullptr;
    if ((what & 1u) && (k == 0 || e->cfg.has_mtp)) TRY(get_graph(e, n, k, sampled, bucket, PH_DRAFT | PH_VERIFY, st, &g));
    if (what & 2u) { TRY(get_graph(e, n, k, sampled, bucket, PH_VERIFY | (k ? PH_CALLER_ND : 0u), st, &g)); TRY(get_graph(e, n, k, sampled, bucket, PH_VERIFY, st, &g)); }
    if (what & 4u) TRY(get_graph(e, n, k, sampled, bucket, PH_VERIFY | PH_DRY | (k ? PH_CALLER_ND : 0u), st, &g));
    if ((what & 8u) && k && e->cfg.has_mtp) TRY(get_graph(e, n, k, sampled, 0, PH_DRAFT, st, &g));
    return WB_OK;
}

extern "C" int32_t wein_b200_engine_prefill(wein_b200_engine *e, uint32_t n, const uint32_t *host_slots, const uint32_t *host_tokens,
                                            const uint32_t *host_lens, void *stream) {
    WB_CHECK_ARG(e && host_slots && host_tokens && host_lens && n >= 1 && n <= e->cfg.max_seqs, "prefill: bad batch");
    cudaStream_t st = (cudaStream_t)stream;
    TRY(set_slots(e, n, host_slots, st));
    // where every slot stands now (a slot may be prefilled again, or after rounds): sizes the attention grid and the limit check
    std::vector<uint32_t> pos0(n, 0);
    CUDA_TRY(cudaStreamSynchronize(st));
    for (uint32_t i = 0; i < n; i++) CUDA_TRY(cudaMemcpy(&pos0[i], e->d_pos + host_slots[i], 4, cudaMemcpyDeviceToHost));
    std::vector<uint64_t> off(n + 1, 0);
    uint32_t max_len = 0;
    bool sampled = false;
    for (uint32_t i = 0; i < n; i++) {
        WB_CHECK_ARG(host_lens[i] >= 1, "prefill: empty prompt for slot %u", host_slots[i]);
        if ((uint64_t)pos0[i] + host_lens[i] + 1 > e->h_limit[host_slots[i]]) {
            wb_set_error("prefill: slot %u at position %u cannot take %u more tokens (limit %u from its admitted pages)", host_slots[i], pos0[i],
                         host_lens[i], e->h_limit[host_slots[i]]);
            return WB_ERR_CAPACITY;
        }
        off[i + 1] = off[i] + host_lens[i];
        max_len = host_lens[i] > max_len ? host_lens[i] : max_len;
        sampled |= e->h_temp[host_slots[i]] > 0.0f;
    }
    for (uint64_t t = 0; t < off[n]; t++) WB_CHECK_ARG(host_tokens[t] < e->V, "prefill: token id %u outside the vocabulary", host_tokens[t]);
    const uint32_t P = e->P;
    std::vector<uint32_t> done(n, 0);
    uint32_t *h_cnt = e->h_stage, *h_last = e->h_stage + n, *h_tok = e->h_stage + 2 * n;
    for (uint32_t base = 0; base < max_len; base += P) {
        uint32_t T = 0, n_lg = 0, max_ctx = 1;
        CUDA_TRY(cudaStreamSynchronize(st));
        for (uint32_t i = 0; i < n; i++) {
            uint32_t rem = host_lens[i] - done[i], c = rem < P ? rem : P;
            h_cnt[i] = c;
            h_last[i] = (c > 0 && c == rem) ? 1u : 0u;
            n_lg += h_last[i];
            for (uint32_t j = 0; j < c; j++) h_tok[T++] = host_tokens[off[i] + done[i] + j];
            done[i] += c;
            if (c && pos0[i] + done[i] > max_ctx) max_ctx = pos0[i] + done[i];
        }
        uint32_t *h_lgslot = h_tok + T;
        for (uint32_t i = 0, q = 0; i < n; i++) if (h_last[i]) h_lgslot[q++] = host_slots[i];
        if (n_lg) CUDA_TRY(cudaMemcpyAsync(e->d_mtp_tok, h_lgslot, (size_t)n_lg * 4, cudaMemcpyHostToDevice, st));
        CUDA_TRY(cudaMemcpyAsync(e->d_cnt_in, h_cnt, (size_t)n * 4, cudaMemcpyHostToDevice, st));
        CUDA_TRY(cudaMemcpyAsync(e->d_last_in, h_last, (size_t)n * 4, cudaMemcpyHostToDevice, st));
        CUDA_TRY(cudaMemcpyAsync(e->d_tok_in, h_tok, (size_t)T * 4, cudaMemcpyHostToDevice, st));
        WB_LAUNCH((prefill_prep_kernel), 1, 1, 0, st, e->d_slots, slot_state(e), e->d_cnt_in, e->d_tok_in, e->d_last_in, n, e->rows_per_slot, e->P, e->d_tok,
                                             e->d_pos_rows, e->d_seq_rows, e->d_row_start, e->d_row_count, e->d_in_row, e->d_out_base,
                                             e->d_lg_rows, e->d_lg_of);
        WB_LAUNCH_CHECK();
        if (max_ctx > e->bpr * 16) max_ctx = e->bpr * 16;
        TRY(forward(e, T, n, P, max_ctx, n_lg, false, false, st));
        if (n_lg > 0) {
            if (!sampled) {
                const uint32_t split = am_split(n_lg);
                TRY(wein_b200_argmax_partials(e->logits, e->d_iota, e->am_part, e->V, n_lg, split, st));
                TRY(wb_argmax_finish(e->am_part, split, e->d_first_tok, 1, 0, n_lg, st));
            } else {
                // the first token of a sequence: drawn from the filtered distribution of the last prompt position
                FilterArgs f{};
                f.logits = e->logits; f.rows = nullptr; f.rows_per_seq = 1; f.temp = e->d_temp; f.top_k = e->d_top_k; f.top_p = e->d_top_p;
                f.n = e->V; f.s = n_lg; f.out_ids = e->p_ids; f.out_probs = e->p_probs; f.out_n = e->p_n; f.out_mul = 1; f.out_off = 0;
                f.sample_out = e->d_first_tok; f.sample_mul = 1; f.sample_off = 0; f.seed = e->d_seed; f.round = e->d_round; f.position = 0;
                f.row_seq = e->d_mtp_tok;  // slot of each finishing sequence, uploaded with the chunk tables
                TRY(wb_topk_filter_args(f, st));
            }
        }
        WB_LAUNCH((prefill_commit_kernel), n, 128, 0, st, e->d_slots, slot_state(e), e->d_cnt_in, e->d_row_start, e->d_out_base, e->d_lg_of, e->d_first_tok,
                                                e->x, e->H);
        WB_LAUNCH_CHECK();
    }
    CUDA_TRY(cudaStreamSynchronize(st));
    return WB_OK;
}

// One readback for the whole batch of the most recent round: host_out [n, 4 + k_max + 1] = per batch row the accept
// length a, the position, the tokens emitted since admission, the round's a+1 tokens (unused words 0xFFFFFFFF) and the slot's
// status word.  One small kernel, one copy to pinned memory, one synchronisation.
extern "C" int32_t wein_b200_engine_read_round(wein_b200_engine *e, uint32_t *host_out, uint32_t host_words, void *stream) {
    WB_CHECK_ARG(e && host_out, "engine_read_round: null pointer");
    WB_CHECK_ARG(e->last_n > 0, "engine_read_round: no round has run yet");
    const uint32_t n = e->last_n, stride = 4 + e->P;
    WB_CHECK_ARG(host_words >= n * stride, "engine_read_round: %u words given, %u needed", host_words, n * stride);
    cudaStream_t st = (cudaStream_t)stream;
    WB_LAUNCH((round_pack_kernel), (n + 127) / 128, 128, 0, st, e->d_slots, slot_state(e), e->d_accept_len, e->d_row_count, e->d_out_tokens, n, e->last_P, e->P,
                                            e->d_pack);
    WB_LAUNCH_CHECK();
    CUDA_TRY(cudaMemcpyAsync(e->h_pack, e->d_pack, (size_t)n * stride * 4, cudaMemcpyDeviceToHost, st));
    CUDA_TRY(cudaStreamSynchronize(st));
    memcpy(host_out, e->h_pack, (size_t)n * stride * 4);
    return WB_OK;
}

extern "C" int32_t wein_b200_engine_read(wein_b200_engine *e, uint32_t slot, uint32_t *host_tokens, uint32_t cap, uint32_t *host_n_tokens,
                                         uint32_t *host_pos, uint64_t *host_stats3, void *stream) {
    WB_CHECK_ARG(e && slot < e->cfg.max_seqs, "engine_read: slot out of range");
    cudaStream_t st = (cudaStream_t)stream;
    CUDA_TRY(cudaStreamSynchronize(st));
    uint32_t oc = 0, pos = 0;
    CUDA_TRY(cudaMemcpy(&oc, e->d_out_count + slot, 4, cudaMemcpyDeviceToHost));
    CUDA_TRY(cudaMemcpy(&pos, e->d_pos + slot, 4, cudaMemcpyDeviceToHost));
    if (host_n_tokens) *host_n_tokens = oc;
    if (host_pos) *host_pos = pos;
    if (host_stats3) CUDA_TRY(cudaMemcpy(host_stats3, e->d_stats + (size_t)slot * STATS_WORDS, 24, cudaMemcpyDeviceToHost));
    if (host_tokens && cap) {
        // the most recent min(cap, emitted, ring size) tokens, oldest first
        uint32_t nread = oc < cap ? oc : cap;
        if (nread > RING_CAP) nread = RING_CAP;
        uint32_t start = (oc - nread) % RING_CAP, first = nread < RING_CAP - start ? nread : RING_CAP - start;
        const uint32_t *ring = e->d_ring + (size_t)slot * RING_CAP;
        if (first) CUDA_TRY(cudaMemcpy(host_tokens, ring + start, (size_t)first * 4, cudaMemcpyDeviceToHost));
        if (nread > first) CUDA_TRY(cudaMemcpy(host_tokens + first, ring, (size_t)(nread - first) * 4, cudaMemcpyDeviceToHost));
    }
    return WB_OK;
}

// The speculation counters of a slot (spec_stats / spec_k_stats of the reference, qwen.rs:4257-4259, :2670), WEIN_B200_STATS_WORDS
// words: rounds, drafts, accepted, fallbacks, draft-length switches, rounds by draft count [8], rounds by accept length [9],
// the last draft count, one spare.  Synchronises the stream.
extern "C" int32_t wein_b200_engine_stats(wein_b200_engine *e, uint32_t slot, uint64_t *host_stats, void *stream) {
    WB_CHECK_ARG(e && slot < e->cfg.max_seqs && host_stats, "engine_stats: bad argument");
    CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
    CUDA_TRY(cudaMemcpy(host_stats, e->d_stats + (size_t)slot * STATS_WORDS, STATS_WORDS * 8, cudaMemcpyDeviceToHost));
    return WB_OK;
}

// Device status word of a slot (WEIN_B200_STATUS_* bits); clear != 0 resets it after the read.  Synchronises the stream.
extern "C" int32_t wein_b200_engine_status(wein_b200_engine *e, uint32_t slot, uint32_t *host_status, uint32_t clear, void *stream) {
    WB_CHECK_ARG(e && slot < e->cfg.max_seqs && host_status, "engine_status: bad argument");
    cudaStream_t st = (cudaStream_t)stream;
    CUDA_TRY(cudaStreamSynchronize(st));
    CUDA_TRY(cudaMemcpy(host_status, e->d_status + slot, 4, cudaMemcpyDeviceToHost));
    if (clear) {
        WB_LAUNCH((clear_status_kernel), 1, 1, 0, st, e->d_status, slot);
        WB_LAUNCH_CHECK();
    }
    return WB_OK;
}

// Phase timers (spec_timing_ms of the reference, qwen.rs:4277-4279): with on != 0, rounds run eagerly (use_graph = 0) record
// events around the draft phase, the verify forward and acceptance + commit; host_ms3 (optional) receives the totals in
// milliseconds since the timers were last switched on.  Graph replays are not broken down.
extern "C" int32_t wein_b200_engine_timing(wein_b200_engine *e, uint32_t on, double *host_ms3) {
    WB_CHECK_ARG(e != nullptr, "engine_timing: null engine");
    fold_timing(e);
    if (host_ms3) for (int i = 0; i < 3; i++) host_ms3[i] = e->ms_phase[i];
    if (on && !e->timing) for (int i = 0; i < 3; i++) e->ms_phase[i] = 0.0;
    e->timing = on != 0;
    return WB_OK;
}
