"""GPU parity of the tolerance-class kernels: verify attention and the skinny GEMM.

Tolerances are the reference's own: online-softmax attention rel2 <= 3e-3, peak <= 1.5e-2
(crates/wein-kernel/tests/ops_m0.rs:968-977); GEMM |got - ref| <= max(2^-7 |ref|, 2^-11) against an f64
product (crates/wein-kernel/tests/gemm.rs:11)."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests.gpu_util import dev, norm_err, rand_bf16, u16

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from inferulm_b200 import ops as o
    return o


def test_paged_attn_golden_within_online_tolerance(ops, golden):
    g = golden
    tokens = g["paged_attn.seq_ids"].size
    out = torch.zeros(g["paged_attn.out"].size, dtype=torch.int16, device="cuda")
    kvh, hd = int(g["paged_attn.kv_heads"]), int(g["paged_attn.head_dim"])
    scratch = torch.zeros(ops.attn_scratch_bytes(tokens, kvh, hd, 16) // 4, dtype=torch.float32, device="cuda")
    ops.paged_attn(dev(g["paged_attn.q"]), dev(g["paged_attn.k_cache"]), dev(g["paged_attn.v_cache"]),
                   dev(g["paged_attn.block_table"]), dev(g["paged_attn.seq_ids"]), dev(g["paged_attn.positions"]), out,
                   float(g["paged_attn.q_scale"]), int(g["paged_attn.bpr"]), int(g["paged_attn.block_size"]),
                   int(g["paged_attn.q_heads"]), kvh, hd, tokens, scratch)
    rel2, peak = norm_err(orc.bf16_to_f32(u16(out)), orc.bf16_to_f32(g["paged_attn.out"]))
    assert rel2 <= 3e-3 and peak <= 1.5e-2, (rel2, peak)


def _attn_case(rs, ctx_lens, cnt, q_heads=16, kv_heads=4, hd=256, garbage=True):
    nseq = len(ctx_lens)
    he = kv_heads * hd
    bpr = max((l + cnt + 15) // 16 for l in ctx_lens) + 1
    n_pages = nseq * bpr + 3
    perm = rs.permutation(n_pages)
    bt = perm[: nseq * bpr].astype(np.uint32).reshape(nseq, bpr)
    k_pool, v_pool = rand_bf16(rs, n_pages * 16 * he), rand_bf16(rs, n_pages * 16 * he)
    if garbage:  # slots past each sequence's end hold NaN: they must never reach the output
        kp, vp = k_pool.reshape(n_pages, 16, he), v_pool.reshape(n_pages, 16, he)
        for s, l in enumerate(ctx_lens):
            end = l + cnt
            pg, off = end // 16, end % 16
            if pg < bpr:
                kp[bt[s, pg], off:] = 0x7FC0
                vp[bt[s, pg], off:] = 0x7FC0
    seq_ids = np.repeat(np.arange(nseq), cnt).astype(np.uint32)
    positions = np.concatenate([np.arange(l, l + cnt) for l in ctx_lens]).astype(np.uint32)
    q = rand_bf16(rs, nseq * cnt * q_heads * hd)
    return dict(q=q, k=k_pool, v=v_pool, bt=bt.reshape(-1), seq_ids=seq_ids, positions=positions, bpr=bpr,
                row_start=(np.arange(nseq) * cnt).astype(np.uint32), row_count=np.full(nseq, cnt, np.uint32))


def _run_attn(ops, c, n_spans, cnt, max_ctx, seg_pages, gate=None, spans=None):
    out = torch.zeros(c["q"].size, dtype=torch.int16, device="cuda")
    max_segs = ((max_ctx + 15) // 16 + seg_pages - 1) // seg_pages
    scratch = torch.zeros(ops.attn_scratch_bytes(n_spans, 4, 256, max_segs) // 4, dtype=torch.float32, device="cuda")
    rs_, rc_ = (c["row_start"], c["row_count"]) if spans is None else spans
    ops.attn_verify(dev(c["q"]), dev(c["k"]), dev(c["v"]), dev(c["bt"]), dev(c["seq_ids"]), dev(c["positions"]), dev(rs_),
                    dev(rc_), dev(gate) if gate is not None else None, out, 1.0 / 16.0, c["bpr"], 16, 16, 4, 256, n_spans, cnt,
                    max_ctx, seg_pages, scratch)
    return u16(out)


@pytest.mark.parametrize("ctx_lens,cnt,seg_pages", [([508], 4, 4), ([508], 4, 64), ([0, 3, 17, 300], 4, 2), ([1100, 40], 5, 4),
                                                    ([2000], 8, 16), ([15, 16, 31], 1, 1)])
def test_attn_verify_vs_oracle(ops, ctx_lens, cnt, seg_pages):
    """The unit shape of the reference's first benchmark configuration (16 q / 4 kv heads, d = 256, 16-token pages, positions 508..511) and ragged
    variants: empty context, page boundaries, two m-tiles (k = 4 and 7 drafts), one or many segments."""
    rs = np.random.default_rng(len(ctx_lens) * 100 + cnt)
    c = _attn_case(rs, ctx_lens, cnt)
    want = orc.paged_attn(c["q"], c["k"], c["v"], c["bt"], c["seq_ids"], c["positions"], 1.0 / 16.0, c["bpr"], 16, 16, 4, 256,
                          threads=8)
    got = orc.bf16_to_f32(_run_attn(ops, c, len(ctx_lens), cnt, max(ctx_lens) + cnt, seg_pages))
    assert np.isfinite(got).all()
    rel2, peak = norm_err(got, orc.bf16_to_f32(want))
    assert rel2 <= 3e-3 and peak <= 1.5e-2, (rel2, peak)
    g2 = got.reshape(-1, 256); w2 = orc.bf16_to_f32(want).reshape(-1, 256)
    row_rel = np.sqrt(((g2 - w2) ** 2).sum(1) / (w2 ** 2).sum(1)).max()
    assert row_rel <= 1e-2, row_rel  # worst row, as the reference's per-row gate


def test_attn_verify_batch_shape_invariance_and_gate(ops):
    """Row (seq, pos) gives the same bits whether it is verified inside a k+1-row chain, alone as a one-token
    step, next to other chains, or with a larger grid bound (o41 / o42 of the reference's kernel tests: the same
    row gives the same bits whatever its batch neighbours).  The fused output gate equals sigmul."""
    rs = np.random.default_rng(77)
    for cnt in (4, 7):
        c = _attn_case(rs, [600, 90, 1500], cnt)
        full = _run_attn(ops, c, 3, cnt, 1500 + cnt, 4)
        n = 16 * 256
        # each row alone (chains of length 1), generous grid bound
        T = 3 * cnt
        single = _run_attn(ops, c, T, 1, c["bpr"] * 16, 4, spans=(np.arange(T, dtype=np.uint32), np.ones(T, np.uint32)))
        assert np.array_equal(full, single), cnt
        # one chain alone
        one = _run_attn(ops, c, 1, cnt, 1500 + cnt, 4, spans=(c["row_start"][1:2], c["row_count"][1:2]))
        assert np.array_equal(one[cnt * n:2 * cnt * n], full[cnt * n:2 * cnt * n])
        # a short chain next to long ones (the second m-tile of its CTA has no rows)
        short = _run_attn(ops, c, 3, cnt, 1500 + cnt, 4, spans=(c["row_start"], np.array([cnt, 2, cnt], np.uint32)))
        assert np.array_equal(short[:cnt * n], full[:cnt * n]) and np.array_equal(short[2 * cnt * n:], full[2 * cnt * n:])
        assert np.array_equal(short[cnt * n:(cnt + 2) * n], full[cnt * n:(cnt + 2) * n])
        gate = rand_bf16(rs, c["q"].size, 2.0)
        gated = _run_attn(ops, c, 3, cnt, 1500 + cnt, 4, gate=gate)
        assert np.array_equal(gated, orc.sigmul(full, gate))


GEMM_SHAPES = [(4, 12352, 2560), (1, 2560, 4096), (4, 2560, 9216), (8, 18432, 2560), (5, 10240, 2560), (3, 2560, 5120),
               (20, 2560, 4096), (32, 1024, 2560), (4, 40, 64), (40, 2560, 2560), (128, 4096, 2560)]


@pytest.mark.parametrize("m,n,k", GEMM_SHAPES)
def test_gemm_wt_tolerance(ops, m, n, k):
    rs = np.random.default_rng(m * 7 + n + k)
    a, w = rand_bf16(rs, m * k, 1.0), rand_bf16(rs, n * k, 0.05)
    ref = (orc.bf16_to_f32(a).reshape(m, k).astype(np.float64) @ orc.bf16_to_f32(w).reshape(n, k).astype(np.float64).T).reshape(-1)
    scratch = torch.zeros(ops.gemm_scratch_bytes(n) // 4, dtype=torch.int32, device="cuda")
    for sc in (None, scratch):
        c = torch.zeros(m * n, dtype=torch.int16, device="cuda")
        ops.gemm_wt(dev(a), dev(w), c, m, n, k, sc)
        got = orc.bf16_to_f32(u16(c)).astype(np.float64)
        tol = np.maximum(2.0 ** -7 * np.abs(ref), 2.0 ** -11)
        assert (np.abs(got - ref) <= tol).all(), float((np.abs(got - ref) / tol).max())
    assert int(scratch[:4096].abs().sum()) == 0  # tile counters re-armed


def test_gemm_wt_small_oracle_and_batch_invariance(ops):
    """Against the oracle's own f64 GEMM on a small case; and a row's bits do not depend on the batch:
    row 0 of an m = 4 product equals the m = 1 product (verify row == plain decode row)."""
    rs = np.random.default_rng(5)
    m, n, k = 4, 320, 2560
    a, w = rand_bf16(rs, m * k, 1.0), rand_bf16(rs, n * k, 0.05)
    ref = orc.gemm_wt(a, w, m, n, k, threads=8)
    c4 = torch.zeros(m * n, dtype=torch.int16, device="cuda")
    ops.gemm_wt(dev(a), dev(w), c4, m, n, k)
    got = orc.bf16_to_f32(u16(c4)).astype(np.float64)
    assert (np.abs(got - ref) <= np.maximum(2.0 ** -7 * np.abs(ref), 2.0 ** -11)).all()
    for mm in (1, 9, 17, 32):
        rows = np.concatenate([a[:k]] + [rand_bf16(rs, k) for _ in range(mm - 1)]) if mm > 1 else a[:k]
        c = torch.zeros(mm * n, dtype=torch.int16, device="cuda")
        ops.gemm_wt(dev(rows), dev(w), c, mm, n, k)
        assert np.array_equal(u16(c)[:n], u16(c4)[:n]), mm


TC_SHAPES = [(40, 12352, 2560), (128, 2560, 4096), (33, 2560, 9216), (160, 2560, 5120), (128, 10240, 2560), (4, 12352, 2560),
             (1, 2560, 4096), (16, 40, 64), (17, 520, 576), (49, 100, 128), (256, 1000, 512), (300, 384, 320), (128, 151936, 2560)]


@pytest.mark.parametrize("m,n,k", TC_SHAPES)
def test_tensor_memory_gemm_tolerance_and_batch_invariance(ops, m, n, k):
    """The tcgen05 kernel (weights as the M operand, accumulators in tensor memory, tensor-map copies, k split over a cluster)
    against the f64 product within the reference's GEMM criterion (crates/wein-kernel/tests/gemm.rs:11): the model's shapes,
    ragged n and k (zero-filled boxes), m above one 256-row chunk.  A row's bits do not depend on the rows it is batched
    with: row 0 alone, and rows 0..7 with other neighbours, give the same words."""
    rs = np.random.default_rng(m * 11 + n + k)
    a, w = rand_bf16(rs, m * k, 1.0), rand_bf16(rs, n * k, 0.05)
    wd = dev(w)
    c = torch.full((m * n,), 0x4100, dtype=torch.int16, device="cuda")
    ops.gemm_wt(dev(a), wd, c, m, n, k, tc=True)
    got = orc.bf16_to_f32(u16(c)).astype(np.float64).reshape(m, n)
    af, wf = orc.bf16_to_f32(a).reshape(m, k).astype(np.float64), orc.bf16_to_f32(w).reshape(n, k).astype(np.float64)
    ref = af @ wf.T
    tol = np.maximum(2.0 ** -7 * np.abs(ref), 2.0 ** -11)
    assert (np.abs(got - ref) <= tol).all(), float((np.abs(got - ref) / tol).max())
    c1 = torch.zeros(n, dtype=torch.int16, device="cuda")
    ops.gemm_wt(dev(a[:k]), wd, c1, 1, n, k, tc=True)
    assert np.array_equal(u16(c1), u16(c)[:n])
    if m >= 8:
        mm = 24
        rows = np.concatenate([a[: 8 * k], rand_bf16(rs, (mm - 8) * k)])
        c2 = torch.zeros(mm * n, dtype=torch.int16, device="cuda")
        ops.gemm_wt(dev(rows), wd, c2, mm, n, k, tc=True)
        assert np.array_equal(u16(c2)[: 8 * n], u16(c)[: 8 * n])
    assert ops.gemm_wait_timeouts() == 0


def test_tensor_memory_gemm_split_depends_on_the_weight_shape_only(ops):
    """The k split (cluster size) fixes the order in which a row's partial sums are added, so it must come from (n, k) and
    the device alone: the same for every row count, and for the plain and SwiGLU forms of a shape family."""
    for n, k in [(2560, 9216), (2560, 4096), (12352, 2560), (10240, 2560), (151936, 2560), (2560, 5120), (1544, 512)]:
        splits = {ops.gemm_plan(m, n, k)[1] for m in (1, 8, 31, 32, 33, 40, 128, 160, 256, 300)}
        assert len(splits) == 1, (n, k, splits)
    assert len({ops.gemm_plan(m, 9216, 2560, True)[1] for m in (1, 4, 40, 128, 256)}) == 1


@pytest.mark.parametrize("m,inter,k", [(128, 9216, 2560), (40, 9216, 2560), (8, 9216, 2560), (1, 1000, 576), (50, 1024, 512)])
def test_tensor_memory_gemm_swiglu_matches_operator_chain(ops, m, inter, k):
    """gate|up + SwiGLU through the tensor-memory kernel == its own plain products followed by the oracle's silu_mul, bit for bit."""
    rs = np.random.default_rng(m + inter + k)
    a, w = rand_bf16(rs, m * k, 1.0), rand_bf16(rs, 2 * inter * k, 0.05)
    ad, wd = dev(a), dev(w)
    gu = torch.zeros(m * 2 * inter, dtype=torch.int16, device="cuda")
    ops.gemm_wt(ad, wd, gu, m, 2 * inter, k, tc=True)
    guh = u16(gu).reshape(m, 2 * inter)
    want = orc.silu_mul(np.ascontiguousarray(guh[:, :inter]).reshape(-1), np.ascontiguousarray(guh[:, inter:]).reshape(-1))
    out = torch.zeros(m * inter, dtype=torch.int16, device="cuda")
    ops.gemm_swiglu(ad, wd, out, m, inter, k, tc=True)
    assert np.array_equal(u16(out), want)
    assert ops.gemm_wait_timeouts() == 0


def test_attn_verify_long_context_full_size(ops):
    """BASELINE long-context shape: one chain of k+1 = 5 rows against a 32,768-token paged KV.  Checked against the oracle
    (tolerance class) and through the size-independent property that a chain row equals the same row verified alone."""
    rs = np.random.default_rng(4)
    ctx, cnt = 32763, 5
    c = _attn_case(rs, [ctx], cnt)
    want = orc.paged_attn(c["q"], c["k"], c["v"], c["bt"], c["seq_ids"], c["positions"], 1.0 / 16.0, c["bpr"], 16, 16, 4, 256, threads=8)
    full = _run_attn(ops, c, 1, cnt, ctx + cnt, 128)
    rel2, peak = norm_err(orc.bf16_to_f32(full), orc.bf16_to_f32(want))
    assert rel2 <= 3e-3 and peak <= 1.5e-2, (rel2, peak)
    single = _run_attn(ops, c, cnt, 1, c["bpr"] * 16, 128, spans=(np.arange(cnt, dtype=np.uint32), np.ones(cnt, np.uint32)))
    assert np.array_equal(full, single)


def test_zero_sized_calls_are_accepted(ops):
    """Empty inputs (no rows / no tokens) return success without launching, like the reference's launch wrappers."""
    z16 = torch.zeros(64, dtype=torch.int16, device="cuda")
    z32 = torch.zeros(64, dtype=torch.int32, device="cuda")
    zf = torch.zeros(64, dtype=torch.float32, device="cuda")
    ops.gemm_wt(z16, z16, z16, 0, 32, 32)
    ops.embed(z32, z16, z16, 32, 0)
    ops.rms_norm_zc(z16, z16, z16, 0, 32, 1e-6)
    ops.add(z16, z16, z16, 0)
    ops.kv_scatter(z16, z16, z32, z32, z32, z16, z16, 1, 16, 32, 0)
    ops.deltanet(z16, z16, z16, z16, z16, zf, z16, z16, z16, z32, z32, z32, 0, 1, 1, 128, 128, 0, 1e-6, z32, 1)
    ops.attn_verify(z16, z16, z16, z32, z32, z32, z32, z32, None, z16, 1.0, 4, 16, 4, 1, 64, 0, 1, 16, 4, zf)
    ops.argmax_rows(z16, z32, torch.zeros(64, dtype=torch.int64, device="cuda"), z32, 8, 0)
    torch.cuda.synchronize()
