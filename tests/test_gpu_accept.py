"""GPU parity of the acceptance kernels: bit-exact token ids / accept lengths against the oracle, plus the
seeded chi-square check that rejection sampling preserves the target distribution."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests.gpu_util import dev, host, rand_bf16

pytestmark = pytest.mark.gpu
V = 151936


@pytest.fixture(scope="module")
def ops():
    from inferulm_b200 import ops as o
    return o


def _filter(ops, x, n, s, temp, top_k, top_p, rows_per_seq=1, sample=None):
    ids = torch.zeros(s * 64, dtype=torch.int32, device="cuda")
    probs = torch.zeros(s * 64, dtype=torch.float32, device="cuda")
    cnt = torch.zeros(s, dtype=torch.int32, device="cuda")
    tok = torch.zeros(s, dtype=torch.int32, device="cuda") if sample else None
    seed, rnd, position = sample if sample else (None, None, 0)
    ops.topk_filter(dev(x), None, None, rows_per_seq, dev(np.asarray(temp, np.float32)), dev(np.asarray(top_k, np.uint32)),
                    dev(np.asarray(top_p, np.float32)), n, s, ids, probs, cnt, tok, dev(seed) if sample else None,
                    dev(rnd) if sample else None, position)
    return (host(ids, np.uint32).reshape(s, 64), host(probs, np.float32).reshape(s, 64), host(cnt, np.uint32),
            host(tok, np.uint32) if sample else None)


@pytest.mark.parametrize("n,temp,top_k,top_p", [(33, 1.0, 4, 0.9), (257, 0.7, 64, 1.0), (1000, 1.3, 8, 0.5), (513, 1.0, 1, 1.0),
                                                (V, 0.7, 50, 0.9), (V, 1.0, 64, 1.0), (248320, 0.7, 20, 0.95)])
def test_topk_filter_bit_exact(ops, n, temp, top_k, top_p):
    """The shapes of the reference's sampler test k10 (crates/wein-kernel/tests/ops_sample.rs:392-417) and the
    BASELINE vocabulary; bf16 logits tie often, so the lowest-index tie rule is exercised on every row."""
    s = 5
    x = orc.vec_bf16(0xD4 + n, s * n, 5.0)
    ids, probs, cnt, _ = _filter(ops, x, n, s, [temp] * s, [top_k] * s, [top_p] * s)
    for r in range(s):
        keep, wi, wp = orc.filtered_dist(x[r * n:(r + 1) * n], n, temp, top_k, top_p)
        assert cnt[r] == keep
        assert np.array_equal(ids[r], wi), r
        assert np.array_equal(probs[r].view(np.uint32), wp.view(np.uint32)), r


def test_topk_filter_degenerate_rows(ops):
    """All-equal logits (every element ties at the threshold), top_k = 0 (in-band error), greedy rows."""
    n = 5000
    x = np.concatenate([np.full(n, 0x3E80, np.uint16), orc.vec_bf16(1, n, 3.0), orc.vec_bf16(2, n, 3.0)])
    ids, probs, cnt, _ = _filter(ops, x, n, 3, [1.0, 1.0, 0.0], [10, 0, 7], [1.0, 1.0, 1.0])
    assert cnt[0] == 10 and list(ids[0][:10]) == list(range(10))
    assert np.allclose(probs[0][:10], 0.1)
    assert cnt[1] == 0 and ids[1][0] == 0xFFFFFFFF
    assert cnt[2] == 1 and ids[2][0] == orc.argmax_rows(x, [2], n)[0] and probs[2][0] == 1.0


def test_draft_sampling_matches_oracle(ops):
    n, s = 4096, 6
    x = orc.vec_bf16(0xA1, s * n, 3.0)
    seed = np.arange(s, dtype=np.uint64) * 977 + 5
    rnd = np.arange(s, dtype=np.uint64) + 3
    ids, probs, cnt, tok = _filter(ops, x, n, s, [0.8] * s, [16] * s, [0.9] * s, sample=(seed, rnd, 2))
    for r in range(s):
        assert tok[r] == orc.draft_sample(ids[r], probs[r], int(cnt[r]), int(seed[r]), int(rnd[r]), 2)


def test_accept_greedy_bit_exact(ops):
    """The acceptance unit of the reference's first benchmark configuration: bf16 logits [4, 151936] ~ N(0,1), drafts = argmax of rows 0..2 with forced mismatch variants."""
    rs = np.random.default_rng(0)
    B, k = 5, 3
    x = rand_bf16(rs, B * (k + 1) * V).reshape(B * (k + 1), V)
    x[2, 77] = x[2, 40000] = 0x4120  # a tie at the top of one row: the lower index wins
    tgt = orc.argmax_rows(x.reshape(-1), np.arange(B * (k + 1)), V, threads=8).reshape(B, k + 1)
    assert tgt[0, 2] == 77
    drafts = tgt[:, :k].copy()
    drafts[1, 0] += 1          # reject at once
    drafts[2, 2] = 5           # accept 2
    drafts[3, 1] = 40000       # accept 1
    nd = np.array([3, 3, 3, 3, 2], np.uint32)  # the last chain carries only 2 drafts
    scratch = torch.zeros(B * (k + 1) * 32, dtype=torch.int64, device="cuda")
    al = torch.zeros(B, dtype=torch.int32, device="cuda")
    out = torch.zeros(B * (k + 1), dtype=torch.int32, device="cuda")
    tg = torch.zeros(B * (k + 1), dtype=torch.int32, device="cuda")
    ops.accept_greedy(dev(x.reshape(-1)), dev(np.arange(B * (k + 1), dtype=np.uint32)), dev(drafts.reshape(-1)), dev(nd), V, B, k,
                      scratch, al, out, tg)
    got_a, got_out = host(al, np.uint32), host(out, np.uint32).reshape(B, k + 1)
    assert np.array_equal(host(tg, np.uint32).reshape(B, k + 1)[:4], tgt[:4])
    for b in range(B):
        a, em = orc.accept_greedy(drafts[b, :nd[b]], tgt[b])
        assert got_a[b] == a
        assert list(got_out[b, :a + 1]) == list(em)
        assert (got_out[b, a + 1:] == 0xFFFFFFFF).all()
    assert list(got_a) == [3, 0, 2, 1, 2]


def test_accept_sampled_bit_exact_and_mixed_greedy(ops):
    rs = np.random.default_rng(1)
    B, k, n = 64, 3, 3000
    temp = np.where(np.arange(B) % 8 == 7, 0.0, 0.7).astype(np.float32)
    top_k = np.full(B, 50, np.uint32); top_p = np.full(B, 0.9, np.float32)
    tl = rand_bf16(rs, B * (k + 1) * n, 2.0)
    noise = rs.standard_normal((B, k, n)).astype(np.float32) * 0.7
    dl = orc.f32_to_bf16((orc.bf16_to_f32(tl).reshape(B, k + 1, n)[:, :k] + noise).reshape(-1))
    seed = (np.arange(B, dtype=np.uint64) + 1) * 0x9E3779B97F4A7C15 % (1 << 63)
    rnd = np.arange(B, dtype=np.uint64) * 3 + 1
    pi, pp, pn, _ = _filter(ops, tl, n, B * (k + 1), temp, top_k, top_p, rows_per_seq=k + 1)
    # draft rows are laid out [B][k]; each draft step samples with its chain position
    qi = np.zeros((B, k, 64), np.uint32); qp = np.zeros((B, k, 64), np.float32); qn = np.zeros((B, k), np.uint32)
    drafts = np.zeros((B, k), np.uint32)
    dlr = dl.reshape(B, k, n)
    for j in range(k):
        i_, p_, n_, t_ = _filter(ops, dlr[:, j].reshape(-1), n, B, temp, top_k, top_p, sample=(seed, rnd, j))
        qi[:, j], qp[:, j], qn[:, j], drafts[:, j] = i_, p_, n_, t_
    al = torch.zeros(B, dtype=torch.int32, device="cuda")
    out = torch.zeros(B * (k + 1), dtype=torch.int32, device="cuda")
    ops.accept_sampled(dev(drafts.reshape(-1)), None, dev(pi.reshape(-1)), dev(pp.reshape(-1)), dev(pn), dev(qi.reshape(-1)),
                       dev(qp.reshape(-1)), dev(qn.reshape(-1)), dev(temp), dev(seed), dev(rnd), B, k, al, out)
    got_a, got_out = host(al, np.uint32), host(out, np.uint32).reshape(B, k + 1)
    pi, pp, pn = pi.reshape(B, k + 1, 64), pp.reshape(B, k + 1, 64), pn.reshape(B, k + 1)
    seen = set()
    for b in range(B):
        if temp[b] > 0:
            a, em = orc.accept_sampled(drafts[b], pi[b], pp[b], pn[b], qi[b], qp[b], qn[b], int(seed[b]), int(rnd[b]))
        else:
            a, em = orc.accept_greedy(drafts[b], pi[b, :, 0])
        assert got_a[b] == a, b
        assert list(got_out[b, :a + 1]) == list(em), b
        seen.add(a)
    assert len(seen) >= 3  # the noise level exercises rejections and acceptances


def test_rejection_sampling_chi_square_on_device(ops):
    """Distribution preservation, measured on the device kernels: the first emitted token of 200k seeded rounds
    follows the filtered target distribution whatever the draft distribution (alpha = 1e-4)."""
    from scipy.stats import chi2
    n, k, B = 16, 1, 200_000
    rs = np.random.default_rng(0)
    pl, ql = rand_bf16(rs, n, 1.5), rand_bf16(rs, n, 1.5)
    temp, top_k, top_p = 0.9, 12, 0.95
    pn_, pids, pp_ = orc.filtered_dist(pl, n, temp, top_k, top_p)
    expect = np.zeros(n); expect[pids[:pn_]] = pp_[:pn_]
    # one shared target row pair and one shared draft row, B sequences with different seeds
    tl = np.concatenate([pl, pl])
    pi, pp, pn, _ = _filter(ops, tl, n, 2, [temp], [top_k], [top_p], rows_per_seq=2)
    seed = np.arange(B, dtype=np.uint64) + 12345
    rnd = np.zeros(B, np.uint64)
    qi1, qp1, qn1, _ = _filter(ops, ql, n, 1, [temp], [top_k], [top_p])
    # per-sequence draft token through the device sampler (same distribution, different seeds)
    x = np.tile(ql, B)
    _, _, _, drafts = _filter(ops, x, n, B, [temp] * B, [top_k] * B, [top_p] * B, sample=(seed, rnd, 0))
    al = torch.zeros(B, dtype=torch.int32, device="cuda")
    out = torch.zeros(B * 2, dtype=torch.int32, device="cuda")
    ops.accept_sampled(dev(drafts), None, dev(np.tile(pi.reshape(-1), B)), dev(np.tile(pp.reshape(-1), B)), dev(np.tile(pn, B)),
                       dev(np.tile(qi1.reshape(-1), B)), dev(np.tile(qp1.reshape(-1), B)), dev(np.tile(qn1, B)),
                       dev(np.full(B, temp, np.float32)), dev(seed), dev(rnd), B, k, al, out)
    first = host(out, np.uint32).reshape(B, 2)[:, 0]
    cnt = np.bincount(first, minlength=n).astype(np.float64)
    sup = expect > 0
    assert cnt[~sup].sum() == 0
    chi = ((cnt[sup] - B * expect[sup]) ** 2 / (B * expect[sup])).sum()
    assert chi < chi2.ppf(1 - 1e-4, sup.sum() - 1), chi
    qfull = np.zeros(n); qfull[qi1[0][:qn1[0]]] = qp1[0][:qn1[0]]
    assert abs(host(al, np.uint32).mean() - np.minimum(expect, qfull).sum()) < 0.01


def _sample(ops, x, n, s, temp, top_k, top_p, seed, rng_dev):
    out = torch.zeros(s, dtype=torch.int32, device="cuda")
    ops.sample_rows(dev(x), dev(np.arange(s, dtype=np.uint32)), dev(np.arange(s, dtype=np.uint32)), dev(np.asarray(temp, np.float32)),
                    dev(np.asarray(top_k, np.uint32)), dev(np.asarray(top_p, np.float32)), dev(np.asarray(seed, np.uint64)), rng_dev, out, n, s)
    return host(out, np.uint32)


def test_sample_rows_matches_reference_sampler_bitwise(ops):
    """k10 of crates/wein-kernel/tests/ops_sample.rs:392-417 (kernel == reference, random logits / parameters / seeds), run
    over several consecutive calls so the PCG state carried in the device buffer is exercised, plus k1 (temp = 0 == argmax)."""
    for (s, n, tk, tp, temp) in [(6, 33, 4, 0.9, 1.0), (5, 257, 64, 1.0, 0.7), (4, 1000, 8, 0.5, 1.3), (3, 513, 1, 1.0, 1.0), (4, V, 50, 0.9, 0.7)]:
        x = orc.vec_bf16(0xD4, s * n, 5.0)
        seeds = np.array([0x7000 + j * 977 for j in range(s)], np.uint64)
        rng_dev = torch.zeros(s, dtype=torch.int64, device="cuda")
        rng_ref = np.zeros(s, np.uint64)
        for call in range(4):
            got = _sample(ops, x, n, s, [temp] * s, [tk] * s, [tp] * s, seeds, rng_dev)
            want = orc.sample_rows(x, np.arange(s), n, [temp] * s, [tk] * s, [tp] * s, seeds, np.arange(s), rng_ref)
            assert np.array_equal(got, want), (s, n, tk, tp, temp, call)
        assert np.array_equal(host(rng_dev, np.uint64), rng_ref)
    x = orc.vec_bf16(0x51, 3 * 1024, 4.0)
    rng_dev = torch.zeros(3, dtype=torch.int64, device="cuda")
    got = _sample(ops, x, 1024, 3, [0.0] * 3, [0] * 3, [1.0] * 3, [1] * 3, rng_dev)
    assert np.array_equal(got, orc.argmax_rows(x, np.arange(3), 1024))
    assert int(rng_dev.abs().sum()) == 0                      # greedy rows do not advance the RNG
    bad = _sample(ops, x, 1024, 3, [1.0] * 3, [0] * 3, [1.0] * 3, [1] * 3, rng_dev)
    assert (bad == 0xFFFFFFFF).all()


def test_sample_rows_chi_square(ops):
    """k8 of ops_sample.rs:350-387 on the device: 0.5/0.3/0.15/0.05, 200k draws, chi-square below 21.108 (dof 3, alpha 1e-4)."""
    s, n = 512, 4
    logits = orc.f32_to_bf16(np.log(np.array([0.5, 0.3, 0.15, 0.05], np.float32)))
    x = np.tile(logits, s)
    rng_dev = torch.zeros(s, dtype=torch.int64, device="cuda")
    seeds = 0xABC000 + np.arange(s, dtype=np.uint64)
    cnt = np.zeros(n)
    for _ in range(391):
        cnt += np.bincount(_sample(ops, x, n, s, [1.0] * s, [64] * s, [1.0] * s, seeds, rng_dev), minlength=n)
    p = np.exp(orc.bf16_to_f32(logits).astype(np.float64)); p /= p.sum()
    chi = ((cnt - cnt.sum() * p) ** 2 / (cnt.sum() * p)).sum()
    assert chi < 21.108, chi
