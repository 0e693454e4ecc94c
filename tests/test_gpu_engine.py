"""GPU tests of the step level (wein_b200_engine_*): the contracts of the reference's executor tests
(crates/wein-exec/tests/qwen.rs qs9 / qs10 / qs12 / qs13) restated on random-init weights, plus a comparison with the
CPU mirror of the forward built from the oracle."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests.gpu_util import host, norm_err

pytestmark = pytest.mark.gpu


def small_shape(**kw):
    from inferulm_b200.engine import ModelShape
    d = dict(hidden=512, n_layers=4, q_heads=8, kv_heads=2, head_dim=64, rot_dim=32, inter=1024, vocab=4096, lin_k_heads=2,
             lin_v_heads=4, full_every=4)
    d.update(kw)
    return ModelShape(**d)


@pytest.fixture(scope="module")
def small_weights():
    from inferulm_b200.engine import SyntheticWeights
    return SyntheticWeights(small_shape(), seed=0, std=0.05)


def _prompt(n, vocab, seed=0):
    return np.random.default_rng(seed).integers(0, vocab, n).astype(np.uint32)


def _run(weights, prompt, n_new, k, use_graph, state_f32=True, max_seqs=1, slot=0, temp=0.0, top_k=0, top_p=1.0, seed=0, max_pos=1024):
    from inferulm_b200.engine import Engine
    eng = Engine(weights, max_seqs=max_seqs, k_max=3, max_pos=max_pos, state_f32=state_f32)
    eng.admit(slot, len(prompt) + n_new + 8, temp=temp, top_k=top_k, top_p=top_p, seed=seed, rng=np.random.default_rng(5))
    eng.prefill([slot], [prompt])
    rounds = eng.generate([slot], n_new, k, use_graph=use_graph)
    toks, pos, stats = eng.read(slot)
    return eng, toks, pos, stats, rounds


def test_forward_matches_cpu_mirror(small_weights):
    """Prefill + plain decode against the CPU mirror (q5 of the reference's executor tests: logits within tolerance,
    argmax equal wherever the margin exceeds the error).  The GEMMs are tolerance-class, everything else bit-exact."""
    from tests.ref_model import RefModel
    w = small_weights
    prompt = _prompt(21, w.shape.vocab, 1)
    ref = RefModel(w, state_f32=True, max_pos=1024)
    for t in prompt:
        lg = ref.forward_token(int(t))
    eng, toks, pos, _, _ = _run(w, prompt, 1, 0, False)
    assert pos == len(prompt)
    # logits of the last prompt position are still in the engine's buffer (row 0)
    got = orc.bf16_to_f32(host(eng.buffer("logits")[: w.shape.vocab], np.uint16))
    want = orc.bf16_to_f32(lg)
    rel2, peak = norm_err(got, want)
    assert rel2 < 3e-2 and peak < 6e-2, (rel2, peak)
    err = np.abs(got - want).max()
    srt = np.sort(want)
    if srt[-1] - srt[-2] > 4 * err:
        assert toks[0] == int(np.argmax(want))
    # recurrent state of the committed row, first DeltaNet layer, against the mirror (f32 pool)
    row = int(host(eng.buffer("state_row", torch.int32), np.uint32)[0])
    n = w.shape.lin_v_heads * 128 * 128
    st = host(eng.buffer("lin_state:0", torch.float32)[row * n:(row + 1) * n], np.float32)
    r2, pk = norm_err(st, ref.lin_state[0])
    assert r2 < 2e-2 and pk < 5e-2, (r2, pk)
    eng.close()


@pytest.mark.parametrize("use_graph", [False, True])
@pytest.mark.parametrize("state_f32", [True, False])
def test_spec_greedy_equals_plain_greedy(small_weights, use_graph, state_f32):
    """qs10: greedy speculative output == non-speculative greedy output, token for token -- and here bit for bit in
    every buffer, because no kernel's arithmetic depends on the batch shape."""
    w = small_weights
    prompt = _prompt(37, w.shape.vocab, 2)
    n_new = 40
    e0, t0, p0, s0, r0 = _run(w, prompt, n_new, 0, use_graph, state_f32)
    e3, t3, p3, s3, r3 = _run(w, prompt, n_new, 3, use_graph, state_f32)
    assert len(t0) >= n_new and len(t3) >= n_new
    assert np.array_equal(t0[:n_new], t3[:n_new])
    assert s0["drafts"] == 0 and s3["drafts"] == 3 * s3["rounds"]
    assert p3 == len(prompt) + len(t3) - 1 and p0 == len(prompt) + len(t0) - 1
    e0.close(); e3.close()


def _copy_model():
    """A model whose greedy continuation repeats the pending token and whose MTP head agrees: every output projection
    is zero (the residual stream stays the token embedding) and the MTP fc copies the normalised embedding."""
    from inferulm_b200.engine import SyntheticWeights
    w = SyntheticWeights(small_shape(), seed=3, std=0.05)
    with torch.no_grad():
        for d in w.layers + [w.mtp["layer"]]:
            d["wd"].zero_()
            (d["o"] if d["full"] else d["out"]).zero_()
        h = w.shape.hidden
        w.mtp["fc"].zero_()
        w.mtp["fc"][:, :h] = torch.eye(h, dtype=torch.bfloat16, device="cuda")
        w.norm_f.zero_(); w.mtp["norm"].zero_(); w.mtp["pre_e"].zero_()
    torch.cuda.synchronize()
    return w


def test_full_acceptance_and_state_rows():
    """qs9 / qs13: when every draft is accepted a round emits k+1 tokens, and the committed state row equals the row
    a plain run reaches after the same tokens (bitwise), round after round (row swap between the two banks)."""
    w = _copy_model()
    prompt = _prompt(19, w.shape.vocab, 4)
    e0, t0, p0, s0, _ = _run(w, prompt, 33, 0, True)
    e3, t3, p3, s3, r3 = _run(w, prompt, 33, 3, True)
    assert np.array_equal(t0[:33], t3[:33])
    assert s3["accepted"] == s3["drafts"] > 0, s3          # the copy model accepts everything
    assert len(t3) == 1 + 4 * s3["rounds"]
    # advance the plain run to the same position, then compare the committed recurrent + conv state rows bit for bit
    while e0.counts([0])[0][1] < p3:
        e0.spec_step([0], 0, p3 + 4)
    assert e0.counts([0])[0][1] == p3
    n = w.shape.lin_v_heads * 128 * 128
    cdn = (2 * w.shape.lin_k_heads * 128 + w.shape.lin_v_heads * 128) * 3
    for li in range(3):
        r0 = int(host(e0.buffer("state_row", torch.int32), np.uint32)[0]); r3_ = int(host(e3.buffer("state_row", torch.int32), np.uint32)[0])
        a = host(e0.buffer(f"lin_state:{li}", torch.float32)[r0 * n:(r0 + 1) * n], np.uint32)
        b = host(e3.buffer(f"lin_state:{li}", torch.float32)[r3_ * n:(r3_ + 1) * n], np.uint32)
        assert np.array_equal(a, b), li
        ca = host(e0.buffer(f"conv_state:{li}")[r0 * cdn:(r0 + 1) * cdn], np.uint16)
        cb = host(e3.buffer(f"conv_state:{li}")[r3_ * cdn:(r3_ + 1) * cdn], np.uint16)
        assert np.array_equal(ca, cb), li
    e0.close(); e3.close()


def test_batch_of_chains_matches_single_runs(small_weights):
    """qs12: four chains in one forward give each sequence the tokens it gets alone (different prompt lengths)."""
    from inferulm_b200.engine import Engine
    w = small_weights
    prompts = [_prompt(n, w.shape.vocab, 10 + n) for n in (5, 33, 16, 47)]
    eng = Engine(w, max_seqs=4, k_max=3, max_pos=512)
    rng = np.random.default_rng(9)
    for s, p in enumerate(prompts):
        eng.admit(s, len(p) + 40, rng=rng)
    eng.prefill([0, 1, 2, 3], prompts)
    eng.generate([0, 1, 2, 3], 24, 3)
    for s, p in enumerate(prompts):
        toks, pos, _ = eng.read(s)
        _, t1, _, _, _ = _run(w, p, 24, 0, True, max_pos=512)
        assert np.array_equal(toks[:24], t1[:24]), s
    # slots in a different order and a smaller batch reuse the same state
    eng.spec_step([2, 0], 3, 200)
    eng.close()


def test_mtp_drafts_match_cpu_mirror(small_weights):
    """The device draft chain (hidden stash -> k MTP forwards with the hidden chained through the head's own normalised
    output, qwen.rs:2805-2848) against the CPU mirror: every draft and every chained hidden row.  The draft phase runs
    alone (engine_draft) for k = 1, 2, 3, so the buffers still hold draft k-1's logits and normalised hidden; the mirror
    is fed the device's own earlier drafts, so one close call cannot hide a later comparison."""
    from inferulm_b200.engine import Engine
    from tests.ref_model import RefModel
    w = small_weights
    H, V = w.shape.hidden, w.shape.vocab
    prompt = _prompt(9, V, 6)
    ref = RefModel(w, state_f32=True, max_pos=256)
    for t in prompt:
        ref.forward_token(int(t))
    eng = Engine(w, max_seqs=1, k_max=3, max_pos=256)
    eng.admit(0, 64)
    eng.prefill([0], [prompt])
    pending = int(eng.read(0)[0][0])
    # stashed hidden of the last prompt position: same rounding points as the mirror, GEMM-tolerance apart
    hid = host(eng.buffer("hid")[:H], np.uint16)
    r2, pk = norm_err(orc.bf16_to_f32(hid), orc.bf16_to_f32(ref.last_hidden))
    assert r2 < 2e-2, (r2, pk)
    checked = 0
    for k in (1, 2, 3):
        out = torch.zeros(k, dtype=torch.int32, device="cuda")
        torch.cuda.synchronize()           # `out` was filled on torch's stream; the engine writes it on its own
        eng.draft([0], k, out=out, use_graph=(k == 2))
        torch.cuda.synchronize()
        drafts = host(out, np.uint32)
        assert np.array_equal(drafts, host(eng.buffer("drafts", torch.int32), np.uint32)[:k])
        want = ref.mtp_draft(hid, pending, k, len(prompt), force=[int(d) for d in drafts])   # device stash, device tokens
        tok_ref, lg_ref, hid_ref = want[k - 1]
        lg = orc.bf16_to_f32(host(eng.buffer("logits")[:V], np.uint16))
        r2, pk = norm_err(lg, orc.bf16_to_f32(lg_ref))
        assert r2 < 3e-2 and pk < 6e-2, (k, r2, pk)
        n2 = orc.bf16_to_f32(host(eng.buffer("n2")[:H], np.uint16))
        r2, pk = norm_err(n2, orc.bf16_to_f32(hid_ref))
        assert r2 < 2e-2 and pk < 5e-2, (k, r2, pk)
        srt = np.sort(orc.bf16_to_f32(lg_ref))
        if srt[-1] - srt[-2] > 4 * np.abs(lg - orc.bf16_to_f32(lg_ref)).max():
            assert drafts[k - 1] == tok_ref, k
            checked += 1
        assert (drafts < V).all()
    assert checked >= 1
    # nothing was committed by the draft phase
    assert eng.read(0)[1] == len(prompt) and eng.read(0)[2]["rounds"] == 0
    eng.close()


def _hidden_copy_model():
    """As _copy_model(), but the MTP head reads ONLY the hidden half of its input (fc = [0 | I]): a draft is right only if
    the hidden row reached the head -- the stash of the committed position for draft 0, the head's own normalised output
    for every later draft."""
    w = _copy_model()
    with torch.no_grad():
        h = w.shape.hidden
        w.mtp["fc"].zero_()
        w.mtp["fc"][:, h:] = torch.eye(h, dtype=torch.bfloat16, device="cuda")
        w.mtp["pre_h"].zero_()
    torch.cuda.synchronize()
    return w


def test_hidden_chaining_carries_the_drafts():
    """Full acceptance with a head that sees nothing but the chained hidden, for three sequences in a permuted slot order
    (a draft row must read its own slot's stash and its own row of the previous draft's output)."""
    from inferulm_b200.engine import Engine
    w = _hidden_copy_model()
    V = w.shape.vocab
    eng = Engine(w, max_seqs=3, k_max=3, max_pos=256)
    slots = [2, 0, 1]
    prompts = {s: _prompt(7 + 5 * s, V, 40 + s) for s in slots}
    for s in slots:
        eng.admit(s, 200)
    eng.prefill(slots, [prompts[s] for s in slots])
    eng.generate(slots, 25, 3)
    for s in slots:
        toks, pos, st = eng.read(s)
        assert st["drafts"] > 0 and st["accepted"] == st["drafts"], (s, st)
        assert (toks == prompts[s][-1]).all()       # the copy model repeats its last token
    eng.close()


def test_sampled_rounds_are_seeded_and_valid(small_weights):
    """Sampled acceptance end to end: same seed -> same tokens (graph or eager), other seed -> other tokens, every
    emitted id inside the vocabulary, counters consistent."""
    w = small_weights
    prompt = _prompt(23, w.shape.vocab, 7)
    kw = dict(temp=0.8, top_k=20, top_p=0.9)
    _, ta, pa, sa, _ = _run(w, prompt, 30, 3, True, seed=11, **kw)
    _, tb, pb, sb, _ = _run(w, prompt, 30, 3, False, seed=11, **kw)
    _, tc, _, _, _ = _run(w, prompt, 30, 3, True, seed=12, **kw)
    assert np.array_equal(ta[:30], tb[:30]) and sa == sb
    assert not np.array_equal(ta[:30], tc[:30])
    assert (ta < w.shape.vocab).all()
    assert len(ta) == 1 + sa["rounds"] + sa["accepted"]
    assert pa == len(prompt) + len(ta) - 1


def test_engine_rejects_bad_arguments(small_weights):
    from inferulm_b200.engine import Engine
    from inferulm_b200.lib import WeinB200Error
    eng = Engine(small_weights, max_seqs=2, k_max=3, max_pos=128)
    with pytest.raises(WeinB200Error):
        eng.admit(5, 32)                       # slot out of range
    with pytest.raises(WeinB200Error):
        eng.admit(0, 32, pages=[10 ** 6])      # page outside the pool
    with pytest.raises(WeinB200Error):
        eng.admit(0, 32, temp=1.0, top_k=0)    # whole-vocabulary sampling is not built
    eng.admit(0, 64)
    with pytest.raises(WeinB200Error):
        eng.read_round(1)                      # no round has run yet
    with pytest.raises(WeinB200Error):
        eng.spec_step([0], 5, 64)              # k > k_max
    with pytest.raises(WeinB200Error):
        eng.spec_step([0, 0], 1, 64)           # slot listed twice
    with pytest.raises(WeinB200Error):
        eng.prefill([0], [np.array([99999999], np.uint32)])  # token outside the vocabulary
    eng.close()


def test_max_draft_length_k7(small_weights):
    """The longest supported chain (k = 7, 8 verify rows, two attention m-tiles): speculative == plain greedy."""
    from inferulm_b200.engine import Engine
    w = small_weights
    prompt = _prompt(29, w.shape.vocab, 8)
    outs = []
    for k in (0, 7):
        eng = Engine(w, max_seqs=1, k_max=7, max_pos=512)
        eng.admit(0, 400)
        eng.prefill([0], [prompt])
        eng.generate([0], 30, k)
        outs.append(eng.read(0)[0][:30])
        eng.close()
    assert np.array_equal(outs[0], outs[1])


def test_adaptive_draft_length_keeps_greedy_output(small_weights):
    """Host-paced rounds with the adaptive policy choosing k: whatever lengths it picks (random weights make the MTP
    head miss, so it falls to k = 1, switches drafting off and probes again), the tokens equal plain greedy decoding."""
    from inferulm_b200.engine import Engine
    w = small_weights
    prompt = _prompt(31, w.shape.vocab, 9)
    eng = Engine(w, max_seqs=1, k_max=3, max_pos=512)
    eng.admit(0, 400)
    eng.prefill([0], [prompt])
    eng.generate([0], 40, 0)
    want = eng.read(0)[0][:40]
    eng.close()
    eng = Engine(w, max_seqs=1, k_max=3, max_pos=512)
    eng.admit(0, 400)
    eng.prefill([0], [prompt])
    rounds, ks = eng.generate_adaptive([0], 40, 3)
    got = eng.read(0)[0][:40]
    eng.close()
    assert np.array_equal(got, want)
    assert rounds == len(ks) and ks[0] == 2 and set(ks) <= {0, 1, 2, 3}
    assert 0 in ks and 1 in ks            # drafting was switched off and probed again


def test_read_round_matches_per_slot_reads(small_weights):
    """The one-copy readback of a round agrees with the per-slot reads: accept length, position, emitted count, tokens."""
    from inferulm_b200.engine import Engine
    w = small_weights
    eng = Engine(w, max_seqs=3, k_max=3, max_pos=256)
    slots = [2, 0, 1]
    for s in slots:
        eng.admit(s, 200)
    eng.prefill(slots, [_prompt(40 + s, w.shape.vocab, 5 + s) for s in slots])
    before = {s: eng.read(s)[0] for s in slots}
    for k in (3, 1, 0):
        eng.spec_step(slots, k, 64)
        rr = eng.read_round(len(slots))
        assert rr.shape == (3, 4 + 4)
        for b, s in enumerate(slots):
            toks, pos, st = eng.read(s)
            a = int(rr[b, 0])
            assert a <= k and int(rr[b, 1]) == pos and int(rr[b, 2]) == len(toks)
            assert np.array_equal(rr[b, 3:3 + a + 1], toks[len(before[s]):])
            assert (rr[b, 3 + a + 1:-1] == 0xFFFFFFFF).all() and rr[b, -1] == 0
            before[s] = toks
    eng.close()


def test_baseline_shape_spec_equals_plain():
    """qs10 (crates/wein-exec/tests/qwen.rs:908) on the model shape the benchmark runs: hidden 2560, 24 + 8 layers,
    vocabulary 151,936, random-init weights.  Greedy k = 3 through graph replay == plain greedy, 32 tokens."""
    from inferulm_b200.engine import Engine, ModelShape, SyntheticWeights
    w = SyntheticWeights(ModelShape(), seed=0, std=0.02)
    prompt = _prompt(48, w.shape.vocab, 21)
    outs = []
    for k in (0, 3):
        eng = Engine(w, max_seqs=1, k_max=3, max_pos=512)
        eng.admit(0, 160)
        eng.prefill([0], [prompt])
        eng.generate([0], 32, k, use_graph=True)
        toks, pos, st = eng.read(0)
        outs.append(toks[:32].copy())
        assert pos == len(prompt) + len(toks) - 1
        eng.close()
    assert np.array_equal(outs[0], outs[1])
    del w
    torch.cuda.empty_cache()


def test_baseline_shape_batch8_k4_spec_equals_plain():
    """The long-context configuration's batch on the benchmark's model shape: 8 sequences, k = 4, 40 verify rows, so every
    product runs on the tensor-memory GEMM with its cluster k-split (n = 2560) and two-tile CTAs.  Greedy speculative ==
    plain greedy at the same batch, token for token."""
    from inferulm_b200.engine import Engine, ModelShape, SyntheticWeights
    w = SyntheticWeights(ModelShape(), seed=1, std=0.02)
    B, k = 8, 4
    prompts = [_prompt(9 + 5 * i, w.shape.vocab, 300 + i) for i in range(B)]
    outs = []
    for kk in (0, k):
        eng = Engine(w, max_seqs=B, k_max=k, max_pos=256)
        for s in range(B):
            eng.admit(s, 128)
        eng.prefill(list(range(B)), prompts)
        eng.generate(list(range(B)), 12, kk)
        outs.append([eng.read(s)[0][:12].copy() for s in range(B)])
        eng.close()
    for s in range(B):
        assert np.array_equal(outs[0][s], outs[1][s]), s
    from inferulm_b200 import ops
    assert ops.gemm_wait_timeouts() == 0 and ops.gdn_wait_timeouts() == 0
    del w
    torch.cuda.empty_cache()


@pytest.mark.parametrize("B,k", [(8, 4), (32, 3)])
def test_greedy_spec_equals_plain_above_32_rows(B, k):
    """North-star bar: greedy speculative output == non-speculative greedy output, token for token, also when the verify
    forward has more than 32 rows (B = 8, k = 4: 40 rows; B = 32, k = 3: 128 rows).  Both runs use the same batch, as the
    reference's own tests equalise the batch shape (crates/wein-exec/tests/qwen.rs:801-804, :903-906); an engine of this
    size multiplies every forward on the tensor-memory GEMM, whose sums do not depend on the row count."""
    from inferulm_b200.engine import Engine, SyntheticWeights
    w = SyntheticWeights(small_shape(), seed=5, std=0.05)
    V = w.shape.vocab
    prompts = [_prompt(5 + (7 * i) % 23, V, 100 + i) for i in range(B)]
    outs = []
    for kk in (0, k):
        eng = Engine(w, max_seqs=B, k_max=k, max_pos=256)
        rng = np.random.default_rng(3)
        for s in range(B):
            eng.admit(s, 120, rng=rng)
        eng.prefill(list(range(B)), prompts)
        eng.generate(list(range(B)), 24, kk)
        outs.append([eng.read(s)[0][:24].copy() for s in range(B)])
        assert all(eng.status(s) == 0 for s in range(B))
        eng.close()
    for s in range(B):
        assert np.array_equal(outs[0][s], outs[1][s]), s
    from inferulm_b200 import ops
    assert ops.gemm_wait_timeouts() == 0 and ops.gdn_wait_timeouts() == 0


def test_spec_verify_with_caller_drafts_and_ragged_chains(small_weights):
    """spec_verify / spec_commit_batch (qwen.rs:2261-2303) with the caller's drafts: per-sequence draft counts, drafts
    that are right, wrong and outside the vocabulary; accept lengths and emitted tokens against the oracle's acceptance
    rule on the engine's own greedy targets; a dry run first, which must commit nothing."""
    from inferulm_b200.engine import Engine
    w = small_weights
    V = w.shape.vocab
    B, k = 4, 3
    prompts = [_prompt(11 + 3 * i, V, 60 + i) for i in range(B)]
    # the greedy continuation of every sequence, from a plain run
    ref = Engine(w, max_seqs=B, k_max=k, max_pos=256)
    for s in range(B):
        ref.admit(s, 100)
    ref.prefill(list(range(B)), prompts)
    ref.generate(list(range(B)), 8, 0)
    cont = [ref.read(s)[0][:8].copy() for s in range(B)]
    ref.close()
    eng = Engine(w, max_seqs=B, k_max=k, max_pos=256)
    for s in range(B):
        eng.admit(s, 100)
    eng.prefill(list(range(B)), prompts)
    # drafts: seq 0 all right (3), seq 1 right, wrong, right (count 3), seq 2 two right but count 1, seq 3 out-of-vocabulary first
    d = np.zeros((B, k), np.uint32)
    for s in range(B):
        d[s] = cont[s][1:1 + k]
    d[1, 1] = (d[1, 1] + 1) % V
    d[3, 0] = 0xFFFFFFF0
    nd = np.array([3, 3, 1, 3], np.uint32)
    want_a = [3, 1, 1, 0]
    dd, ndd = torch.from_numpy(d.view(np.int32)).cuda(), torch.from_numpy(nd.view(np.int32)).cuda()
    slots = list(range(B))
    eng.spec_verify(slots, k, dd, 64, n_drafts=ndd, dry_run=True)
    rr = eng.read_round(B)
    for s in range(B):
        assert int(rr[s, 0]) == want_a[s], (s, rr[s])
        assert eng.read(s)[1] == len(prompts[s]) and eng.read(s)[2]["rounds"] == 0     # nothing committed
    target = host(eng.buffer("target", torch.int32), np.uint32)[: B * (k + 1)].reshape(B, k + 1)
    for use_graph in (False,):
        eng.spec_verify(slots, k, dd, 64, n_drafts=ndd, use_graph=use_graph)
    rr = eng.read_round(B)
    for s in range(B):
        a, toks = orc.accept_greedy(d[s, :nd[s]], target[s, :nd[s] + 1])
        assert a == want_a[s] and int(rr[s, 0]) == a
        assert np.array_equal(rr[s, 3:3 + a + 1], np.asarray(toks, np.uint32))
        got, pos, st = eng.read(s)
        assert np.array_equal(got[:a + 2], cont[s][:a + 2])          # first token + this round's a + 1 tokens: the greedy path
        assert pos == len(prompts[s]) + a + 1 and st["drafts"] == nd[s] and st["accepted"] == a
    # a second round through the graph, engine-made drafts handed back through spec_verify == spec_step
    eng.draft(slots, k)
    eng.spec_verify(slots, k, None, 64, engine_drafts=True, use_graph=True)
    for s in range(B):
        got = eng.read(s)[0]
        assert np.array_equal(got[:len(got)], _greedy_prefix(w, prompts[s], len(got)))
    eng.close()


def _greedy_prefix(w, prompt, n):
    _, t, _, _, _ = _run(w, prompt, n, 0, True, max_pos=256)
    return t[:n]


def test_per_request_draft_length_in_one_round(small_weights):
    """set_spec per request (qwen.rs:2604-2647) and the mixed batch of qs11 (crates/wein-exec/tests/qwen.rs:990): chains of
    3, 1 and 0 drafts in one verify forward; every sequence keeps its greedy output and its own counters."""
    from inferulm_b200.engine import Engine
    w = _copy_model()          # every draft is accepted, so the accept length shows the chain length each slot ran with
    V = w.shape.vocab
    eng = Engine(w, max_seqs=3, k_max=3, max_pos=256)
    prompts = [_prompt(9 + 4 * s, V, 80 + s) for s in range(3)]
    for s in range(3):
        eng.admit(s, 200)
    eng.prefill([0, 1, 2], prompts)
    for s, kk in ((0, 3), (1, 1), (2, 0)):
        eng.set_spec(s, kk)
    for _ in range(5):
        eng.spec_step([0, 1, 2], 3, 128)
    rr = eng.read_round(3)
    assert [int(rr[s, 0]) for s in range(3)] == [3, 1, 0]
    for s, kk in ((0, 3), (1, 1), (2, 0)):
        toks, pos, _ = eng.read(s)
        st = eng.stats(s)
        assert st["rounds"] == 5 and st["drafts"] == 5 * kk and st["accepted"] == 5 * kk and st["by_k"][kk] == 5
        assert st["by_accept"][kk] == 5 and st["k_switches"] == 0 and st["fallbacks"] == 0
        assert len(toks) == 1 + 5 * (kk + 1) and (toks == prompts[s][-1]).all()
    eng.set_spec(1, 2)
    eng.spec_step([0, 1, 2], 3, 128)
    assert eng.stats(1)["k_switches"] == 1 and eng.stats(1)["last_k"] == 2
    eng.close()


def test_position_limit_is_enforced_on_the_device(small_weights):
    """A slot admitted with pages for 48 positions inside an engine of max_pos 128: rounds shorten the chain at the limit
    (status K_CLAMPED, counted as a fallback), then refuse the slot (status POS_LIMIT) without touching its neighbour's
    pages, its own committed state or its position; a prompt that does not fit is rejected on the host."""
    from inferulm_b200.engine import Engine
    from inferulm_b200.lib import WeinB200Error
    w = small_weights
    V = w.shape.vocab
    eng = Engine(w, max_seqs=2, k_max=3, max_pos=128)
    eng.admit(0, 48, pages=[0, 1, 2])
    eng.admit(1, 128, pages=[3, 4, 5, 6, 7, 8, 9, 10])
    with pytest.raises(WeinB200Error):
        eng.prefill([0], [_prompt(48, V, 1)])               # 48 tokens + the next one do not fit 48 positions
    eng.prefill([0, 1], [_prompt(40, V, 1), _prompt(20, V, 2)])
    he = w.shape.kv_heads * w.shape.head_dim
    rounds = 0
    while eng.read(0)[1] < 48 and rounds < 24:
        eng.spec_step([0, 1], 3, 128)
        rounds += 1
    assert eng.read(0)[1] == 48 and eng.status(0) == 2      # reached its last position by shortened chains, never refused
    st = eng.stats(0)
    assert st["fallbacks"] >= 1 and st["by_k"][0] >= 1 and st["rounds"] == rounds
    toks_mid = eng.read(0)[0]
    p1 = eng.read(1)[1]
    kp = host(eng.buffer("k_pool:0"), np.uint16).copy()
    eng.spec_step([0, 1], 3, 128)                           # now refused
    rr = eng.read_round(2)
    assert eng.status(0) & 1 and int(rr[0, -1]) & 1 and (rr[0, 3:-1] == 0xFFFFFFFF).all()
    assert eng.read(0)[1] == 48 and np.array_equal(eng.read(0)[0], toks_mid)
    assert eng.read(1)[1] > p1 and eng.status(1) == 0       # the neighbour went on
    kp2 = host(eng.buffer("k_pool:0"), np.uint16)
    pages0 = kp.reshape(-1, 16 * he)[:3], kp2.reshape(-1, 16 * he)[:3]
    assert np.array_equal(pages0[0], pages0[1])             # the refused slot wrote nothing
    assert eng.status(0, clear=True) & 1 and eng.status(0) == 0
    # generate() stops by itself at the limit
    assert eng.generate([0], 100, 3) == 0
    eng.close()


def test_understated_context_bound_is_flagged_not_fatal(small_weights):
    """ctx_bound below the real position: attention reduces what its grid covers and raises CTX_BOUND in the status word;
    with the right bound the same round is clean."""
    from inferulm_b200.engine import Engine
    w = small_weights
    eng = Engine(w, max_seqs=1, k_max=3, max_pos=1024, attn_seg_pages=4)
    eng.admit(0, 1000)
    eng.prefill([0], [_prompt(300, w.shape.vocab, 3)])
    eng.spec_step([0], 3, 400)
    assert eng.status(0) == 0
    eng.spec_step([0], 3, 40, use_graph=False)              # 40 < 300: three segments instead of five
    assert eng.status(0, clear=True) & 4
    eng.spec_step([0], 3, 400)
    assert eng.status(0) == 0
    eng.close()


def test_warm_makes_rounds_allocation_free(small_weights):
    """After warm() a round of the warmed shape replays its graph without allocating device memory; eager rounds with the
    phase timers on report the three phases."""
    from inferulm_b200.engine import Engine
    w = small_weights
    eng = Engine(w, max_seqs=2, k_max=3, max_pos=256)
    for s in (0, 1):
        eng.admit(s, 200)
    eng.prefill([0, 1], [_prompt(12, w.shape.vocab, 1), _prompt(17, w.shape.vocab, 2)])
    eng.warm([0, 1], 3, 128, what=1 | 2 | 4 | 8)
    eng.spec_step([0, 1], 3, 128)      # the first launch of a kernel may still load its code
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    for _ in range(3):
        eng.spec_step([0, 1], 3, 128)
    eng.read_round(2)
    assert torch.cuda.mem_get_info()[0] == free0
    eng.timing(True)
    for _ in range(2):
        eng.spec_step([0, 1], 3, 128, use_graph=False)
    ms = eng.timing(False)
    assert all(m > 0.0 for m in ms) and ms[1] > ms[2]
    eng.close()
