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
    """The device draft chain (hidden stash -> k MTP forwards with chained hidden) against the CPU mirror."""
    from inferulm_b200.engine import Engine
    from tests.ref_model import RefModel
    w = small_weights
    prompt = _prompt(9, w.shape.vocab, 6)
    ref = RefModel(w, state_f32=True, max_pos=256)
    for t in prompt:
        lg = ref.forward_token(int(t))
    eng = Engine(w, max_seqs=1, k_max=3, max_pos=256)
    eng.admit(0, 64)
    eng.prefill([0], [prompt])
    pending = int(eng.read(0)[0][0])
    # stashed hidden of the last prompt position: same rounding points as the mirror, GEMM-tolerance apart
    hid = host(eng.buffer("hid")[: w.shape.hidden], np.uint16)
    r2, pk = norm_err(orc.bf16_to_f32(hid), orc.bf16_to_f32(ref.last_hidden))
    assert r2 < 2e-2, (r2, pk)
    eng.spec_step([0], 3, 64, use_graph=False)
    drafts = host(eng.buffer("drafts", torch.int32), np.uint32)[:3]
    want = ref.mtp_draft(hid, pending, 3, len(prompt))   # feed the device's own stash: isolates the draft path
    # the first draft depends on one MTP forward only
    lg0 = orc.bf16_to_f32(want[0][1]); srt = np.sort(lg0)
    if srt[-1] - srt[-2] > 0.05:
        assert drafts[0] == want[0][0]
    assert (drafts < w.shape.vocab).all()
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
        assert rr.shape == (3, 3 + 4)
        for b, s in enumerate(slots):
            toks, pos, st = eng.read(s)
            a = int(rr[b, 0])
            assert a <= k and int(rr[b, 1]) == pos and int(rr[b, 2]) == len(toks)
            assert np.array_equal(rr[b, 3:3 + a + 1], toks[len(before[s]):])
            assert (rr[b, 3 + a + 1:] == 0xFFFFFFFF).all()
            before[s] = toks
    eng.close()
