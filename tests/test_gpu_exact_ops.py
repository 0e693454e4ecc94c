"""GPU parity of the bit-exact operators: each CUDA kernel, called through the
C-ABI, must reproduce the oracle's bf16 words exactly on seeded inputs.  The
cases follow the reference's own kernel tests (crates/wein-kernel/tests)."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests.gpu_util import dev, host, rand_bf16, u16

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from inferulm_b200 import ops as o
    return o


def test_golden_vectors_on_device(ops, golden):
    g = golden
    # silu
    out = torch.empty(g["silu.x"].size, dtype=torch.int16, device="cuda")
    ops.silu(dev(g["silu.x"]), out, g["silu.x"].size)
    assert np.array_equal(u16(out), g["silu.out"])
    # kv_scatter into zeroed pools
    he = int(g["kv_scatter.head_elems"])
    kp = torch.zeros(g["kv_scatter.out_k"].size, dtype=torch.int16, device="cuda")
    vp = torch.zeros_like(kp)
    ops.kv_scatter(dev(g["kv_scatter.src_k"]), dev(g["kv_scatter.src_v"]), dev(g["kv_scatter.block_table"]),
                   dev(g["kv_scatter.seq_ids"]), dev(g["kv_scatter.positions"]), kp, vp, int(g["kv_scatter.bpr"]),
                   int(g["kv_scatter.block_size"]), he, g["kv_scatter.seq_ids"].size)
    assert np.array_equal(u16(kp), g["kv_scatter.out_k"]) and np.array_equal(u16(vp), g["kv_scatter.out_v"])


@pytest.mark.parametrize("rows,hidden", [(5, 2560), (64, 256), (7, 128), (3, 96), (2, 9216)])
def test_rms_norm_zc_and_add_norm(ops, rows, hidden):
    rs = np.random.default_rng(rows * 1000 + hidden)
    x, y, w = rand_bf16(rs, rows * hidden, 2.0), rand_bf16(rs, rows * hidden, 2.0), rand_bf16(rs, hidden, 0.3)
    out = torch.empty(rows * hidden, dtype=torch.int16, device="cuda")
    ops.rms_norm_zc(dev(x), dev(w), out, rows, hidden, 1e-6)
    assert np.array_equal(u16(out), orc.rms_norm_zc(x, w, rows, hidden, 1e-6))
    s, n = torch.empty_like(out), torch.empty_like(out)
    ops.add_norm_zc(dev(x), dev(y), dev(w), s, n, rows, hidden, 1e-6)
    ws, wn = orc.add_norm_zc(x, y, w, rows, hidden, 1e-6)
    assert np.array_equal(u16(s), ws) and np.array_equal(u16(n), wn)
    # in place (the executor normalises q/k heads in place)
    xd = dev(x)
    ops.rms_norm_zc(xd, dev(w), xd, rows, hidden, 1e-6)
    assert np.array_equal(u16(xd), orc.rms_norm_zc(x, w, rows, hidden, 1e-6))


def test_rms_norm_gated(ops):
    rs = np.random.default_rng(3)
    rows, hidden = 4 * 32, 128
    x, z = rand_bf16(rs, rows * hidden, 1.5), rand_bf16(rs, rows * hidden, 2.0)
    w = (1.0 + 0.1 * rs.standard_normal(hidden)).astype(np.float32)
    out = torch.empty(rows * hidden, dtype=torch.int16, device="cuda")
    ops.rms_norm_gated(dev(x), dev(z), dev(w), out, rows, hidden, 1e-6)
    assert np.array_equal(u16(out), orc.rms_norm_gated(x, z, w, rows, hidden, 1e-6))


def test_rope_pt(ops):
    rs = np.random.default_rng(4)
    tokens, heads, hd, rot = 6, 16, 256, 64
    cos, sin = orc.rope_table(4096, rot // 2, 1e7, round_bf16=True)
    pos = rs.integers(0, 4096, tokens).astype(np.uint32)
    x = rand_bf16(rs, tokens * heads * hd, 2.0)
    want = orc.rope_pt(x, cos, sin, pos, rot, hd, heads)
    out = torch.empty(x.size, dtype=torch.int16, device="cuda")
    ops.rope_pt(dev(x), dev(cos), dev(sin), dev(pos), out, rot, hd, heads, tokens)
    assert np.array_equal(u16(out), want)
    xd = dev(x)
    ops.rope_pt(xd, dev(cos), dev(sin), dev(pos), xd, rot, hd, heads, tokens)
    assert np.array_equal(u16(xd), want)


def test_elementwise(ops):
    rs = np.random.default_rng(5)
    n = 4 * 9216 + 3
    a, b = rand_bf16(rs, n, 3.0), rand_bf16(rs, n, 3.0)
    a[:4] = orc.f32_to_bf16(np.array([0.0, -0.0, 60.0, -100.0], np.float32))
    out = torch.empty(n, dtype=torch.int16, device="cuda")
    for fn, ref in ((ops.add, orc.add), (ops.mul, orc.mul), (ops.silu_mul, orc.silu_mul), (ops.sigmul, orc.sigmul)):
        fn(dev(a), dev(b), out, n)
        assert np.array_equal(u16(out), ref(a, b)), fn.__name__
    ops.silu(dev(a), out, n)
    assert np.array_equal(u16(out), orc.silu(a))


def test_embed(ops):
    rs = np.random.default_rng(6)
    vocab, hidden = 1000, 2560
    w = rand_bf16(rs, vocab * hidden)
    ids = rs.integers(0, vocab, 9).astype(np.uint32)
    out = torch.empty(9 * hidden, dtype=torch.int16, device="cuda")
    ops.embed(dev(ids), dev(w), out, hidden, 9)
    assert np.array_equal(u16(out), orc.embed(ids, w, hidden))


def test_conv_ops_match_reference_semantics(ops):
    """conv1d_dw + conv_state_roll incl. per-position rows (spec_rows.rs:65-111) and the fused verify kernel."""
    rs = np.random.default_rng(7)
    cd, kernel, st = 8192, 4, 3
    pool_rows = 12
    # two chain spans (4 tokens) and one plain span (3 tokens)
    row_start, row_count = np.array([0, 4, 8], np.uint32), np.array([4, 4, 3], np.uint32)
    row_id, specs = np.array([1, 6, 11], np.uint32), np.array([1, 1, 0], np.uint32)
    tokens = 11
    x, w = rand_bf16(rs, tokens * cd, 2.0), rand_bf16(rs, cd * kernel, 0.5)
    state = rand_bf16(rs, pool_rows * cd * st, 2.0)
    tok_row = np.repeat(row_id, row_count).astype(np.uint32)
    tok_pos = np.concatenate([np.arange(c) for c in row_count]).astype(np.uint32)
    want_out = orc.conv1d_dw(x, w, state, tok_row, tok_pos, cd, kernel)
    want_state = orc.conv_state_roll(x, state, row_start, row_count, row_id, cd, kernel, specs)
    out = torch.empty(tokens * cd, dtype=torch.int16, device="cuda")
    sd = dev(state)
    ops.conv1d_dw(dev(x), dev(w), sd, out, dev(tok_row), dev(tok_pos), cd, kernel, tokens)
    ops.conv_state_roll(dev(x), sd, dev(row_start), dev(row_count), dev(row_id), cd, kernel, 3, dev(specs))
    assert np.array_equal(u16(out), want_out)
    assert np.array_equal(u16(sd), want_state)
    # fused chain kernel: chain spans only, snapshot base = head + 1 reproduces the reference rows
    sd2, out2 = dev(state), torch.zeros_like(out)
    ops.conv_verify(dev(x), cd, dev(w), sd2, out2, dev(row_start[:2]), dev(row_count[:2]), dev(row_id[:2]),
                    dev(row_id[:2] + 1), cd, kernel, 2)
    want2 = orc.conv_state_roll(x, state, row_start[:2], row_count[:2], row_id[:2], cd, kernel, specs[:2])
    assert np.array_equal(u16(sd2), want2)
    assert np.array_equal(u16(out2)[: 8 * cd], want_out[: 8 * cd])


def _gdn_case(rs, spans, kh, vh, pool_rows, scale_state=0.5):
    kd = vd = 128
    tokens = int(sum(c for _, c, _, _ in spans))
    q, k = rand_bf16(rs, tokens * kh * kd, 2.0), rand_bf16(rs, tokens * kh * kd, 2.0)
    v = rand_bf16(rs, tokens * vh * vd, 2.0)
    a, b = rand_bf16(rs, tokens * vh, 1.0), rand_bf16(rs, tokens * vh, 1.0)
    a_log = (rs.standard_normal(vh) * 0.5).astype(np.float32)
    dtb = rand_bf16(rs, vh, 0.5)
    state = rand_bf16(rs, pool_rows * vh * vd * kd, scale_state)
    rs_, rc, rid, sp = (np.array([s[i] for s in spans], np.uint32) for i in range(4))
    return dict(q=q, k=k, v=v, a=a, b=b, a_log=a_log, dtb=dtb, state=state, row_start=rs_, row_count=rc, row_id=rid,
                specs=sp, tokens=tokens, kh=kh, vh=vh)


@pytest.mark.parametrize("vsplit", [1, 2, 4])
def test_deltanet_bf16_pool_bit_exact(ops, vsplit):
    """o20 / o27: mixed plain and chain spans in one call, bit-exact state rows and outputs;
    the result does not depend on how v rows are split over warps."""
    rs = np.random.default_rng(8)
    spans = [(0, 4, 1, 1), (4, 3, 7, 0), (7, 1, 9, 0), (8, 5, 10, 1)]  # (start, count, row, spec)
    c = _gdn_case(rs, spans, kh=2, vh=4, pool_rows=17)
    want_out, want_state = orc.deltanet(c["q"], c["k"], c["v"], c["a"], c["b"], c["a_log"], c["dtb"], c["state"],
                                        c["row_start"], c["row_count"], c["row_id"], c["kh"], c["vh"], 128, 128, 1e-6,
                                        c["specs"])
    sd = dev(c["state"])
    out = torch.zeros(c["tokens"] * c["vh"] * 128, dtype=torch.int16, device="cuda")
    ops.deltanet(dev(c["q"]), dev(c["k"]), dev(c["v"]), dev(c["a"]), dev(c["b"]), dev(c["a_log"]), dev(c["dtb"]), sd, out,
                 dev(c["row_start"]), dev(c["row_count"]), dev(c["row_id"]), len(spans), c["kh"], c["vh"], 128, 128,
                 c["tokens"], 1e-6, dev(c["specs"]), vsplit)
    assert np.array_equal(u16(out), want_out)
    assert np.array_equal(u16(sd), want_state)


def test_deltanet_rejects_other_shapes(ops):
    from inferulm_b200.lib import WeinB200Error
    z = torch.zeros(16, dtype=torch.int16, device="cuda")
    with pytest.raises(WeinB200Error):
        ops.deltanet(z, z, z, z, z, z, z, z, z, z, z, z, 1, 1, 1, 64, 64, 1, 1e-6, z, 1)


def test_gdn_verify_f32_pool_and_strided_inputs(ops):
    """The engine-shaped entry: q/k/v read in place from the conv output [T, 2*keyd+vald], a/b from a wider
    projection buffer, explicit snapshot rows (ping-pong banks), f32 pool.  Outputs must equal the oracle's
    f32-state mode bit for bit (same tree, no rounding on store)."""
    rs = np.random.default_rng(9)
    kh, vh = 16, 32
    spans = [(0, 4, 0, 1), (4, 4, 8, 1)]
    c = _gdn_case(rs, spans, kh, vh, pool_rows=16)
    keyd, vald = kh * 128, vh * 128
    cd = 2 * keyd + vald
    T = c["tokens"]
    qkvc = np.zeros((T, cd), np.uint16)
    qkvc[:, :keyd] = c["q"].reshape(T, keyd)
    qkvc[:, keyd:2 * keyd] = c["k"].reshape(T, keyd)
    qkvc[:, 2 * keyd:] = c["v"].reshape(T, vald)
    ab = np.zeros((T, 96), np.uint16)
    ab[:, 32:64] = c["a"].reshape(T, vh)
    ab[:, 64:96] = c["b"].reshape(T, vh)
    state_f = orc.bf16_to_f32(c["state"]).copy()
    in_row, out_base = np.array([0, 8], np.uint32), np.array([4, 12], np.uint32)  # snapshots land in the other bank
    # oracle: chain semantics with contiguous rows; remap rows afterwards
    pool = state_f.reshape(16, -1)
    want_out = np.zeros(T * vh * 128, np.uint16)
    want_pool = pool.copy()
    for s, (t0, cnt, _, _) in enumerate(spans):
        tmp = np.zeros((cnt + 1, pool.shape[1]), np.float32)
        tmp[0] = pool[in_row[s]]
        sl = slice(t0, t0 + cnt)
        o, st = orc.deltanet(c["q"].reshape(T, -1)[sl], c["k"].reshape(T, -1)[sl], c["v"].reshape(T, -1)[sl],
                             c["a"].reshape(T, -1)[sl], c["b"].reshape(T, -1)[sl], c["a_log"], c["dtb"], tmp.reshape(-1),
                             [0], [cnt], [0], kh, vh, 128, 128, 1e-6, [1], state_mode=1, threads=8)
        want_out[t0 * vh * 128:(t0 + cnt) * vh * 128] = o
        want_pool[out_base[s]:out_base[s] + cnt] = st.reshape(cnt + 1, -1)[1:]
    dq = dev(qkvc.reshape(-1))
    dab = dev(ab.reshape(-1))
    sd = dev(state_f)
    out = torch.zeros(T * vh * 128, dtype=torch.int16, device="cuda")
    for rpw in (0, 8, 16, 32):
        sd.copy_(dev(state_f))
        out.zero_()
        ops.gdn_verify(dq, dq[keyd:], dq[2 * keyd:], cd, cd, cd, dab[32:], dab[64:], 96, dev(c["a_log"]), dev(c["dtb"]), sd, 1,
                       out, dev(c["row_start"]), dev(c["row_count"]), dev(in_row), dev(out_base), None, 2, kh, vh, 128, 128,
                       1e-6, rpw)
        assert np.array_equal(u16(out), want_out), rpw
        assert np.array_equal(host(sd, np.float32), want_pool.reshape(-1)), rpw


def test_argmax_rows_total_order(ops):
    """o21 / k1: ties resolve to the lowest index; every scan order gives the reference's answer."""
    rs = np.random.default_rng(10)
    for s, n in ((1, 7), (5, 300), (3, 1024), (4, 151936), (2, 248320)):
        x = rand_bf16(rs, s * n, 4.0).reshape(s, n)
        x[:, 1:4] = orc.f32_to_bf16(np.array([9.0], np.float32))[0]
        if n > 5000:
            x[1, 5000] = orc.f32_to_bf16(np.array([9.0], np.float32))[0]
            x[0, :] = orc.f32_to_bf16(np.array([-np.inf], np.float32))[0]
        rows = np.arange(s, dtype=np.uint32)[::-1].copy()
        scratch = torch.empty(s * ops.ARGMAX_SPLIT, dtype=torch.int64, device="cuda")
        out = torch.empty(s, dtype=torch.int32, device="cuda")
        ops.argmax_rows(dev(x.reshape(-1)), dev(rows), scratch, out, n, s)
        assert np.array_equal(host(out, np.uint32), orc.argmax_rows(x.reshape(-1), rows, n)), (s, n)


@pytest.mark.parametrize("state_f32", [1, 0])
def test_gdn_layer_fusion_equals_operator_chain(ops, state_f32):
    """The one-launch DeltaNet token mixer against the oracle's operator chain conv1d_dw -> conv_state_roll ->
    deltanet -> rms_norm_gated on the BASELINE layer shape (16 qk / 32 v heads), ragged chain lengths, bit for bit."""
    rs = np.random.default_rng(21)
    kh, vh = 16, 32
    keyd, vald = kh * 128, vh * 128
    cd = 2 * keyd + vald
    ld = cd + vald + 2 * vh
    counts = [4, 1, 8, 3]
    n = len(counts)
    T = sum(counts)
    row_start = np.concatenate([[0], np.cumsum(counts)[:-1]]).astype(np.uint32)
    row_count = np.array(counts, np.uint32)
    pool_rows = n * 16
    in_row = (np.arange(n) * 16 + 2).astype(np.uint32)
    out_base = (np.arange(n) * 16 + 8).astype(np.uint32)
    proj = rand_bf16(rs, T * ld, 1.0).reshape(T, ld)
    conv_w = rand_bf16(rs, cd * 4, 0.5)
    conv_state = rand_bf16(rs, pool_rows * cd * 3, 1.0)
    a_log = (rs.standard_normal(vh) * 0.5).astype(np.float32)
    dtb = rand_bf16(rs, vh, 0.5)
    norm_w = (1 + 0.1 * rs.standard_normal(128)).astype(np.float32)
    st16 = rand_bf16(rs, pool_rows * vh * 128 * 128, 0.3)
    state = orc.bf16_to_f32(st16).copy() if state_f32 else st16
    # oracle chain, span by span (rows remapped: the oracle's chain writes head+1.., ours writes out_base..)
    want_out = np.zeros(T * vald, np.uint16)
    want_conv = conv_state.reshape(pool_rows, -1).copy()
    want_state = state.reshape(pool_rows, -1).copy()
    for s in range(n):
        t0, c = int(row_start[s]), counts[s]
        x = proj[t0:t0 + c, :cd].reshape(-1)
        cs = np.zeros((c + 1, cd * 3), np.uint16); cs[0] = conv_state.reshape(pool_rows, -1)[in_row[s]]
        convd = orc.conv1d_dw(x, conv_w, cs.reshape(-1), [0] * c, list(range(c)), cd, 4).reshape(c, cd)
        rolled = orc.conv_state_roll(x, cs.reshape(-1), [0], [c], [0], cd, 4, [1]).reshape(c + 1, -1)
        want_conv[out_base[s]:out_base[s] + c] = rolled[1:]
        ls = np.zeros((c + 1, vh * 128 * 128), state.dtype); ls[0] = state.reshape(pool_rows, -1)[in_row[s]]
        core, st = orc.deltanet(convd[:, :keyd].reshape(-1), convd[:, keyd:2 * keyd].reshape(-1), convd[:, 2 * keyd:].reshape(-1),
                                proj[t0:t0 + c, cd + vald:cd + vald + vh].reshape(-1), proj[t0:t0 + c, cd + vald + vh:].reshape(-1),
                                a_log, dtb, ls.reshape(-1), [0], [c], [0], kh, vh, 128, 128, 1e-6, [1], state_mode=state_f32, threads=8)
        want_state[out_base[s]:out_base[s] + c] = st.reshape(c + 1, -1)[1:]
        z = proj[t0:t0 + c, cd:cd + vald].reshape(-1)
        want_out[t0 * vald:(t0 + c) * vald] = orc.rms_norm_gated(core, z, norm_w, c * vh, 128, 1e-6)
    cs_d, st_d = dev(conv_state), dev(state)
    out = torch.zeros(T * vald, dtype=torch.int16, device="cuda")
    ops.gdn_layer(dev(proj.reshape(-1)), ld, dev(conv_w), cs_d, dev(a_log), dev(dtb), dev(norm_w), st_d, state_f32, out, dev(row_start),
                  dev(row_count), dev(in_row), dev(out_base), n, kh, vh, 1e-6, 1e-6)
    assert np.array_equal(u16(out), want_out)
    assert np.array_equal(u16(cs_d), want_conv.reshape(-1))
    got_state = host(st_d, np.float32 if state_f32 else np.uint16)
    assert np.array_equal(got_state.view(np.uint32 if state_f32 else np.uint16), want_state.reshape(-1).view(np.uint32 if state_f32 else np.uint16))


@pytest.mark.parametrize("state_f32", [1, 0])
def test_gdn_lite_commit_equals_snapshot(ops, state_f32):
    """Snapshot-lite: the layer kernel in log mode followed by gdn_commit leaves, for every accept length a, bit for bit the
    state row that the snapshot path writes at out_base + a; outputs and conv-state rows do not depend on the mode, and the
    log mode writes no state row at all."""
    rs = np.random.default_rng(33)
    kh, vh = 16, 32
    keyd, vald = kh * 128, vh * 128
    cd = 2 * keyd + vald
    ld = cd + vald + 2 * vh
    counts = [4, 1, 8, 3, 5]
    n = len(counts)
    T = sum(counts)
    row_start = np.concatenate([[0], np.cumsum(counts)[:-1]]).astype(np.uint32)
    row_count = np.array(counts, np.uint32)
    pool_rows = n * 16
    in_row = (np.arange(n) * 16 + 2).astype(np.uint32)
    out_base = (np.arange(n) * 16 + 8).astype(np.uint32)
    proj = rand_bf16(rs, T * ld, 1.0)
    conv_w = rand_bf16(rs, cd * 4, 0.5)
    conv_state = rand_bf16(rs, pool_rows * cd * 3, 1.0)
    a_log = (rs.standard_normal(vh) * 0.5).astype(np.float32)
    dtb = rand_bf16(rs, vh, 0.5)
    norm_w = (1 + 0.1 * rs.standard_normal(128)).astype(np.float32)
    st16 = rand_bf16(rs, pool_rows * vh * 128 * 128, 0.3)
    state = orc.bf16_to_f32(st16).copy() if state_f32 else st16
    sdt = np.float32 if state_f32 else np.uint16
    bits = np.uint32 if state_f32 else np.uint16
    args = (dev(proj), ld, dev(conv_w))
    tabs = (dev(row_start), dev(row_count), dev(in_row), dev(out_base))
    # snapshot path
    cs_a, st_a = dev(conv_state), dev(state)
    out_a = torch.zeros(T * vald, dtype=torch.int16, device="cuda")
    ops.gdn_layer(*args, cs_a, dev(a_log), dev(dtb), dev(norm_w), st_a, state_f32, out_a, *tabs, n, kh, vh, 1e-6, 1e-6)
    snap = host(st_a, sdt).view(bits).reshape(pool_rows, -1)
    # log path
    cs_b, st_b = dev(conv_state), dev(state)
    out_b = torch.zeros(T * vald, dtype=torch.int16, device="cuda")
    log = torch.zeros(T * vh * 264, dtype=torch.float32, device="cuda")
    ops.gdn_layer_lite(*args, cs_b, dev(a_log), dev(dtb), dev(norm_w), st_b, state_f32, out_b, *tabs, n, kh, vh, 1e-6, 1e-6, log)
    assert np.array_equal(u16(out_a), u16(out_b))
    assert np.array_equal(u16(cs_a), u16(cs_b))
    assert np.array_equal(host(st_b, sdt).view(bits), state.view(bits))   # untouched
    for trial, acc in enumerate(([3, 0, 7, 1, 2], [0, 0, 0, 0, 0], [3, 0, 7, 2, 4], [9, 9, 9, 9, 9])):
        st_c = dev(state)
        ops.gdn_commit([st_c], [log], state_f32, tabs[0], tabs[1], tabs[2], tabs[3], dev(np.array(acc, np.uint32)), n, vh)
        got = host(st_c, sdt).view(bits).reshape(pool_rows, -1)
        want = state.view(bits).reshape(pool_rows, -1).copy()
        for s_ in range(n):
            a = min(acc[s_], counts[s_] - 1)
            want[out_base[s_] + a] = snap[out_base[s_] + a]
        assert np.array_equal(got, want), trial


@pytest.mark.parametrize("state_f32,lite,spans", [(1, 1, 12), (0, 1, 12), (1, 0, 12), (0, 0, 12), (1, 1, 3), (1, 1, 40), (0, 0, 40)])
def test_gdn_layer_two_launch_path_equals_one_launch(ops, state_f32, lite, spans):
    """Given a scratch and at least 296 (span, v-head) pairs, the per-token operands (conv + SiLU, l2 norms, k-hat / q-hat,
    gates) are made once per span by a launch of their own and persistent CTAs stream the states through shared memory:
    outputs, conv-state rows, state rows or update records are bit for bit those of the one-launch kernel (12 spans: more
    items than CTAs of the test device would be needed to wrap around, so a case with 40 spans is run too)."""
    rs = np.random.default_rng(44)
    kh, vh = 16, 32
    keyd, vald = kh * 128, vh * 128
    cd = 2 * keyd + vald
    ld = cd + vald + 2 * vh
    counts = ([4, 1, 8, 3, 5, 4, 4, 2, 7, 4, 4, 6] * 4)[:spans]
    if spans == 40:
        counts[5] = counts[17] = counts[39] = 0   # refused slots: spans without rows, among them the last item of a CTA
    n = len(counts)
    T = sum(counts)
    row_start = np.concatenate([[0], np.cumsum(counts)[:-1]]).astype(np.uint32)
    row_count = np.array(counts, np.uint32)
    pool_rows = n * 10
    in_row = (np.arange(n) * 10).astype(np.uint32)
    out_base = (np.arange(n) * 10 + 1).astype(np.uint32)
    proj = rand_bf16(rs, T * ld, 1.0)
    conv_w = rand_bf16(rs, cd * 4, 0.5)
    conv_state = rand_bf16(rs, pool_rows * cd * 3, 1.0)
    a_log = (rs.standard_normal(vh) * 0.5).astype(np.float32)
    dtb = rand_bf16(rs, vh, 0.5)
    norm_w = (1 + 0.1 * rs.standard_normal(128)).astype(np.float32)
    st16 = rand_bf16(rs, pool_rows * vh * 128 * 128, 0.3)
    state = orc.bf16_to_f32(st16).copy() if state_f32 else st16
    tabs = (dev(row_start), dev(row_count), dev(in_row), dev(out_base))
    res = []
    for scratch in (None, torch.zeros(T * vh * 388, dtype=torch.float32, device="cuda")):
        cs, st = dev(conv_state), dev(state)
        out = torch.zeros(T * vald, dtype=torch.int16, device="cuda")
        log = torch.zeros(T * vh * 264, dtype=torch.float32, device="cuda") if lite else None
        ops.gdn_layer_ws(dev(proj), ld, dev(conv_w), cs, dev(a_log), dev(dtb), dev(norm_w), st, state_f32, out, *tabs, n, kh, vh,
                         1e-6, 1e-6, log, scratch)
        res.append((u16(out), u16(cs), host(st, np.float32 if state_f32 else np.uint16).view(np.uint32 if state_f32 else np.uint16),
                    host(log, np.float32).view(np.uint32) if lite else None))
    assert np.array_equal(res[0][0], res[1][0])
    assert np.array_equal(res[0][1], res[1][1])
    assert np.array_equal(res[0][2], res[1][2])
    if lite:
        assert np.array_equal(res[0][3], res[1][3])
    assert ops.gdn_wait_timeouts() == 0


def test_snapshot_lite_entries_reject_bad_arguments_and_accept_empty_calls(ops):
    """gdn_layer_lite needs its log, logs must be 16-byte aligned, gdn_commit needs its tables; empty calls succeed."""
    from inferulm_b200.lib import WeinB200Error
    z16 = torch.zeros(4096, dtype=torch.int16, device="cuda")
    z32 = torch.zeros(64, dtype=torch.int32, device="cuda")
    zf = torch.zeros(4096, dtype=torch.float32, device="cuda")
    args = (z16, 64, z16, z16, zf, z16, zf, zf, 1, z16, z32, z32, z32, z32)
    with pytest.raises(WeinB200Error):
        ops.gdn_layer_lite(*args, 1, 16, 32, 1e-6, 1e-6, None)
    with pytest.raises(WeinB200Error):
        ops.gdn_layer_lite(*args, 1, 16, 32, 1e-6, 1e-6, zf[1:])          # misaligned log
    with pytest.raises(WeinB200Error):
        ops.gdn_layer_ws(*args, 1, 15, 32, 1e-6, 1e-6)                    # v_heads not a multiple of k_heads
    ops.gdn_layer_lite(*args, 0, 16, 32, 1e-6, 1e-6, zf)                   # no spans: nothing launched
    ops.gdn_commit([zf], [zf], 1, z32, z32, z32, z32, z32, 0, 32)          # no spans
    tbl = ops.ptr_table([zf])
    with pytest.raises(WeinB200Error):
        ops.gdn_commit(tbl, tbl, 1, None, z32, z32, z32, z32, 1, 32)       # missing table
    torch.cuda.synchronize()
