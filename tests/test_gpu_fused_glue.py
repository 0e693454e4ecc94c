"""GPU parity of the fused glue kernels the forward passes launch, each against the chain of reference operators it
replaces (crates/wein-exec/src/qwen.rs:3888-3950 full-attention prologue, :4451-4468 MTP input, :4090-4099 SwiGLU),
bit for bit through the C-ABI."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests.gpu_util import dev, rand_bf16, u16

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from inferulm_b200 import ops as o
    return o


@pytest.mark.parametrize("q_heads,kv_heads,hd,rot,tokens", [(16, 4, 256, 64, 5), (8, 2, 64, 32, 9), (4, 4, 128, 128, 3)])
def test_qk_prep_equals_operator_chain(ops, q_heads, kv_heads, hd, rot, tokens):
    """q / gate split + q-norm + k-norm + partial rotary + KV scatter in one launch == embed-gather, rms_norm_zc,
    rope_pt and kv_scatter of the oracle run one after another."""
    rs = np.random.default_rng(q_heads * 100 + hd + tokens)
    qd, he = q_heads * hd, kv_heads * hd
    ld = 2 * qd + 2 * he + 32                      # a wider row than needed: the kernel must honour the stride
    bpr, nseq, max_pos = 6, 3, 6 * 16
    n_pages = nseq * bpr + 2
    rows = rand_bf16(rs, tokens * ld, 1.5).reshape(tokens, ld)
    qn, kn = rand_bf16(rs, hd, 0.3), rand_bf16(rs, hd, 0.3)
    cos, sin = orc.rope_table(max_pos, rot // 2, 1e7, round_bf16=True)
    bt = rs.permutation(n_pages)[: nseq * bpr].astype(np.uint32)
    seq_ids = rs.integers(0, nseq, tokens).astype(np.uint32)
    # distinct (sequence, position) pairs so no two rows land in the same page slot
    kv_pos = np.array([(7 * t + 3) % max_pos for t in range(tokens)], np.uint32)
    rope_pos = np.array([(11 * t + 5) % max_pos for t in range(tokens)], np.uint32)   # draft rows rotate by another index
    k_pool0, v_pool0 = rand_bf16(rs, n_pages * 16 * he), rand_bf16(rs, n_pages * 16 * he)

    qg = rows[:, : 2 * qd].reshape(tokens, q_heads, 2, hd)
    q_raw = np.ascontiguousarray(qg[:, :, 0]).reshape(-1)
    gate_want = np.ascontiguousarray(qg[:, :, 1]).reshape(-1)
    k_raw = np.ascontiguousarray(rows[:, 2 * qd: 2 * qd + he]).reshape(-1)
    v_raw = np.ascontiguousarray(rows[:, 2 * qd + he: 2 * qd + 2 * he]).reshape(-1)
    qh_want = orc.rope_pt(orc.rms_norm_zc(q_raw, qn, tokens * q_heads, hd, 1e-6), cos, sin, rope_pos, rot, hd, q_heads)
    k_want = orc.rope_pt(orc.rms_norm_zc(k_raw, kn, tokens * kv_heads, hd, 1e-6), cos, sin, rope_pos, rot, hd, kv_heads)
    kp_want, vp_want = orc.kv_scatter(k_want, v_raw, bt, seq_ids, kv_pos, k_pool0.copy(), v_pool0.copy(), bpr, 16, he)

    qh = torch.zeros(tokens * qd, dtype=torch.int16, device="cuda")
    gate = torch.zeros_like(qh)
    kp, vp = dev(k_pool0), dev(v_pool0)
    ops.qk_prep(dev(rows.reshape(-1)), ld, dev(qn), dev(kn), dev(cos), dev(sin), dev(rope_pos), dev(kv_pos), dev(seq_ids), dev(bt), bpr,
                qh, gate, kp, vp, tokens, q_heads, kv_heads, hd, rot, 1e-6)
    assert np.array_equal(u16(qh), qh_want)
    assert np.array_equal(u16(gate), gate_want)
    assert np.array_equal(u16(kp), kp_want) and np.array_equal(u16(vp), vp_want)


@pytest.mark.parametrize("rows,hidden,gather", [(4, 2560, True), (7, 512, False), (3, 4096, True)])
def test_mtp_cat_equals_operator_chain(ops, rows, hidden, gather):
    """[norm(embed[tok]) | norm(hidden row)] == embed gather + 2 x rms_norm_zc + concatenation of the oracle."""
    rs = np.random.default_rng(rows + hidden)
    vocab, pool_rows = 97, 11
    emb = rand_bf16(rs, vocab * hidden, 0.5)
    hid = rand_bf16(rs, pool_rows * hidden, 2.0)
    pre_e, pre_h = rand_bf16(rs, hidden, 0.3), rand_bf16(rs, hidden, 0.3)
    tok = rs.integers(0, vocab, rows).astype(np.uint32)
    hid_rows = rs.permutation(pool_rows)[:rows].astype(np.uint32) if gather else None
    e = orc.rms_norm_zc(orc.embed(tok, emb, hidden), pre_e, rows, hidden, 1e-6).reshape(rows, hidden)
    src = hid.reshape(pool_rows, hidden)[hid_rows if gather else np.arange(rows)]
    h = orc.rms_norm_zc(np.ascontiguousarray(src).reshape(-1), pre_h, rows, hidden, 1e-6).reshape(rows, hidden)
    want = np.concatenate([e, h], axis=1).reshape(-1)
    cat = torch.zeros(rows * 2 * hidden, dtype=torch.int16, device="cuda")
    ops.mtp_cat(dev(tok), dev(emb), dev(hid), dev(hid_rows) if gather else None, dev(pre_e), dev(pre_h), cat, rows, hidden, 1e-6)
    assert np.array_equal(u16(cat), want)


@pytest.mark.parametrize("rows,inter,pad", [(4, 9216, 0), (33, 1024, 64), (1, 34, 2)])
def test_silu_mul_rows_equals_silu_mul(ops, rows, inter, pad):
    rs = np.random.default_rng(rows + inter)
    ld = 2 * inter + pad
    gu = rand_bf16(rs, rows * ld, 2.0).reshape(rows, ld)
    want = orc.silu_mul(np.ascontiguousarray(gu[:, :inter]).reshape(-1), np.ascontiguousarray(gu[:, inter:2 * inter]).reshape(-1))
    out = torch.zeros(rows * inter, dtype=torch.int16, device="cuda")
    ops.silu_mul_rows(dev(gu.reshape(-1)), ld, out, rows, inter)
    assert np.array_equal(u16(out), want)


@pytest.mark.parametrize("m,inter,k", [(4, 9216, 2560), (1, 9216, 2560), (20, 1024, 512), (32, 9216, 2560)])
def test_gemm_swiglu_default_path(ops, m, inter, k):
    """The gate|up projection with the SwiGLU epilogue on the kernel the engine launches by default: bit-equal to its own
    plain product over [gate; up] followed by the oracle's silu_mul, and the plain product within the reference's GEMM
    criterion against an f64 product (crates/wein-kernel/tests/gemm.rs:11)."""
    rs = np.random.default_rng(m * 7 + inter + k)
    a, w = rand_bf16(rs, m * k, 1.0), rand_bf16(rs, 2 * inter * k, 0.05)
    ad, wd = dev(a), dev(w)
    gu = torch.zeros(m * 2 * inter, dtype=torch.int16, device="cuda")
    ops.gemm_wt(ad, wd, gu, m, 2 * inter, k)
    guh = u16(gu).reshape(m, 2 * inter)
    ref = orc.bf16_to_f32(a).reshape(m, k).astype(np.float64) @ orc.bf16_to_f32(w).reshape(2 * inter, k).astype(np.float64).T
    got = orc.bf16_to_f32(guh.reshape(-1)).astype(np.float64).reshape(m, 2 * inter)
    assert (np.abs(got - ref) <= np.maximum(2.0 ** -7 * np.abs(ref), 2.0 ** -11)).all()
    want = orc.silu_mul(np.ascontiguousarray(guh[:, :inter]).reshape(-1), np.ascontiguousarray(guh[:, inter:]).reshape(-1))
    out = torch.zeros(m * inter, dtype=torch.int16, device="cuda")
    ops.gemm_swiglu(ad, wd, out, m, inter, k)
    assert np.array_equal(u16(out), want)
