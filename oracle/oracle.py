"""ctypes front end of the CPU oracle (oracle/wein_oracle.c).

Test infrastructure only: imported by tests/, the smoke check and the
CPU-baseline leg of the benchmark.  Arrays are numpy: bf16 tensors travel as
uint16 bit patterns, exactly like the reference's own golden files.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libwein_oracle.so")


def build(force=False):
    src = os.path.join(_HERE, "wein_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libwein_oracle.so"], stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = C.CDLL(_SO)
        _lib.orc_bf16_to_f32.restype = C.c_float
        _lib.orc_bf16_to_f32.argtypes = [C.c_uint16]
        _lib.orc_f32_to_bf16.restype = C.c_uint16
        _lib.orc_f32_to_bf16.argtypes = [C.c_float]
        for name in ("orc_expf", "orc_log2f", "orc_softplus"):
            getattr(_lib, name).restype = C.c_float
            getattr(_lib, name).argtypes = [C.c_float]
        _lib.orc_splitmix_f32.restype = C.c_float
        _lib.orc_splitmix_f32.argtypes = [C.c_uint64]
        _lib.orc_rng_seed.restype = C.c_uint64
        _lib.orc_rng_seed.argtypes = [C.c_uint64]
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _u16(a):
    return np.ascontiguousarray(a, dtype=np.uint16)


def _u32(a):
    return np.ascontiguousarray(a, dtype=np.uint32)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


I64 = C.c_int64
F32 = C.c_float
INT = C.c_int


def bf16_to_f32(x):
    """Exact widening of bf16 bit patterns (uint16) to float32."""
    return (np.asarray(x, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(x):
    """Round-to-nearest-even narrowing, the reference's formula (reference.rs:19-23)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


def vec_bf16(seed_hi, n, scale):
    out = np.empty(n, np.uint16)
    lib().orc_vec_bf16(C.c_uint64(seed_hi), I64(n), F32(scale), _p(out))
    return out


def expf(x):
    return float(lib().orc_expf(x))


def splitmix_f32(seed):
    return float(lib().orc_splitmix_f32(seed))


def _ew2(fn, a, b):
    a, b = _u16(a), _u16(b)
    out = np.empty_like(a)
    fn(_p(a), _p(b), _p(out), I64(a.size))
    return out


def silu(x):
    x = _u16(x)
    out = np.empty_like(x)
    lib().orc_silu(_p(x), _p(out), I64(x.size))
    return out


def add(a, b):
    return _ew2(lib().orc_add, a, b)


def mul(a, b):
    return _ew2(lib().orc_mul, a, b)


def silu_mul(g, u):
    return _ew2(lib().orc_silu_mul, g, u)


def sigmul(x, g):
    return _ew2(lib().orc_sigmul, x, g)


def embed(ids, w, hidden):
    ids, w = _u32(ids), _u16(w)
    out = np.empty(ids.size * hidden, np.uint16)
    lib().orc_embed(_p(ids), _p(w), _p(out), I64(ids.size), I64(hidden))
    return out


def rms_norm(x, w, rows, hidden, eps):
    x, w = _u16(x), _u16(w)
    out = np.empty(rows * hidden, np.uint16)
    lib().orc_rms_norm(_p(x), _p(w), _p(out), I64(rows), I64(hidden), F32(eps))
    return out


def rms_norm_zc(x, w, rows, hidden, eps):
    x, w = _u16(x), _u16(w)
    out = np.empty(rows * hidden, np.uint16)
    lib().orc_rms_norm_zc(_p(x), _p(w), _p(out), I64(rows), I64(hidden), F32(eps))
    return out


def add_norm_zc(a, b, w, rows, hidden, eps):
    a, b, w = _u16(a), _u16(b), _u16(w)
    s = np.empty(rows * hidden, np.uint16)
    n = np.empty(rows * hidden, np.uint16)
    lib().orc_add_norm_zc(_p(a), _p(b), _p(w), _p(s), _p(n), I64(rows), I64(hidden), F32(eps))
    return s, n


def rms_norm_gated(x, z, w, rows, hidden, eps):
    x, z, w = _u16(x), _u16(z), _f32(w)
    out = np.empty(rows * hidden, np.uint16)
    lib().orc_rms_norm_gated(_p(x), _p(z), _p(w), _p(out), I64(rows), I64(hidden), F32(eps))
    return out


def rope_table(max_pos, rot_pairs, base, round_bf16=False):
    cos = np.empty(max_pos * rot_pairs, np.float32)
    sin = np.empty(max_pos * rot_pairs, np.float32)
    lib().orc_rope_table(I64(max_pos), I64(rot_pairs), C.c_double(base), _p(cos), _p(sin))
    if round_bf16:  # the executor rounds the table to bf16 first (qwen.rs:1581-1586)
        cos = bf16_to_f32(f32_to_bf16(cos))
        sin = bf16_to_f32(f32_to_bf16(sin))
    return cos, sin


def rope(q, k, cos, sin, pos, rot_dim):
    q, k, cos, sin, pos = _u16(q), _u16(k), _f32(cos), _f32(sin), _u32(pos)
    oq, ok = np.empty_like(q), np.empty_like(k)
    lib().orc_rope(_p(q), _p(k), _p(cos), _p(sin), _p(pos), I64(pos.size), I64(rot_dim), _p(oq), _p(ok))
    return oq, ok


def rope_pt(x, cos, sin, pos, rot_dim, head_dim, heads):
    x, cos, sin, pos = _u16(x), _f32(cos), _f32(sin), _u32(pos)
    out = np.empty_like(x)
    lib().orc_rope_pt(_p(x), _p(cos), _p(sin), _p(pos), I64(pos.size), I64(rot_dim), I64(head_dim), I64(heads), _p(out))
    return out


def kv_scatter(src_k, src_v, block_table, seq_ids, positions, k_pool, v_pool, bpr, block_size, head_elems):
    """Writes into copies of the given pools and returns them."""
    src_k, src_v = _u16(src_k), _u16(src_v)
    bt, sid, pos = _u32(block_table), _u32(seq_ids), _u32(positions)
    k_pool, v_pool = _u16(k_pool).copy(), _u16(v_pool).copy()
    lib().orc_kv_scatter(_p(src_k), _p(src_v), _p(bt), _p(sid), _p(pos), I64(pos.size), I64(bpr), I64(block_size),
                         I64(head_elems), _p(k_pool), _p(v_pool))
    return k_pool, v_pool


def paged_attn(q, k_cache, v_cache, block_table, seq_ids, positions, q_scale, bpr, block_size, q_heads, kv_heads,
               head_dim, threads=1):
    q, k_cache, v_cache = _u16(q), _u16(k_cache), _u16(v_cache)
    bt, sid, pos = _u32(block_table), _u32(seq_ids), _u32(positions)
    out = np.empty(pos.size * q_heads * head_dim, np.uint16)
    lib().orc_paged_attn(_p(q), _p(k_cache), _p(v_cache), _p(bt), _p(sid), _p(pos), _p(out), F32(q_scale), I64(bpr),
                         I64(block_size), I64(q_heads), I64(kv_heads), I64(head_dim), I64(pos.size), INT(threads))
    return out


def conv1d_dw(x, w, state_in, tok_row, tok_pos, conv_dim, kernel):
    x, w, state_in = _u16(x), _u16(w), _u16(state_in)
    tr, tp = _u32(tok_row), _u32(tok_pos)
    out = np.empty(tr.size * conv_dim, np.uint16)
    lib().orc_conv1d_dw(_p(x), _p(w), _p(state_in), _p(tr), _p(tp), I64(tr.size), I64(conv_dim), I64(kernel), _p(out))
    return out


def conv_state_roll(x, state, row_start, row_count, row_id, conv_dim, kernel, specs):
    """Returns the new state pool (a copy)."""
    x, state = _u16(x), _u16(state).copy()
    rs, rc, rid, sp = _u32(row_start), _u32(row_count), _u32(row_id), _u32(specs)
    lib().orc_conv_state_roll(_p(x), _p(state), _p(rs), _p(rc), _p(rid), _p(sp), I64(rs.size), I64(conv_dim), I64(kernel))
    return state


def deltanet(q, k, v, a, b, a_log, dt_bias, state, row_start, row_count, row_id, k_heads, v_heads, k_dim, v_dim,
             l2_eps, specs, state_mode=0, threads=1):
    """state: uint16 pool (state_mode 0) or float32 pool (1: fused, 2: separate mul/add).
    Returns (core_out, new_state_pool)."""
    q, k, v, a, b = _u16(q), _u16(k), _u16(v), _u16(a), _u16(b)
    a_log, dt_bias = _f32(a_log), _u16(dt_bias)
    state = (_u16(state) if state_mode == 0 else _f32(state)).copy()
    rs, rc, rid, sp = _u32(row_start), _u32(row_count), _u32(row_id), _u32(specs)
    total = int((rs.astype(np.int64) + rc).max()) if rs.size else 0
    out = np.zeros(total * v_heads * v_dim, np.uint16)
    lib().orc_deltanet(_p(q), _p(k), _p(v), _p(a), _p(b), _p(a_log), _p(dt_bias), _p(state), INT(state_mode), _p(out),
                       _p(rs), _p(rc), _p(rid), _p(sp), I64(rs.size), I64(k_heads), I64(v_heads), I64(k_dim),
                       I64(v_dim), F32(l2_eps), INT(threads))
    return out, state


def argmax_rows(x, rows, n, threads=1):
    x, rows = _u16(x), _u32(rows)
    out = np.empty(rows.size, np.uint32)
    lib().orc_argmax_rows(_p(x), _p(rows), I64(rows.size), I64(n), _p(out), INT(threads))
    return out


def rng_seed(seed):
    return int(lib().orc_rng_seed(C.c_uint64(seed)))


def sample_rows(x, rows, n, temp, top_k, top_p, seed, slots, rng):
    """rng (uint64 array) is advanced in place, like the device buffer."""
    x, rows = _u16(x), _u32(rows)
    temp, top_k, top_p = _f32(temp), _u32(top_k), _f32(top_p)
    seed = np.ascontiguousarray(seed, dtype=np.uint64)
    slots = _u32(slots)
    assert rng.dtype == np.uint64 and rng.flags.c_contiguous
    out = np.empty(rows.size, np.uint32)
    lib().orc_sample_rows(_p(x), _p(rows), I64(rows.size), I64(n), _p(temp), _p(top_k), _p(top_p), _p(seed), _p(slots),
                          _p(rng), _p(out))
    return out


def gemm_wt(a, w, m, n, k, threads=1):
    a, w = _u16(a), _u16(w)
    c = np.empty(m * n, np.float64)
    lib().orc_gemm_wt(_p(a), _p(w), _p(c), I64(m), I64(n), I64(k), INT(threads))
    return c


def gemm_wt_bf16(a, w, m, n, k, threads=1):
    a, w = _u16(a), _u16(w)
    c = np.empty(m * n, np.uint16)
    lib().orc_gemm_wt_bf16(_p(a), _p(w), _p(c), I64(m), I64(n), I64(k), INT(threads))
    return c


def accept_greedy(drafts, target):
    drafts, target = _u32(drafts), _u32(target)
    k = drafts.size
    emitted = np.zeros(k + 1, np.uint32)
    lib().orc_accept_greedy.restype = INT
    a = lib().orc_accept_greedy(_p(drafts), INT(k), _p(target), _p(emitted))
    return a, emitted[: a + 1]


def philox4x32(ctr, key):
    ctr, key = _u32(ctr), _u32(key)
    out = np.empty(4, np.uint32)
    lib().orc_philox4x32(_p(ctr), _p(key), _p(out))
    return out


def spec_uniforms(seed, rnd, position, stream):
    u = np.empty(4, np.float32)
    lib().orc_spec_uniforms(C.c_uint64(seed), C.c_uint64(rnd), C.c_uint32(position), C.c_uint32(stream), _p(u))
    return u


def filtered_dist(x, n, temp, top_k, top_p):
    x = _u16(x)
    ids = np.empty(64, np.uint32)
    probs = np.empty(64, np.float32)
    lib().orc_filtered_dist.restype = INT
    keep = lib().orc_filtered_dist(_p(x), I64(n), F32(temp), C.c_uint32(top_k), F32(top_p), _p(ids), _p(probs))
    return keep, ids, probs


def draft_sample(ids, probs, n, seed, rnd, position):
    ids, probs = _u32(ids), _f32(probs)
    lib().orc_draft_sample.restype = C.c_uint32
    return int(lib().orc_draft_sample(_p(ids), _p(probs), INT(n), C.c_uint64(seed), C.c_uint64(rnd), C.c_uint32(position)))


def accept_sampled(drafts, p_ids, p_probs, p_n, q_ids, q_probs, q_n, seed, rnd):
    drafts = _u32(drafts)
    k = drafts.size
    p_ids, p_probs, q_ids, q_probs = _u32(p_ids), _f32(p_probs), _u32(q_ids), _f32(q_probs)
    p_n = np.ascontiguousarray(p_n, dtype=np.int32)
    q_n = np.ascontiguousarray(q_n, dtype=np.int32)
    emitted = np.zeros(k + 1, np.uint32)
    lib().orc_accept_sampled.restype = INT
    a = lib().orc_accept_sampled(_p(drafts), INT(k), _p(p_ids), _p(p_probs), _p(p_n), _p(q_ids), _p(q_probs), _p(q_n),
                                 C.c_uint64(seed), C.c_uint64(rnd), _p(emitted))
    return a, emitted[: a + 1]
