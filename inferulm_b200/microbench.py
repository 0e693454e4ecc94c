"""Small, self-contained cases of the hot kernels: CUDA-event timing and the target of `ncu` captures.

    python -m inferulm_b200.microbench gemm|gemm_wt|gdn|gdn_lite|attn|accept|filter [--reps N] [--set NAME=INT ...]

Each case holds well under 2 GB on the device, rotates its big operands through more than the 126 MB L2 so DRAM
figures mean something, launches the kernel a handful of times (eagerly: one kernel per launch, easy to select with
`ncu -k`), and prints one JSON line with the achieved algorithmic GB/s.  The algorithmic bytes are the ones the design
notes give per kernel: weights once for the GEMM, (1 + positions) x 64 KiB per head for the DeltaNet state, the cached
K and V rows once per chain for attention, the logits rows once for acceptance.
"""
import argparse
import json

import numpy as np
import torch

from . import ops

KH, VH = 16, 32
KEYD, VALD = KH * 128, VH * 128
CD = 2 * KEYD + VALD
LD = CD + VALD + 2 * VH


def _time(fn, n_launch, reps):
    for i in range(min(2, n_launch)):
        fn(i)
    torch.cuda.synchronize()
    best = 1e9
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(n_launch):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) / n_launch)
    return best * 1e-3


def _graph_time(one, n_mat, reps):
    """Seconds per launch of `one(i)`, i = 0..n_mat-1, replayed as one CUDA graph (the host's launch rate stays out)."""
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        one(0)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        for i in range(n_mat):
            one(i)
    return _time(lambda i: g.replay(), 1, reps) / n_mat


def case_gemm(reps, m=4, inter=9216, k=2560, n_mat=8, tc=-1, graph=1):
    """gate|up projection with the SwiGLU epilogue (the round's dominant launch), 8 matrices of 94 MB in rotation.
    tc = 1 forces the tensor-memory kernel, 0 the register-streaming kernel (m <= 32), -1 = by m; graph = 0 launches eagerly
    (one kernel per launch, easy to select with `ncu -k`; the host launch gap is then inside the time)."""
    tc = (m > 32) if tc < 0 else bool(tc)
    ws = [torch.randn(2 * inter, k, device="cuda").to(torch.bfloat16) * 0.02 for _ in range(n_mat)]
    a = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    out = torch.empty(m, inter, dtype=torch.bfloat16, device="cuda")
    one = lambda i: ops.gemm_swiglu(a, ws[i], out, m, inter, k, tc=tc)
    sec = _graph_time(one, n_mat, reps) if graph else _time(one, n_mat, reps)
    byt = 2 * inter * k * 2 + m * k * 2 + m * inter * 2
    return dict(kernel=("ugemm_kernel" if tc else "wgemm_kernel") + " (gate|up + SwiGLU)", m=m, n=2 * inter, k=k, us=sec * 1e6, bytes=byt, gbs=byt / sec / 1e9,
                timeouts=ops.gemm_wait_timeouts(), graph=bool(graph), plan=ops.gemm_plan(m, inter, k, True) if tc else None)


def case_gemm_wt(reps, m=128, n=2560, k=9216, tc=-1, graph=1):
    """A plain product C[m,n] = A W^T over enough matrices to exceed L2 several times; graph = 1 replays the launches as one
    CUDA graph so the host's launch rate does not enter the kernel time."""
    tc = (m > 32) if tc < 0 else bool(tc)
    n_mat = max(4, int(1.5e9 // (n * k * 2)))
    n_mat = min(n_mat, 48)
    ws = [torch.randn(n, k, device="cuda").to(torch.bfloat16) * 0.02 for _ in range(n_mat)]
    a = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    one = lambda i: ops.gemm_wt(a, ws[i], out, m, n, k, tc=tc)
    byt = n * k * 2 + m * k * 2 + m * n * 2
    sec = _graph_time(one, n_mat, reps) if graph else _time(one, n_mat, reps)
    return dict(kernel="ugemm_kernel" if tc else "wgemm_kernel", m=m, n=n, k=k, us=sec * 1e6, bytes=byt, gbs=byt / sec / 1e9, matrices=n_mat,
                timeouts=ops.gemm_wait_timeouts(), plan=ops.gemm_plan(m, n, k) if tc else None)


def case_gdn(reps, B=32, P=4, n_layers=2):
    """One DeltaNet layer (fused conv + recurrence + gated norm), f32 state, B chains of P positions."""
    T = B * P
    proj = torch.randn(T, LD, device="cuda").to(torch.bfloat16)
    conv_w = (torch.randn(CD, 4, device="cuda") * 0.3).to(torch.bfloat16)
    rows = B * 2 * P
    a_log = torch.randn(VH, device="cuda")
    dtb = torch.randn(VH, device="cuda").to(torch.bfloat16)
    nw = torch.ones(128, device="cuda")
    states = [torch.randn(rows * VH * 128 * 128, device="cuda") * 0.1 for _ in range(n_layers)]
    convs = [torch.randn(rows * CD * 3, device="cuda").to(torch.bfloat16) for _ in range(n_layers)]
    out = torch.empty(T * VALD, dtype=torch.bfloat16, device="cuda")
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    rs, rc = i32([b * P for b in range(B)]), i32([P] * B)
    ir, ob = i32([b * 2 * P for b in range(B)]), i32([b * 2 * P + P for b in range(B)])
    pf = proj.view(-1)
    sec = _time(lambda i: ops.gdn_layer(pf, LD, conv_w, convs[i], a_log, dtb, nw, states[i], 1, out, rs, rc, ir, ob, B, KH, VH, 1e-6, 1e-6),
                n_layers, reps)
    byt = B * VH * (1 + P) * 65536 + B * (1 + P) * CD * 3 * 2 + T * LD * 2 + T * VALD * 2
    return dict(kernel="gdn_layer_kernel<f32>", batch=B, positions=P, us=sec * 1e6, bytes=byt, gbs=byt / sec / 1e9)


def case_gdn_lite(reps, B=32, P=4, n_layers=2, accept=3):
    """Snapshot-lite pair: the layer kernel in log mode (state only read, 1 KiB update record per position and head) and
    the commit kernel that replays records 0..accept on the input state and stores the one kept row, over n_layers layers."""
    T = B * P
    proj = torch.randn(T, LD, device="cuda").to(torch.bfloat16)
    conv_w = (torch.randn(CD, 4, device="cuda") * 0.3).to(torch.bfloat16)
    rows = B * 2 * P
    a_log = torch.randn(VH, device="cuda")
    dtb = torch.randn(VH, device="cuda").to(torch.bfloat16)
    nw = torch.ones(128, device="cuda")
    states = [torch.randn(rows * VH * 128 * 128, device="cuda") * 0.1 for _ in range(n_layers)]
    convs = [torch.randn(rows * CD * 3, device="cuda").to(torch.bfloat16) for _ in range(n_layers)]
    logs = [torch.zeros(T * VH * 264, device="cuda") for _ in range(n_layers)]
    kq = torch.zeros(T * VH * 388, device="cuda")
    out = torch.empty(T * VALD, dtype=torch.bfloat16, device="cuda")
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    rs, rc = i32([b * P for b in range(B)]), i32([P] * B)
    ir, ob = i32([b * 2 * P for b in range(B)]), i32([b * 2 * P + P for b in range(B)])
    acc = i32([accept] * B)
    pf = proj.view(-1)
    sec_layer = _time(lambda i: ops.gdn_layer_ws(pf, LD, conv_w, convs[i], a_log, dtb, nw, states[i], 1, out, rs, rc, ir, ob, B, KH, VH,
                                                 1e-6, 1e-6, logs[i], kq), n_layers, reps)
    sp, lp = ops.ptr_table(states), ops.ptr_table(logs)
    sec_commit = _time(lambda i: ops.gdn_commit(sp, lp, 1, rs, rc, ir, ob, acc, B, VH), 1, reps)
    byt_layer = B * VH * 65536 + B * P * VH * 1056 + B * (1 + P) * CD * 3 * 2 + T * LD * 2 + T * VALD * 2
    byt_commit = n_layers * B * VH * (2 * 65536 + (accept + 1) * 1056)
    return dict(kernel="gdn_pre_kernel + gdn_layer_kernel<f32> (log mode); gdn_commit_kernel<f32>", batch=B, positions=P, layer_us=sec_layer * 1e6,
                layer_bytes=byt_layer, layer_gbs=byt_layer / sec_layer / 1e9, commit_layers=n_layers, commit_us=sec_commit * 1e6,
                commit_bytes=byt_commit, commit_gbs=byt_commit / sec_commit / 1e9)


def case_attn(reps, B=8, ctx=8192, P=4, n_pools=2, seg_pages=16):
    """Paged GQA verify attention: B chains of P query positions against ctx cached tokens, 16 q / 4 kv heads, d = 256."""
    qh, kvh, hd = 16, 4, 256
    he = kvh * hd
    bpr = (ctx + P + 15) // 16
    n_pages = B * bpr
    pools = [(torch.randn(n_pages * 16 * he, device="cuda").to(torch.bfloat16), torch.randn(n_pages * 16 * he, device="cuda").to(torch.bfloat16))
             for _ in range(n_pools)]
    rs = np.random.default_rng(0)
    bt = torch.from_numpy(rs.permutation(n_pages).astype(np.int32)).cuda()
    T = B * P
    q = torch.randn(T * qh * hd, device="cuda").to(torch.bfloat16)
    seq = torch.arange(B, dtype=torch.int32, device="cuda").repeat_interleave(P)
    pos = (torch.arange(P, dtype=torch.int32, device="cuda") + ctx).repeat(B)
    row_start = torch.arange(B, dtype=torch.int32, device="cuda") * P
    row_count = torch.full((B,), P, dtype=torch.int32, device="cuda")
    out = torch.empty_like(q)
    max_ctx = ctx + P
    max_segs = ((max_ctx + 15) // 16 + seg_pages - 1) // seg_pages
    scratch = torch.empty(ops.attn_scratch_bytes(B, kvh, hd, max_segs) // 4, dtype=torch.float32, device="cuda")
    sec = _time(lambda i: ops.attn_verify(q, pools[i][0], pools[i][1], bt, seq, pos, row_start, row_count, None, out, 1.0 / 16.0, bpr, 16, qh,
                                          kvh, hd, B, P, max_ctx, seg_pages, scratch), n_pools, reps)
    byt = B * 2 * he * 2 * (ctx + P)
    return dict(kernel="attn_verify_kernel<256> + attn_combine_kernel", batch=B, ctx=ctx, positions=P, seg_pages=seg_pages, us=sec * 1e6,
                bytes=byt, gbs=byt / sec / 1e9)


def case_accept(reps, B=32, k=3, V=151936, n_buf=4):
    """Greedy acceptance over B x (k+1) bf16 logits rows of the 151,936-token vocabulary."""
    T = B * (k + 1)
    logits = [torch.randn(T * V, device="cuda").to(torch.bfloat16) for _ in range(n_buf)]
    rows = torch.arange(T, dtype=torch.int32, device="cuda")
    drafts = torch.randint(0, V, (B * k,), dtype=torch.int32, device="cuda")
    scratch = torch.empty(T * 32, dtype=torch.int64, device="cuda")
    al = torch.empty(B, dtype=torch.int32, device="cuda")
    out = torch.empty(T, dtype=torch.int32, device="cuda")
    sec = _time(lambda i: ops.accept_greedy(logits[i], rows, drafts, None, V, B, k, scratch, al, out), n_buf, reps)
    byt = T * V * 2
    return dict(kernel="argmax_p1_kernel + accept_kernel", batch=B, k=k, vocab=V, us=sec * 1e6, bytes=byt, gbs=byt / sec / 1e9)


def case_filter(reps, S=128, V=151936, top_k=50, n_buf=3):
    """Temperature / top-k / top-p filter of S bf16 logits rows (one CTA per row) into compact renormalised distributions."""
    logits = [torch.randn(S * V, device="cuda").to(torch.bfloat16) for _ in range(n_buf)]
    rows = torch.arange(S, dtype=torch.int32, device="cuda")
    temp = torch.full((S,), 0.7, device="cuda")
    tk = torch.full((S,), top_k, dtype=torch.int32, device="cuda")
    tp = torch.full((S,), 0.9, device="cuda")
    ids = torch.zeros(S * 64, dtype=torch.int32, device="cuda")
    pr = torch.zeros(S * 64, device="cuda")
    nn = torch.zeros(S, dtype=torch.int32, device="cuda")
    sec = _time(lambda i: ops.topk_filter(logits[i], rows, rows, 1, temp, tk, tp, V, S, ids, pr, nn), n_buf, reps)
    byt = 2 * S * V * 2   # two passes over the row
    return dict(kernel="topk_filter_kernel", rows=S, vocab=V, top_k=top_k, us=sec * 1e6, bytes=byt, gbs=byt / sec / 1e9,
                kept_mean=float(nn.float().mean()))


CASES = dict(gemm=case_gemm, gemm_wt=case_gemm_wt, gdn=case_gdn, gdn_lite=case_gdn_lite, attn=case_attn, accept=case_accept, filter=case_filter)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=sorted(CASES))
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--set", action="append", default=[], metavar="NAME=INT", help="override a case parameter, e.g. --set ctx=32768")
    args = ap.parse_args()
    torch.manual_seed(0)
    kw = {k: int(v) for k, v in (kv.split("=") for kv in args.set)}
    print(json.dumps(CASES[args.case](args.reps, **kw)))


if __name__ == "__main__":
    main()
