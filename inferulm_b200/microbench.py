"""Small, self-contained cases of the hot kernels: CUDA-event timing and the target of `ncu` captures.

    python -m inferulm_b200.microbench gemm|gdn|attn|accept [--reps N]

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


def case_gemm(reps, m=4, inter=9216, k=2560, n_mat=8):
    """gate|up projection with the SwiGLU epilogue (the round's dominant launch), m = 4 rows, 8 matrices of 94 MB."""
    ws = [torch.randn(2 * inter, k, device="cuda").to(torch.bfloat16) * 0.02 for _ in range(n_mat)]
    a = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    out = torch.empty(m, inter, dtype=torch.bfloat16, device="cuda")
    scratch = torch.zeros(ops.gemm_scratch_bytes(2 * inter) // 4, dtype=torch.int32, device="cuda")
    sec = _time(lambda i: ops.gemm_swiglu(a, ws[i], out, m, inter, k, scratch), n_mat, reps)
    byt = 2 * inter * k * 2 + m * k * 2 + m * inter * 2
    return dict(kernel="wgemm_kernel (gate|up + SwiGLU)", m=m, n=2 * inter, k=k, us=sec * 1e6, bytes=byt, gbs=byt / sec / 1e9,
                note="eager launches: the host launch gap is inside the time; bench.py times the same kernel by graph replay")


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


CASES = dict(gemm=case_gemm, gdn=case_gdn, attn=case_attn, accept=case_accept)


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
