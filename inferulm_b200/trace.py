"""What each kernel of a captured speculative round adds to the round's critical path.

    python -m inferulm_b200.build --trace
    WEIN_B200_TRACE=1 python -m inferulm_b200.trace [--prompt 1024] [--k 3] [--rounds 4]

Uses the diagnostic twin of the library, in which block 0 of every kernel records the global timer when its dependency wait
returns.  Kernels of a round run in dependency order, so the time between two consecutive stamps is the critical-path share of
the earlier kernel (its own run time plus the completion-to-wake-up latency of its successor).  Batch 1, greedy.  Prints the
median interval per kernel class over the timed rounds.  A diagnostic: its numbers are not benchmark values.
"""
import argparse
import collections
import ctypes as C
import os

import numpy as np
import torch

UNITS = "capi ops_exact gdn accept fused_glue attn gemm gemm_stream engine".split()


def round_labels(shape, k):
    """Kernel classes of one round in launch order (k draft forwards, then the verify forward, acceptance and commit)."""
    lab = []
    for _ in range(k):
        lab += ["mtp_prep", "mtp_cat", "gemm fc", "norm", "gemm qg|k|v", "qk_prep", "attn_verify", "attn_combine", "gemm o", "add_norm",
                "gemm gate|up", "gemm down", "add_norm", "gemm lm_head", "argmax_p1", "argmax_finish"]
    lab += ["verify_prep", "embed", "norm"]
    for l in range(shape.n_layers):
        if shape.is_full(l):
            lab += ["gemm qg|k|v", "qk_prep", "attn_verify", "attn_combine", "gemm o", "add_norm", "gemm gate|up", "gemm down", "add_norm"]
        else:
            lab += ["gemm qkv|z|a|b", "gdn_layer", "gemm out", "add_norm", "gemm gate|up", "gemm down", "add_norm"]
    lab += ["gemm lm_head", "argmax_p1", "accept", "gdn_commit", "commit"]
    return lab


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--prompt", type=int, default=1024)
    ap.add_argument("--k", type=int, default=3)
    ap.add_argument("--rounds", type=int, default=4)
    args = ap.parse_args()
    if os.environ.get("WEIN_B200_TRACE") != "1":
        raise SystemExit("set WEIN_B200_TRACE=1 (and build the diagnostic library with `python -m inferulm_b200.build --trace`)")
    from .engine import Engine, ModelShape, SyntheticWeights
    from .lib import load
    lib = load()
    buf = torch.zeros(16384, dtype=torch.int64, device="cuda")
    for u in UNITS:
        getattr(lib, f"wb_trace_set_{u}")(C.c_void_p(buf.data_ptr()))
    shape = ModelShape()
    weights = SyntheticWeights(shape, seed=0, std=0.02)
    k, prompt = args.k, args.prompt
    eng = Engine(weights, max_seqs=1, k_max=k, max_pos=prompt + (args.rounds + 10) * (k + 1) + 64, state_f32=True)
    rs = np.random.default_rng(0)
    eng.admit(0, eng.max_pos, rng=rs)
    eng.prefill([0], [rs.integers(0, shape.vocab, prompt).astype(np.uint32)])
    bound = prompt
    for _ in range(6):
        bound += k + 1
        eng.spec_step([0], k, bound, use_graph=1)
    torch.cuda.synchronize()
    buf.zero_()
    torch.cuda.synchronize()
    for _ in range(args.rounds + 1):     # one extra round closes the last interval of the last timed round
        bound += k + 1
        eng.spec_step([0], k, bound, use_graph=1)
    torch.cuda.synchronize()
    h = buf.cpu().numpy()
    n = int(h[0] & 0xFFFFFFFF)
    labels = round_labels(shape, k)
    per = len(labels)
    if n != per * (args.rounds + 1):
        raise SystemExit(f"{n} stamps for {args.rounds + 1} rounds of {per} kernels: the round's kernel list has changed")
    t = h[1:1 + n].astype(np.int64)
    iv = np.diff(t)[: per * args.rounds].reshape(args.rounds, per)
    med = np.median(iv, axis=0) / 1000.0
    agg = collections.OrderedDict()
    for lab, v in zip(labels, med):
        agg.setdefault(lab, []).append(v)
    total = med.sum()
    print(f"round: {total:.1f} us over {per} kernels (median of {args.rounds} rounds, prompt {prompt}, k = {k})")
    print(f"{'kernel class':18s} {'n':>4s} {'total us':>9s} {'share':>6s} {'avg us':>7s} {'min':>6s} {'max':>6s}")
    for lab, vs in sorted(agg.items(), key=lambda kv: -sum(kv[1])):
        print(f"{lab:18s} {len(vs):4d} {sum(vs):9.1f} {100 * sum(vs) / total:5.1f}% {np.mean(vs):7.2f} {min(vs):6.2f} {max(vs):6.2f}")
    eng.close()


if __name__ == "__main__":
    main()
