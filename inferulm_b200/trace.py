"""What each kernel of a captured speculative round adds to the round's critical path.

    python -m inferulm_b200.build --trace
    WEIN_B200_TRACE=1 python -m inferulm_b200.trace [--batch 1] [--prompt 1024] [--k 3] [--rounds 4] [--temp 0]

Uses the diagnostic twin of the library, in which block 0 of every kernel records the global timer when its dependency wait
returns, together with the call site of the wait (source file and line, which identify the kernel).  Kernels of a round run in
dependency order, so the time between two consecutive stamps is the critical-path share of the earlier kernel: its own run time
plus the completion-to-wake-up latency of its successor -- and plus any kernel in between that carries no stamp (the library
GEMMs that forwards of more than 32 rows use: their time shows up in the interval of the kernel in front of them).  Prints the
median interval per kernel over the timed rounds.  A diagnostic: its numbers are not benchmark values.
"""
import argparse
import collections
import ctypes as C
import os
import re

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
UNITS = "capi ops_exact gdn accept fused_glue attn gemm gemm_stream engine".split()


def file_id(name):
    h = 2166136261
    for ch in name.encode():
        h = ((h ^ ch) * 16777619) & 0xFFFFFFFF
    return h


def _kernel_name(text):
    """Name of the __global__ function declared on this line (a __launch_bounds__(...) clause may sit in front of it)."""
    i = text.find("__launch_bounds__")
    if i >= 0:
        j, depth = text.find("(", i), 0
        while j >= 0 and j < len(text):
            depth += text[j] == "("
            depth -= text[j] == ")"
            j += 1
            if depth == 0:
                break
        text = text[:i] + text[j:]
    m = re.search(r"__global__\s+void\s+(\w+)\s*\(", text)
    return m.group(1) if m else None


def call_sites():
    """(file id, line) of every dependency wait -> name of the __global__ function around it."""
    sites = {}
    for fn in os.listdir(os.path.join(HERE, "csrc")):
        if not fn.endswith(".cu"):
            continue
        kernel = None
        for no, text in enumerate(open(os.path.join(HERE, "csrc", fn)).read().split("\n"), start=1):
            if "__global__" in text:
                kernel = _kernel_name(text) or kernel
            if "PDL_ENTRY()" in text or "pdl_wait()" in text:
                sites[(file_id(fn), no)] = kernel or f"{fn}:{no}"
    return sites


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--prompt", type=int, default=1024)
    ap.add_argument("--k", type=int, default=3)
    ap.add_argument("--rounds", type=int, default=4)
    ap.add_argument("--temp", type=float, default=0.0)
    args = ap.parse_args()
    if os.environ.get("WEIN_B200_TRACE") != "1":
        raise SystemExit("set WEIN_B200_TRACE=1 (and build the diagnostic library with `python -m inferulm_b200.build --trace`)")
    from .engine import Engine, ModelShape, SyntheticWeights
    from .lib import load
    lib = load()
    buf = torch.zeros(65536, dtype=torch.int64, device="cuda")
    for u in UNITS:
        getattr(lib, f"wb_trace_set_{u}")(C.c_void_p(buf.data_ptr()))
    shape = ModelShape()
    weights = SyntheticWeights(shape, seed=0, std=0.02)
    B, k, prompt = args.batch, args.k, args.prompt
    eng = Engine(weights, max_seqs=B, k_max=k, max_pos=prompt + (args.rounds + 10) * (k + 1) + 64, state_f32=True)
    rs = np.random.default_rng(0)
    slots = list(range(B))
    for s in slots:
        eng.admit(s, eng.max_pos, temp=args.temp, top_k=50 if args.temp > 0 else 0, top_p=0.9 if args.temp > 0 else 1.0, seed=s, rng=rs)
    eng.prefill(slots, [rs.integers(0, shape.vocab, prompt).astype(np.uint32) for _ in slots])
    bound = prompt
    for _ in range(6):
        bound += k + 1
        eng.spec_step(slots, k, bound, use_graph=1)
    torch.cuda.synchronize()
    buf.zero_()
    torch.cuda.synchronize()
    for _ in range(args.rounds + 1):     # one extra round closes the last interval of the last timed round
        bound += k + 1
        eng.spec_step(slots, k, bound, use_graph=1)
    torch.cuda.synchronize()
    h = buf.cpu().numpy()
    n = int(h[0] & 0xFFFFFFFF)
    if n % (args.rounds + 1):
        raise SystemExit(f"{n} stamps do not divide into {args.rounds + 1} equal rounds")
    per = n // (args.rounds + 1)
    t = h[1:1 + 2 * n:2].astype(np.int64)
    tag = h[2:2 + 2 * n:2].astype(np.uint64)
    sites = call_sites()
    names = [sites.get((int(x) >> 32, int(x) & 0xFFFFFFFF), hex(int(x))) for x in tag[:per]]
    iv = np.diff(t)[: per * args.rounds].reshape(args.rounds, per)
    med = np.median(iv, axis=0) / 1000.0
    agg = collections.OrderedDict()
    for name, v in zip(names, med):
        agg.setdefault(name, []).append(v)
    total = med.sum()
    print(f"round: {total:.1f} us over {per} stamped kernels (median of {args.rounds} rounds, batch {B}, prompt {prompt}, k = {k}, temp {args.temp})")
    print(f"{'kernel':28s} {'n':>4s} {'total us':>9s} {'share':>6s} {'avg us':>7s} {'min':>6s} {'max':>6s}")
    for name, vs in sorted(agg.items(), key=lambda kv: -sum(kv[1])):
        print(f"{name:28s} {len(vs):4d} {sum(vs):9.1f} {100 * sum(vs) / total:5.1f}% {np.mean(vs):7.2f} {min(vs):6.2f} {max(vs):6.2f}")
    eng.close()


if __name__ == "__main__":
    main()
