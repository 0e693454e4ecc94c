"""Benchmark of the MTP draft -> verify -> accept round on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c3]

A "step" is one speculative round (k draft forwards, one verify forward over k+1 positions, device acceptance and
commit) over one batch of sequences.  Workload c2 (default, BASELINE config 1): synthetic Qwen3.5-4B-shape hybrid
decoder, random-init bf16 weights N(0, 0.02), greedy MTP k = 3, batch 1, 1024-token uniform-random prompt.  With
N > 1 every rank runs its own sequences on its own GPU (no collective on the data path): weak scaling.

One JSON line is printed by rank 0.  `value` = emitted ("accepted") tokens per second over the K timed rounds,
replayed as CUDA graphs with all inputs resident; `e2e` = the same rounds driven through the public step API with the
per-round host inputs uploaded from pinned memory and the per-round results (tokens, accept counters) read back.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: batch, k, prompt, temp, top_k, top_p
    "c2": dict(batch=1, k=3, prompt=1024, temp=0.0, top_k=0, top_p=1.0,
               desc="Qwen3.5-4B-shape hybrid decoder (24 GDN + 8 GQA, hidden 2560, FFN 9216, vocab 151936), greedy MTP k=3, batch 1, 1024-token prompt"),
    "c4": dict(batch=8, k=4, prompt=32768, temp=0.0, top_k=0, top_p=1.0,
               desc="same model, long context: batch 8, 32768-token prompts (paged bf16 KV, 16-token pages) + f32 recurrent state, greedy k=4"),
    "c3": dict(batch=32, k=3, prompt=2048, temp=0.7, top_k=50, top_p=0.9,
               desc="same model, batch 32, sampled acceptance T=0.7 top-k 50 top-p 0.9, k=3, 2048-token prompts"),
}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler(threading.Thread):
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        super().__init__(daemon=True)
        self.idx, self.rows, self.stop_flag = gpu_index, [], False

    def run(self):
        while not self.stop_flag:
            try:
                out = subprocess.run(["nvidia-smi", f"--id={self.idx}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.rows.append([c.strip() for c in out.split(",")])
            except Exception:
                pass
            time.sleep(0.1)

    def summary(self):
        sm = [float(r[1]) for r in self.rows if r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if r[2].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7), ("sw_power_cap", 8)):
                if len(r) > col and r[col].lower().startswith("active"):
                    reasons.add(name)
        return dict(sm_mhz=float(np.median(sm)) if sm else None, sm_max_mhz=max(mx) if mx else None, reasons=sorted(reasons),
                    samples=len(self.rows))


# ------------------------------------------------------------------------------------------------ CPU baseline (oracle)
def cpu_unit(threads, shape, P=4, ctx=512):
    """Times the reference's CPU kernels (oracle port) on the BASELINE unit: one gated-DeltaNet layer over P positions,
    one GQA layer against a ctx-token paged KV, greedy acceptance over P x vocab logits, and one gate|up projection
    (f64-accumulate GEMM) as the GEMM sample.  Returns seconds per piece."""
    from oracle import oracle as orc
    rs = np.random.default_rng(0)
    kh, vh, kd, vd = shape.lin_k_heads, shape.lin_v_heads, shape.lin_k_dim, shape.lin_v_dim
    r16 = lambda n, sc=1.0: orc.f32_to_bf16((rs.standard_normal(n) * sc).astype(np.float32))
    q, k, v = r16(P * kh * kd), r16(P * kh * kd), r16(P * vh * vd)
    a, b = r16(P * vh), r16(P * vh)
    a_log, dtb = rs.standard_normal(vh).astype(np.float32) * 0.5, r16(vh, 0.5)
    state = (rs.standard_normal((P + 1) * vh * vd * kd) * 0.1).astype(np.float32)
    t = {}
    t0 = time.perf_counter()
    orc.deltanet(q, k, v, a, b, a_log, dtb, state, [0], [P], [0], kh, vh, kd, vd, 1e-6, [1], state_mode=1, threads=threads)
    t["gdn_layer"] = time.perf_counter() - t0
    qh, kvh, hd = shape.q_heads, shape.kv_heads, shape.head_dim
    pages = (ctx + 15) // 16
    kc, vc = r16(pages * 16 * kvh * hd), r16(pages * 16 * kvh * hd)
    qq = r16(P * qh * hd)
    t0 = time.perf_counter()
    orc.paged_attn(qq, kc, vc, rs.permutation(pages).astype(np.uint32), [0] * P, list(range(ctx - P, ctx)), 1.0 / 16.0, pages, 16, qh, kvh, hd,
                   threads=threads)
    t["gqa_layer"] = time.perf_counter() - t0
    lg = r16(P * shape.vocab)
    t0 = time.perf_counter()
    tg = orc.argmax_rows(lg, np.arange(P), shape.vocab, threads=threads)
    orc.accept_greedy(tg[:P - 1], tg)
    t["accept"] = time.perf_counter() - t0
    n, kk = 2 * shape.inter // 8, shape.hidden      # one eighth of a gate|up projection
    A, W = r16(P * kk), r16(n * kk, 0.02)
    t0 = time.perf_counter()
    orc.gemm_wt_bf16(A, W, P, n, kk, threads=threads)
    t["gemm_sample"] = time.perf_counter() - t0
    t["gemm_sample_macs"] = P * n * kk
    return t


def cpu_round_seconds(t, shape, batch, k, ctx):
    """Scales the unit timings to one full round (verify forward of k+1 rows + k draft forwards) of `batch` sequences."""
    P = k + 1
    n_full = sum(shape.is_full(l) for l in range(shape.n_layers))
    n_lin = shape.n_layers - n_full
    macs_verify = (shape.weight_bytes() // 2) * P * batch
    macs_draft = (shape.mtp_bytes() // 2) * batch * k
    gemm = (macs_verify + macs_draft) / t["gemm_sample_macs"] * t["gemm_sample"]
    attn = n_full * t["gqa_layer"] * batch * (ctx / 512.0)
    return gemm + batch * n_lin * t["gdn_layer"] + attn + batch * t["accept"]


def run_reference(args, wl):
    """The reference's CPU implementation of the path (C port of its reference.rs kernels, the Rust toolchain being
    absent), all host threads, each step = one bounded sample unit scaled to a full round."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from inferulm_b200.engine import ModelShape
    shape = ModelShape()
    threads = os.cpu_count() or 1
    for _ in range(min(args.warmup, 1)):
        cpu_unit(threads, shape)
    secs = []
    t_all = time.perf_counter()
    for _ in range(min(args.steps, 8)):
        u = cpu_unit(threads, shape)
        secs.append(cpu_round_seconds(u, shape, wl["batch"], wl["k"], wl["prompt"]))
    wall = time.perf_counter() - t_all
    sec = float(np.median(secs))
    value = wl["batch"] * 1.0 / sec      # one token per sequence per round (draft acceptance of random weights ~ 0)
    line = dict(metric="accepted_tok_per_s", value=value, unit="tok/s", n_gpus=args.gpus, steps=args.steps, warmup=args.warmup,
                ms_per_step=sec * 1e3, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="bf16", data="synthetic",
                impl="reference", config=dict(workload=wl["desc"], name=args.workload),
                cpu_baseline=dict(value=value, unit="tok/s", cores=threads, kind="port",
                                  sample=f"BASELINE unit (1 GDN layer x4 positions, 1 GQA layer ctx 512, accept 4x151936, 1/8 gate|up GEMM) "
                                         f"scaled to a full round; {wall:.1f} s of CPU work"),
                e2e=dict(value=value, unit="tok/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------ our arm
def run_ours(args, wl):
    import torch
    import torch.distributed as dist
    from inferulm_b200.engine import Engine, ModelShape, SyntheticWeights

    from inferulm_b200 import dist_util as du
    rank, world, local = du.rank_world()
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    shape = ModelShape()
    weights = SyntheticWeights(shape, seed=0, std=0.02)
    B, k, prompt_len = wl["batch"], wl["k"], wl["prompt"]
    rounds_total = args.warmup + args.steps
    max_pos = prompt_len + 2 * (rounds_total + 8) * (k + 1) + 64
    eng = Engine(weights, max_seqs=B, k_max=k, max_pos=max_pos, state_f32=True)
    rs = np.random.default_rng(7000 + rank)
    prompts = du.rank_prompts(rank, B, prompt_len, shape.vocab)
    slots = list(range(B))
    for s in slots:
        eng.admit(s, max_pos, temp=wl["temp"], top_k=wl["top_k"], top_p=wl["top_p"], seed=rank * 1000 + s, rng=rs)
    eng.prefill(slots, prompts)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(nrounds, mode):
        """mode 'graph': back-to-back replays, no host work between rounds.  mode 'e2e': every round re-uploads its host
        inputs (the slot table, from pinned memory) and reads its results back (tokens emitted, position, counters)."""
        cnt0 = eng.counts(slots)
        bound = max(p for _, p in cnt0)
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(eng.stream):
            ev0.record(eng.stream)
            for _ in range(nrounds):
                bound = min(bound + k + 1, max_pos)
                eng.spec_step(slots, k, bound, use_graph=3 if mode == "e2e" else 1)
                if mode == "e2e":
                    eng.read_round(len(slots))
            ev1.record(eng.stream)
        barrier()
        ms = ev0.elapsed_time(ev1)
        cnt1 = eng.counts(slots)
        toks = sum(c1 - c0 for (c0, _), (c1, _) in zip(cnt0, cnt1))
        return ms, toks

    timed(args.warmup, "graph")
    sampler = ClockSampler(local)
    sampler.start()
    if args.profile:
        torch.cuda.profiler.start()
    ms, toks = timed(args.steps, "graph")
    if args.profile:
        torch.cuda.profiler.stop()
    sampler.stop_flag = True
    launches = eng.last_launches() * args.steps
    ctx_now = max(p for _, p in eng.counts(slots))
    # the verify step alone (verify forward over k+1 rows + acceptance + commit): the same round with the draft forwards
    # skipped through the library's measurement hook (the verify rows then carry stale draft tokens: timing only)
    import ctypes as C
    eng.lib.wein_b200_engine_ablate(C.c_uint32(16))
    timed(min(args.warmup, 3), "graph")
    ms_verify, _ = timed(args.steps, "graph")
    eng.lib.wein_b200_engine_ablate(C.c_uint32(int(os.environ.get("WEIN_B200_ABLATE", "0"))))
    timed(min(args.warmup, 3), "e2e")
    ms_e2e, toks_e2e = timed(args.steps, "e2e")

    dev0 = torch.device("cuda", local)
    ms_max, toks_all = du.reduce_job(ms, toks, dev0)
    ms_e2e_max, toks_e2e_all = du.reduce_job(ms_e2e, toks_e2e, dev0)
    ms_verify_max, _ = du.reduce_job(ms_verify, 0, dev0)
    stats = [eng.read(s, cap=1)[2] for s in slots]
    acc = sum(s["accepted"] for s in stats) / max(1, sum(s["drafts"] for s in stats))

    # ---- roofline of the dominant kernel: the weight-streaming GEMM, timed alone over the 32 layers' gate|up
    # matrices (94 MB each, 3 GB in rotation: every launch reads its weights from HBM, not from L2)
    peak, peak_kind = peaks()
    from inferulm_b200 import ops
    P = k + 1
    M = B * P
    a_in = torch.randn(M, shape.hidden, device="cuda").to(torch.bfloat16)
    fused = M <= 32   # the engine's launch for this projection: skinny GEMM with the SwiGLU epilogue, else cuBLASLt
    c_out = torch.empty(M, shape.inter if fused else 2 * shape.inter, dtype=torch.bfloat16, device="cuda")
    scratch = torch.zeros(ops.gemm_scratch_bytes(2 * shape.inter) // 4, dtype=torch.int32, device="cuda")
    gus = [d["gu"] for d in weights.layers]

    def one(g):
        if fused:
            ops.gemm_swiglu(a_in, g, c_out, M, shape.inter, shape.hidden, scratch)
        else:
            ops.gemm_wt(a_in, g, c_out, M, 2 * shape.inter, shape.hidden, scratch)

    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for g in gus[:3]:
            one(g)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()   # replayed as a graph so the host's launch rate does not enter the kernel time
    with torch.cuda.graph(graph, stream=side):
        for g in gus:
            one(g)
    graph.replay()
    torch.cuda.synchronize()
    gemm_ms = 1e9
    for _ in range(3):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        gemm_ms = min(gemm_ms, e0.elapsed_time(e1) / len(gus))
    gemm_bytes = 2 * shape.inter * shape.hidden * 2 + M * shape.hidden * 2 + M * (shape.inter if fused else 2 * shape.inter) * 2
    achieved = gemm_bytes / (gemm_ms * 1e-3) / 1e9
    kernel_name = (f"wgemm_kernel (gate|up + SwiGLU) m={M} n={2 * shape.inter} k={shape.hidden}" if fused
                   else f"cuBLASLt gate|up m={M} n={2 * shape.inter} k={shape.hidden}")

    # ---- algorithmic bytes of one round: verify step (weights + state + conv + KV + logits) + k draft forwards
    n_full = sum(shape.is_full(l) for l in range(shape.n_layers))
    n_lin = shape.n_layers - n_full
    st_row = shape.lin_v_heads * 128 * 128 * 4
    conv_row = (2 * shape.lin_k_heads * 128 + shape.lin_v_heads * 128) * 3 * 2
    kv_tok = 2 * shape.kv_heads * shape.head_dim * 2
    # DeltaNet state: with three or more positions the engine logs per-position updates and materialises one state per chain
    # (read by the layer, read + written by the commit: 3 rows, plus the 1056-byte records written and read back); below
    # that, and with WEIN_B200_LITE=0, one row is read and a snapshot per position written (1 + P rows)
    lite = P >= 3 and os.environ.get("WEIN_B200_LITE", "1") != "0"
    state_bytes = (3 * st_row + 2 * P * shape.lin_v_heads * 1056) if lite else (1 + P) * st_row
    verify_bytes = (shape.weight_bytes() + B * n_lin * (state_bytes + (1 + P) * conv_row) + B * n_full * kv_tok * (ctx_now + P)
                    + 2 * B * P * shape.vocab * 2)
    round_bytes = verify_bytes + k * shape.mtp_bytes()
    step_s = ms_max * 1e-3 / args.steps

    if rank == 0:
        cpu = None
        if world == 1 or True:
            threads = os.cpu_count() or 1
            t0 = time.perf_counter()
            u = cpu_unit(threads, shape)
            sec = cpu_round_seconds(u, shape, B, k, ctx_now)
            per_round = toks / max(1, args.steps) / B
            cpu = dict(value=B * per_round / sec, unit="tok/s", cores=threads, kind="port",
                       sample=f"BASELINE unit (1 GDN layer x{P} positions, 1 GQA layer ctx 512, accept {P}x{shape.vocab}, 1/8 gate|up GEMM) "
                              f"scaled to one round at ctx {ctx_now}; {time.perf_counter() - t0:.1f} s of CPU work")
        line = dict(metric="accepted_tok_per_s", value=toks_all / (ms_max * 1e-3), unit="tok/s", n_gpus=world, steps=args.steps,
                    warmup=args.warmup, ms_per_step=ms_max / args.steps, higher_is_better=True, scaling="weak", vs_baseline=None,
                    dtype="bf16", data="synthetic",
                    config=dict(workload=wl["desc"], name=args.workload, batch_per_gpu=B, k=k, prompt=prompt_len, ctx_at_timing=ctx_now,
                                l2="per-round working set (7.9 GB of weights) exceeds L2; no flush needed", state="f32",
                                draft_acceptance=acc, tokens_per_round=toks / max(1, args.steps) / B,
                                # the round is one fixed graph: its time does not depend on how many drafts are accepted, so
                                # the same measurement gives the rate at any acceptance; random weights sit at the floor
                                tok_s_if_every_draft_were_accepted=world * B * (k + 1) / (ms_max / args.steps * 1e-3)),
                    e2e=dict(value=toks_e2e_all / (ms_e2e_max * 1e-3), unit="tok/s", h2d_bytes_per_step=4 * B,
                             d2h_bytes_per_step=B * 4 * (3 + k + 1), ms_per_step=ms_e2e_max / args.steps),
                    gpu_launches=launches,
                    roofline=dict(bound="hbm", achieved=achieved, peak=peak, unit="GB/s", frac=achieved / peak,
                                  traffic=(97.6e6 if fused and M == 4 else None),  # ncu dram read+write per launch, profiles/wgemm_gateup_swiglu_m4.md
                                  kernel=kernel_name, peak_kind=peak_kind,
                                  us_per_launch=gemm_ms * 1e3),
                    verify_step=dict(us=ms_verify_max / args.steps * 1e3, bytes=verify_bytes,
                                     achieved_gbs=verify_bytes / (ms_verify_max / args.steps * 1e-3) / 1e9,
                                     frac_of_measured_peak=verify_bytes / (ms_verify_max / args.steps * 1e-3) / 1e9 / peak,
                                     frac_of_8tbs=verify_bytes / (ms_verify_max / args.steps * 1e-3) / 8e12),
                    state_traffic=("update records + one committed state per chain (3 state rows per layer)" if lite
                                   else "one state snapshot per position (1 + P state rows per layer)"),
                    step_roofline=dict(verify_bytes=verify_bytes, round_bytes=round_bytes, round_us=step_s * 1e6,
                                       achieved_gbs=round_bytes / step_s / 1e9, frac_of_measured_peak=round_bytes / step_s / 1e9 / peak,
                                       frac_of_8tbs=round_bytes / step_s / 8e12),
                    cpu_baseline=cpu, clocks=sampler.summary())
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    eng.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--prompt", type=int, default=0, help="override the workload's prompt length (profiling captures use a short one)")
    ap.add_argument("--profile", action="store_true", help="bracket the timed rounds with cudaProfilerStart/Stop (for ncu --profile-from-start off)")
    args = ap.parse_args()
    wl = dict(WORKLOADS[args.workload])
    if args.prompt:
        wl["prompt"] = args.prompt
    if args.impl == "reference":
        run_reference(args, wl)
    else:
        run_ours(args, wl)


if __name__ == "__main__":
    main()
