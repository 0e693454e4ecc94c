"""Python harness around the step-level C-ABI (wein_b200_engine_*).

It plays the role the reference's test / probe harness plays for Qwen35Executor
(crates/wein-exec/examples/qwen_spec_probe.rs:193-283): build a model, admit
sequences, prefill, run speculative rounds, read tokens and counters.  torch is
used only to own device memory (the synthetic weights) and the CUDA stream.
"""
import ctypes as C
from dataclasses import dataclass, field

import numpy as np
import torch

from .lib import check, load

MAX_LAYERS = 64


class ModelCfg(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("hidden", "n_layers", "q_heads", "kv_heads", "head_dim", "rot_dim", "inter", "vocab",
                                          "lin_k_heads", "lin_v_heads", "lin_k_dim", "lin_v_dim", "conv_kernel")] + [
        ("rms_eps", C.c_float), ("l2_eps", C.c_float), ("rope_theta", C.c_double), ("layer_is_full", C.c_uint8 * MAX_LAYERS),
        ("has_mtp", C.c_uint32), ("max_seqs", C.c_uint32), ("k_max", C.c_uint32), ("max_pos", C.c_uint32), ("n_pages", C.c_uint32),
        ("state_f32", C.c_uint32), ("attn_seg_pages", C.c_uint32), ("state_snapshots", C.c_uint32)]


_LAYER_FIELDS = ("ln1", "ln2", "wg", "wu", "wd", "qg", "k", "v", "qn", "kn", "o", "qkv", "z", "a", "b", "conv", "a_log", "dt_bias",
                 "norm", "out")


class LayerWeights(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in _LAYER_FIELDS]


class Weights(C.Structure):
    _fields_ = [("embed", C.c_void_p), ("norm_f", C.c_void_p), ("layers", LayerWeights * MAX_LAYERS), ("mtp_pre_e", C.c_void_p),
                ("mtp_pre_h", C.c_void_p), ("mtp_fc", C.c_void_p), ("mtp_norm", C.c_void_p), ("mtp_layer", LayerWeights)]


@dataclass
class ModelShape:
    """Qwen3.5-4B text backbone shape (crates/wein-model/src/config.rs:17-46); full attention at every 4th layer."""
    hidden: int = 2560
    n_layers: int = 32
    q_heads: int = 16
    kv_heads: int = 4
    head_dim: int = 256
    rot_dim: int = 64
    inter: int = 9216
    vocab: int = 151936
    lin_k_heads: int = 16
    lin_v_heads: int = 32
    lin_k_dim: int = 128
    lin_v_dim: int = 128
    conv_kernel: int = 4
    rms_eps: float = 1e-6
    l2_eps: float = 1e-6
    rope_theta: float = 1e7
    full_every: int = 4
    has_mtp: bool = True
    layer_types: list = field(default_factory=list)

    def is_full(self, l):
        if self.layer_types:
            return bool(self.layer_types[l])
        return (l + 1) % self.full_every == 0

    def weight_bytes(self):
        """bf16 bytes one verify forward streams: every layer matrix + the tied embedding once."""
        h, ii = self.hidden, self.inter
        qd, he = self.q_heads * self.head_dim, self.kv_heads * self.head_dim
        keyd, vald = self.lin_k_heads * self.lin_k_dim, self.lin_v_heads * self.lin_v_dim
        mlp = 3 * ii * h
        full = (2 * qd + 2 * he) * h + h * qd + mlp
        lin = (2 * keyd + vald + vald + 2 * self.lin_v_heads) * h + h * vald + mlp
        n_full = sum(self.is_full(l) for l in range(self.n_layers))
        return 2 * (n_full * full + (self.n_layers - n_full) * lin + self.vocab * h)

    def mtp_bytes(self):
        h, ii = self.hidden, self.inter
        qd, he = self.q_heads * self.head_dim, self.kv_heads * self.head_dim
        return 2 * ((2 * qd + 2 * he) * h + h * qd + 3 * ii * h + 2 * h * h + self.vocab * h)


def _randn_bf16(gen, shape, std):
    t = torch.empty(shape, dtype=torch.bfloat16, device="cuda")
    t.normal_(0.0, std, generator=gen)
    return t


class SyntheticWeights:
    """Random-init bf16 weights N(0, std) of the given shape; the projection matrices of a layer are allocated
    adjacently (qkv|z|a|b, qg|k|v, wg|wu) so the engine multiplies each group in one launch."""

    def __init__(self, shape: ModelShape, seed=0, std=0.02):
        self.shape = s = shape
        g = torch.Generator(device="cuda")
        g.manual_seed(seed)
        self.keep = []
        self.c = Weights()
        h, ii = s.hidden, s.inter
        self.embed = _randn_bf16(g, (s.vocab, h), std)
        self.norm_f = _randn_bf16(g, (h,), std)
        self.c.embed, self.c.norm_f = self.embed.data_ptr(), self.norm_f.data_ptr()
        self.layers = []
        for l in range(s.n_layers):
            d = self._layer(g, s.is_full(l), std)
            self.layers.append(d)
            self._fill(self.c.layers[l], d)
        if s.has_mtp:
            self.mtp = dict(pre_e=_randn_bf16(g, (h,), std), pre_h=_randn_bf16(g, (h,), std), fc=_randn_bf16(g, (h, 2 * h), std),
                            norm=_randn_bf16(g, (h,), std), layer=self._layer(g, True, std))
            self.c.mtp_pre_e, self.c.mtp_pre_h = self.mtp["pre_e"].data_ptr(), self.mtp["pre_h"].data_ptr()
            self.c.mtp_fc, self.c.mtp_norm = self.mtp["fc"].data_ptr(), self.mtp["norm"].data_ptr()
            self._fill(self.c.mtp_layer, self.mtp["layer"])
        torch.cuda.synchronize()

    def _layer(self, g, full, std):
        s = self.shape
        h, ii = s.hidden, s.inter
        d = dict(full=full, ln1=_randn_bf16(g, (h,), std), ln2=_randn_bf16(g, (h,), std))
        gu = _randn_bf16(g, (2 * ii, h), std)
        d["gu"], d["wg"], d["wu"] = gu, gu[:ii], gu[ii:]
        d["wd"] = _randn_bf16(g, (h, ii), std)
        if full:
            qd, he = s.q_heads * s.head_dim, s.kv_heads * s.head_dim
            p = _randn_bf16(g, (2 * qd + 2 * he, h), std)
            d["proj"], d["qg"], d["k"], d["v"] = p, p[:2 * qd], p[2 * qd:2 * qd + he], p[2 * qd + he:]
            d["qn"], d["kn"] = _randn_bf16(g, (s.head_dim,), std), _randn_bf16(g, (s.head_dim,), std)
            d["o"] = _randn_bf16(g, (h, qd), std)
        else:
            keyd, vald, vh = s.lin_k_heads * s.lin_k_dim, s.lin_v_heads * s.lin_v_dim, s.lin_v_heads
            cd = 2 * keyd + vald
            p = _randn_bf16(g, (cd + vald + 2 * vh, h), std)
            d["proj"], d["qkv"], d["z"], d["a"], d["b"] = p, p[:cd], p[cd:cd + vald], p[cd + vald:cd + vald + vh], p[cd + vald + vh:]
            d["conv"] = _randn_bf16(g, (cd, s.conv_kernel), 0.3)
            d["a_log"] = torch.empty(vh, dtype=torch.float32, device="cuda").uniform_(-1.0, 1.0, generator=g)
            d["dt_bias"] = _randn_bf16(g, (vh,), 0.5)
            d["norm"] = 1.0 + 0.1 * torch.randn(s.lin_v_dim, dtype=torch.float32, device="cuda", generator=g)
            d["out"] = _randn_bf16(g, (h, vald), std)
        return d

    @staticmethod
    def _fill(cw, d):
        for n in _LAYER_FIELDS:
            setattr(cw, n, d[n].data_ptr() if n in d else None)


class Engine:
    def __init__(self, weights: SyntheticWeights, max_seqs=1, k_max=3, max_pos=4096, n_pages=None, state_f32=True, attn_seg_pages=0,
                 state_snapshots=False):
        s = weights.shape
        self.weights, self.shape = weights, s
        self.lib = load()
        self.lib.wein_b200_engine_buffer.restype = C.c_void_p
        self.lib.wein_b200_engine_device_bytes.restype = C.c_uint64
        cfg = ModelCfg()
        for n in ("hidden", "n_layers", "q_heads", "kv_heads", "head_dim", "rot_dim", "inter", "vocab", "lin_k_heads", "lin_v_heads",
                  "lin_k_dim", "lin_v_dim", "conv_kernel", "rms_eps", "l2_eps", "rope_theta"):
            setattr(cfg, n, getattr(s, n))
        for l in range(s.n_layers):
            cfg.layer_is_full[l] = 1 if s.is_full(l) else 0
        self.bpr = (max_pos + 15) // 16
        self.n_pages = n_pages if n_pages is not None else max_seqs * self.bpr
        cfg.has_mtp, cfg.max_seqs, cfg.k_max, cfg.max_pos, cfg.n_pages = int(s.has_mtp), max_seqs, k_max, max_pos, self.n_pages
        cfg.state_f32, cfg.attn_seg_pages, cfg.state_snapshots = int(state_f32), attn_seg_pages, int(state_snapshots)
        self.cfg, self.max_seqs, self.k_max, self.max_pos = cfg, max_seqs, k_max, max_pos
        # rounds are replayed as CUDA graphs, which cannot be captured on the legacy default stream
        self.stream = torch.cuda.Stream()
        self.h = C.c_void_p()
        check(self.lib.wein_b200_engine_create(C.byref(cfg), C.byref(weights.c), C.byref(self.h)))
        self._free_pages = list(range(self.n_pages))
        self._cap = {}   # slot -> position limit (16 x admitted pages, at most max_pos)

    def close(self):
        if self.h:
            self.lib.wein_b200_engine_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _stream(self):
        return C.c_void_p(self.stream.cuda_stream)

    def device_bytes(self):
        return int(self.lib.wein_b200_engine_device_bytes(self.h))

    def admit(self, slot, n_tokens_cap, temp=0.0, top_k=0, top_p=1.0, seed=0, pages=None, rng=None):
        """Gives the slot pages for n_tokens_cap positions (taken from the free list, shuffled when rng is given)."""
        need = (n_tokens_cap + 15) // 16
        if pages is None:
            if rng is not None:
                rng.shuffle(self._free_pages)
            pages, self._free_pages = self._free_pages[:need], self._free_pages[need:]
            assert len(pages) == need, "out of KV pages"
        arr = (C.c_uint32 * len(pages))(*pages)
        check(self.lib.wein_b200_engine_admit(self.h, C.c_uint32(slot), arr, C.c_uint32(len(pages)), C.c_float(temp), C.c_uint32(top_k),
                                              C.c_float(top_p), C.c_uint64(seed), self._stream()))
        self._cap[slot] = min(self.max_pos, 16 * len(pages))
        return pages

    def resume(self, slot, position, pending_token):
        """Starts an admitted slot at `position` (KV pages and state row written by the caller: a prefix-cache hit)."""
        check(self.lib.wein_b200_engine_resume(self.h, C.c_uint32(slot), C.c_uint32(position), C.c_uint32(pending_token), self._stream()))

    def set_spec(self, slot, k):
        """Per-request draft length: later rounds verify min(round k, k) drafts for the slot (0 = plain decode row)."""
        check(self.lib.wein_b200_engine_set_spec(self.h, C.c_uint32(slot), C.c_uint32(k), self._stream()))

    def prefill(self, slots, prompts):
        slots = list(slots)
        toks = np.concatenate([np.asarray(p, np.uint32) for p in prompts]).astype(np.uint32)
        lens = np.array([len(p) for p in prompts], np.uint32)
        sl = np.array(slots, np.uint32)
        check(self.lib.wein_b200_engine_prefill(self.h, C.c_uint32(len(slots)), sl.ctypes.data_as(C.c_void_p), toks.ctypes.data_as(C.c_void_p),
                                                lens.ctypes.data_as(C.c_void_p), self._stream()))

    def spec_step(self, slots, k, ctx_bound, use_graph=True):
        sl = np.asarray(slots, np.uint32)
        check(self.lib.wein_b200_engine_spec_step(self.h, C.c_uint32(sl.size), sl.ctypes.data_as(C.c_void_p), C.c_uint32(k),
                                                  C.c_uint32(min(ctx_bound, self.max_pos)), C.c_uint32(int(use_graph)), self._stream()))

    def draft(self, slots, k, out=None, use_graph=True):
        """The draft phase alone: k MTP forwards; `out` (int32 CUDA tensor [n, k], optional) receives the drafts."""
        sl = np.asarray(slots, np.uint32)
        check(self.lib.wein_b200_engine_draft(self.h, C.c_uint32(sl.size), sl.ctypes.data_as(C.c_void_p), C.c_uint32(k),
                                              C.c_void_p(out.data_ptr() if out is not None else 0), C.c_uint32(int(use_graph)), self._stream()))

    VERIFY_GRAPH, VERIFY_FORCE_SLOTS, VERIFY_DRY_RUN, VERIFY_ENGINE_DRAFTS = 1, 2, 4, 8

    def spec_verify(self, slots, k, drafts, ctx_bound, n_drafts=None, q=None, use_graph=True, dry_run=False, engine_drafts=False):
        """Verify + accept + commit with the caller's drafts: int32 CUDA tensors drafts [n, k], n_drafts [n] (optional),
        q = (ids [n, k, 64] int32, probs [n, k, 64] float32, counts [n, k] int32) (optional)."""
        sl = np.asarray(slots, np.uint32)
        flags = (self.VERIFY_GRAPH if use_graph else 0) | (self.VERIFY_DRY_RUN if dry_run else 0) | (self.VERIFY_ENGINE_DRAFTS if engine_drafts else 0)
        p = lambda t: C.c_void_p(t.data_ptr() if t is not None else 0)
        qi, qp, qn = q if q is not None else (None, None, None)
        check(self.lib.wein_b200_engine_spec_verify(self.h, C.c_uint32(sl.size), sl.ctypes.data_as(C.c_void_p), C.c_uint32(k), p(drafts), p(n_drafts),
                                                    p(qi), p(qp), p(qn), C.c_uint32(min(ctx_bound, self.max_pos)), C.c_uint32(flags), self._stream()))

    def warm(self, slots, k, ctx_bound, what=1):
        """Captures the graphs of later rounds of this shape (what: 1 spec_step, 2 spec_verify, 4 dry-run verify, 8 draft)."""
        sl = np.asarray(slots, np.uint32)
        check(self.lib.wein_b200_engine_warm(self.h, C.c_uint32(sl.size), sl.ctypes.data_as(C.c_void_p), C.c_uint32(k),
                                             C.c_uint32(min(ctx_bound, self.max_pos)), C.c_uint32(what), self._stream()))

    STATS_WORDS = 24

    def stats(self, slot):
        """All speculation counters of a slot: rounds, drafts, accepted, fallbacks, k switches, rounds by draft count,
        rounds by accept length."""
        w = (C.c_uint64 * self.STATS_WORDS)()
        check(self.lib.wein_b200_engine_stats(self.h, C.c_uint32(slot), w, self._stream()))
        v = [int(x) for x in w]
        return dict(rounds=v[0], drafts=v[1], accepted=v[2], fallbacks=v[3], k_switches=v[4], by_k=v[5:13], by_accept=v[13:22], last_k=v[22])

    def status(self, slot, clear=False):
        v = C.c_uint32()
        check(self.lib.wein_b200_engine_status(self.h, C.c_uint32(slot), C.byref(v), C.c_uint32(int(clear)), self._stream()))
        return v.value

    def timing(self, on):
        """Switches the phase timers of eager rounds on / off; returns the totals (draft, forward, finish) in ms so far."""
        ms = (C.c_double * 3)()
        check(self.lib.wein_b200_engine_timing(self.h, C.c_uint32(int(on)), ms))
        return tuple(float(x) for x in ms)

    def read(self, slot, cap=8192):
        toks = np.zeros(cap, np.uint32)
        n, pos = C.c_uint32(), C.c_uint32()
        stats = (C.c_uint64 * 3)()
        check(self.lib.wein_b200_engine_read(self.h, C.c_uint32(slot), toks.ctypes.data_as(C.c_void_p), C.c_uint32(cap), C.byref(n),
                                             C.byref(pos), stats, self._stream()))
        return toks[: min(n.value, cap)].copy(), pos.value, dict(rounds=int(stats[0]), drafts=int(stats[1]), accepted=int(stats[2]))

    def read_round(self, n):
        """One readback for the batch of the most recent round: array [n, 4 + k_max + 1] of
        (accept length, position, tokens emitted since admission, the round's tokens padded with 0xFFFFFFFF, status word)."""
        stride = 4 + self.k_max + 1
        out = np.empty(n * stride, np.uint32)
        check(self.lib.wein_b200_engine_read_round(self.h, out.ctypes.data_as(C.c_void_p), C.c_uint32(out.size), self._stream()))
        return out.reshape(n, stride)

    def last_launches(self):
        return int(self.lib.wein_b200_engine_last_launches(self.h))

    def buffer(self, name, dtype=torch.int16):
        """Zero-copy view of an engine-owned device buffer (tests and profiling)."""
        nbytes = C.c_uint64()
        p = self.lib.wein_b200_engine_buffer(self.h, name.encode(), C.byref(nbytes))
        if not p:
            raise KeyError(name)
        n = nbytes.value // torch.empty(0, dtype=dtype).element_size()
        tstr = {torch.int16: "<i2", torch.int32: "<i4", torch.int64: "<i8", torch.float32: "<f4", torch.uint8: "|u1"}[dtype]

        class _Holder:
            __cuda_array_interface__ = dict(shape=(n,), typestr=tstr, data=(p, False), version=3)

        return torch.as_tensor(_Holder(), device="cuda")

    def counts(self, slots):
        """(tokens emitted, position) per slot; synchronises the stream."""
        out = []
        for s in slots:
            n, pos = C.c_uint32(), C.c_uint32()
            check(self.lib.wein_b200_engine_read(self.h, C.c_uint32(s), None, C.c_uint32(0), C.byref(n), C.byref(pos), None, self._stream()))
            out.append((n.value, pos.value))
        return out

    def generate(self, slots, n_new, k, use_graph=True):
        """Runs rounds until every slot has emitted n_new tokens since admission; returns the number of rounds.
        No readback sits between the rounds of a burst: the context bound handed to the attention grid is advanced on
        the host by the worst case (k+1 positions per round) and re-based whenever the counters are read."""
        slots = list(slots)
        rounds = 0
        while True:
            cnt = self.counts(slots)
            left = n_new - min(c for c, _ in cnt)
            bound = max(p for _, p in cnt)
            # rounds that certainly stay below every slot's position limit (a round advances a slot by at most k + 1)
            room = min((self._cap.get(s, self.max_pos) - p) // (k + 1) for s, (_, p) in zip(slots, cnt))
            if left <= 0 or room <= 0:
                return rounds
            burst = min(max(1, left // (k + 1)), room)
            for _ in range(burst):
                bound = min(bound + k + 1, self.max_pos)
                self.spec_step(slots, k, bound, use_graph)
                rounds += 1

    def generate_adaptive(self, slots, n_new, k_cap, use_graph=True):
        """As generate(), with each slot's draft length chosen per round by the reference's adaptive policy
        (spec_policy.SpecPolicy, one state per slot, qwen.rs:2510-2568): the round drafts as far as its most optimistic slot
        and every slot verifies its own number of drafts (set_spec), as the reference's per-request k.  The policy needs
        each round's accept counts, so the counters are read back after every round: the host-paced mode the reference
        runs in.  Returns (rounds, list of the round k used)."""
        from .spec_policy import SpecPolicy, batch_k
        slots = list(slots)
        k_max = self.k_max
        pol = {s: SpecPolicy(k_cap=k_cap, engine_k_max=k_max) for s in slots}
        prev = {s: self.read(s, cap=1)[2] for s in slots}
        ks = []
        while True:
            cnt = self.counts(slots)
            bound = max(p for _, p in cnt)
            for p in pol.values():
                p.before_step()
            k = batch_k(pol.values())
            room = min(self._cap.get(s, self.max_pos) - p for s, (_, p) in zip(slots, cnt))
            if n_new - min(c for c, _ in cnt) <= 0 or room < k + 1:
                return len(ks), ks
            for s in slots:
                self.set_spec(s, pol[s].k)
            self.spec_step(slots, k, min(bound + k + 1, self.max_pos), use_graph)
            ks.append(k)
            for s in slots:
                st = self.read(s, cap=1)[2]
                pol[s].observe(st["accepted"] - prev[s]["accepted"], st["drafts"] - prev[s]["drafts"])
                prev[s] = st
