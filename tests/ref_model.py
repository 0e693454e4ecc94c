"""CPU mirror of the hybrid decoder forward, built from the oracle's operators.

Follows the reference's own CPU model mirror (crates/wein-exec/src/qwen_ref.rs:162-275): one token at a time, the
same operator order and bf16 rounding points as the device forward, GEMMs accumulated in f64 and rounded once.
Test infrastructure only.
"""
import numpy as np

from oracle import oracle as orc


def _np16(t):
    """torch bf16 / int16 tensor -> uint16 numpy bit patterns."""
    import torch
    if t.dtype == torch.bfloat16:
        t = t.view(torch.int16)
    return t.detach().cpu().contiguous().numpy().view(np.uint16).reshape(-1)


def _npf(t):
    return t.detach().cpu().contiguous().numpy().astype(np.float32).reshape(-1)


class RefModel:
    def __init__(self, weights, state_f32=True, max_pos=4096, threads=8):
        self.s = s = weights.shape
        self.th = threads
        self.state_mode = 1 if state_f32 else 0
        self.embed = _np16(weights.embed)
        self.norm_f = _np16(weights.norm_f)
        self.layers = [self._conv_layer(d) for d in weights.layers]
        if s.has_mtp:
            m = weights.mtp
            self.mtp = dict(pre_e=_np16(m["pre_e"]), pre_h=_np16(m["pre_h"]), fc=_np16(m["fc"]), norm=_np16(m["norm"]),
                            layer=self._conv_layer(m["layer"]))
        self.cos, self.sin = orc.rope_table(max_pos, s.rot_dim // 2, s.rope_theta, round_bf16=True)
        self.reset()

    @staticmethod
    def _conv_layer(d):
        out = {}
        for k, v in d.items():
            if k in ("full",):
                out[k] = v
            elif k in ("a_log", "norm"):
                out[k] = _npf(v)
            elif k in ("gu", "proj"):
                continue
            else:
                out[k] = _np16(v)
        return out

    def reset(self):
        s = self.s
        self.pos = 0
        n_full = sum(1 for l in self.layers if l["full"])
        n_lin = len(self.layers) - n_full
        self.k_cache = [np.zeros(0, np.uint16) for _ in range(n_full)]
        self.v_cache = [np.zeros(0, np.uint16) for _ in range(n_full)]
        cd = 2 * s.lin_k_heads * s.lin_k_dim + s.lin_v_heads * s.lin_v_dim
        self.conv_state = [np.zeros(cd * 3, np.uint16) for _ in range(n_lin)]
        n = s.lin_v_heads * s.lin_v_dim * s.lin_k_dim
        self.lin_state = [np.zeros(n, np.float32 if self.state_mode else np.uint16) for _ in range(n_lin)]
        self.last_hidden = None

    def _gemm(self, a, w, m, n, k):
        return orc.gemm_wt_bf16(a, w, m, n, k, threads=self.th)

    def _attn_block(self, w, n1, k_cache, v_cache, rope_pos, kv_list):
        """Single-token full-attention block; kv_list = (k_cache, v_cache) python lists of per-token rows."""
        s = self.s
        h, qh, kvh, hd = s.hidden, s.q_heads, s.kv_heads, s.head_dim
        qg = self._gemm(n1, w["qg"], 1, 2 * qh * hd, h).reshape(qh, 2, hd)
        q, gate = qg[:, 0].reshape(-1), qg[:, 1].reshape(-1)
        q = orc.rms_norm_zc(q, w["qn"], qh, hd, s.rms_eps)
        k = orc.rms_norm_zc(self._gemm(n1, w["k"], 1, kvh * hd, h), w["kn"], kvh, hd, s.rms_eps)
        v = self._gemm(n1, w["v"], 1, kvh * hd, h)
        q = orc.rope_pt(q, self.cos, self.sin, [rope_pos], s.rot_dim, hd, qh)
        k = orc.rope_pt(k, self.cos, self.sin, [rope_pos], s.rot_dim, hd, kvh)
        kc = np.concatenate([k_cache, k])
        vc = np.concatenate([v_cache, v])
        ntok = kc.size // (kvh * hd)
        pages = (ntok + 15) // 16
        pad = pages * 16 * kvh * hd - kc.size
        attn = orc.paged_attn(q, np.concatenate([kc, np.zeros(pad, np.uint16)]), np.concatenate([vc, np.zeros(pad, np.uint16)]),
                              np.arange(pages, dtype=np.uint32), [0], [ntok - 1], 1.0 / np.sqrt(np.float32(hd)), pages, 16, qh, kvh, hd,
                              threads=self.th)
        agated = orc.sigmul(attn, gate)
        return self._gemm(agated, w["o"], 1, h, qh * hd), kc, vc

    def _mlp(self, w, n2):
        s = self.s
        g = self._gemm(n2, w["wg"], 1, s.inter, s.hidden)
        u = self._gemm(n2, w["wu"], 1, s.inter, s.hidden)
        return self._gemm(orc.silu_mul(g, u), w["wd"], 1, s.hidden, s.inter)

    def forward_token(self, token):
        """Advances the state by one token; returns the bf16 logits row (uint16) of this position."""
        s = self.s
        h = s.hidden
        x = orc.embed([token], self.embed, h)
        fi = li = 0
        for w in self.layers:
            n1 = orc.rms_norm_zc(x, w["ln1"], 1, h, s.rms_eps)
            if w["full"]:
                o, self.k_cache[fi], self.v_cache[fi] = self._attn_block(w, n1, self.k_cache[fi], self.v_cache[fi], self.pos, None)
                fi += 1
            else:
                kh, vh, kd, vd = s.lin_k_heads, s.lin_v_heads, s.lin_k_dim, s.lin_v_dim
                keyd, vald = kh * kd, vh * vd
                cd = 2 * keyd + vald
                qkv = self._gemm(n1, w["qkv"], 1, cd, h)
                convd = orc.conv1d_dw(qkv, w["conv"], self.conv_state[li], [0], [0], cd, 4)
                self.conv_state[li] = orc.conv_state_roll(qkv, self.conv_state[li], [0], [1], [0], cd, 4, [0])
                z = self._gemm(n1, w["z"], 1, vald, h)
                a = self._gemm(n1, w["a"], 1, vh, h)
                b = self._gemm(n1, w["b"], 1, vh, h)
                core, self.lin_state[li] = orc.deltanet(convd[:keyd], convd[keyd:2 * keyd], convd[2 * keyd:], a, b, w["a_log"], w["dt_bias"],
                                                        self.lin_state[li], [0], [1], [0], kh, vh, kd, vd, s.l2_eps, [0],
                                                        state_mode=self.state_mode, threads=self.th)
                normed = orc.rms_norm_gated(core, z, w["norm"], vh, vd, s.rms_eps)
                o = self._gemm(normed, w["out"], 1, h, vald)
                li += 1
            h2 = orc.add(x, o)
            n2 = orc.rms_norm_zc(h2, w["ln2"], 1, h, s.rms_eps)
            x = orc.add(h2, self._mlp(w, n2))
        self.last_hidden = x
        xn = orc.rms_norm_zc(x, self.norm_f, 1, h, s.rms_eps)
        self.pos += 1
        return self._gemm(xn, self.embed, 1, s.vocab, h)

    def mtp_draft(self, hidden, tokens_first, k, start_pos, force=None):
        """k greedy drafts of the MTP head (crates/wein-exec/src/qwen.rs:2805-2848, :4435-4522): a clean chain per
        round (chain-local KV), absolute rotary positions, hidden chained through the head's own normalised output.
        Returns per draft (token, logits, normalised hidden fed to the next draft); force[i], when given, replaces draft
        i as the token fed to draft i + 1 (teacher forcing with another implementation's drafts)."""
        s = self.s
        h = s.hidden
        m = self.mtp
        w = m["layer"]
        kc = vc = np.zeros(0, np.uint16)
        hid, tok, out = hidden, tokens_first, []
        for i in range(k):
            e = orc.rms_norm_zc(orc.embed([tok], self.embed, h), m["pre_e"], 1, h, s.rms_eps)
            hh = orc.rms_norm_zc(hid, m["pre_h"], 1, h, s.rms_eps)
            x = self._gemm(np.concatenate([e, hh]), m["fc"], 1, h, 2 * h)
            n1 = orc.rms_norm_zc(x, w["ln1"], 1, h, s.rms_eps)
            o, kc, vc = self._attn_block(w, n1, kc, vc, start_pos + i, None)
            h2 = orc.add(x, o)
            n2 = orc.rms_norm_zc(h2, w["ln2"], 1, h, s.rms_eps)
            x = orc.add(h2, self._mlp(w, n2))
            n2 = orc.rms_norm_zc(x, m["norm"], 1, h, s.rms_eps)
            logits = self._gemm(n2, self.embed, 1, s.vocab, h)
            tok = int(orc.argmax_rows(logits, [0], s.vocab)[0])
            out.append((tok, logits, n2))
            if force is not None:
                tok = int(force[i])
            hid = n2
        return out
