"""Adaptive draft length, host side: the reference's per-request policy restated.

Follows `Qwen35Executor::spec_policy_step` (crates/wein-exec/src/qwen.rs:2510-2568), `set_spec` (:2604-2647) and the
probe countdown at the top of `step` (:5263-5280) with the constants of :76-105.  The reference keeps this logic on the
host and so does this package: it only decides the `k` handed to `Engine.spec_step`; nothing here touches the device.

Per request the policy tracks an exponential moving average of accepted / drafted per round:

* EMA >= 0.45 -> k = 3, 0.30 <= EMA < 0.45 -> k = 2, below -> k = 1;
* a round counts as "low" when its own ratio is < 0.15 AND the EMA is < 0.30; three low rounds in a row switch drafting
  off (k = 0) and arm a probe: after 2 << min(off_tries - 1, 3) plain decode steps one round with k = 1 is tried.  The
  reference means the gap to double (2, 4, 8, 16) when a request keeps being switched off, but it clears `off_tries` in every
  round that does not switch off, the two failing rounds before the next switch-off included, so the gap it actually arms
  is 2; this restatement keeps that behaviour;
* a request starts at k = min(cap, 2) until the first round has been observed (the first ratio seeds the EMA).

One difference, stated: the reference clamps to its global maximum of 8 only, so the policy may raise k above the cap given
to `set_spec`; here k is also clamped to the engine's `k_max`, because the engine sizes its chain rows for that many drafts.
"""
from dataclasses import dataclass
from typing import Optional

import numpy as np

F32 = np.float32   # the reference computes ratio and average in f32: thresholds are compared on the same roundings
EMA_ALPHA = F32(0.3)
K_ON = F32(0.45)
K_MID = F32(0.30)
OFF_RATIO = F32(0.15)
OFF_RUNS = 3
PROBE_STEPS = 2
K_COLD = 2
K_MAX = 8
ANCHOR_IDLE = 8


@dataclass
class SpecPolicy:
    """State of one request.  `k` is the draft length to use for its next round (0 = plain decode step)."""
    k_cap: int                      # the k asked for by the caller (set_spec's argument)
    engine_k_max: int = K_MAX       # chain rows the engine was built for
    adaptive: bool = True
    k: int = 0
    ema: Optional[float] = None
    low_run: int = 0
    off_tries: int = 0
    probe: int = 0
    idle: int = 0
    switches: int = 0

    def __post_init__(self):
        cap = min(self.k_cap, K_MAX, self.engine_k_max)
        self.auto = self.adaptive and cap > 0
        self.k = min(cap, K_COLD) if self.auto else cap

    def before_step(self) -> bool:
        """Call once per decode step before choosing k (qwen.rs:5263-5280).  While drafting is off, counts the probe down and
        re-opens with k = 1 when it reaches zero.  Returns True when the request has been off for ANCHOR_IDLE steps, the point
        at which the reference moves its state back to the block-table row (nothing to do for this engine)."""
        if not self.auto:
            return False
        if self.k != 0:
            self.idle = 0
            return False
        if self.probe > 0:
            self.probe -= 1
            self.idle += 1
        else:
            self.k = 1
        if self.idle >= ANCHOR_IDLE:
            self.idle = 0
            return True
        return False

    def observe(self, accepted: int, drafts: int) -> int:
        """Feed the outcome of a round (qwen.rs:2510-2568); returns the k of the next round."""
        if drafts == 0 or not self.auto:
            return self.k
        ratio = F32(accepted) / F32(drafts)
        self.ema = ratio if self.ema is None else F32(F32(EMA_ALPHA * ratio) + F32(F32(F32(1.0) - EMA_ALPHA) * F32(self.ema)))
        ema = self.ema
        self.low_run = self.low_run + 1 if (ratio < OFF_RATIO and ema < K_MID) else 0
        k = 3 if ema >= K_ON else (2 if ema >= K_MID else 1)
        if self.low_run >= OFF_RUNS:
            k = 0
            self.off_tries += 1
            self.low_run = 0
            self.probe = PROBE_STEPS << min(self.off_tries - 1, 3)
        else:
            self.off_tries = 0
        k = min(k, K_MAX, self.engine_k_max)
        if k != self.k:
            self.switches += 1
        self.k = k
        return k


def batch_k(policies) -> int:
    """The round's shape: the batch drafts as far as its most optimistic request.  Every slot still verifies its own draft
    length inside that round (`Engine.set_spec`), as the reference verifies chains of different lengths in one forward."""
    return max((p.k for p in policies), default=0)
