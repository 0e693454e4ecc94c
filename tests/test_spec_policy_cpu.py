"""Host-side adaptive draft length: the reference's policy (crates/wein-exec/src/qwen.rs:2510-2568, :2604-2647, :5263-5280)
replayed on scripted acceptance sequences."""
import numpy as np

from inferulm_b200.spec_policy import SpecPolicy, batch_k


def test_cold_start_and_bands():
    p = SpecPolicy(k_cap=3)
    assert p.k == 2                      # cold start: min(cap, 2)
    assert p.observe(2, 2) == 3          # first ratio seeds the average: 1.0 -> top band
    assert abs(float(p.ema) - 1.0) < 1e-7
    assert p.observe(0, 3) == 3          # 0.3*0 + 0.7*1.0 = 0.7
    assert p.observe(0, 3) == 3          # 0.49
    assert p.observe(0, 3) == 2          # 0.343 -> middle band
    assert p.observe(0, 2) == 1          # 0.2401 -> lowest band, first low round (ratio < 0.15 and average < 0.30)
    assert p.low_run == 1
    assert p.switches == 3


def test_switch_off_needs_three_low_rounds_and_low_average():
    p = SpecPolicy(k_cap=3)
    p.observe(0, 2)                      # average 0.0
    assert p.k == 1 and p.low_run == 1
    p.observe(1, 1)                      # a hit resets the run (ratio 1.0)
    assert p.low_run == 0
    for _ in range(2):
        p.observe(0, 1)
    assert p.k == 1 and p.low_run == 2   # average 0.147, then 0.103
    p.observe(0, 1)
    assert p.k == 0 and p.low_run == 0 and p.off_tries == 1 and p.probe == 2


def test_unlucky_rounds_with_healthy_average_do_not_switch_off():
    p = SpecPolicy(k_cap=3)
    p.observe(3, 3)                      # average 1.0
    for _ in range(3):
        p.observe(0, 3)                  # 0.7, 0.49, 0.343: ratio is low but the average is not below 0.30
    assert p.k == 2 and p.low_run == 0


def test_probe_gap_as_the_reference_computes_it():
    """gap = 2 << min(off_tries - 1, 3).  As written in the reference, every round that does not switch drafting off clears
    off_tries -- including the two failing rounds that precede the next switch-off -- so consecutive switch-offs all arm
    the same gap of 2 steps; the doubling only shows if off_tries is carried in from outside."""
    p = SpecPolicy(k_cap=3)
    for _ in range(3):
        while p.k != 0:
            p.observe(0, max(p.k, 1))
        assert p.off_tries == 1 and p.probe == 2
        steps = 0
        while p.k == 0:
            p.before_step()
            steps += 1
        assert steps == 3 and p.k == 1     # two plain steps, then the probing round opens with k = 1
    for tries, gap in ((1, 4), (2, 8), (3, 16), (7, 16)):
        q = SpecPolicy(k_cap=3)
        q.observe(0, 2)
        q.observe(0, 1)
        q.off_tries = tries                # set after the rounds that would clear it
        q.low_run = 2
        q.observe(0, 1)
        assert q.k == 0 and q.probe == gap


def test_anchor_signal_after_eight_idle_steps():
    p = SpecPolicy(k_cap=3)
    p.observe(0, 2)
    p.observe(0, 1)
    p.off_tries, p.low_run = 3, 2
    p.observe(0, 1)
    assert p.k == 0 and p.probe == 16
    flags = [p.before_step() for _ in range(10)]
    assert flags.index(True) == 7 and flags.count(True) == 1


def test_fixed_k_when_not_adaptive_and_engine_clamp():
    p = SpecPolicy(k_cap=5, adaptive=False)
    assert p.k == 5 and p.observe(0, 5) == 5 and not p.before_step()
    q = SpecPolicy(k_cap=8, engine_k_max=2)
    assert q.k == 2
    q.observe(2, 2)
    assert q.k == 2                      # the band says 3, the engine holds two drafts
    assert batch_k([p, q]) == 5 and batch_k([]) == 0


def test_threshold_uses_f32_rounding():
    p = SpecPolicy(k_cap=3)
    p.observe(9, 20)                     # 0.45 in f32 == the f32 constant 0.45: top band
    assert p.ema.dtype == np.float32 and p.k == 3
