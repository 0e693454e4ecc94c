"""CPU checks of the benchmark's host side: the CPU arm runs a whole round through the oracle's kernels, and the
byte accounting of a verify step follows the formula the roofline fraction is quoted on."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def _tiny():
    from inferulm_b200.engine import ModelShape
    return ModelShape(hidden=256, n_layers=4, q_heads=4, kv_heads=2, head_dim=64, rot_dim=32, inter=512, vocab=1024, lin_k_heads=2,
                      lin_v_heads=4, full_every=4)


def test_cpu_round_runs_every_piece_of_a_round():
    import bench
    cr = bench.CpuRound(_tiny(), batch=2, k=2, ctx=40, threads=2)
    assert cr.run() > 0.0
    assert cr.run() > 0.0      # repeatable: a run leaves the synthetic inputs as they were


def test_verify_bytes_follow_the_formula():
    import bench
    from inferulm_b200.engine import ModelShape
    s = ModelShape()
    b, lite = bench.verify_bytes_of(s, 1, 3, 1152, snapshots=True)
    # weights + 24 layers x (1 + P) state rows and conv rows + 8 layers x KV of (L + P) tokens + logits written and read
    want = s.weight_bytes() + 24 * 5 * (2097152 + 49152) + 8 * 4096 * (1152 + 4) + 2 * 4 * 151936 * 2
    assert not lite and b == want
    assert abs(s.weight_bytes() - 7_918_024_192) < 3_000_000      # the matrices of the model shape (small vectors and conv taps excluded)
    b2, lite2 = bench.verify_bytes_of(s, 1, 3, 1152)
    assert lite2 and b2 < b
