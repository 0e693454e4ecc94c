"""The N > 1 path of the benchmark on CPU: two gloo ranks, sequence sharding, max-time / sum-tokens reduction."""
import os
import socket

import numpy as np
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    import torch.distributed as dist
    from inferulm_b200 import dist_util as du
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    r, w, _ = du.rank_world()
    mine = du.shard_sequences(5, r, w)
    packed = du.pack_sequences([9, 1, 8, 2, 7, 3], w)
    prompts = du.rank_prompts(r, 2, 8, 1000)
    ms, toks = du.reduce_job(10.0 + 5 * r, 100 * (r + 1))
    out.put((r, mine, [p.tolist() for p in prompts], ms, toks, packed))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_sharding_and_reduction():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    (r0, s0, p0, ms0, t0, k0), (r1, s1, p1, ms1, t1, k1) = res
    assert k0 == k1 == [[0, 5, 3, 1], [2, 4]]               # every rank computes the same longest-first packing (loads 15 / 15)
    assert s0 == [0, 2, 4] and s1 == [1, 3]                 # round-robin, disjoint, complete
    assert p0 != p1                                         # ranks run different sequences
    assert ms0 == ms1 == 15.0 and t0 == t1 == 300.0         # max of the times, sum of the tokens, same on every rank


def test_single_process_reduce_is_identity():
    from inferulm_b200 import dist_util as du
    assert du.reduce_job(3.5, 7) == (3.5, 7.0)
    assert du.shard_sequences(3, 0, 1) == [0, 1, 2]
    a, b = du.rank_prompts(0, 1, 4, 50), du.rank_prompts(0, 1, 4, 50)
    assert np.array_equal(a[0], b[0])


def test_longest_first_packing_balances_log_uniform_costs():
    """256 sequences with log-uniform prompt lengths over 8 ranks: complete, disjoint, and balanced to a few percent."""
    from inferulm_b200 import dist_util as du
    rs = np.random.default_rng(0)
    costs = np.exp(rs.uniform(np.log(256), np.log(8192), 256)).astype(np.int64) + 256
    for world in (1, 2, 4, 8):
        bins = du.pack_sequences(costs, world)
        assert sorted(i for b in bins for i in b) == list(range(256))
        loads = [int(costs[b].sum()) for b in bins]
        assert max(loads) <= 1.03 * (sum(loads) / world)
        assert all(int(costs[b[0]]) >= int(costs[b[-1]]) for b in bins if b)      # each rank starts with its longest
