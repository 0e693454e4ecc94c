"""Multi-GPU plumbing of the benchmark: sequences are sharded across ranks with no collective on the data path; the only
communication is the timing barrier and the reduction of each rank's (time, tokens) pair at the end."""
import os

import numpy as np


def rank_world():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))


def shard_sequences(n_total, rank, world):
    """Sequence i of a global batch goes to rank i mod world (round-robin; sequences are independent)."""
    return [i for i in range(n_total) if i % world == rank]


def pack_sequences(costs, world):
    """Longest-first greedy bin packing: sequences sorted by cost (prompt + output tokens), largest first, each to the rank
    with the least cost so far (ties to the lowest rank).  Returns one list of sequence indices per rank, in the order the
    rank runs them.  Deterministic, so every rank computes the same assignment without communicating."""
    costs = np.asarray(costs, dtype=np.int64)
    order = sorted(range(costs.size), key=lambda i: (-int(costs[i]), i))
    load = [0] * world
    bins = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda j: (load[j], j))
        bins[r].append(i)
        load[r] += int(costs[i])
    return bins


def rank_prompts(rank, batch, prompt_len, vocab, base_seed=1000):
    """The prompts of one rank: seeded by the rank so that ranks run different sequences."""
    rs = np.random.default_rng(base_seed + rank)
    return [rs.integers(0, vocab, prompt_len).astype(np.uint32) for _ in range(batch)]


def reduce_job(ms_local, tokens_local, device=None):
    """(max over ranks of the step time, sum over ranks of the tokens): whole-job throughput = tokens / max time."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(ms_local), float(tokens_local)
    t = torch.tensor([float(ms_local)], dtype=torch.float64, device=device)
    s = torch.tensor([float(tokens_local)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dist.all_reduce(s, op=dist.ReduceOp.SUM)
    return float(t.item()), float(s.item())
