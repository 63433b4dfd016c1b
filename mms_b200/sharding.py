"""Candidate sharding over the GPUs of one box and the search's final argmax.

The path shards with no data-path collective: candidates are independent
and every rank holds the whole trace.  The only exchange is what the
reference does with the score list after `get_scores` — `np.argmax`
(alpa_serve/placement_policy/model_parallelism.py:349-351) or a top-k by
`np.argsort` (base_policy.py:462) — so ranks exchange either one
(score, index) pair each, or their score slices.  One process per GPU,
`torch.distributed` (NCCL on GPUs, gloo in the CPU tests).
"""
from typing import List, Sequence, Tuple

import numpy as np
import torch
import torch.distributed as dist


def shard_bounds(n: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous slice [lo, hi) of n candidates for `rank`; sizes differ by at most 1."""
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def _world(group=None):
    if not (dist.is_available() and dist.is_initialized()):
        return 0, 1
    return dist.get_rank(group), dist.get_world_size(group)


def _device_for(group=None):
    backend = dist.get_backend(group) if dist.is_initialized() else "gloo"
    return torch.device("cuda", torch.cuda.current_device()) if backend == "nccl" \
        else torch.device("cpu")


def argmax_over_ranks(local_scores: Sequence[float], first_index: int, group=None):
    """(best score, its index in the global candidate list).  Equals
    `np.argmax` over the concatenation of all ranks' slices: the FIRST
    maximum wins.  An empty slice contributes (-inf, a huge index)."""
    rank, world = _world(group)
    local = np.asarray(local_scores, dtype=np.float64)
    if len(local):
        k = int(np.argmax(local))
        pair = [float(local[k]), float(first_index + k)]
    else:
        pair = [-np.inf, float(2 ** 52)]
    if world == 1:
        return pair[0], int(pair[1])
    dev = _device_for(group)
    mine = torch.tensor(pair, dtype=torch.float64, device=dev)
    every = torch.empty(2 * world, dtype=torch.float64, device=dev)
    dist.all_gather_into_tensor(every, mine, group=group)
    every = every.cpu().numpy().reshape(world, 2)
    best = every[:, 0].max()
    idx = every[every[:, 0] == best, 1].min()        # first maximum over the global order
    return float(best), int(idx)


def gather_scores(local_scores: Sequence[float], n_total: int, group=None) -> List[float]:
    """All ranks' score slices in global candidate order (contiguous shards
    as cut by shard_bounds), for callers that need a top-k."""
    rank, world = _world(group)
    local = np.asarray(local_scores, dtype=np.float64)
    if world == 1:
        return [np.float64(x) for x in local]
    dev = _device_for(group)
    width = (n_total + world - 1) // world
    mine = torch.full((width,), float("nan"), dtype=torch.float64, device=dev)
    mine[:len(local)] = torch.from_numpy(local).to(dev)
    every = torch.empty(width * world, dtype=torch.float64, device=dev)
    dist.all_gather_into_tensor(every, mine, group=group)
    every = every.cpu().numpy().reshape(world, width)
    out = []
    for r in range(world):
        lo, hi = shard_bounds(n_total, r, world)
        out.extend(np.float64(x) for x in every[r, :hi - lo])
    return out


class ShardedEvaluator:
    """`get_scores` of a PlacementEvaluator over all ranks: each rank scores
    its contiguous slice of the list and every rank gets the full list back,
    so a search loop that runs identically on all ranks stays in step.
    `evaluator` needs a `get_scores(list) -> list` method."""

    def __init__(self, evaluator, group=None):
        self.evaluator = evaluator
        self.group = group

    def get_scores(self, sols):
        rank, world = _world(self.group)
        lo, hi = shard_bounds(len(sols), rank, world)
        local = self.evaluator.get_scores(list(sols[lo:hi])) if hi > lo else []
        return gather_scores(local, len(sols), self.group)

    def best(self, sols):
        rank, world = _world(self.group)
        lo, hi = shard_bounds(len(sols), rank, world)
        local = self.evaluator.get_scores(list(sols[lo:hi])) if hi > lo else []
        return argmax_over_ranks(local, lo, self.group)
