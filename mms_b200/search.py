"""Placement searches on top of the batched GPU evaluator.

Host-side mirror of the search loops that generate the candidate lists:
alpa_serve/placement_policy/base_policy.py:329-479 (fast greedy, beam
search), model_parallelism.py:208-242,294-479 (ModelParallelismGreedy,
ModelParallelismSearch) and selective_replication.py:126-203.  The decisions
are the reference's, taken from the same numbers; what changes is how often
the simulator is called: independent searches advance in LOCKSTEP so that
every step scores all their candidates in one GPU launch instead of one
simulator call each.
"""
import gc
import math
import time
from bisect import bisect_left, bisect_right
from typing import List, Sequence

import numpy as np

from .placement import (ClusterEnv, ModelData, ModelPlacement, PlacementEvaluator,
                        gen_train_workload, _weight_mem)
from .profiling import ParallelConfig
from .workload import eps


def get_factors(n: int) -> List[int]:
    """All divisors of n, ascending (alpa_serve/util.py:74-85)."""
    small = [i for i in range(1, int(math.sqrt(n)) + 1) if n % i == 0]
    return sorted(set(small + [n // i for i in small]))


def get2tok(n: int) -> List[int]:
    """Powers of two up to n (util.py:142-150)."""
    assert n > 0
    out = [1]
    while out[-1] * 2 <= n:
        out.append(out[-1] * 2)
    return out


def decompose2tok(n: int) -> List[int]:
    """The powers of two that sum to n, ascending (util.py:153-161)."""
    return [1 << k for k in range(n.bit_length()) if (n >> k) & 1]


def _weights(configs, model_datas):
    return {c: [_weight_mem(d, c) for d in model_datas] for c in set(configs)}


def _group_mem(sol, weight):
    return [sum(weight[c][m] for m in ms) for c, ms in zip(sol.group_configs, sol.group_models)]


def fast_greedy_lockstep(init_sols: Sequence[ModelPlacement], model_datas, cluster_env,
                         evaluator: PlacementEvaluator, verbose: int = 0) -> List[ModelPlacement]:
    """replica_placement_fast_greedy (base_policy.py:329-400) for several
    independent starting placements at once.  Every iteration simulates the
    current placement of every unfinished chain in one batch, then each chain
    adds the most under-served model that fits to its least loaded group."""
    mem_budget = cluster_env.mem_budget
    sols = list(init_sols)
    weights = [_weights(s.group_configs, model_datas) for s in sols]
    active = list(range(len(sols)))
    it = 0
    while active:
        enc, res = evaluator.evaluate([sols[k] for k in active])
        still = []
        for row, k in enumerate(active):
            sol, weight = sols[k], weights[k]
            g_n = int(enc.num_groups[row])
            mreq = res.model_num_requests[row]
            goodputs = res.model_num_good[row] / (mreq + eps)
            unserved = mreq * (1 - goodputs)
            model_ids = np.argsort(unserved)[::-1]
            group_ids = np.argsort(res.group_num_requests[row, :g_n])
            group_mem = _group_mem(sol, weight)
            pick = None
            for g in group_ids:
                c = sol.group_configs[g]
                for m in model_ids:
                    if m not in sol.group_models[g] and weight[c][m] + group_mem[g] <= mem_budget:
                        pick = (int(g), int(m))
                        break
                if pick:
                    break
            if pick is None:
                continue
            sols[k] = sol.add_model(*pick).normalize()
            still.append(k)
        if verbose >= 2:
            print(f"greedy iter {it}: {len(still)} of {len(sols)} chains still growing")
        active = still
        it += 1
    return sols


def replica_placement_fast_greedy(init_sol, model_datas, cluster_env, workload, evaluator,
                                  verbose: int = 0):
    """Same signature as base_policy.py:329."""
    if evaluator is None:
        evaluator = PlacementEvaluator(model_datas, cluster_env, workload, "fast_simulator", False)
    return fast_greedy_lockstep([init_sol], model_datas, cluster_env, evaluator, verbose)[0]


def _is_normalized(sol) -> bool:
    """True when `sol` is what ModelPlacement.normalize() returns: tuples all
    the way down, models ascending inside each group, groups ascending by
    their model tuple."""
    cfgs, models = sol.group_configs, sol.group_models
    if type(cfgs) is not tuple or type(models) is not tuple:
        return False
    prev = None
    for ms in models:
        if type(ms) is not tuple or (prev is not None and ms < prev):
            return False
        if any(ms[i] > ms[i + 1] for i in range(len(ms) - 1)):
            return False
        prev = ms
    return True


def _expand(sol, weight, num_models, mem_budget, visited):
    """All placements one (group, model) addition away from `sol` that fit
    the budget (strictly, base_policy.py:450) and were not seen before, each
    normalized (base_policy.py:29-35).  A normalized `sol` — every placement a
    search makes after its first step — is not re-sorted per addition: the new
    model is inserted into its group's tuple, and the group into the sorted
    rest, where the stable sort of normalize() would put it."""
    out = []
    group_mem = _group_mem(sol, weight)
    seen = set()
    fast = _is_normalized(sol)
    cfgs, models = sol.group_configs, sol.group_models
    for g in range(len(cfgs)):
        c = cfgs[g]
        # A later group with the same config and models yields, model by model,
        # placements whose group_models were just produced by the earlier one:
        # the `visited` test below would drop every one of them.
        kind = (c, tuple(models[g]))
        if kind in seen:
            continue
        seen.add(kind)
        if fast:
            mine = models[g]
            rest_m, rest_c = models[:g] + models[g + 1:], cfgs[:g] + cfgs[g + 1:]
        for m in range(num_models):
            if weight[c][m] + group_mem[g] < mem_budget and m not in models[g]:
                if fast:
                    k = bisect_left(mine, m)
                    grown = mine[:k] + (m,) + mine[k:]
                    # groups with an equal tuple keep their order: those that stood before
                    # group g stay before it
                    lo = bisect_left(rest_m, grown)
                    at = lo + max(0, min(bisect_right(rest_m, grown), g) - lo)
                    new_models = rest_m[:at] + (grown,) + rest_m[at:]
                    if new_models in visited:
                        continue
                    visited.add(new_models)
                    out.append(ModelPlacement(rest_c[:at] + (c,) + rest_c[at:], new_models))
                    continue
                nxt = sol.add_model(g, m).normalize()
                if nxt.group_models not in visited:
                    visited.add(nxt.group_models)
                    out.append(nxt)
    return out


def beam_search_lockstep(init_sols: Sequence[ModelPlacement], model_datas, cluster_env,
                         evaluator: PlacementEvaluator, beam_size: int, verbose: int = 0,
                         on_layer=None) -> List[ModelPlacement]:
    """replica_placement_beam_search (base_policy.py:403-479) for several
    starting placements at once: one `get_scores` call per layer covers the
    expansions of every search that is still running.  `on_layer(n, seconds)`
    is told the size and wall time of each layer."""
    num_models = len(model_datas)
    mem_budget = cluster_env.mem_budget
    n = len(init_sols)
    weights = [_weights(s.group_configs, model_datas) for s in init_sols]
    beams = [[s] for s in init_sols]
    best_score = [-1] * n
    best_sol = list(init_sols)
    visited = [set() for _ in range(n)]
    active = list(range(n))
    # The search keeps tens of thousands of small tuples alive (the visited
    # sets); a full collection walking them costs tens of milliseconds, more
    # than a layer, and finds nothing: none of these objects form cycles.
    gc_was_on = gc.isenabled()
    gc.disable()
    try:
        return _beam_layers(active, beams, best_score, best_sol, visited, weights, num_models,
                            mem_budget, evaluator, beam_size, verbose, on_layer)
    finally:
        if gc_was_on:
            gc.enable()


def _beam_layers(active, beams, best_score, best_sol, visited, weights, num_models, mem_budget,
                 evaluator, beam_size, verbose, on_layer):
    while active:
        tic = time.time()
        layers, owner = [], []
        for k in active:
            nxt = []
            for sol in beams[k]:
                nxt.extend(_expand(sol, weights[k], num_models, mem_budget, visited[k]))
            layers.append(nxt)
            owner.extend([k] * len(nxt))
        flat = [s for layer in layers for s in layer]
        if not flat:
            break
        scores = evaluator.get_scores(flat)
        still, pos = [], 0
        for k, layer in zip(active, layers):
            mine = scores[pos:pos + len(layer)]
            pos += len(layer)
            if not layer:
                continue
            order = np.argsort(mine)[::-1][:beam_size]
            beams[k] = []
            for idx in order:
                beams[k].append(layer[idx])
                if mine[idx] > best_score[k]:
                    best_score[k] = mine[idx]
                    best_sol[k] = layer[idx]
            still.append(k)
        if on_layer:
            on_layer(len(flat), time.time() - tic)
        if verbose >= 1:
            print(f"beam layer: {len(flat)} candidates, {len(still)} searches running")
        active = still
    return best_sol


def replica_placement_beam_search(init_sol, model_datas, cluster_env, workload, evaluator,
                                  beam_size: int, verbose: int = 0):
    """Same signature as base_policy.py:403."""
    if evaluator is None:
        evaluator = PlacementEvaluator(model_datas, cluster_env, workload, "fast_simulator", False)
    return beam_search_lockstep([init_sol], model_datas, cluster_env, evaluator, beam_size,
                                verbose)[0]


class BasePlacementPolicy:
    """base_policy.py:87-140."""

    def __init__(self, verbose: int = 0):
        self.verbose = verbose

    def place_models(self, controller, cluster_env, model_datas, train_workload=None):
        placement, debug_info = self.solve_placement(model_datas, cluster_env, train_workload)
        self.place_models_impl(controller, cluster_env, model_datas, placement)
        placement.verify(model_datas, cluster_env)
        return placement

    def place_models_impl(self, controller, cluster_env, model_datas, placement):
        """Creates the mesh groups and replicas on a controller object
        (base_policy.py:109-140); nothing to do for a placement schedule."""
        if hasattr(placement, "placements") or controller is None:
            return
        per_node = cluster_env.num_devices_per_node
        for g, config in enumerate(placement.group_configs):
            devices = int(np.prod(config))
            if devices <= per_node:
                shape = (1, devices)
            else:
                assert devices % per_node == 0
                shape = (devices // per_node, per_node)
            controller.create_mesh_group_manager.remote(g, shape)
        controller.sync()
        for g, models in enumerate(placement.group_models):
            for m in models:
                controller.create_replica.remote(model_datas[m].name, g,
                                                 [placement.group_configs[g]])
        controller.sync()


def _empty(configs):
    return ModelPlacement(list(configs), [[] for _ in configs])


class SelectiveReplicationGreedy(BasePlacementPolicy):
    """selective_replication.py:126-153: one device per group, fast greedy."""

    def solve_placement(self, model_datas, cluster_env, train_workload=None):
        if train_workload is None:
            train_workload = gen_train_workload(model_datas)
        evaluator = PlacementEvaluator(model_datas, cluster_env, train_workload)
        sol = _empty([ParallelConfig(1, 1, 1)] * cluster_env.num_devices)
        return replica_placement_fast_greedy(sol, model_datas, cluster_env, train_workload,
                                             evaluator, self.verbose), None


class SelectiveReplicationSearch(BasePlacementPolicy):
    """selective_replication.py:179-203: one device per group, beam search of width 3."""

    def __init__(self, verbose: int = 0):
        super().__init__(verbose)
        self.beam_size = 3

    def solve_placement(self, model_datas, cluster_env, train_workload=None):
        if train_workload is None:
            train_workload = gen_train_workload(model_datas)
        evaluator = PlacementEvaluator(model_datas, cluster_env, train_workload)
        sol = _empty([ParallelConfig(1, 1, 1)] * cluster_env.num_devices)
        return replica_placement_beam_search(sol, model_datas, cluster_env, train_workload,
                                             evaluator, self.beam_size, self.verbose), None


class ModelParallelismGreedy(BasePlacementPolicy):
    """model_parallelism.py:208-241: equal pipeline groups, fast greedy."""

    def __init__(self, group_size: int = 2, verbose: int = 0):
        super().__init__(verbose)
        self.group_size = group_size

    def solve_placement(self, model_datas, cluster_env, train_workload=None):
        if train_workload is None:
            train_workload = gen_train_workload(model_datas)
        evaluator = PlacementEvaluator(model_datas, cluster_env, train_workload)
        assert cluster_env.num_devices % self.group_size == 0
        groups = cluster_env.num_devices // self.group_size
        sol = _empty([ParallelConfig(1, 1, self.group_size)] * groups)
        return replica_placement_fast_greedy(sol, model_datas, cluster_env, train_workload,
                                             evaluator, self.verbose), None


class ModelParallelismSearch(BasePlacementPolicy):
    """model_parallelism.py:294-351,459-479 without separation and
    evolutionary search: every way of cutting the cluster into equal
    power-of-two groups (plus a power-of-two remainder) gets a fast-greedy
    placement — all of them advanced in lockstep — and the best-scoring one
    wins (first maximum, like np.argmax)."""

    def __init__(self, max_bs: int = 1, max_pp: int = 8, max_op: int = 4, verbose: int = 0):
        super().__init__(verbose)
        self.max_bs, self.max_pp, self.max_op = max_bs, max_pp, max_op

    def enumerate_group_configs_uneven(self, cluster_env):
        """model_parallelism.py:459-479."""
        sols = []
        devices, per_node = cluster_env.num_devices, cluster_env.num_devices_per_node
        for size in get2tok(devices):
            if size > per_node and size % per_node != 0:
                continue
            regular = devices // size
            rest = decompose2tok(devices % size)
            for pp in get_factors(size):
                op = size // pp
                if pp > self.max_pp or op > self.max_op:
                    continue
                sols.append(_empty([ParallelConfig(1, op, pp)] * regular +
                                   [ParallelConfig(1, 1, s) for s in rest]))
        return sols

    def solve_placement_one_eco(self, model_datas, cluster_env, train_workload):
        evaluator = PlacementEvaluator(model_datas, cluster_env, train_workload)
        sols = fast_greedy_lockstep(self.enumerate_group_configs_uneven(cluster_env),
                                    model_datas, cluster_env, evaluator, self.verbose)
        scores = evaluator.get_scores(sols)
        return sols[int(np.argmax(scores))], {}

    def solve_placement(self, model_datas, cluster_env, train_workload=None):
        if train_workload is None:
            train_workload = gen_train_workload(model_datas)
        return self.solve_placement_one_eco(model_datas, cluster_env, train_workload)
