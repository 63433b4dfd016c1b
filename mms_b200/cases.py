"""Seeded synthetic evaluation cases (models, trace, candidate placements).

These stand in for the profiling database and the production traces the
reference's experiments load from files: same shapes, sizes and value
distributions, generated from numpy seeds.  Used by the benchmark and the
tests; every case is described by plain containers of this package, which
the reference's own classes can consume as well (duck typing).
"""
import dataclasses
from typing import List

import numpy as np

from .placement import ClusterEnv, ModelData, ModelPlacement
from .profiling import GB, LatencyMemData, ParallelConfig, ProfilingResult, synthetic_profile
from .workload import GammaProcess, Workload


@dataclasses.dataclass
class Case:
    name: str
    model_datas: List[ModelData]
    cluster_env: ClusterEnv
    workload: Workload
    placements: List[ModelPlacement]
    batch_sizes: tuple = (1,)


def merged_gamma_trace(model_datas, duration, base_seed) -> Workload:
    """One Gamma process per model, seed = base_seed + model index, merged by
    arrival time (the convention of base_policy.py:277-279)."""
    parts = [GammaProcess(d.rate, d.cv).generate_workload(d.name, 0, duration, slo=d.slo,
                                                          seed=base_seed + i)
             for i, d in enumerate(model_datas)]
    return Workload.merge(*parts)


def fixed_pipeline_case(duration=3600.0, base_seed=0) -> Case:
    """8 devices as 4 groups of pipeline degree 2; 8 equal models (0.15 s on
    one device, 2 x 0.075 s on two), two models per group; Gamma arrivals at
    2 req/s per model with CV 4; SLO 5 x 0.15 s."""
    prof = ProfilingResult("toy-150ms", {
        ParallelConfig(1, 1, 1): LatencyMemData({1: [0.15]}, {1: [0.0]}, [2 * GB]),
        ParallelConfig(1, 1, 2): LatencyMemData({1: [0.075, 0.075]}, {1: [0.0, 0.0]},
                                                [1 * GB, 1 * GB]),
    })
    datas = [ModelData(f"m{i}", 0.75, 2.0, 4.0, prof) for i in range(8)]
    placement = ModelPlacement([ParallelConfig(1, 1, 2)] * 4, [[0, 1], [2, 3], [4, 5], [6, 7]])
    return Case("fixed-4x-pp2", datas, ClusterEnv(8, 13 * GB),
                merged_gamma_trace(datas, duration, base_seed), [placement])


SIZE_CLASSES = ((0.05, 2.6), (0.15, 5.2), (0.40, 13.4))   # (single-device seconds, GB)


def zipf_rates(n, total_rate, alpha=0.9):
    w = 1.0 / np.arange(1, n + 1) ** alpha
    return total_rate * w / w.sum()


def mixed_models(num_models=32, total_rate=50.0, cv=3.0, slo_scale=5.0, batch_sizes=(1,),
                 classes=SIZE_CLASSES) -> List[ModelData]:
    """Models cycling through the size classes; model i gets the i-th largest
    Zipf(0.9) share of the total rate and an SLO of slo_scale x its
    single-device latency."""
    rates = zipf_rates(num_models, total_rate)
    datas = []
    for i in range(num_models):
        lat, size = classes[i % len(classes)]
        prof = synthetic_profile(f"class{i % len(classes)}", lat, size * GB,
                                 batch_sizes=batch_sizes)
        datas.append(ModelData(f"m{i}", slo_scale * lat, float(rates[i]), cv, prof))
    return datas


def random_placements(model_datas, num_devices, mem_budget, count, seed,
                      group_sizes=(1, 2, 4, 8), max_models_per_group=4) -> List[ModelPlacement]:
    """`count` random placements: pipeline-parallel group sizes drawn until
    they add up to num_devices; each group takes up to max_models_per_group
    distinct random models while their per-device weights fit the budget."""
    rng = np.random.RandomState(seed)
    M = len(model_datas)
    out = []
    for _ in range(count):
        left = num_devices
        configs, groups = [], []
        while left > 0:
            fits = [s for s in group_sizes if s <= left]
            p = int(fits[rng.randint(len(fits))])
            left -= p
            cfg = ParallelConfig(1, 1, p)
            want = int(rng.randint(1, max_models_per_group + 1))
            used, chosen = 0.0, []
            for m in rng.permutation(M):
                if len(chosen) >= want:
                    break
                entry = model_datas[m].profiling_result.para_dict.get(cfg)
                if entry is None:
                    continue
                need = max(entry.weight_mem)
                if used + need <= mem_budget:
                    chosen.append(int(m))
                    used += need
            configs.append(cfg)
            groups.append(chosen)
        out.append(ModelPlacement(configs, groups))
    return out


def candidate_batch_case(num_candidates=4096, duration=3600.0, base_seed=0, placement_seed=0,
                         batching=False, num_models=32, num_devices=64,
                         total_rate=50.0, cv=3.0) -> Case:
    """64 devices, 32 models in three size classes, Zipf(0.9) rates summing to
    50 req/s, CV 3, one hour; `num_candidates` random placements under a
    13 GB-per-device budget.  With `batching`, profiles carry batch sizes
    1, 2, 4, 8 with l(b) = l(1) * (0.8 + 0.2 b)."""
    bs = (1, 2, 4, 8) if batching else (1,)
    datas = mixed_models(num_models, total_rate, cv, batch_sizes=bs)
    env = ClusterEnv(num_devices, 13 * GB)
    placements = random_placements(datas, num_devices, env.mem_budget, num_candidates,
                                   placement_seed)
    name = "candidates-batching" if batching else "candidates"
    return Case(name, datas, env, merged_gamma_trace(datas, duration, base_seed), placements, bs)


# eight latency tables over the three size classes: (single-device seconds, GB)
SEARCH_CLASSES = ((0.04, 2.6), (0.05, 2.6), (0.06, 2.6), (0.12, 5.2), (0.15, 5.2), (0.18, 5.2),
                  (0.35, 13.4), (0.40, 13.4))


def greedy_search_case(slo_scale=5.0, num_models=56, num_devices=64, total_rate=80.0, cv=4.0,
                       duration=1800.0, base_seed=1) -> Case:
    """The full placement search problem: 64 devices, 56 models over eight
    latency tables, Zipf(0.9) shares of 80 req/s, CV 4, 30 minutes, seed 1.
    Profiles exist for pipeline degrees 1, 2, 4, 8 (operator parallelism 1),
    so the search's partitions are 64x1, 32x2, 16x4 and 8x8 devices."""
    datas = mixed_models(num_models, total_rate, cv, slo_scale, classes=SEARCH_CLASSES)
    env = ClusterEnv(num_devices, 13 * GB)
    return Case("greedy-search", datas, env, merged_gamma_trace(datas, duration, base_seed), [])


SWEEP_RATE_SCALES = (0.5, 1.0, 2.0, 4.0)
SWEEP_CVS = (1.0, 2.0, 4.0, 8.0)


@dataclasses.dataclass
class SweepCase:
    model_datas: List[ModelData]
    cluster_env: ClusterEnv
    placement: ModelPlacement
    duration: float
    total_rate: float

    def cell(self, t: int):
        """(rate scale, CV) of trace t: 16 cells, trace t is in cell t mod 16."""
        return SWEEP_RATE_SCALES[t % 4], SWEEP_CVS[(t // 4) % 4]

    def trace(self, t: int) -> Workload:
        """Trace t: base seed t, the rates of all models scaled and the CV set
        as its cell says."""
        scale, cv = self.cell(t)
        scaled = [ModelData(d.name, d.slo, d.rate * scale, cv, d.profiling_result)
                  for d in self.model_datas]
        return merged_gamma_trace(scaled, self.duration, base_seed=t)


def sweep_case(duration=3600.0, total_rate=278.0, placement_seed=0) -> SweepCase:
    """Robustness sweep: ONE 64-device placement of the 32 models of
    candidate_batch_case, scored on many traces; at rate scale 1 the models
    share `total_rate` req/s (about a million requests per hour-long trace)."""
    datas = mixed_models(32, total_rate, 1.0)
    env = ClusterEnv(64, 13 * GB)
    placement = random_placements(datas, 64, env.mem_budget, 1, placement_seed)[0]
    return SweepCase(datas, env, placement, duration, total_rate)


def replacement_case(duration=900.0, base_seed=3):
    """A placement schedule (ModelPlacementWithReplacement, base_policy.py:58-68)
    for approximate_one_case: 16 devices, 8 models, three placements of four
    groups each that take over at 0 s, 300 s and 600 s.  Returns (model_datas,
    cluster_env, workload, start_times, placements)."""
    datas = mixed_models(8, 30.0, 3.0)
    env = ClusterEnv(16, 13 * GB)
    c2, c4, c8 = (ParallelConfig(1, 1, p) for p in (2, 4, 8))
    placements = [
        ModelPlacement([c4, c4, c4, c4], [[0, 3, 6], [1, 4, 7], [0, 3, 1], [4, 6, 7]]),
        ModelPlacement([c8, c4, c2, c2], [[2, 5, 0, 1], [3, 4, 6, 7], [0, 3], [1, 6]]),
        ModelPlacement([c4, c4, c4, c4], [[0, 1, 3], [4, 6, 7], [0, 1, 3], [4, 6, 7]]),
    ]
    return datas, env, merged_gamma_trace(datas, duration, base_seed), [0.0, 300.0, 600.0], placements
