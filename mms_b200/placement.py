"""Placement datatypes and the batched PlacementEvaluator.

Mirror of alpa_serve/placement_policy/base_policy.py:18-264.  The evaluator
keeps the reference's constructor and its get_scores / get_stats contract
(list of candidate placements in, list of scores or stats tuples out), but
scores the whole list with one GPU launch instead of one simulator call per
candidate (base_policy.py:175-189).
"""
import dataclasses
from typing import List, Sequence

import numpy as np

from . import engine
from .profiling import ParallelConfig, ProfilingResult  # noqa: F401 (re-exported)
from .simulator import fast_stats, workload_arrays
from .workload import GammaProcess, Workload, eps

inf = 1e100      # alpa_serve/util.py:23


@dataclasses.dataclass
class ModelPlacement:
    """base_policy.py:18-55: the parallel config of every device group and
    the model ids each group serves."""
    group_configs: Sequence[ParallelConfig]
    group_models: Sequence[Sequence[int]]

    def add_model(self, group_id: int, model_id: int):
        models = list(self.group_models)
        models[group_id] = list(models[group_id]) + [model_id]
        return ModelPlacement(self.group_configs, models)

    def normalize(self):
        """Sort the models inside each group, then the groups by their model
        tuple (base_policy.py:29-35)."""
        models = tuple(tuple(sorted(ms)) for ms in self.group_models)
        order = sorted(range(len(models)), key=lambda i: models[i])
        return ModelPlacement(tuple(self.group_configs[i] for i in order),
                              tuple(models[i] for i in order))

    def copy(self):
        return ModelPlacement(list(self.group_configs), [list(ms) for ms in self.group_models])

    def verify(self, model_datas, cluster_env):
        """base_policy.py:41-55: every group fits the memory budget and holds
        each model at most once."""
        for c, ms in zip(self.group_configs, self.group_models):
            mem = sum(_weight_mem(model_datas[m], c) for m in ms)
            assert mem <= cluster_env.mem_budget
            assert len(set(ms)) == len(ms)


@dataclasses.dataclass
class ModelPlacementWithReplacement:
    """base_policy.py:58-68: placements[k] is in force from start_times[k]."""
    start_times: List[float]
    placements: List[ModelPlacement]

    def verify(self, model_datas, cluster_env):
        for p in self.placements:
            p.verify(model_datas, cluster_env)

    def __str__(self):
        return f"ModelPlacementWithReplacement(num_segments={len(self.placements)})"


@dataclasses.dataclass
class ModelData:
    """base_policy.py:71-77."""
    name: str
    slo: float
    rate: float
    cv: float
    profiling_result: ProfilingResult


@dataclasses.dataclass
class ClusterEnv:
    """base_policy.py:80-84."""
    num_devices: int
    mem_budget: float
    num_devices_per_node: int = 8


def _weight_mem(model_data, config):
    entry = model_data.profiling_result.para_dict.get(config)
    return max(entry.weight_mem) if entry is not None else inf


def gen_train_workload(model_datas, seed: int = 0, simulation_min_duration: float = 100,
                       simulation_min_samples: int = 30000) -> Workload:
    """The trace a search trains on when none is given (base_policy.py:267-281):
    one Gamma process per model, seed + model index, merged."""
    total_rate = sum(d.rate for d in model_datas)
    duration = max(simulation_min_duration, simulation_min_samples / total_rate)
    parts = [GammaProcess(d.rate, d.cv).generate_workload(d.name, 0, duration=duration,
                                                          slo=d.slo, seed=seed + i)
             for i, d in enumerate(model_datas)]
    return Workload.merge(*parts)


class PlacementEvaluator:
    """Scores candidate placements on the GPU (base_policy.py:143-264).

    `method` must be "fast_simulator" (the only method the reference's
    searches use); `parallel` is accepted for signature compatibility and
    ignored — the batch is the parallelism.
    """

    def __init__(self, model_datas, cluster_env, workload, method: str = "fast_simulator",
                 parallel: bool = False, device=None, options=None):
        if method != "fast_simulator":
            raise NotImplementedError("only the fast_simulator method runs on the GPU")
        self.parallel = parallel
        self.model_datas = model_datas
        self.cluster_env = cluster_env
        self.workload = workload
        self.method = method
        workload.cached_data = None                    # base_policy.py:155
        workload.enable_simulator_cache = True         # base_policy.py:170
        self.model_names = tuple(d.name for d in model_datas)
        self.prof_ress = tuple(d.profiling_result for d in model_datas)
        model_ids, slos = workload_arrays(workload, self.model_names)
        workload.cached_data = (model_ids, slos, self.model_names, self.prof_ress)
        self.trace = engine.DeviceTrace(workload.arrivals, model_ids, slos,
                                        len(self.model_names), device=device)
        self.table = engine.LatencyTable(self.prof_ress)
        self.options = options          # engine.sim_options(...) or None
        # A long list is encoded and launched in parts.  The first part only has
        # to cover the host's work on the second, so it is the smaller one; more
        # and smaller parts cost more on the GPU (shorter chunks, more run-in)
        # than the encoding they hide.
        self.pipeline_parts = 2
        self.pipeline_min_part = 768    # placements per part, at least
        self.pipeline_shares = (3, 5)   # relative sizes of the parts (None: equal)
        # placements with mirror candidates as a launch of their own inside a
        # part: one flag, or one per part.  Only the last part needs it: the
        # serial repairs of an earlier part run beside the parts behind it anyway.
        self.pipeline_split = (False, True)
        self._streams = []
        self.last_resimulated = None
        self.last_h2d_bytes = 0
        self.last_d2h_bytes = 0

    # -- the batched core ---------------------------------------------------
    def evaluate(self, sols: Sequence[ModelPlacement], pinned=False):
        """Scores the whole list; returns (batch, BatchResult) where `batch`
        has B, num_groups and num_replicas.  A long list goes to the GPU in
        `pipeline_parts` parts, each on a stream of its own, so that the host
        encodes the next part while the GPU simulates the previous ones."""
        n = len(sols)
        parts = max(1, min(self.pipeline_parts, n // self.pipeline_min_part))
        if parts == 1:
            enc = engine.encode_placements(sols, self.table, len(self.model_names))
            res, h2d, d2h = engine.run_batch(self.trace, enc, self.table, pinned=pinned,
                                             options=self.options)
            self.last_h2d_bytes, self.last_d2h_bytes = h2d, d2h
            self.last_resimulated = res.resimulated
            return enc, res
        import torch
        dev = self.trace.device
        while len(self._streams) < parts:
            self._streams.append(torch.cuda.Stream(device=dev))
        main = torch.cuda.current_stream(dev)
        shares = self.pipeline_shares
        if shares is None or len(shares) != parts:
            shares = (1,) * parts
        total, run, bounds = float(sum(shares)), 0.0, [0]
        for share in shares:
            run += share
            bounds.append(min(n, int(round(n * run / total))))
        bounds[-1] = n
        split = self.pipeline_split
        if isinstance(split, (bool, int)):
            split = (bool(split),) * parts
        elif len(split) != parts:
            split = (False,) * (parts - 1) + (True,)
        encs, jobs = [], []
        for k in range(parts):
            enc = engine.encode_placements(sols[bounds[k]:bounds[k + 1]], self.table,
                                           len(self.model_names))
            self._streams[k].wait_stream(main)           # the trace was uploaded there
            with torch.cuda.stream(self._streams[k]):
                jobs.append(engine.submit_batch(self.trace, enc, self.table, pinned=pinned,
                                                options=self.options, split=split[k],
                                                crowded=k + 1 < parts))
            encs.append(enc)
        done = [engine.collect_batch(job) for job in jobs]
        for k in range(parts):
            main.wait_stream(self._streams[k])
        res = engine.BatchResult.concatenate([d[0] for d in done])
        self.last_h2d_bytes = sum(d[1] for d in done)
        self.last_d2h_bytes = sum(d[2] for d in done)
        self.last_resimulated = res.resimulated
        return engine.BatchSummary(encs), res

    def scores_from(self, enc, res) -> List[float]:
        """goodput - latency_mean/10000 + num_replicas/1e6 (base_policy.py:225-226)
        with goodput = np.mean(good), latency_mean = np.mean(finish - start)."""
        n = self.trace.num_requests
        goodput = res.good_total.astype(np.float64) / n
        latency_mean = res.latency_sum / n
        scores = goodput - latency_mean / 10000 + enc.num_replicas / 1000000
        return [np.float64(s) for s in scores]

    # -- the reference's interface --------------------------------------------
    def get_scores(self, sols: Sequence[ModelPlacement]) -> List[float]:
        if not len(sols):
            return []
        enc, res = self.evaluate(sols)
        return self.scores_from(enc, res)

    def get_stats(self, sols: Sequence[ModelPlacement]):
        """[(goodput, per-model goodput, group_num_requests, StatsResult)]
        per candidate (base_policy.py:228-264)."""
        if not len(sols):
            return []
        enc, res = self.evaluate(sols)
        start = self.trace.host_arrivals
        out = []
        for b in range(enc.B):
            g = int(enc.num_groups[b])
            stats = fast_stats(self.model_names, start, res.latency_sum[b], res.good_total[b],
                               res.model_num_requests[b], res.model_num_good[b],
                               res.group_num_requests[b, :g])
            out.append((stats.goodput, [x.goodput for x in stats.per_model_stats],
                        stats.group_num_requests, stats))
        return out


class TraceSweep:
    """One placement scored on many traces — the robustness sweeps that call
    `approximate_one_case(..., fast_stats=True)` once per trace
    (alpa_serve/simulator/controller.py:308-407) — with the traces as the
    batch: `batch` of them are uploaded side by side and simulated in one
    launch, every GPU thread running the placement on a trace of its own."""

    def __init__(self, model_datas, cluster_env, placement: ModelPlacement, device=None,
                 options=None, batch: int = 256):
        self.model_datas = model_datas
        self.cluster_env = cluster_env
        self.placement = placement
        self.model_names = tuple(d.name for d in model_datas)
        self.table = engine.LatencyTable(tuple(d.profiling_result for d in model_datas))
        self.enc = engine.encode_placements([placement], self.table, len(self.model_names))
        self.device = device
        self.options = options
        self.batch = int(batch)

    def evaluate(self, workloads: Sequence[Workload]):
        """Per trace: (goodput, per-model goodput, group_num_requests), with
        goodput = np.mean(good) and per-model goodput = good / (requests + eps)
        as in fast_stats (controller.py:393-403)."""
        out = []
        M = len(self.model_names)
        for lo in range(0, len(workloads), self.batch):
            part = workloads[lo:lo + self.batch]
            arrays = [workload_arrays(w, self.model_names) for w in part]
            traces = engine.DeviceTraceBatch([w.arrivals for w in part], [a[0] for a in arrays],
                                             [a[1] for a in arrays], M, device=self.device)
            res, _, _ = engine.run_batch(traces, self.enc.repeat(len(part)), self.table,
                                         options=self.options)
            g = int(self.enc.num_groups[0])
            for t in range(len(part)):
                n = int(traces.lengths[t])
                goodput = float(res.good_total[t]) / n if n else 0.0
                per_model = res.model_num_good[t] / (res.model_num_requests[t] + eps)
                out.append((goodput, per_model, tuple(res.group_num_requests[t, :g])))
        return out
