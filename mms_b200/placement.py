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
        # engine.sim_options per part (None: self.options for every part)
        self.pipeline_options = None
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
            opts_k = self.options
            if self.pipeline_options is not None and len(self.pipeline_options) == parts:
                opts_k = self.pipeline_options[k]
            with torch.cuda.stream(self._streams[k]):
                jobs.append(engine.submit_batch(self.trace, enc, self.table, pinned=pinned,
                                                options=opts_k, split=split[k],
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


def length_groups(lengths, slack=1.125, min_group=32):
    """Cuts traces into groups of similar length (each at most `slack` times
    as long as the group's shortest, unless that leaves fewer than
    `min_group`), so that padding every group to its longest trace adds
    little: a list of index arrays, each ascending in length."""
    order = np.argsort(np.asarray(lengths), kind="stable")
    groups, cur = [], []
    for t in order.tolist():
        if cur and lengths[t] > slack * max(lengths[cur[0]], 1) and len(cur) >= min_group:
            groups.append(np.asarray(cur, np.int64))
            cur = []
        cur.append(t)
    if cur:
        groups.append(np.asarray(cur, np.int64))
    return groups


class ResidentSweep:
    """The traces of a sweep on the GPU, grouped by length, every group ready to
    be launched (any number of times) on a stream of its own."""

    def __init__(self, sweep, workloads, cells, eager=False):
        """eager: every group is launched as soon as its traces are on their way
        (longest traces first), so that the uploads of the later groups run
        beside the kernels of the earlier ones; `tally_launched` then joins
        them.  Uploads go through pinned staging buffers."""
        import torch
        self.sweep = sweep
        self.T = len(workloads)
        M = len(sweep.model_names)
        dev = sweep.device if sweep.device is not None else torch.device(
            "cuda", torch.cuda.current_device())
        self.device = torch.device(dev)
        arrays = sweep._arrays(workloads, lazy=eager)
        lengths = np.array([len(w.arrivals) for w in workloads], np.int64)
        self.lengths = lengths
        self.groups = length_groups(lengths)
        if eager:                                   # the longest walk starts first
            self.groups.sort(key=lambda idx: -int(lengths[idx].max()))
        self.h2d_bytes = 0
        self.jobs, self.streams, self.meta = [], [], []
        main = torch.cuda.current_stream(self.device)
        for idx in self.groups:
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(main)
            with torch.cuda.stream(side if eager else main):
                traces = engine.DeviceTraceBatch([workloads[t].arrivals for t in idx],
                                                 [arrays[t][0] for t in idx],
                                                 [arrays[t][1] for t in idx], M,
                                                 device=self.device, staged=eager)
                job = engine.ResidentBatch(traces, sweep.enc.repeat(len(idx)), sweep.table,
                                           options=sweep.options, split=False)
                if eager:
                    job.launch()
            self.h2d_bytes += traces.h2d_bytes + job.h2d_bytes
            self.jobs.append(job)
            self.streams.append(side)
            cell = torch.from_numpy(((sweep.first_trace + idx) % cells).astype(np.int64)).to(
                self.device)
            n = torch.from_numpy(lengths[idx]).to(self.device)
            self.meta.append((cell, n))
        self.cells = cells
        # per cell: good requests, requests, traces (integers: the sums do not depend on order)
        self.tally = torch.zeros((cells, 3), dtype=torch.int64, device=self.device)

    def launch(self):
        """Simulates every group (each on its own stream, all joined behind the
        current one) and tallies per cell; returns the tally tensor."""
        import torch
        main = torch.cuda.current_stream(self.device)
        self.tally.zero_()
        for job, side in zip(self.jobs, self.streams):
            side.wait_stream(main)
            with torch.cuda.stream(side):
                job.launch()
        return self.tally_launched()

    def tally_launched(self):
        """Joins the groups' streams behind the current one and tallies per cell."""
        import torch
        main = torch.cuda.current_stream(self.device)
        self.tally.zero_()
        for side in self.streams:
            main.wait_stream(side)
        for job, (cell, n) in zip(self.jobs, self.meta):
            for j in job.jobs:
                j.stream = main
            good = job.device_outputs()[0][1]
            self.tally.index_add_(0, cell, torch.stack(
                (good, n, torch.ones_like(n)), dim=1))
        return self.tally

    def results(self):
        """BatchResult over all traces in the order they were given."""
        parts = [job.results()[0] for job in self.jobs]
        res = engine.BatchResult()
        for name in engine.BatchResult.__slots__:
            first = getattr(parts[0], name)
            if first is None:
                setattr(res, name, None)
                continue
            whole = np.zeros((self.T,) + first.shape[1:], first.dtype)
            for idx, part in zip(self.groups, parts):
                whole[idx] = getattr(part, name)
            setattr(res, name, whole)
        self.d2h_bytes = sum(int(getattr(p, n).nbytes) for p in parts
                             for n in ("model_num_requests", "model_num_good",
                                       "group_num_requests", "good_total", "status"))
        return res

    def release(self):
        for job in self.jobs:
            job.release()
        self.jobs = []


class TraceSweep:
    """One placement scored on many traces — the robustness sweeps that call
    `approximate_one_case(..., fast_stats=True)` once per trace
    (alpa_serve/simulator/controller.py:308-407) — with the traces as the
    batch: they are uploaded as they are, grouped by length, and every group
    is simulated in one launch, every GPU thread running the placement on a
    trace of its own.  Trace t belongs to cell (first_trace + t) mod cells of
    the sweep's grid; `evaluate_tally` also returns the per-cell sums."""

    def __init__(self, model_datas, cluster_env, placement: ModelPlacement, device=None,
                 options=None, batch: int = 4096, cells: int = 1, first_trace: int = 0):
        self.model_datas = model_datas
        self.cluster_env = cluster_env
        self.placement = placement
        self.model_names = tuple(d.name for d in model_datas)
        self.table = engine.LatencyTable(tuple(d.profiling_result for d in model_datas))
        self.enc = engine.encode_placements([placement], self.table, len(self.model_names))
        self.device = device
        self.options = options
        self.batch = int(batch)
        self.cells = int(cells)
        self.first_trace = int(first_trace)
        # evaluate(): launch each group of traces as soon as it is uploaded (through pinned
        # staging buffers) instead of uploading everything first
        self.eager = True
        self.last_h2d_bytes = self.last_d2h_bytes = 0

    def _arrays(self, workloads, lazy=False):
        """(model_ids, slos) of every workload; numpy does the work outside the
        interpreter lock, so a few threads share it.  lazy: as engine.LazyArrays
        that the upload fills piece by piece (array-backed workloads only)."""
        from concurrent.futures import ThreadPoolExecutor
        import os
        if lazy:
            return [self._lazy_arrays(w) for w in workloads]
        if len(workloads) < 8:
            return [workload_arrays(w, self.model_names) for w in workloads]
        with ThreadPoolExecutor(min(16, os.cpu_count() or 1)) as pool:
            return list(pool.map(lambda w: workload_arrays(w, self.model_names), workloads))

    def _lazy_arrays(self, w):
        if not hasattr(w, "name_index"):
            return workload_arrays(w, self.model_names)
        name2id = {m: i for i, m in enumerate(self.model_names)}
        lut = np.array([name2id.get(n, -1) for n in w.names] or [-1], dtype=np.int32)
        which, slo = w.name_index, w.request_slo

        same = np.array_equal(lut, np.arange(len(lut), dtype=np.int32))

        def fill_ids(out, lo, hi):
            if same:                # the workload lists the models in registration order
                np.copyto(out, which[lo:hi])
            else:
                np.take(lut, which[lo:hi], out=out, mode="clip")    # indices are always in range

        def fill_slos(out, lo, hi):
            np.copyto(out, slo[lo:hi], casting="same_kind")     # f64 -> f32 as astype rounds it
        return (engine.LazyArray(len(which), np.int32, fill_ids),
                engine.LazyArray(len(slo), np.float32, fill_slos))

    def resident(self, workloads: Sequence[Workload]) -> ResidentSweep:
        return ResidentSweep(self, workloads, self.cells)

    def evaluate_tally(self, workloads: Sequence[Workload]):
        """(per-trace results as `evaluate` returns them, per-cell tally i64[cells][3] =
        good requests, requests, traces — on the device)."""
        out = []
        tally = None
        self.last_h2d_bytes = self.last_d2h_bytes = 0
        g = int(self.enc.num_groups[0])
        for lo in range(0, len(workloads), self.batch):
            part = workloads[lo:lo + self.batch]
            first = self.first_trace
            self.first_trace = first + lo
            try:
                run = ResidentSweep(self, part, self.cells, eager=self.eager)
            finally:
                self.first_trace = first
            t = (run.tally_launched() if self.eager else run.launch()).clone()
            tally = t if tally is None else tally + t
            res = run.results()
            engine._check_status(res)
            self.last_h2d_bytes += run.h2d_bytes
            self.last_d2h_bytes += run.d2h_bytes
            run.release()
            for k in range(len(part)):
                n = int(run.lengths[k])
                goodput = float(res.good_total[k]) / n if n else 0.0
                per_model = res.model_num_good[k] / (res.model_num_requests[k] + eps)
                out.append((goodput, per_model, tuple(res.group_num_requests[k, :g])))
        return out, tally

    def evaluate(self, workloads: Sequence[Workload]):
        """Per trace: (goodput, per-model goodput, group_num_requests), with
        goodput = np.mean(good) and per-model goodput = good / (requests + eps)
        as in fast_stats (controller.py:393-403)."""
        return self.evaluate_tally(workloads)[0]
