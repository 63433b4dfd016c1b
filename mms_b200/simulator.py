"""Drop-in simulator entry points, same names and arguments as
alpa_serve/simulator/controller.py:282-798, computed on the GPU.

  simulate_requests_mixed            controller.py:562
  simulate_requests                  controller.py:507
  approximate_one_case_one_placement controller.py:410
  approximate_one_case               controller.py:308
  DummyController                    controller.py:282

Results equal the reference's bit for bit (fp64 finish times, good flags,
int32 counters).  There is no CPU path: without the built extension or a
CUDA device every function raises.
"""
from functools import partial
from typing import Callable

import numpy as np

from . import _native as nat
from . import engine
from .workload import DEFAULT_WARMUP, PerModelStatsResult, StatsResult, eps

inf = 1e100      # alpa_serve/util.py:23

# Batch sizes the batching simulator may form: the module global
# alpa_serve.util.batchsize_config (util.py:13).  Like in the reference it is
# edited in place (`batchsize_config[:] = [1, 2, 4, 8]`).
batchsize_config = [1, 2, 4, 8, 16]


def _counters(res, M, G, b=0):
    mreq = res.model_num_requests[b, :M].astype(np.int32)
    mgood = res.model_num_good[b, :M].astype(np.int32)
    greq = res.group_num_requests[b, :G].astype(np.int32)
    ggood = res.group_num_good[b, :G].astype(np.int32)
    return mreq, mgood, greq, ggood


# How the trace is cut for time-parallel execution; None = library default.
# Results do not depend on it (tests sweep it).
_options = None


def set_chunking(chunk_requests=0, warmup_requests=0):
    """Overrides the chunk length / run-in of the time-parallel execution for
    the entry points of this module (0, 0 restores the default)."""
    global _options
    _options = None if (chunk_requests == 0 and warmup_requests == 0) \
        else engine.sim_options(chunk_requests, warmup_requests)


def _run_dense(finish, good, tstamps, model_ids, slos, m_id2g_id, num_stages, latency,
               num_requests, flags):
    """One candidate in the reference's dense layout; fills finish/good."""
    latency = np.ascontiguousarray(latency, dtype=np.float32)
    M, G, S = latency.shape
    N = int(num_requests)
    trace = engine.DeviceTrace(np.asarray(tstamps)[:N], np.asarray(model_ids)[:N],
                               np.asarray(slos)[:N], M)
    if G == 0 or M == 0:
        finish[:N] = np.asarray(tstamps)[:N]
        good[:N] = False
        z = np.zeros
        return z(M, np.int32), z(M, np.int32), z(G, np.int32), z(G, np.int32)
    off, rep, info, T = engine.encode_dense(m_id2g_id, num_stages, M)
    res, _, _ = engine._launch(trace, 1, M, G, rep.shape[1], T, S, G, off, rep, info,
                               latency, 0, flags | nat.FLAG_PER_REQUEST, True,
                               options=_options)
    finish[:N] = res.finish[0]
    good[:N] = res.good[0]
    return _counters(res, M, G)


def simulate_requests_mixed(finish, good, tstamps, model_ids, slos, m_id2g_id,
                            num_stages, stage_latency, num_requests):
    """controller.py:562-628: FIFO pipeline simulation with SLO dropping.
    Fills `finish` and `good` in place, returns (model_num_requests,
    model_num_good_requests, group_num_requests, group_num_good_requests)."""
    return _run_dense(finish, good, tstamps, model_ids, slos, m_id2g_id, num_stages,
                      stage_latency, num_requests, 0)


def simulate_requests(finish, good, tstamps, model_ids, slos, m_id2g_id,
                      group_max_latency, group_sum_latency, num_requests):
    """controller.py:507-558: the one-clock-per-group variant."""
    gmax = np.asarray(group_max_latency, dtype=np.float32)
    gsum = np.asarray(group_sum_latency, dtype=np.float32)
    pair = np.stack([gsum, gmax], axis=-1)          # [M][G][{sum, max}]
    ones = np.ones(gmax.shape[1], np.int32)
    return _run_dense(finish, good, tstamps, model_ids, slos, m_id2g_id, ones, pair,
                      num_requests, nat.FLAG_LEGACY_CLOCK)


def simulate_requests_mixed_batching(finish, good, tstamps, model_ids, slos, m_id2g_id,
                                     g_id2m_id, num_stages, stage_latency, num_requests):
    """controller.py:631-798: per-model queues, batches formed at dispatch
    under the head request's deadline.  stage_latency is
    [M][G][S][len(batchsize_config)]; g_id2m_id is implied by m_id2g_id and
    only checked for shape."""
    lat = np.ascontiguousarray(stage_latency, dtype=np.float32)
    M, G, S, NB = lat.shape
    if NB != len(batchsize_config):
        raise ValueError("stage_latency's last axis must match batchsize_config")
    N = int(num_requests)
    trace = engine.DeviceTrace(np.asarray(tstamps)[:N], np.asarray(model_ids)[:N],
                               np.asarray(slos)[:N], M)
    if G == 0 or M == 0:
        finish[:N] = np.asarray(tstamps)[:N]
        good[:N] = False
        z = np.zeros
        return z(M, np.int32), z(M, np.int32), z(G, np.int32), z(G, np.int32)
    off, rep, info, T = engine.encode_dense(m_id2g_id, num_stages, M)
    res = engine.launch_batching(trace, 1, M, G, rep.shape[1], T, S, G, off, rep, info, lat, 0,
                                 list(batchsize_config))
    finish[:N] = res.finish[0]
    good[:N] = res.good[0]
    return _counters(res, M, G)


def approximate_one_case_one_placement(placement, model_names, prof_ress, model_ids, slos,
                                       arrivals, mixed=True, enable_batching=False,
                                       rows_on_device=False):
    """controller.py:410-503: simulate one ModelPlacement on one trace.
    Returns (start, finish, good, model_num_requests, model_num_good_requests,
    group_num_requests, group_num_good_requests).  With rows_on_device (no
    counterpart in the reference) finish and good are torch tensors on the GPU
    (f64[N], u8[N]) instead of numpy arrays: nothing per request is downloaded."""
    M = len(model_names)
    G = len(placement.group_configs)
    N = len(arrivals)
    arrivals = np.asarray(arrivals, dtype=np.float64)
    if rows_on_device and mixed and G > 0:
        trace = engine.DeviceTrace(arrivals, model_ids, slos, M)
        table = engine.LatencyTable(prof_ress, list(batchsize_config) if enable_batching else None)
        enc = engine.encode_placements([placement], table, M)
        if enable_batching:
            res = engine.run_batch_batching(trace, enc, table, per_request=False,
                                            rows_on_device=True)
        else:
            res, _, _ = engine.run_batch(trace, enc, table, per_request=True, group_good=True,
                                         options=_options, rows_on_device=True)
        return (arrivals, res.finish_device[0], res.good_device[0]) + tuple(_counters(res, M, G))
    finish = np.empty(N, dtype=np.float64)
    good = np.empty(N, dtype=bool)
    if not mixed:
        max_bs = 1
        gmax = np.empty((M, G), np.float32)
        gsum = np.empty((M, G), np.float32)
        with np.errstate(over="ignore"):
            for m in range(M):
                for g in range(G):
                    value = prof_ress[m].para_dict.get(placement.group_configs[g], None)
                    if value:                                  # controller.py:438-443
                        penalty = 0.009 * len(value.latency[max_bs])
                        gmax[m][g] = max(value.latency[max_bs]) * (1 + penalty)
                        gsum[m][g] = sum(value.latency[max_bs]) * (1 + penalty)
                    else:
                        gmax[m][g] = gsum[m][g] = inf
        m2g = np.full((M, max(G, 1)), -1, np.int32)
        fill = [0] * M
        for g, ms in enumerate(placement.group_models):
            for m in ms:
                m2g[m][fill[m]] = g
                fill[m] += 1
        counters = simulate_requests(finish, good, arrivals, model_ids, slos, m2g, gmax, gsum, N)
        return (arrivals, finish, good) + tuple(counters)

    trace = engine.DeviceTrace(arrivals, model_ids, slos, M)
    table = engine.LatencyTable(prof_ress, list(batchsize_config) if enable_batching else None)
    enc = engine.encode_placements([placement], table, M)
    if enable_batching and G > 0:
        res = engine.run_batch_batching(trace, enc, table)
        finish[:] = res.finish[0]
        good[:] = res.good[0]
        return (arrivals, finish, good) + tuple(_counters(res, M, G))
    if G == 0:
        z = np.zeros
        return (arrivals, arrivals.copy(), np.zeros(N, bool), trace.model_hist.cpu().numpy()[:M],
                z(M, np.int32), z(0, np.int32), z(0, np.int32))
    res, _, _ = engine.run_batch(trace, enc, table, per_request=True, group_good=True,
                                 options=_options)
    finish[:] = res.finish[0]
    good[:] = res.good[0]
    return (arrivals, finish, good) + tuple(_counters(res, M, G))


class DummyController:
    """Collects the ProfilingResult of every registered model
    (controller.py:282-305).  Each method also answers to `.remote(...)`,
    like the reference's install_remote_methods makes them."""

    def __init__(self):
        self.name2profiling = {}
        for name in ("register_model", "create_mesh_group_manager", "create_replica"):
            _add_remote(self, name)

    def register_model(self, name: str, model_def: Callable):
        assert isinstance(model_def, partial)
        for a in model_def.args:
            if hasattr(a, "para_dict"):
                self.name2profiling[name] = a
                break

    def create_mesh_group_manager(self, *args, **kwargs):
        pass

    def create_replica(self, *args, **kwargs):
        pass

    def sync(self):
        pass


def _add_remote(obj, name):
    bound = getattr(obj, name)

    def call(*args, **kwargs):
        return bound(*args, **kwargs)
    call.remote = bound
    setattr(obj, name, call)


def workload_arrays(workload, model_names):
    """(model_ids i32[N], slos f32[N]) of a workload for a model registration
    order (controller.py:334-336).  Works on this package's array-backed
    Workload and on any object with a `requests` list."""
    name2id = {m: i for i, m in enumerate(model_names)}
    if hasattr(workload, "name_index"):
        lut = np.array([name2id.get(n, -1) for n in workload.names] or [-1], dtype=np.int32)
        ids = lut[workload.name_index] if len(workload.name_index) else np.empty(0, np.int32)
        return ids.astype(np.int32), workload.request_slo.astype(np.float32)
    ids = np.array([name2id.get(r.model_name, -1) for r in workload.requests], dtype=np.int32)
    slos = np.array([r.slo for r in workload.requests], dtype=np.float32)
    return ids, slos


def fast_stats(model_names, start, finish_minus_start_sum, good_total, model_num_requests,
               model_num_good, group_num_requests) -> StatsResult:
    """The no-warm-up statistics of controller.py:393-403, from the reduced
    quantities the GPU returns: np.mean(good) = good_total / N and
    np.mean(finish - start) = (numpy-ordered sum) / N."""
    n = len(start)
    interval = start[-1] - start[0]
    per_model = [PerModelStatsResult(
        model_names[i], model_num_requests[i],
        model_num_good[i] / (model_num_requests[i] + eps),
        model_num_requests[i] / interval, 0, 0, 0, 0, [], [], [])
        for i in range(len(model_names))]
    goodput = np.float64(good_total) / n
    latency_mean = np.float64(finish_minus_start_sum) / n
    return StatsResult(per_model, tuple(group_num_requests), goodput, latency_mean, n,
                       n / interval)


class DeviceColumn:
    """Stands where compute_stats puts a per-request array of one model
    (PerModelStatsResult.latency, .request_starts, .request_finishes,
    workload.py:347-349).  The per-request outputs stay on the GPU; the array is
    downloaded and cut out when somebody looks at it."""

    def __init__(self, fetch, length):
        self._fetch, self._length, self._value = fetch, int(length), None

    def _get(self):
        if self._value is None:
            self._value = self._fetch()
            self._fetch = None
        return self._value

    def __array__(self, dtype=None, copy=None):
        v = np.asarray(self._get())
        return v.astype(dtype) if dtype is not None and v.dtype != dtype else v

    def __len__(self):
        return self._length

    def __getitem__(self, key):
        return self._get()[key]

    def __iter__(self):
        return iter(self._get())


def device_stats(workload, start, finish_dev, good_dev, warmup) -> StatsResult:
    """Workload.compute_stats (workload.py:308-354) from per-request outputs
    that are still on the GPU (finish f64[N], good u8[N] torch tensors): the
    numbers come from mms_compute_stats, the per-request arrays of the result
    are DeviceColumns."""
    import torch
    arrivals = np.asarray(workload.arrivals, dtype=np.float64)
    which = np.asarray(workload.name_index, dtype=np.int32)
    n = len(arrivals)
    lo, hi = 0, n
    if n > 1:
        skip = int(warmup / (arrivals[-1] - arrivals[0]) * n)
        if skip > 0:
            lo, hi = skip, max(n - skip, skip)
    window = hi - lo
    dev = finish_dev.device
    d_arr = torch.from_numpy(np.ascontiguousarray(start, dtype=np.float64)).to(dev)
    d_which = torch.from_numpy(which).to(dev)
    K = len(workload.names)
    st = engine.device_compute_stats(d_arr, d_which, K, finish_dev.reshape(1, -1),
                                     good_dev.reshape(1, -1), lo, window)
    start_w, which_w = np.asarray(start)[lo:hi], which[lo:hi]
    # names in order of first appearance, then a stable sort by request count (:321-326)
    _, first = np.unique(which_w, return_index=True)
    seen = [int(k) for k in which_w[np.sort(first)]]
    ordered = sorted(seen, key=lambda k: int(st["num_requests"][k]))
    host = {}

    def rows():
        if not host:
            host["finish"] = finish_dev.cpu().numpy()[lo:hi]
            host["good"] = good_dev.cpu().numpy()[lo:hi].astype(bool)
        return host["finish"], host["good"]

    def column(k, what):
        def fetch():
            fin, good = rows()
            pick = (which_w == k) & good
            if not pick.any():
                return [0] if what == "latency" else start_w[pick]
            return {"latency": lambda: fin[pick] - start_w[pick], "start": lambda: start_w[pick],
                    "finish": lambda: fin[pick]}[what]()
        return fetch

    per_model = []
    for k in ordered:
        count, ok = int(st["num_requests"][k]), int(st["num_good"][0, k])
        goodput = np.float64(ok) / count
        if ok > 0:
            with np.errstate(divide="ignore"):
                throughput = ok / (st["last_start"][0, k] - st["first_start"][0, k])
            mean, std = st["latency_mean"][0, k], st["latency_std"][0, k]
            p90, p99 = st["latency_p90"][0, k], st["latency_p99"][0, k]
        else:                      # latency = [0] in the reference (:339-341)
            zero = np.sort([0])
            throughput, mean, std, p90, p99 = 0, np.mean([0]), np.std([0]), zero[0], zero[0]
        per_model.append(PerModelStatsResult(
            workload.names[k], count, goodput, throughput, mean, std, p90, p99,
            DeviceColumn(column(k, "latency"), max(ok, 1)), DeviceColumn(column(k, "start"), ok),
            DeviceColumn(column(k, "finish"), ok)))
    return StatsResult(per_model, None, np.float64(st["good_total"][0]) / window,
                       st["latency_sum"][0] / window, window,
                       window / (start_w[-1] - start_w[0]))


def approximate_one_case(case, seed: int = 0, warmup: int = DEFAULT_WARMUP, debug: bool = False,
                         fast_stats: bool = False, enable_batching: bool = False):
    """controller.py:308-407.  `case` is the reference's ServingCase triple
    (register_models, generate_workload, place_models)."""
    register_models, generate_workload, place_models = case
    workload = generate_workload()

    if workload.enable_simulator_cache and workload.cached_data:
        model_ids, slos, model_names, prof_ress = workload.cached_data
        placement = place_models(None)
    else:
        controller = DummyController()
        register_models(controller)
        placement = place_models(controller)
        model_names, prof_ress = zip(*controller.name2profiling.items())
        model_ids, slos = workload_arrays(workload, model_names)
        if workload.enable_simulator_cache:
            workload.cached_data = (model_ids, slos, model_names, prof_ress)

    # compute_stats runs on the GPU when the workload is array-backed: the per-request
    # outputs then never leave the device
    on_device = (not fast_stats and hasattr(workload, "name_index") and len(workload) > 1
                 and all(len(p.group_configs) > 0
                         for p in getattr(placement, "placements", [placement])))
    run = partial(approximate_one_case_one_placement, enable_batching=enable_batching,
                  rows_on_device=on_device)
    if hasattr(placement, "placements"):          # ModelPlacementWithReplacement
        arrivals = workload.arrivals
        change_times = list(placement.start_times[1:]) + [inf]
        # controller.py:353-371: a segment ends at the first arrival that is
        # later than the next change time; clocks restart from zero.
        bounds = [0]
        pt = 0
        for i in range(len(arrivals)):
            if arrivals[i] > change_times[pt]:
                bounds.append(i)
                pt += 1
        bounds.append(len(arrivals))
        parts = [run(placement.placements[k], model_names, prof_ress,
                     model_ids[bounds[k]:bounds[k + 1]], slos[bounds[k]:bounds[k + 1]],
                     arrivals[bounds[k]:bounds[k + 1]]) for k in range(len(bounds) - 1)]
        start = np.concatenate([p[0] for p in parts])
        if on_device:
            import torch
            finish = torch.cat([p[1] for p in parts])
            good = torch.cat([p[2] for p in parts])
        else:
            finish = np.concatenate([p[1] for p in parts])
            good = np.concatenate([p[2] for p in parts])
        model_num_requests = np.sum([p[3] for p in parts], axis=0)
        model_num_good = np.sum([p[4] for p in parts], axis=0)
        group_num_requests = np.sum([p[5] for p in parts], axis=0)
    else:
        (start, finish, good, model_num_requests, model_num_good,
         group_num_requests, _) = run(placement, model_names, prof_ress, model_ids, slos,
                                      workload.arrivals)

    if fast_stats:
        interval = start[-1] - start[0]
        per_model = [PerModelStatsResult(
            model_names[i], model_num_requests[i],
            model_num_good[i] / (model_num_requests[i] + eps),
            model_num_requests[i] / interval, 0, 0, 0, 0, [], [], [])
            for i in range(len(model_names))]
        stats = StatsResult(per_model, tuple(group_num_requests), np.mean(good),
                            np.mean(finish - start), len(start), len(start) / interval)
    elif on_device:
        stats = device_stats(workload, start, finish, good, warmup)
        stats.group_num_requests = tuple(group_num_requests)
    else:
        stats = workload.compute_stats(start, finish, good, warmup)
        stats.group_num_requests = tuple(group_num_requests)
    return stats, placement
