"""Benchmark of the placement-evaluation hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload: the batched candidate evaluation — 4096 random placements of 32
models on 64 devices scored against one one-hour Gamma trace (about 180 k
requests).  One step = one pass of the simulator over the whole batch.
Metric: candidate-placements x requests simulated per second.  Prints one
JSON line.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "candidate_placements_x_requests_per_sec"
UNIT = "candidate*request/s"
BYTES_PER_UNIT = 16          # f64 arrival + i32 model id + f32 slo, read once per candidate
NUM_CANDIDATES = 4096
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one sim_stream_kernel launch (the dominant
# kernel: the launch over the 3695 placements without mirror candidates) on the default
# workload, from profiles/launch_list_candidates4096_3600s.md
STREAM_KERNEL_DRAM_BYTES = 39151616 + 1057084928


_REAL_STDOUT = None


def quiet_stdout():
    """Libraries write banners to stdout (NCCL prints its version on the first
    collective): everything but the result line goes to stderr."""
    global _REAL_STDOUT
    if _REAL_STDOUT is None:
        sys.stdout.flush()
        _REAL_STDOUT = os.dup(1)
        os.dup2(2, 1)


def emit(line):
    """The ONE JSON line of the contract, on the real stdout."""
    text = (json.dumps(line) + "\n").encode()
    sys.stdout.flush()
    if _REAL_STDOUT is None:
        os.write(1, text)
    else:
        os.write(_REAL_STDOUT, text)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--candidates", type=int, default=NUM_CANDIDATES)
    ap.add_argument("--duration", type=float, default=3600.0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--greedy-steps", type=int, default=3,
                    help="also time this many steps of the full greedy placement search (0 = skip)")
    ap.add_argument("--chunk", type=int, default=0, help="requests per chunk (0 auto, <0 one)")
    ap.add_argument("--run-in", type=int, default=0, help="run-in requests per chunk (0 auto)")
    ap.add_argument("--rounds", type=int, default=0, help="validate+repair rounds (0 auto)")
    ap.add_argument("--repair-segments", type=int, default=0,
                    help="segments a repair runs per round (0 auto, <0 no cap)")
    ap.add_argument("--workload", default="candidates", choices=["candidates", "sweep"],
                    help="candidates: 4096 placements x one trace (the headline); sweep: one "
                         "placement x many traces (robustness sweep)")
    ap.add_argument("--traces", type=int, default=256, help="sweep: traces per GPU")
    ap.add_argument("--placement-seed", type=int, default=-1,
                    help="seed of the candidate list (default: the rank)")
    ap.add_argument("--no-split", action="store_true",
                    help="one launch per step even when some placements have mirror candidates")
    ap.add_argument("--no-mirrors", action="store_true",
                    help="no mirror candidates for placements with interchangeable groups")
    return ap.parse_args()


def hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Polls nvidia-smi for SM clocks and throttle reasons while a region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, index=0):
        self.index = index
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _poll(self):
        try:
            out = subprocess.run(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout
            f = [x.strip() for x in out.strip().splitlines()[0].split(",")]
            self.samples.append(float(f[0]))
            self.max_mhz = float(f[1])
            for name, v in zip(self.NAMES, f[2:]):
                if v.lower().startswith("active"):
                    self.reasons.add(name)
        except Exception:
            pass

    def _run(self):
        while not self._stop.is_set():
            self._poll()
            self._stop.wait(0.1)

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=10)

    def summary(self):
        return {"sm_mhz": float(np.median(self.samples)) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def build_case(args, placement_seed):
    from mms_b200 import cases
    return cases.candidate_batch_case(num_candidates=args.candidates, duration=args.duration,
                                      placement_seed=placement_seed)


def dense_batch(case, count):
    """Dense per-candidate tables for the CPU checker (untimed set-up)."""
    from mms_b200.simulator import workload_arrays
    from oracle import tables
    names = [d.name for d in case.model_datas]
    profs = [d.profiling_result for d in case.model_datas]
    mids, slos = workload_arrays(case.workload, names)
    sols = case.placements[:count]
    G = max(len(p.group_configs) for p in sols)
    M = len(profs)
    m2g = np.full((len(sols), M, G), -1, np.int32)
    ns = np.ones((len(sols), G), np.int32)
    S = max(c.pp for p in sols for c in p.group_configs)
    lat = np.full((len(sols), M, G, S), np.float32(np.inf), np.float32)
    for b, p in enumerate(sols):
        a, _, n, l = tables.dense_tables(p, profs)
        g = len(n)
        m2g[b, :, :g] = a[:, :g]
        ns[b, :g] = n
        lat[b, :, :g, :l.shape[2]] = l
    return mids, slos, m2g, ns, lat


_dense_cache = {}


def cpu_port_rate(case, count, threads):
    """Times the C restatement of the reference's numba kernel (plus the
    reductions the score needs) over `count` candidates on `threads` host
    threads.  Table construction is set-up, not timed.  Returns units per
    second and the seconds taken."""
    from oracle import cpu
    key = (id(case), count)
    if key not in _dense_cache:
        _dense_cache[key] = dense_batch(case, count)
    mids, slos, m2g, ns, lat = _dense_cache[key]
    arr = case.workload.arrivals
    cpu.score_batch(arr, mids, slos, m2g[:threads], ns[:threads], lat[:threads], threads)
    t0 = time.perf_counter()
    cpu.score_batch(arr, mids, slos, m2g, ns, lat, threads)
    dt = time.perf_counter() - t0
    return count * len(arr) / dt, dt


def run_reference(args):
    """The reference's CPU implementation of the path (here: the C port of
    its numba kernel, all host threads), on the same workload and metric."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    case = build_case(args, 0)
    threads = os.cpu_count() or 1
    per_step = min(args.candidates, max(threads * 16, 256))
    rates = []
    for i in range(args.warmup + args.steps):
        rate, dt = cpu_port_rate(case, per_step, threads)
        if i >= args.warmup:
            rates.append((rate, dt))
    value = float(np.mean([r for r, _ in rates]))
    ms = float(np.mean([d for _, d in rates])) * 1e3
    sample = f"{per_step} of {args.candidates} candidates x {len(case.workload)} requests per step"
    emit({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64",
        "data": "synthetic",
        "config": {"workload": "candidate-batch: 64 devices, 32 models, 4096 placements, "
                               "1 h Gamma trace", "num_candidates": args.candidates,
                   "num_requests": len(case.workload), "sample": sample},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    })


def run_b200(args):
    import ctypes

    import torch
    import torch.distributed as dist
    from mms_b200 import _native as nat
    from mms_b200 import engine
    from mms_b200.placement import PlacementEvaluator

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    # every rank scores its own 4096 candidates (weak scaling) on the same trace
    case = build_case(args, placement_seed=rank if args.placement_seed < 0 else args.placement_seed)
    ev = PlacementEvaluator(case.model_datas, case.cluster_env, case.workload, device=dev,
                            options=engine.sim_options(args.chunk, args.run_in, args.rounds, args.repair_segments))
    N, B = ev.trace.num_requests, len(case.placements)
    L = nat.lib()

    # ---- device-resident arm: tables already in HBM, time the C-ABI call(s) ----
    # B placements are scored; the ones with interchangeable groups bring mirror candidates
    # and go into a launch of their own beside the rest (engine.ResidentBatch)
    enc = engine.encode_placements(case.placements, ev.table, len(ev.model_names))
    opts = engine.sim_options(args.chunk, args.run_in, args.rounds, args.repair_segments)
    resident = engine.ResidentBatch(ev.trace, enc, ev.table, options=opts,
                                    mirrors=not args.no_mirrors, split=not args.no_split)
    n_mirrors = sum(job.B - job.Bs for job in resident.jobs)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)   # > 126 MB of L2
    best = torch.zeros(2, dtype=torch.float64, device=dev)
    gathered = torch.zeros(2 * world, dtype=torch.float64, device=dev)
    part_index = [None if idx is None else torch.from_numpy(idx).to(dev)
                  for idx, _, _ in resident.device_outputs()]

    own_done = torch.cuda.Event(enable_timing=True)     # this rank's kernels, before the exchange

    def step():
        resident.launch()
        own_done.record()
        if world > 1:   # the search's argmax over all ranks' candidates
            best[0] = -1e300
            for pos, (_, good, lat_sum) in zip(part_index, resident.device_outputs()):
                score = good.double() / N - lat_sum / N / 10000
                top = torch.max(score, dim=0)
                where = top.indices if pos is None else pos[top.indices]
                better = top.values > best[0]
                best[1] = torch.where(better, (where + rank * B).double(), best[1])
                best[0] = torch.where(better, top.values, best[0])
            dist.all_gather_into_tensor(gathered, best)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        flush.zero_()
        step()
    barrier()
    times, own_times = [], []
    nat.check(L.mms_profile_begin(), "mms_profile_begin")     # events around the stream kernel
    with ClockSampler(local) as clk:
        for _ in range(args.steps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            step()
            e1.record()
            e1.synchronize()
            times.append(e0.elapsed_time(e1))
            own_times.append(e0.elapsed_time(own_done))
    barrier()
    k_launches, k_ms = ctypes.c_int32(0), ctypes.c_float(0.0)
    each = np.zeros(256, np.float32)
    nat.check(L.mms_profile_end(ctypes.byref(k_launches), ctypes.byref(k_ms), each.ctypes.data,
                                len(each)), "mms_profile_end")
    # the dominant kernel: the stream kernel of the step's largest launch (with a split step,
    # launch 0 holds the placements with mirror candidates and launch 1 the rest)
    per_step = len(resident.jobs)
    big = int(np.argmax([job.Bs for job in resident.jobs]))
    stream_kernel_ms = float(np.mean(each[big:k_launches.value:per_step]))
    kernel_units = resident.jobs[big].Bs * N
    total_ms = torch.tensor([sum(times)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(total_ms, op=dist.ReduceOp.MAX)
    total_ms = float(total_ms.item())
    by_rank = torch.tensor([float(np.mean(own_times))], dtype=torch.float64, device=dev)
    if world > 1:
        all_ranks = torch.zeros(world, dtype=torch.float64, device=dev)
        dist.all_gather_into_tensor(all_ranks, by_rank)
        by_rank = all_ranks
    by_rank = [round(float(x), 3) for x in by_rank.tolist()]
    final, _ = resident.results()
    assert not np.any(final.status), "kernel status words are not clean"
    redo = final.resimulated
    units_per_step = B * N * world
    value = units_per_step * args.steps / (total_ms * 1e-3)

    # ---- end-to-end arm: host buffers in, scores out, through the evaluator ----
    e2e_times, h2d, d2h = [], 0, 0
    for i in range(2 + min(args.steps, 3)):
        barrier()
        t0 = time.perf_counter()
        ev.trace = engine.DeviceTrace(case.workload.arrivals, ev.workload.cached_data[0],
                                      ev.workload.cached_data[1], len(ev.model_names), dev)
        scores = ev.get_scores(case.placements)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        if i >= 2:
            e2e_times.append(dt)
        h2d = ev.trace.h2d_bytes + ev.last_h2d_bytes
        d2h = ev.last_d2h_bytes
    e2e_t = torch.tensor([float(np.mean(e2e_times))], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(e2e_t, op=dist.ReduceOp.MAX)
    e2e_value = units_per_step / float(e2e_t.item())

    greedy = greedy_step_timing(args, dev) if (world == 1 and args.greedy_steps > 0) else None
    if rank == 0:
        peak, which = hbm_peak()
        # the dominant kernel (sim_stream_kernel), timed by CUDA events on its own stream
        # inside the timed steps; the whole call (all kernels) is reported beside it
        achieved = kernel_units * BYTES_PER_UNIT / (stream_kernel_ms * 1e-3) / 1e9
        call_achieved = B * N * BYTES_PER_UNIT / (np.mean(times) * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f64", "data": "synthetic",
            "config": {"workload": "candidate-batch: 64 devices, 32 models, 4096 placements "
                                   "per GPU, 1 h Gamma trace (Zipf 0.9 rates, 50 req/s, CV 3)",
                       "num_candidates_per_gpu": B, "num_requests": N,
                       "parallelism": f"candidates sharded over {world} GPU(s)",
                       "l2": "256 MiB buffer written between timed steps"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak,
                         "traffic": (STREAM_KERNEL_DRAM_BYTES
                                     if (B, args.duration, per_step) == (NUM_CANDIDATES, 3600.0, 2)
                                     else None),
                         "traffic_unit": "bytes per sim_stream_kernel launch (ncu, DRAM read+write)",
                         "kernel": "sim_stream_kernel", "kernel_ms": stream_kernel_ms,
                         "kernel_launches_timed": int(k_launches.value) // per_step,
                         "whole_call": {"achieved": call_achieved, "frac": call_achieved / peak,
                                        "ms": float(np.mean(times))},
                         "peak_source": which, "bytes_per_unit": BYTES_PER_UNIT,
                         "algorithmic_bytes_per_launch": kernel_units * BYTES_PER_UNIT},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": int(h2d),
                    "d2h_bytes_per_step": int(d2h)},
            # segment leaves, rows, stream, (validate, resolve, two forms of repair) per
            # round, two forms of chain, count, requests per model
            "gpu_launches": ((7 + 4 * (args.rounds if args.rounds > 0 else 4)) * args.steps
                             * len(resident.jobs)),
            "mirror_candidates_per_gpu": int(n_mirrors),
            "launches_per_step": len(resident.jobs),
            # each rank's own kernels per step, before the exchange of the best score
            "kernel_ms_per_step_by_rank": by_rank,
            "chunks_resimulated_per_candidate": float(np.mean(redo)),
            "chunks_resimulated_hist": np.bincount(redo).tolist(),
            "clocks": clk.summary(),
            "best_score": float(np.max(scores)),
        }
        if greedy:
            line["greedy_step"] = greedy
        if not args.no_cpu_baseline and world == 1:      # single-GPU runs only
            count = min(B, 3072)       # about 10 s of one host core
            rate, dt = cpu_port_rate(case, count, 1)
            line["cpu_baseline"] = {
                "value": rate, "unit": UNIT, "cores": 1, "kind": "port",
                "sample": f"{count} of {B} candidates x {N} requests, {dt:.1f} s"}
        emit(line)
    if world > 1:
        dist.destroy_process_group()


def greedy_step_timing(args, dev):
    """Wall time per step of the full greedy placement search (64 devices, 56
    models): every step expands all (partition, group, model) additions of the
    four pipeline partitions and scores them in one launch."""
    import torch
    from mms_b200 import cases, search
    from mms_b200.placement import PlacementEvaluator
    case = cases.greedy_search_case()
    ev = PlacementEvaluator(case.model_datas, case.cluster_env, case.workload, device=dev)
    starts = search.ModelParallelismSearch(max_op=1).enumerate_group_configs_uneven(
        case.cluster_env)
    layers = []

    class Enough(Exception):
        pass

    def on_layer(n, seconds):
        torch.cuda.synchronize()
        layers.append((n, seconds))
        if len(layers) >= args.greedy_steps + 1:
            raise Enough()
    try:
        search.beam_search_lockstep(starts, case.model_datas, case.cluster_env, ev, 1,
                                    on_layer=on_layer)
    except Enough:
        pass
    timed = layers[1:] or layers            # the first step also warms up
    n = float(np.mean([x[0] for x in timed]))
    sec = float(np.mean([x[1] for x in timed]))
    return {"ms_per_step": sec * 1e3, "candidates_per_step": n,
            "num_requests": len(case.workload), "partitions": len(starts),
            "value": n * len(case.workload) / sec, "unit": UNIT,
            "includes": "host expansion and dedup, encoding, H2D, kernels, D2H, top-1 per partition"}


def run_sweep(args):
    """One placement x many traces per GPU (trace t of rank r is global trace
    r * traces + t); same metric, 1 unit = 1 trace x 1 request."""
    import ctypes

    import torch
    import torch.distributed as dist
    from mms_b200 import _native as nat
    from mms_b200 import cases, engine
    from mms_b200.placement import TraceSweep
    from mms_b200.simulator import workload_arrays

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    duration = args.duration if args.duration != 3600.0 else 720.0
    case = cases.sweep_case(duration=duration)
    T = args.traces
    workloads = [case.trace(rank * T + t) for t in range(T)]
    sweep = TraceSweep(case.model_datas, case.cluster_env, case.placement, device=dev, batch=T,
                       options=engine.sim_options(args.chunk, args.run_in, args.rounds,
                                                  args.repair_segments))
    names = sweep.model_names
    arrays = [workload_arrays(w, names) for w in workloads]
    units = int(sum(len(w.arrivals) for w in workloads))
    L = nat.lib()

    # ---- device-resident arm ----
    traces = engine.DeviceTraceBatch([w.arrivals for w in workloads], [a[0] for a in arrays],
                                     [a[1] for a in arrays], len(names), device=dev)
    enc = sweep.enc.repeat(T)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    jobs = []

    def step():
        job = engine.submit_batch(traces, enc, sweep.table, options=sweep.options)
        jobs.append(job)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def drain():
        out = None
        while jobs:
            out = engine.collect_batch(jobs.pop())[0]
        return out

    for _ in range(max(args.warmup, 3)):
        flush.zero_()
        step()
        drain()
    barrier()
    times = []
    nat.check(L.mms_profile_begin(), "mms_profile_begin")
    with ClockSampler(local) as clk:
        for _ in range(args.steps):
            flush.zero_()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            step()                      # tables are uploaded inside (a few hundred KB)
            e1.record()
            e1.synchronize()
            times.append(e0.elapsed_time(e1))
            res = drain()
    barrier()
    k_launches, k_ms = ctypes.c_int32(0), ctypes.c_float(0.0)
    nat.check(L.mms_profile_end(ctypes.byref(k_launches), ctypes.byref(k_ms), None, 0),
              "mms_profile_end")
    stream_kernel_ms = k_ms.value / max(k_launches.value, 1)
    total_ms = torch.tensor([sum(times)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(total_ms, op=dist.ReduceOp.MAX)
    total_ms = float(total_ms.item())
    all_units = torch.tensor([units], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(all_units)
    all_units = float(all_units.item())
    value = all_units * args.steps / (total_ms * 1e-3)

    # ---- end-to-end arm: host traces in, goodputs out (and the tallies combined) ----
    e2e_times = []
    for i in range(3):
        barrier()
        t0 = time.perf_counter()
        got = sweep.evaluate(workloads)
        tally = torch.zeros(16, 2, dtype=torch.float64, device=dev)   # per cell: sum, count
        for t, g in enumerate(got):
            cell = (rank * T + t) % 16
            tally[cell, 0] += g[0]
            tally[cell, 1] += 1
        if world > 1:
            dist.all_reduce(tally)
        torch.cuda.synchronize()
        if i >= 1:
            e2e_times.append(time.perf_counter() - t0)
    e2e_t = torch.tensor([float(np.mean(e2e_times))], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(e2e_t, op=dist.ReduceOp.MAX)
    e2e_value = all_units / float(e2e_t.item())
    goodputs = np.array([g[0] for g in got])
    assert np.array_equal(goodputs, res.good_total / traces.lengths), "resident and e2e arms differ"

    if rank == 0:
        peak, which = hbm_peak()
        achieved = units * BYTES_PER_UNIT / (stream_kernel_ms * 1e-3) / 1e9
        call_achieved = units * BYTES_PER_UNIT / (np.mean(times) * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f64", "data": "synthetic",
            "config": {"workload": f"trace-sweep: one 64-device placement of 32 models x {T} traces "
                                   f"per GPU ({duration:.0f} s Gamma traces, 16 cells of rate scale "
                                   "{0.5,1,2,4} x CV {1,2,4,8}, 278 req/s at scale 1)",
                       "traces_per_gpu": T, "requests_per_gpu": units,
                       "padded_requests_per_trace": traces.num_requests,
                       "parallelism": f"traces sharded over {world} GPU(s)",
                       "l2": "256 MiB buffer written between timed steps"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": None,
                         "kernel": "sim_stream_kernel", "kernel_ms": stream_kernel_ms,
                         "kernel_launches_timed": int(k_launches.value),
                         "whole_call": {"achieved": call_achieved, "frac": call_achieved / peak,
                                        "ms": float(np.mean(times))},
                         "peak_source": which, "bytes_per_unit": BYTES_PER_UNIT,
                         "algorithmic_bytes_per_launch": units * BYTES_PER_UNIT},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": int(traces.h2d_bytes),
                    "d2h_bytes_per_step": int(T * (2 * len(names) + enc.G + 4) * 4)},
            "gpu_launches": (7 + 4 * (args.rounds if args.rounds > 0 else 4)) * args.steps,
            "chunks_resimulated_per_trace": float(np.mean(res.resimulated)),
            "clocks": clk.summary(),
            "goodput_mean_per_cell": [float(np.mean(goodputs[c::16])) for c in range(16)],
        }
        if not args.no_cpu_baseline and world == 1:
            from oracle import tables
            profs = [d.profiling_result for d in case.model_datas]
            t0 = time.perf_counter()
            done = 0
            for t in range(T):
                tables.one_placement(case.placement, profs, arrays[t][0], arrays[t][1],
                                     workloads[t].arrivals)
                done += len(workloads[t].arrivals)
                if time.perf_counter() - t0 > 10.0:
                    break
            dt = time.perf_counter() - t0
            line["cpu_baseline"] = {"value": done / dt, "unit": UNIT, "cores": 1, "kind": "port",
                                    "sample": f"{done} requests of the first traces, {dt:.1f} s"}
        emit(line)
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse_args()
    quiet_stdout()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "sweep":
        run_sweep(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
