"""Benchmark of the placement-evaluation hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
                    [--workload candidates|batching|greedy|sweep] [--scaling weak|strong]

Workloads (one JSON line each; `candidates` is the default and the headline):

  candidates  4096 random placements of 32 models on 64 devices scored against
              one one-hour Gamma trace (about 180 k requests).  One step = one
              pass of the simulator over the whole batch, followed by the
              search's argmax.  Weak scaling: every GPU scores a list of its
              own; strong scaling: one list of 4096 split over the GPUs.
  batching    1024 such placements with batch sizes 1/2/4/8 (the batching
              simulator).
  greedy      the placement search on 64 devices and 56 models: every step
              expands all (partition, group, model) additions and scores them
              in one launch; wall time per step.
  sweep       one placement scored on many traces (robustness sweep), traces
              sharded over the GPUs, goodput tallies combined at the end.

Metric: candidate-placements x requests simulated per second.  Every line
carries the roofline of its dominant kernel (timed with CUDA events inside
the run), the same work on the host cores (`cpu_baseline`: the reference's own
numba/Python code where it can be imported, else the C restatement of it), an
end-to-end figure from host buffers, and a parity check of the timed outputs
against the CPU checker.  A single-GPU run of the default workload also
carries short runs of the other three under "configs".
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
BYTES_PER_UNIT_FULL = 25     # ... plus f64 finish + u8 good written (per-request outputs)
NUM_CANDIDATES = 4096
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of ONE sim_stream_kernel launch (ncu) on the
# default workload: only valid for the library version and the launch shape it was taken
# with, and reported as null for any other.
STREAM_KERNEL_TRAFFIC = {"abi_version": 9, "candidates": 3695, "requests": 180715,
                         "bytes": 41885184 + 1057393152}

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
    ap.add_argument("--workload", default="candidates",
                    choices=["candidates", "batching", "greedy", "sweep", "stats"])
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="candidates: a list per GPU (weak) or one list split over the GPUs")
    ap.add_argument("--candidates", type=int, default=0,
                    help="placements per step (default 4096; batching: 1024)")
    ap.add_argument("--duration", type=float, default=0.0,
                    help="seconds of trace (default 3600; greedy 1800; sweep 3600)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-configs", action="store_true",
                    help="default workload: leave out the short runs of the other workloads")
    ap.add_argument("--greedy-steps", type=int, default=0,
                    help="greedy: stop after this many steps (0 = the whole search)")
    ap.add_argument("--slo-scale", default="5",
                    help="greedy: SLO as a multiple of the single-device latency, or 'all' for "
                         "the sweep over 2, 3, 5, 8")
    ap.add_argument("--chunk", type=int, default=0, help="requests per chunk (0 auto, <0 one)")
    ap.add_argument("--run-in", type=int, default=0, help="run-in requests per chunk (0 auto)")
    ap.add_argument("--rounds", type=int, default=0, help="validate+repair rounds (0 auto)")
    ap.add_argument("--repair-segments", type=int, default=0,
                    help="segments a repair runs per round (0 auto, <0 no cap)")
    ap.add_argument("--hard", default="",
                    help="candidates: chunk,run-in,rounds,repair-segments of the launch that holds "
                         "the placements with mirror candidates (default: as the others)")
    ap.add_argument("--traces", type=int, default=0, help="sweep: traces per GPU (default 1024)")
    ap.add_argument("--placement-seed", type=int, default=-1,
                    help="seed of the candidate list (default: the rank; strong scaling: 0)")
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


def host_cores():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


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


class Dist:
    """Rank bookkeeping and the few collectives the bench needs."""

    def __init__(self):
        import torch
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        assert torch.cuda.is_available(), "bench.py needs a CUDA device"
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=self.dev)

    def barrier(self):
        import torch
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    def reduce(self, value, op="max"):
        import torch
        t = torch.tensor([float(value)], dtype=torch.float64, device=self.dev)
        if self.world > 1:
            import torch.distributed as dist
            dist.all_reduce(t, op=dist.ReduceOp.MAX if op == "max" else dist.ReduceOp.SUM)
        return float(t.item())

    def gather(self, values):
        """All ranks' equally long f64 vectors, [world][len], on every rank."""
        import torch
        t = torch.as_tensor(np.asarray(values, np.float64), device=self.dev)
        if self.world == 1:
            return t.cpu().numpy()[None, :]
        import torch.distributed as dist
        out = torch.empty(self.world * t.numel(), dtype=torch.float64, device=self.dev)
        dist.all_gather_into_tensor(out, t)
        return out.cpu().numpy().reshape(self.world, -1)

    def close(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------
# The same work on the host cores
# ---------------------------------------------------------------------------------------------

def reference_modules():
    """The reference's own modules (numba kernels, PlacementEvaluator) when they
    can be imported here — a checkout, or the private copy under oracle/_ref —
    else (None, reason)."""
    try:
        import numba  # noqa: F401
    except Exception as e:      # the reference's kernels are numba-jitted
        return None, f"numba is not importable ({e.__class__.__name__})"
    from oracle import reference
    if not reference.available():
        return None, "no reference checkout and no oracle/_ref copy on this machine"
    try:
        return reference.load(), None
    except Exception as e:
        return None, f"the reference failed to import: {e!r}"[:200]


def dense_inputs(case, placements):
    """(model_ids, slos, m2g, num_stages, latency) for the C checker (untimed set-up)."""
    from mms_b200.simulator import workload_arrays
    from oracle import tables
    names = [d.name for d in case.model_datas]
    profs = [d.profiling_result for d in case.model_datas]
    mids, slos = workload_arrays(case.workload, names)
    m2g, ns, lat = tables.dense_tables_batch(placements, profs)
    return mids, slos, m2g, ns, lat


def port_scores(case, placements, threads):
    """The C restatement of the reference's numba kernel plus the reductions
    the score needs, for every placement, on `threads` host threads.  Returns
    (dict of result arrays, seconds of the timed call)."""
    from oracle import cpu, tables
    mids, slos, m2g, ns, lat = dense_inputs(case, placements)
    arr = case.workload.arrivals
    warm = min(len(placements), max(threads, 1))
    cpu.score_batch(arr, mids, slos, m2g[:warm], ns[:warm], lat[:warm], threads)
    t0 = time.perf_counter()
    good, lsum, mgood, greq = cpu.score_batch(arr, mids, slos, m2g, ns, lat, threads)
    dt = time.perf_counter() - t0
    scores = np.array([tables.score_from_sums(p, g, s, len(arr))
                       for p, g, s in zip(placements, good, lsum)], np.float64)
    return {"good_total": good, "latency_sum": lsum, "model_num_good": mgood,
            "group_num_requests": greq, "scores": scores}, dt


def parity_against_port(case, placements, res, scores, threads, rows=None):
    """Compares the GPU's reductions for `placements` (rows `rows` of `res`)
    with the C checker's, bit for bit.  Returns the parity record and the
    checker's throughput."""
    want, dt = port_scores(case, placements, threads)
    rows = np.arange(len(placements)) if rows is None else np.asarray(rows)
    G = want["group_num_requests"].shape[1]
    bad = np.zeros(len(placements), bool)
    bad |= res.good_total[rows] != want["good_total"]
    bad |= res.latency_sum[rows].view(np.uint64) != want["latency_sum"].view(np.uint64)
    bad |= np.any(res.model_num_good[rows] != want["model_num_good"], axis=1)
    greq = res.group_num_requests[rows]
    width = min(G, greq.shape[1])
    bad |= np.any(greq[:, :width] != want["group_num_requests"][:, :width], axis=1)
    bad |= np.asarray(scores, np.float64)[rows].view(np.uint64) != want["scores"].view(np.uint64)
    rate = len(placements) * len(case.workload) / dt
    return ({"checked": int(len(placements)), "mismatches": int(bad.sum()),
             "against": "C restatement of the reference's simulator (oracle/), "
                        f"{threads} host threads",
             "compared": "good_total, latency_sum (fp64 bits), model_num_good, "
                         "group_num_requests, score (fp64 bits)"}, rate, dt)


_REF_STATE = {}


def _ref_worker_scores(bounds):
    lo, hi = bounds
    st = _REF_STATE
    return [float(x) for x in st["ev"].get_scores(st["placements"][lo:hi])]


def reference_rate(case, placements, cores, steps=1, warmup=0):
    """Times the reference's own path — PlacementEvaluator.get_scores
    (base_policy.py:175-226: Python table building, the numba kernel, the
    fast statistics) — over `placements` on `cores` host cores (worker
    processes forked after the numba kernels are compiled; the reference is
    single-threaded).  Returns (scores, seconds per step list, kernel-only
    requests per second of simulate_requests_mixed on one core)."""
    import multiprocessing
    from oracle import reference
    ref = reference.load()
    sub = type(case)(case.name, case.model_datas, case.cluster_env, case.workload, placements)
    rdatas, renv, rw, rpls = reference.to_reference_case(sub)
    ev = ref.base_policy.PlacementEvaluator(rdatas, renv, rw, "fast_simulator", False)
    ev.get_scores(rpls[:2])                      # compiles the kernels, fills the workload cache
    # the numba kernel alone, warm, on the first placement (controller.py:561-628), with
    # the dense tables of controller.py:418-476 built beforehand
    from oracle import tables
    mids, slos = rw.cached_data[0], rw.cached_data[1]
    m2g, _, ns, lat = tables.dense_tables(placements[0], [d.profiling_result for d in rdatas])
    n_req = len(rw.arrivals)
    fin, good = np.empty(n_req, np.float64), np.empty(n_req, bool)
    t0 = time.perf_counter()
    reps = 0
    while time.perf_counter() - t0 < 0.5:
        ref.controller.simulate_requests_mixed(fin, good, rw.arrivals, mids, slos, m2g, ns, lat,
                                               n_req)
        reps += 1
    per_call = (time.perf_counter() - t0) / reps
    _REF_STATE.update(ev=ev, placements=rpls)
    n = len(rpls)
    times, scores = [], None
    if cores <= 1:
        for i in range(warmup + steps):
            t0 = time.perf_counter()
            scores = [float(x) for x in ev.get_scores(rpls)]
            if i >= warmup:
                times.append(time.perf_counter() - t0)
    else:
        step = max(1, min(32, n // (4 * cores)))
        slices = [(lo, min(n, lo + step)) for lo in range(0, n, step)]
        ctx = multiprocessing.get_context("fork")
        with ctx.Pool(cores) as pool:
            pool.map(_ref_worker_scores, slices[:cores])           # workers are up
            for i in range(warmup + steps):
                t0 = time.perf_counter()
                parts = pool.map(_ref_worker_scores, slices, chunksize=1)
                if i >= warmup:
                    times.append(time.perf_counter() - t0)
            scores = [x for part in parts for x in part]
    return np.array(scores, np.float64), times, len(rw.arrivals) / per_call


def candidates_config(args, world, B, N, strong):
    """The `config` object of the candidates workload; the same text in both arms."""
    per = "split over the GPUs" if strong else "per GPU"
    return {"workload": f"candidate-batch: 64 devices, 32 models, {args.candidates} random "
                        f"placements {per}, {args.duration:.0f} s Gamma trace (Zipf 0.9 rates, "
                        "50 req/s, CV 3), score-only",
            "num_candidates": args.candidates, "num_requests": N,
            "scaling": "strong" if strong else "weak",
            "l2": "256 MiB buffer written between timed steps (GPU arm)"}


def run_reference(args):
    """The reference's CPU implementation of the path on all host cores of this
    machine, same workload and metric: its own numba code where the reference
    can be imported, else the C restatement of it."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from mms_b200 import cases
    cores = host_cores()
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    if args.workload != "candidates":
        emit({"impl": "reference", "unavailable":
              f"the reference arm times the default workload only (got {args.workload})"})
        return
    case = cases.candidate_batch_case(num_candidates=args.candidates, duration=args.duration,
                                      placement_seed=max(args.placement_seed, 0))
    N = len(case.workload)
    ref, why = reference_modules()
    extra = {}
    if ref is not None:
        _, times, kernel_rate = reference_rate(case, case.placements, cores, args.steps,
                                               args.warmup)
        kind = "reference"
        how = (f"all {args.candidates} candidates x {N} requests per step through the "
               "reference's PlacementEvaluator.get_scores (Python table building + numba "
               f"simulate_requests_mixed + fast statistics), {cores} worker processes")
        extra["numba_kernel_only_requests_per_sec_one_core"] = kernel_rate
    else:
        times = []
        for i in range(args.warmup + args.steps):
            _, dt = port_scores(case, case.placements, cores)
            if i >= args.warmup:
                times.append(dt)
        kind = "port"
        how = (f"all {args.candidates} candidates x {N} requests per step through the C "
               f"restatement of the reference's numba kernel, {cores} host threads "
               f"(the reference itself: {why})")
    value = args.candidates * N / float(np.mean(times))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT,
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": float(np.mean(times)) * 1e3, "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": candidates_config(args, world, args.candidates, N, args.scaling == "strong"),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind,
                         "sample": how},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    line.update(extra)
    emit(line)


# ---------------------------------------------------------------------------------------------
# candidates: 4096 placements x one trace (the headline)
# ---------------------------------------------------------------------------------------------

def run_candidates(args, D):
    import ctypes

    import torch
    from mms_b200 import _native as nat
    from mms_b200 import cases, engine
    from mms_b200.placement import PlacementEvaluator
    from mms_b200.sharding import shard_bounds

    rank, world, dev = D.rank, D.world, D.dev
    strong = args.scaling == "strong"
    seed = (max(args.placement_seed, 0) if strong
            else (rank if args.placement_seed < 0 else args.placement_seed))
    case = cases.candidate_batch_case(num_candidates=args.candidates, duration=args.duration,
                                      placement_seed=seed)
    lo, hi = shard_bounds(args.candidates, rank, world) if strong else (0, args.candidates)
    mine = case.placements[lo:hi]
    first_index = lo if strong else rank * args.candidates
    opts = engine.sim_options(args.chunk, args.run_in, args.rounds, args.repair_segments)
    ev = PlacementEvaluator(case.model_datas, case.cluster_env, case.workload, device=dev,
                            options=opts)
    N, B = ev.trace.num_requests, len(mine)
    L = nat.lib()

    # ---- device-resident arm: tables already in HBM, time the C-ABI call(s) ----
    # B placements are scored; the ones with interchangeable groups bring mirror candidates
    # and go into a launch of their own beside the rest (engine.ResidentBatch)
    enc = engine.encode_placements(mine, ev.table, len(ev.model_names))
    hard = engine.sim_options(*[int(x) for x in args.hard.split(",")]) if args.hard else None
    resident = engine.ResidentBatch(ev.trace, enc, ev.table, options=opts,
                                    mirrors=not args.no_mirrors, split=not args.no_split,
                                    hard_options=hard)
    n_mirrors = sum(job.B - job.Bs for job in resident.jobs)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)   # > 126 MB of L2
    best = torch.zeros(2, dtype=torch.float64, device=dev)
    gathered = torch.zeros(2 * world, dtype=torch.float64, device=dev)
    replicas, index_map = [], []
    for idx, _, _ in resident.device_outputs():
        rows = np.arange(B) if idx is None else idx
        replicas.append(torch.from_numpy(enc.num_replicas[rows].astype(np.int64)).to(dev))
        index_map.append(None if idx is None else torch.from_numpy(idx.astype(np.int64)).to(dev))
    own_done = torch.cuda.Event(enable_timing=True)     # this rank's simulation, before the argmax

    def ptr(t):
        return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)

    def step():
        resident.launch()
        own_done.record()
        # the search's selection (np.argmax over get_scores): on the device per launch, then
        # over the ranks
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        for k, (_, good, lat_sum) in enumerate(resident.device_outputs()):
            nat.check(L.mms_argmax_scores(ptr(good), ptr(lat_sum), ptr(replicas[k]), N,
                                          int(good.numel()), ptr(index_map[k]), first_index,
                                          1 if k else 0, ptr(best), st), "mms_argmax_scores")
        if world > 1:
            import torch.distributed as dist
            dist.all_gather_into_tensor(gathered, best)
        else:
            gathered.copy_(best)

    for _ in range(max(args.warmup, 3)):
        flush.zero_()
        step()
    D.barrier()
    times, own_times = [], []
    nat.profile_begin()
    with ClockSampler(D.local) as clk:
        for _ in range(args.steps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            step()
            e1.record()
            e1.synchronize()
            times.append(e0.elapsed_time(e1))
            own_times.append(e0.elapsed_time(own_done))
    D.barrier()
    span_ms, span_tag = nat.profile_end()
    # the dominant kernel: the stream kernel of the step's largest launch (with a split step,
    # launch 0 holds the placements with mirror candidates and launch 1 the rest)
    per_step = len(resident.jobs)
    big = int(np.argmax([job.Bs for job in resident.jobs]))
    stream_ms = span_ms[span_tag == nat.PROFILE_STREAM]
    chain_ms = span_ms[span_tag == nat.PROFILE_CHAIN]
    stream_kernel_ms = float(np.mean(stream_ms[big::per_step])) if len(stream_ms) else float("nan")
    chain_kernel_ms = float(np.max(chain_ms)) if len(chain_ms) else 0.0
    call_ms = span_ms[span_tag == nat.PROFILE_CALL]
    call_ms_by_launch = [round(float(np.mean(call_ms[k::per_step])), 3) for k in range(per_step)]
    stream_ms_by_launch = [round(float(np.mean(stream_ms[k::per_step])), 3) for k in range(per_step)]
    chain_ms_by_launch = [round(float(np.mean(chain_ms[k::per_step])), 3) for k in range(per_step)] \
        if len(chain_ms) == len(stream_ms) else []
    kernel_units = resident.jobs[big].Bs * N
    total_ms = D.reduce(sum(times), "max")
    by_rank = [round(float(x), 3) for x in D.gather([float(np.mean(own_times))])[:, 0]]
    final, _ = resident.results()
    assert not np.any(final.status), "kernel status words are not clean"
    scores = np.array(ev.scores_from(enc, final), np.float64)
    redo = final.resimulated
    total_units = (args.candidates if strong else args.candidates * world) * N
    value = total_units * args.steps / (total_ms * 1e-3)

    # ---- what the timed steps computed, against the checker -------------------------------
    # every rank's scores go to rank 0: the argmax the steps exchanged must be np.argmax over
    # all of them; rank 0 then checks every reduction of its own candidates against the C
    # checker, and (several ranks) the winner's score on whichever rank's list it is
    width = -(-args.candidates // world) if strong else args.candidates
    padded = np.full(width, -np.inf)
    padded[:B] = scores
    every = D.gather(padded)
    pairs = gathered.cpu().numpy().reshape(world, 2)
    parity = argmax_checked = None
    if rank == 0:
        if strong:
            flat = np.concatenate([every[r, :shard_bounds(args.candidates, r, world)[1]
                                         - shard_bounds(args.candidates, r, world)[0]]
                                   for r in range(world)])
        else:
            flat = every.reshape(-1)
        want_idx = int(np.argmax(flat))
        top = pairs[:, 0].max()
        got_idx = int(pairs[pairs[:, 0] == top, 1].min())
        argmax_checked = bool(got_idx == want_idx and top == flat[want_idx])
        assert argmax_checked, ("argmax over ranks", got_idx, want_idx, top, flat[want_idx])
        if not args.no_cpu_baseline:
            threads = host_cores()
            parity, port_rate, port_dt = parity_against_port(case, mine, final, scores, threads)
            parity["port_rate"] = port_rate
            if world > 1:
                # the winner, wherever it was scored
                if strong:
                    wcase, wpos = case, want_idx
                else:
                    wrank, wpos = divmod(want_idx, args.candidates)
                    wcase = case if wrank == 0 else cases.candidate_batch_case(
                        num_candidates=args.candidates, duration=args.duration,
                        placement_seed=wrank if args.placement_seed < 0 else args.placement_seed)
                wres, _ = port_scores(wcase, [wcase.placements[wpos]], 1)
                parity["winner_score_equals_checker"] = bool(wres["scores"][0] == top)
                parity["mismatches"] += 0 if parity["winner_score_equals_checker"] else 1
            if strong and world > 1:
                # all ranks' scores of the one list
                allw, _ = port_scores(case, case.placements, threads)
                diff = int(np.sum(allw["scores"].view(np.uint64) != flat.view(np.uint64)))
                parity["checked_all_ranks"] = int(len(flat))
                parity["mismatches"] += diff

    # ---- end-to-end arm: host buffers in, scores out, through the evaluator ----
    e2e_times, h2d, d2h = [], 0, 0
    e2e_scores = None
    for i in range(2 + min(args.steps, 3)):
        D.barrier()
        t0 = time.perf_counter()
        ev.trace = engine.DeviceTrace(case.workload.arrivals, ev.workload.cached_data[0],
                                      ev.workload.cached_data[1], len(ev.model_names), dev)
        e2e_scores = ev.get_scores(mine)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        if i >= 2:
            e2e_times.append(dt)
        h2d = ev.trace.h2d_bytes + ev.last_h2d_bytes
        d2h = ev.last_d2h_bytes
    e2e_value = total_units / D.reduce(float(np.mean(e2e_times)), "max")
    assert np.array_equal(np.array(e2e_scores, np.float64).view(np.uint64), scores.view(np.uint64)), \
        "the end-to-end arm and the resident arm disagree"

    line = None
    if rank == 0:
        peak, which = hbm_peak()
        achieved = kernel_units * BYTES_PER_UNIT / (stream_kernel_ms * 1e-3) / 1e9
        call_achieved = B * N * BYTES_PER_UNIT / (np.mean(times) * 1e-3) / 1e9
        t = STREAM_KERNEL_TRAFFIC
        traffic = t["bytes"] if (t["abi_version"] == L.mms_abi_version() and
                                 (t["candidates"], t["requests"]) == (resident.jobs[big].Bs, N)) else None
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": total_ms / args.steps, "higher_is_better": True,
            "scaling": "strong" if strong else "weak",
            "vs_baseline": None, "dtype": "f64", "data": "synthetic",
            "config": candidates_config(args, world, args.candidates, N, strong),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak,
                         "achieved_is": "algorithmic bytes (16 B per candidate and request) over "
                                        "the kernel's CUDA-event time; the trace is shared and "
                                        "L2-resident, so DRAM traffic is far lower",
                         "traffic": traffic,
                         "traffic_unit": "bytes per sim_stream_kernel launch (ncu, DRAM read+write)",
                         "dram_gbs": (traffic / (stream_kernel_ms * 1e-3) / 1e9) if traffic else None,
                         "kernel": "sim_stream_kernel", "kernel_ms": stream_kernel_ms,
                         "kernel_candidates": int(resident.jobs[big].Bs),
                         "kernel_launches_timed": int(len(stream_ms)) // per_step,
                         "chain_kernel_ms_max": chain_kernel_ms,
                         # per launch of a step, in launch order (they overlap on the GPU)
                         "call_ms_by_launch": call_ms_by_launch,
                         "stream_kernel_ms_by_launch": stream_ms_by_launch,
                         "chain_kernel_ms_by_launch": chain_ms_by_launch,
                         "whole_call": {"achieved": call_achieved, "frac": call_achieved / peak,
                                        "ms": float(np.mean(times))},
                         "peak_source": which, "bytes_per_unit": BYTES_PER_UNIT,
                         "algorithmic_bytes_per_launch": kernel_units * BYTES_PER_UNIT},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": int(h2d),
                    "d2h_bytes_per_step": int(d2h)},
            # clear, tables, stream, (validate, resolve, two forms of repair) per round, two
            # forms of chain, count, requests per model — per launch — and the argmax
            "gpu_launches": ((7 + 4 * (args.rounds if args.rounds > 0 else 4) + 1) * args.steps
                             * len(resident.jobs)),
            "mirror_candidates_per_gpu": int(n_mirrors),
            "launches_per_step": len(resident.jobs),
            # each rank's simulation per step, before the selection and its exchange
            "kernel_ms_per_step_by_rank": by_rank,
            "chunks_resimulated_per_candidate": float(np.mean(redo)),
            "chunks_resimulated_hist": np.bincount(redo).tolist(),
            "clocks": clk.summary(),
            "best_score": float(np.max(flat)),
            "argmax_checked": argmax_checked,
        }
        if parity is not None:
            line["parity"] = parity
        if not args.no_cpu_baseline and world == 1:      # single-GPU runs only
            line.update(candidates_cpu_baseline(case, mine, scores))
            line["vs_cpu_baseline"] = value / line["cpu_baseline"]["value"]
    return line


def candidates_cpu_baseline(case, placements, gpu_scores):
    """cpu_baseline of the candidates workload on ONE host core: the
    reference's own path over a sample (and its scores against the GPU's),
    else the C restatement."""
    N = len(case.workload)
    ref, why = reference_modules()
    if ref is not None:
        count = min(len(placements), 1024)       # about 10 s of one host core
        ref_scores, times, kernel_rate = reference_rate(case, placements[:count], 1)
        dt = times[0]
        same = ref_scores.view(np.uint64) == np.asarray(gpu_scores[:count], np.float64).view(np.uint64)
        return {"cpu_baseline": {
                    "value": count * N / dt, "unit": UNIT, "cores": 1, "kind": "reference",
                    "sample": f"first {count} of {len(placements)} candidates x {N} requests through "
                              "the reference's PlacementEvaluator.get_scores (Python table "
                              f"building + numba kernel), {dt:.1f} s",
                    "numba_kernel_only_requests_per_sec": kernel_rate},
                "parity_reference": {"checked": int(count), "mismatches": int(np.sum(~same)),
                                     "against": "scores of the reference's own evaluator (fp64 bits)"}}
    count = min(len(placements), 3072)
    _, dt = port_scores(case, placements[:count], 1)
    return {"cpu_baseline": {
        "value": count * N / dt, "unit": UNIT, "cores": 1, "kind": "port",
        "sample": f"{count} of {len(placements)} candidates x {N} requests, {dt:.1f} s "
                  f"(the reference itself: {why})"}}


# ---------------------------------------------------------------------------------------------
# batching: 1024 placements, batch sizes 1/2/4/8
# ---------------------------------------------------------------------------------------------

def run_batching(args, D, candidates=1024, duration=3600.0, steps=None, cpu=True):
    import torch
    from mms_b200 import _native as nat
    from mms_b200 import cases, engine
    from mms_b200.simulator import workload_arrays

    rank, world, dev = D.rank, D.world, D.dev
    steps = steps or args.steps
    case = cases.candidate_batch_case(num_candidates=candidates, duration=duration,
                                      placement_seed=rank, batching=True)
    names = [d.name for d in case.model_datas]
    profs = [d.profiling_result for d in case.model_datas]
    mids, slos = workload_arrays(case.workload, names)
    arr = case.workload.arrivals
    N, B = len(arr), len(case.placements)
    bs = list(case.batch_sizes)

    trace = engine.DeviceTrace(arr, mids, slos, len(names), dev)
    table = engine.LatencyTable(profs, bs)
    enc = engine.encode_placements(case.placements, table, len(names))
    job = engine.resident_batching(trace, enc, table)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for _ in range(3):
        flush.zero_()
        job.launch()
    D.barrier()
    times = []
    nat.profile_begin()
    with ClockSampler(D.local) as clk:
        for _ in range(steps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            job.launch()
            e1.record()
            e1.synchronize()
            times.append(e0.elapsed_time(e1))
    D.barrier()
    span_ms, span_tag = nat.profile_end()
    stream_ms = span_ms[span_tag == nat.PROFILE_BATCH_STREAM]
    chain_ms = span_ms[span_tag == nat.PROFILE_BATCH_CHAIN]
    res, _ = job.results(per_request=False)
    assert not np.any(res.status), "kernel status words are not clean"
    total_ms = D.reduce(sum(times), "max")
    value = B * N * world * steps / (total_ms * 1e-3)

    # end to end: host tables and trace in, reductions out
    e2e_times = []
    h2d = d2h = 0
    for i in range(3):
        D.barrier()
        t0 = time.perf_counter()
        tr = engine.DeviceTrace(arr, mids, slos, len(names), dev)
        tb = engine.LatencyTable(profs, bs)
        e = engine.encode_placements(case.placements, tb, len(names))
        j = engine.resident_batching(tr, e, tb).launch()
        r2, d2h = j.results(per_request=False)
        if i >= 1:
            e2e_times.append(time.perf_counter() - t0)
        h2d = tr.h2d_bytes + j.h2d_bytes + tb.host.nbytes
    e2e_value = B * N * world / D.reduce(float(np.mean(e2e_times)), "max")
    assert r2.latency_sum.tobytes() == res.latency_sum.tobytes()

    if rank != 0:
        return None
    peak, which = hbm_peak()
    k_ms = float(np.mean(stream_ms)) if len(stream_ms) else float("nan")
    dominant, dom_ms = "batch_stream_kernel", k_ms
    if len(chain_ms) and float(np.mean(chain_ms)) > k_ms:
        dominant, dom_ms = "batch_chain_kernel", float(np.mean(chain_ms))
    achieved = B * N * BYTES_PER_UNIT_FULL / (dom_ms * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps,
        "warmup": 3, "ms_per_step": total_ms / steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": f"candidate-batch with batching: 64 devices, 32 models, {B} random "
                               f"placements per GPU, batch sizes {bs}, l(b) = l(1)(0.8 + 0.2 b), "
                               f"{duration:.0f} s Gamma trace (50 req/s, CV 3)",
                   "num_candidates": B, "num_requests": N,
                   "l2": "256 MiB buffer written between timed steps"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "traffic": None, "kernel": dominant,
                     "kernel_ms": dom_ms, "stream_kernel_ms": k_ms,
                     "chain_kernel_ms": float(np.mean(chain_ms)) if len(chain_ms) else 0.0,
                     "peak_source": which, "bytes_per_unit": BYTES_PER_UNIT_FULL,
                     "algorithmic_bytes_per_launch": B * N * BYTES_PER_UNIT_FULL},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(d2h)},
        "gpu_launches": 6 * steps,
        "chunks_resimulated_per_candidate": float(np.mean(res.resimulated)),
        "clocks": clk.summary(),
    }
    if cpu:
        line.update(batching_checks(case, res, profs, mids, slos, arr, bs))
    return line


def batching_checks(case, res, profs, mids, slos, arr, bs):
    """Parity of a sample of candidates against the C checker (threads), the
    checker's rate on one thread, and the reference's pure-Python simulator on
    a slice of the trace."""
    from concurrent.futures import ThreadPoolExecutor
    from oracle import tables
    N = len(arr)
    threads = host_cores()
    sample = list(range(0, len(case.placements), max(1, len(case.placements) // 128)))[:128]

    def one(b):
        return tables.one_placement(case.placements[b], profs, mids, slos, arr, bs)

    t0 = time.perf_counter()
    one(sample[0])
    t_one = time.perf_counter() - t0
    with ThreadPoolExecutor(threads) as pool:       # the C call releases the GIL
        outs = list(pool.map(one, sample))
    bad = 0
    for b, (fin, good, mreq, mgood, greq, ggood) in zip(sample, outs):
        ok = (res.good_total[b] == np.count_nonzero(good)
              and res.latency_sum[b] == float(np.add.reduce(fin - arr))
              and np.array_equal(res.model_num_good[b], mgood)
              and np.array_equal(res.model_num_requests[b], mreq)
              and np.array_equal(res.group_num_requests[b, :len(greq)], greq)
              and np.array_equal(res.group_num_good[b, :len(ggood)], ggood))
        bad += 0 if ok else 1
    out = {"parity": {"checked": len(sample), "mismatches": int(bad),
                      "against": "C restatement of simulate_requests_mixed_batching (oracle/)",
                      "compared": "good_total, latency_sum (fp64), all four counter arrays"},
           "cpu_baseline": {"value": N / t_one, "unit": UNIT, "cores": 1, "kind": "port",
                            "sample": f"1 candidate x {N} requests, {t_one:.2f} s"}}
    ref, why = reference_modules()
    if ref is not None:
        # the reference's batching simulator is interpreted Python (about 0.1 M requests/s):
        # a slice of the trace for one placement
        from oracle import reference
        n = min(N, 40000)
        sub = type(case)(case.name, case.model_datas, case.cluster_env, case.workload,
                         case.placements[:1], case.batch_sizes)
        rdatas, _, _, rpls = reference.to_reference_case(sub)
        ref.util.batchsize_config[:] = bs
        names = [d.name for d in rdatas]
        rprofs = [d.profiling_result for d in rdatas]
        t0 = time.perf_counter()
        ref.controller.approximate_one_case_one_placement(rpls[0], names, rprofs, mids[:n],
                                                          slos[:n], arr[:n], enable_batching=True)
        dt = time.perf_counter() - t0
        out["cpu_baseline"] = {"value": n / dt, "unit": UNIT, "cores": 1, "kind": "reference",
                               "sample": f"1 candidate x the first {n} requests through the "
                                         "reference's pure-Python simulate_requests_mixed_batching, "
                                         f"{dt:.1f} s", "port_value": N / t_one}
    return out


# ---------------------------------------------------------------------------------------------
# greedy: the placement search, wall time per step
# ---------------------------------------------------------------------------------------------

class RecordingEvaluator:
    """Passes get_scores through and keeps the first lists (for the checker)."""

    def __init__(self, ev, keep_units):
        self.ev, self.keep_units, self.kept, self.units = ev, keep_units, [], 0

    def get_scores(self, sols):
        scores = self.ev.get_scores(sols)
        if self.units < self.keep_units:
            self.kept.append((list(sols), list(scores)))
            self.units += len(sols)
        return scores

    def __getattr__(self, name):
        return getattr(self.ev, name)


def run_greedy(args, D, slo_scale=5.0, max_steps=0, duration=1800.0, cpu=True):
    """The lockstep beam search (beam 1) over the four pipeline partitions of 64
    devices (operator parallelism 1: 64x1, 32x2, 16x4, 8x8), 56 models."""
    import torch
    from mms_b200 import _native as nat
    from mms_b200 import cases, search
    from mms_b200.placement import PlacementEvaluator
    dev = D.dev
    case = cases.greedy_search_case(slo_scale=slo_scale, duration=duration)
    N = len(case.workload)
    ev = RecordingEvaluator(PlacementEvaluator(case.model_datas, case.cluster_env, case.workload,
                                               device=dev), keep_units=1500)
    starts = search.ModelParallelismSearch(max_op=1).enumerate_group_configs_uneven(
        case.cluster_env)
    layers = []

    class Enough(Exception):
        pass

    def on_layer(n, seconds):
        layers.append((n, seconds))
        if max_steps and len(layers) >= max_steps + 1:
            raise Enough()

    best = None
    nat.profile_begin()
    t0 = time.perf_counter()
    with ClockSampler(D.local) as clk:
        try:
            best = search.beam_search_lockstep(starts, case.model_datas, case.cluster_env, ev, 1,
                                               on_layer=on_layer)
        except Enough:
            pass
        torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    span_ms, span_tag = nat.profile_end()
    timed = layers[1:] or layers            # the first step also warms up
    cands = float(np.sum([x[0] for x in timed]))
    sec = float(np.sum([x[1] for x in timed]))
    stream_ms = span_ms[span_tag == nat.PROFILE_STREAM]
    peak, which = hbm_peak()
    units_all = float(np.sum([x[0] for x in layers])) * N
    # every launch of the search is bracketed, unless there were more than the library keeps
    k_ms = float(np.sum(stream_ms))
    complete = 0 < len(span_ms) < 2048
    achieved = (units_all * BYTES_PER_UNIT / (k_ms * 1e-3) / 1e9) if (k_ms and complete) else 0.0
    line = {
        "metric": METRIC, "value": cands * N / sec, "unit": UNIT, "n_gpus": 1,
        "steps": len(timed), "warmup": 1, "ms_per_step": sec / len(timed) * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64",
        "data": "synthetic",
        "config": {"workload": "greedy placement search: 64 devices, 56 models over eight latency "
                               f"tables, Zipf 0.9 shares of 80 req/s, CV 4, {duration:.0f} s, seed 1, "
                               f"SLO {slo_scale:g}x; beam search of width 1 over the 4 pipeline "
                               "partitions (operator parallelism 1; the config defines no latency "
                               "for operator parallelism), all advanced in lockstep, "
                               + ("whole search" if not max_steps else f"first {max_steps} steps"),
                   "num_requests": N, "partitions": len(starts), "slo_scale": slo_scale,
                   "candidates_per_step_mean": cands / len(timed),
                   "candidates_per_step_max": int(max(x[0] for x in layers))},
        "greedy_step_ms": sec / len(timed) * 1e3,
        "search_wall_s": wall, "search_steps": len(layers),
        "includes": "host expansion and dedup, encoding, H2D, kernels, D2H, top-1 per partition",
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "traffic": None, "kernel": "sim_stream_kernel",
                     "kernel_ms": k_ms / max(1, len(stream_ms)),
                     "kernel_launches_timed": int(len(stream_ms)), "peak_source": which,
                     "bytes_per_unit": BYTES_PER_UNIT},
        "e2e": {"value": cands * N / sec, "unit": UNIT,
                "h2d_bytes_per_step": int(ev.ev.last_h2d_bytes),
                "d2h_bytes_per_step": int(ev.ev.last_d2h_bytes)},
        "gpu_launches": int(len(span_ms)),
        "clocks": clk.summary(),
    }
    if best is not None:
        final = ev.ev.get_scores(best)
        line["best_score"] = float(np.max(final))
        line["best_partition_groups"] = int(len(best[int(np.argmax(final))].group_configs))
    if cpu and ev.kept:
        # the same step lists through the checker on one host thread: time and scores
        flat = [s for sols, _ in ev.kept for s in sols]
        got = np.array([x for _, sc in ev.kept for x in sc], np.float64)
        want, dt = port_scores(case, flat, 1)
        line["parity"] = {"checked": len(flat),
                          "mismatches": int(np.sum(want["scores"].view(np.uint64) != got.view(np.uint64))),
                          "against": "scores from the C restatement (oracle/), fp64 bits",
                          "steps_checked": len(ev.kept)}
        gpu_sec = float(np.sum([x[1] for x in layers[:len(ev.kept)]]))
        line["cpu_baseline"] = {
            "value": len(flat) * N / dt, "unit": UNIT, "cores": 1, "kind": "port",
            "sample": f"the candidate lists of the first {len(ev.kept)} steps ({len(flat)} "
                      f"placements x {N} requests): {dt:.2f} s on one host thread (simulation "
                      f"only) against {gpu_sec:.3f} s here (whole steps)"}
    return line


# ---------------------------------------------------------------------------------------------
# sweep: one placement x many traces
# ---------------------------------------------------------------------------------------------

def run_sweep(args, D, traces=1024, duration=3600.0, steps=None, cpu=True):
    """One placement x many traces per GPU (trace t of rank r is global trace
    r * traces + t); 1 unit = 1 trace x 1 request.  The tallies per cell are
    combined over the ranks inside the timed step."""
    import torch
    from mms_b200 import _native as nat
    from mms_b200 import cases, engine
    from mms_b200.placement import TraceSweep
    from mms_b200.simulator import workload_arrays

    rank, world, dev = D.rank, D.world, D.dev
    steps = steps or args.steps
    case = cases.sweep_case(duration=duration)
    T = traces
    t_gen = time.perf_counter()
    workloads = [case.trace(rank * T + t) for t in range(T)]
    t_gen = time.perf_counter() - t_gen
    opts = engine.sim_options(args.chunk, args.run_in, args.rounds, args.repair_segments)
    sweep = TraceSweep(case.model_datas, case.cluster_env, case.placement, device=dev,
                       options=opts, cells=16, first_trace=rank * T)
    names = sweep.model_names
    units = int(sum(len(w.arrivals) for w in workloads))

    # ---- device-resident arm: the traces are in HBM, one step = simulate all + tally ----
    resident = sweep.resident(workloads)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def step():
        tally = resident.launch()
        if world > 1:
            import torch.distributed as dist
            dist.all_reduce(tally)
        return tally

    for _ in range(max(min(args.warmup, 3), 1)):
        flush.zero_()
        step()
    D.barrier()
    times = []
    nat.profile_begin()
    with ClockSampler(D.local) as clk:
        for _ in range(steps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            tally = step()
            e1.record()
            e1.synchronize()
            times.append(e0.elapsed_time(e1))
    D.barrier()
    span_ms, span_tag = nat.profile_end()
    res = resident.results()
    total_ms = D.reduce(sum(times), "max")
    all_units = D.reduce(units, "sum")
    value = all_units * steps / (total_ms * 1e-3)
    # groups run side by side on streams of their own: the step lasts as long as its
    # longest group, whose chain kernel (one trace to a warp, walked from end to end where
    # the load never lets the state settle) is the dominant launch
    n_groups = len(resident.groups)
    group_units = [int(resident.lengths[idx].sum()) for idx in resident.groups]
    stream_all = span_ms[span_tag == nat.PROFILE_STREAM]
    chain_all = span_ms[span_tag == nat.PROFILE_CHAIN]
    stream_by_group = [float(np.mean(stream_all[g::n_groups])) for g in range(n_groups)] \
        if len(stream_all) == steps * n_groups else []
    chain_by_group = [float(np.mean(chain_all[g::n_groups])) for g in range(n_groups)] \
        if len(chain_all) == steps * n_groups else []
    tally_host = tally.cpu().numpy()
    resident.release()

    # ---- end-to-end arm: host traces in, goodputs out, tallies combined ----
    e2e_times = []
    got = None
    for i in range(2):
        D.barrier()
        t0 = time.perf_counter()
        got, tl = sweep.evaluate_tally(workloads)
        if world > 1:
            import torch.distributed as dist
            dist.all_reduce(tl)
        torch.cuda.synchronize()
        if i >= 1 or steps == 1:
            e2e_times.append(time.perf_counter() - t0)
    e2e_value = all_units / D.reduce(float(np.mean(e2e_times)), "max")
    goodputs = np.array([g[0] for g in got])
    lengths = np.array([len(w.arrivals) for w in workloads])
    assert np.array_equal(goodputs, res.good_total / lengths), "resident and e2e arms differ"

    if rank != 0:
        return None
    peak, which = hbm_peak()
    if chain_by_group and max(chain_by_group) >= max(stream_by_group or [0.0]):
        g = int(np.argmax(chain_by_group))
        dominant, dom_ms, dom_units = "sim_chain_kernel", chain_by_group[g], group_units[g]
    elif stream_by_group:
        g = int(np.argmax(stream_by_group))
        dominant, dom_ms, dom_units = "sim_stream_kernel", stream_by_group[g], group_units[g]
    else:
        dominant, dom_ms, dom_units = "whole step", float(np.mean(times)), units
    achieved = dom_units * BYTES_PER_UNIT / (dom_ms * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps,
        "warmup": max(min(args.warmup, 3), 1), "ms_per_step": total_ms / steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64",
        "data": "synthetic",
        "config": {"workload": f"trace-sweep: one 64-device placement of 32 models x {T} traces "
                               f"per GPU ({duration:.0f} s Gamma traces, 16 cells of rate scale "
                               "{0.5,1,2,4} x CV {1,2,4,8}, 278 req/s at scale 1), traces of one "
                               "rate scale per launch",
                   "traces_per_gpu": T, "requests_per_gpu": units,
                   "parallelism": f"traces sharded over {world} GPU(s); per-cell tallies "
                                  "all-reduced inside the timed step",
                   "l2": "256 MiB buffer written between timed steps",
                   "host_trace_generation_s": t_gen},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "traffic": None, "kernel": dominant,
                     "kernel_ms": dom_ms, "kernel_units": dom_units,
                     "launches_side_by_side": n_groups,
                     "stream_kernel_ms_by_group": stream_by_group,
                     "chain_kernel_ms_by_group": chain_by_group,
                     "requests_by_group": group_units, "peak_source": which,
                     "bytes_per_unit": BYTES_PER_UNIT,
                     "algorithmic_bytes_per_launch": dom_units * BYTES_PER_UNIT},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": int(sweep.last_h2d_bytes),
                "d2h_bytes_per_step": int(sweep.last_d2h_bytes)},
        "gpu_launches": (7 + 4 * (args.rounds if args.rounds > 0 else 4)) * n_groups * steps,
        "chunks_resimulated_per_trace": float(np.mean(res.resimulated)),
        "clocks": clk.summary(),
        "goodput_mean_per_cell": [float(x) for x in (tally_host[:, 0] / np.maximum(tally_host[:, 1], 1))],
    }
    if cpu:
        from oracle import tables
        profs = [d.profiling_result for d in case.model_datas]
        t0 = time.perf_counter()
        done, bad, checked = 0, 0, 0
        order = list(range(0, T, max(1, T // 32)))       # traces of every cell
        for t in order:
            a = workload_arrays(workloads[t], names)
            out = tables.one_placement(case.placement, profs, a[0], a[1], workloads[t].arrivals)
            done += len(workloads[t].arrivals)
            checked += 1
            ok = (res.good_total[t] == np.count_nonzero(out[1])
                  and np.array_equal(res.model_num_good[t], out[3])
                  and np.array_equal(res.group_num_requests[t, :len(out[4])], out[4]))
            bad += 0 if ok else 1
            if time.perf_counter() - t0 > 20.0:
                break
        dt = time.perf_counter() - t0
        line["cpu_baseline"] = {"value": done / dt, "unit": UNIT, "cores": 1, "kind": "port",
                                "sample": f"{checked} traces ({done} requests), {dt:.1f} s"}
        line["parity"] = {"checked": checked, "mismatches": bad,
                          "against": "C restatement (oracle/), per trace: good_total, "
                                     "model_num_good, group_num_requests"}
    return line


def run_stats(args, D, candidates=8, duration=3600.0, steps=5):
    """Workload.compute_stats (workload.py:308-354) of `candidates` placements'
    per-request outputs: mms_compute_stats on rows that never left the GPU,
    against the host route (download 9 bytes per request, then the checker's
    numpy statistics, which are the reference's own numpy calls)."""
    import torch
    from mms_b200 import cases, engine
    from mms_b200.simulator import workload_arrays
    from oracle import stats as ostats

    dev = D.dev
    case = cases.candidate_batch_case(num_candidates=candidates, duration=duration)
    w = case.workload
    names = [d.name for d in case.model_datas]
    profs = [d.profiling_result for d in case.model_datas]
    mids, slos = workload_arrays(w, names)
    trace = engine.DeviceTrace(w.arrivals, mids, slos, len(names), dev)
    table = engine.LatencyTable(profs)
    enc = engine.encode_placements(case.placements, table, len(names))
    res, _, _ = engine.run_batch(trace, enc, table, per_request=True, group_good=True,
                                 rows_on_device=True)
    B, N = res.finish_device.shape
    lo, hi = ostats.window(w.arrivals, 10.0)
    d_which = torch.from_numpy(np.asarray(w.name_index, np.int32)).to(dev)
    K = len(w.names)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    times, wall = [], []
    for i in range(3 + steps):
        flush.zero_()
        torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        st = engine.device_compute_stats(trace.arrivals, d_which, K, res.finish_device,
                                         res.good_device, lo, hi - lo)
        e1.record()
        e1.synchronize()
        if i >= 3:
            times.append(e0.elapsed_time(e1))
            wall.append((time.perf_counter() - t0) * 1e3)
    # the host route, for every placement: download the rows, numpy statistics
    t0 = time.perf_counter()
    fin = res.finish_device.cpu().numpy()
    good = res.good_device.cpu().numpy().astype(bool)
    t_down = time.perf_counter() - t0
    t0 = time.perf_counter()
    mismatches = 0
    index = {n: k for k, n in enumerate(w.names)}
    for b in range(B):
        per_model, overall = ostats.compute_stats(w.arrivals, w.name_index, w.names, w.arrivals,
                                                  fin[b], good[b], 10.0)
        for p in per_model:
            k = index[p["name"]]
            for field in ("latency_mean", "latency_std", "latency_p90", "latency_p99"):
                mismatches += st[field][b, k].tobytes() != np.float64(p[field]).tobytes()
            mismatches += int(st["num_good"][b, k]) != round(p["goodput"] * p["num_requests"])
        mismatches += (st["latency_sum"][b] / (hi - lo)) != overall[1]
        mismatches += np.float64(st["good_total"][b]) / (hi - lo) != overall[0]
    t_numpy = time.perf_counter() - t0
    assert mismatches == 0, f"{mismatches} statistics differ from the checker's"
    ms = float(np.mean(times))
    # read once by the compaction per model and candidate from L2, from HBM about once:
    # finish 8 + good 1 + arrivals 8 + model id 4 per request, plus the compacted latencies
    # written once and read four times (two sums, two selections of eight passes each: L2)
    return {
        "workload": f"compute_stats of {B} placements, {N} requests, {K} models, warm-up 10 s",
        "device_ms": ms, "device_wall_ms": float(np.mean(wall)),
        "requests_per_s": B * (hi - lo) / (ms * 1e-3),
        "d2h_bytes": int(st["d2h_bytes"]),
        "host_route_ms": (t_down + t_numpy) * 1e3, "host_download_ms": t_down * 1e3,
        "host_numpy_ms": t_numpy * 1e3, "host_d2h_bytes": int(fin.nbytes + good.nbytes),
        "parity": {"against": "numpy statistics of the downloaded rows (checker)",
                   "mismatches": int(mismatches)},
    }


def guarded(name, fn):
    """A short run of another workload inside the default line: its failure must
    not lose the headline."""
    t0 = time.perf_counter()
    try:
        out = fn()
    except Exception as e:      # noqa: BLE001
        import traceback
        traceback.print_exc()
        return {"error": f"{e.__class__.__name__}: {e}"[:300]}
    if out is not None:
        out["bench_seconds"] = time.perf_counter() - t0
    return out


def main():
    args = parse_args()
    quiet_stdout()
    if not args.candidates:
        args.candidates = 1024 if args.workload == "batching" else NUM_CANDIDATES
    if not args.duration:
        args.duration = 1800.0 if args.workload == "greedy" else 3600.0
    if args.impl == "reference":
        run_reference(args)
        return
    D = Dist()
    if args.workload == "batching":
        line = run_batching(args, D, args.candidates, args.duration, cpu=not args.no_cpu_baseline)
    elif args.workload == "greedy":
        if args.slo_scale == "all":
            line = None
            sweep = {}
            for scale in (2.0, 3.0, 5.0, 8.0):
                one = run_greedy(args, D, scale, args.greedy_steps, args.duration,
                                 cpu=not args.no_cpu_baseline and scale == 5.0)
                sweep[f"{scale:g}"] = {k: one[k] for k in ("value", "greedy_step_ms", "search_wall_s",
                                                           "search_steps", "best_score")
                                       if k in one}
                if scale == 5.0:
                    line = one
            line["slo_sweep"] = sweep
        else:
            line = run_greedy(args, D, float(args.slo_scale), args.greedy_steps, args.duration,
                              cpu=not args.no_cpu_baseline)
    elif args.workload == "stats":
        # not a contract line: the figures of the compute_stats path alone
        line = run_stats(args, D, 8, args.duration, steps=args.steps) if D.rank == 0 else None
    elif args.workload == "sweep":
        line = run_sweep(args, D, args.traces or 1024, args.duration,
                         cpu=not args.no_cpu_baseline)
    else:
        line = run_candidates(args, D)
        if (line is not None and D.world == 1 and not args.no_configs
                and args.scaling == "weak"):
            # short runs of the other workloads, so that one command shows all of them
            line["configs"] = {
                "batching": guarded("batching", lambda: run_batching(
                    args, D, 1024, 3600.0, steps=3, cpu=not args.no_cpu_baseline)),
                "greedy": guarded("greedy", lambda: run_greedy(
                    args, D, 5.0, max_steps=24, cpu=not args.no_cpu_baseline)),
                "sweep": guarded("sweep", lambda: run_sweep(
                    args, D, 256, 360.0, steps=2, cpu=not args.no_cpu_baseline)),
                "compute_stats": guarded("compute_stats", lambda: run_stats(args, D)),
            }
    if line is not None:
        emit(line)
    D.close()


if __name__ == "__main__":
    main()
