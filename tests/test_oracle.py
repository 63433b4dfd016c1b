"""The CPU checker against the golden outputs of the live reference."""
import hashlib

import numpy as np
import pytest

from mms_b200 import cases
from mms_b200.simulator import workload_arrays
from oracle import cpu, tables


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def same_counters(got, g):
    for arr, key in zip(got, ("model_num_requests", "model_num_good", "group_num_requests",
                              "group_num_good")):
        assert np.array_equal(arr, g[key]), key


def test_mixed_kernel_matches_numba(golden):
    g = golden("kernel_mixed")
    N = len(g["tstamps"])
    fin = np.empty(N); good = np.empty(N, bool)
    got = cpu.simulate_requests_mixed(fin, good, g["tstamps"], g["model_ids"], g["slos"],
                                      g["m_id2g_id"], g["num_stages"], g["stage_latency"], N)
    assert fin.tobytes() == g["finish"].tobytes()      # bit-exact fp64
    assert np.array_equal(good, g["good"])
    same_counters(got, g)
    assert 0.2 < good.mean() < 0.95                    # both branches are exercised


def test_legacy_kernel_matches_numba(golden):
    g = golden("kernel_legacy")
    N = len(g["tstamps"])
    fin = np.empty(N); good = np.empty(N, bool)
    got = cpu.simulate_requests(fin, good, g["tstamps"], g["model_ids"], g["slos"],
                                g["m_id2g_id"], g["group_max_latency"],
                                g["group_sum_latency"], N)
    assert fin.tobytes() == g["finish"].tobytes()
    assert np.array_equal(good, g["good"])
    same_counters(got, g)


def test_batching_kernel_matches_python_reference(golden):
    g = golden("kernel_batching")
    N = len(g["tstamps"])
    fin = np.empty(N); good = np.empty(N, bool)
    got = cpu.simulate_requests_mixed_batching(
        fin, good, g["tstamps"], g["model_ids"], g["slos"], g["m_id2g_id"], g["g_id2m_id"],
        g["num_stages"], g["stage_latency"], N, tuple(g["batchsize_config"]))
    assert fin.tobytes() == g["finish"].tobytes()
    assert np.array_equal(good, g["good"])
    same_counters(got, g)


def test_fixed_pipeline_case_full_size(golden):
    g = golden("case_fixed_pipeline")
    case = cases.fixed_pipeline_case()
    w = case.workload
    assert len(w) == int(g["num_requests"])
    assert sha(w.arrivals) == str(g["arrivals_sha256"])   # numpy's Gamma stream is unchanged
    names = [d.name for d in case.model_datas]
    profs = [d.profiling_result for d in case.model_datas]
    mids, slos = workload_arrays(w, names)
    assert sha(mids) == str(g["model_ids_sha256"])
    fin, good, mreq, mgood, greq, ggood = tables.one_placement(
        case.placements[0], profs, mids, slos, w.arrivals)
    assert sha(fin) == str(g["finish_sha256"])
    assert sha(good.astype(np.uint8)) == str(g["good_sha256"])
    same_counters((mreq, mgood, greq, ggood), g)
    assert np.mean(good) == float(g["goodput"])
    assert cpu.latency_mean(fin, w.arrivals) == float(g["latency_mean"])
    assert tables.score(case.placements[0], fin, good, w.arrivals) == float(g["score"])


def test_candidate_batch_scores(golden):
    g = golden("case_candidates")
    case = cases.candidate_batch_case(num_candidates=int(g["num_candidates"]),
                                      duration=float(g["duration"]))
    w = case.workload
    assert sha(w.arrivals) == str(g["arrivals_sha256"])
    names = [d.name for d in case.model_datas]
    profs = [d.profiling_result for d in case.model_datas]
    mids, slos = workload_arrays(w, names)
    for b, p in enumerate(case.placements):
        fin, good, mreq, mgood, greq, _ = tables.one_placement(p, profs, mids, slos, w.arrivals)
        assert tables.score(p, fin, good, w.arrivals) == g["scores"][b]
        assert np.array_equal(greq, g["group_num_requests"][b, :len(greq)])
        assert np.array_equal(mgood / (mreq + 1e-6), g["model_goodput"][b])
        if b < 4:
            assert fin.tobytes() == g["finish_first4"][b].tobytes()
            assert np.array_equal(good, g["good_first4"][b])


def test_candidate_batch_with_batching(golden):
    g = golden("case_candidates_batching")
    case = cases.candidate_batch_case(num_candidates=int(g["num_candidates"]),
                                      duration=float(g["duration"]), batching=True)
    w = case.workload
    assert sha(w.arrivals) == str(g["arrivals_sha256"])
    names = [d.name for d in case.model_datas]
    profs = [d.profiling_result for d in case.model_datas]
    mids, slos = workload_arrays(w, names)
    for b, p in enumerate(case.placements):
        fin, good, mreq, mgood, greq, ggood = tables.one_placement(
            p, profs, mids, slos, w.arrivals, batchsize_config=(1, 2, 4, 8))
        assert fin.tobytes() == g["finish"][b].tobytes(), b
        assert np.array_equal(good, g["good"][b])
        assert np.array_equal(mreq, g["model_num_requests"][b])
        assert np.array_equal(mgood, g["model_num_good"][b])
        assert np.array_equal(greq, g["group_num_requests"][b, :len(greq)])
        assert np.array_equal(ggood, g["group_num_good"][b, :len(ggood)])


@pytest.mark.parametrize("n", [0, 1, 5, 7, 8, 9, 100, 127, 128, 129, 136, 1000, 4097, 57949,
                               180715])
def test_pairwise_sum_is_numpys_order(n):
    a = np.random.RandomState(n).gamma(0.3, 1.0, size=n)
    assert cpu.pairwise_sum(a) == float(np.add.reduce(a))
    if n:
        assert cpu.pairwise_sum(a) / n == float(np.mean(a))


def test_placement_schedule_fast_stats(golden):
    """approximate_one_case with a ModelPlacementWithReplacement
    (controller.py:346-403): the trace is split at the first arrival later
    than each change time, every part starts from idle clocks, counters add
    up.  The checker, driven that way, reproduces the reference's StatsResult."""
    g = golden("case_replacement")
    datas, env, w, starts, pls = cases.replacement_case()
    assert hashlib.sha256(np.ascontiguousarray(w.arrivals).tobytes()).hexdigest() == str(g["arrivals_sha256"])
    names = [d.name for d in datas]
    profs = [d.profiling_result for d in datas]
    mids, slos = workload_arrays(w, names)
    arr = w.arrivals
    change = list(starts[1:]) + [np.inf]
    bounds, pt = [0], 0
    for i in range(len(arr)):
        if arr[i] > change[pt]:
            bounds.append(i)
            pt += 1
    bounds.append(len(arr))
    parts = [tables.one_placement(pls[k], profs, mids[bounds[k]:bounds[k + 1]],
                                  slos[bounds[k]:bounds[k + 1]], arr[bounds[k]:bounds[k + 1]])
             for k in range(len(pls))]
    finish = np.concatenate([p[0] for p in parts])
    good = np.concatenate([p[1] for p in parts])
    mreq = np.sum([p[2] for p in parts], axis=0)
    mgood = np.sum([p[3] for p in parts], axis=0)
    greq = np.sum([p[4] for p in parts], axis=0)
    interval = arr[-1] - arr[0]
    assert np.mean(good) == float(g["fast_goodput"])
    assert np.mean(finish - arr) == float(g["fast_latency_mean"])
    assert len(arr) == int(g["fast_num_requests"])
    assert len(arr) / interval == float(g["fast_request_rate"])
    assert np.array_equal(greq, g["fast_group_num_requests"])
    assert np.array_equal(mreq, g["fast_model_num_requests"])
    assert np.array_equal(mgood / (mreq + 1e-6), g["fast_model_goodput"])
    assert np.array_equal(mreq / interval, g["fast_model_throughput"])


def test_compute_stats_checker_matches_reference(golden):
    """oracle.stats.compute_stats against what the reference's
    Workload.compute_stats (workload.py:308-354) returned for the simulator
    outputs stored in case_candidates.npz, two warm-up lengths."""
    from mms_b200 import cases
    from oracle import stats
    g, c = golden("case_stats"), golden("case_candidates")
    w = cases.candidate_batch_case(num_candidates=48, duration=120.0).workload
    assert sha(w.arrivals) == str(c["arrivals_sha256"])
    for wi, warmup in enumerate(g["warmups"]):
        for b in range(4):
            per_model, overall = stats.compute_stats(
                w.arrivals, w.name_index, w.names, w.arrivals, c["finish_first4"][b],
                c["good_first4"][b], float(warmup))
            tag = f"w{wi}_b{b}"
            assert [p["name"] for p in per_model] == list(g[f"{tag}_names"])
            for field in stats.FIELDS:
                got = np.array([p[field] for p in per_model], np.float64)
                assert np.array_equal(got, g[f"{tag}_{field}"]), (tag, field)
            assert np.array_equal(np.array(overall, np.float64), g[f"{tag}_overall"])


def test_host_compute_stats_equals_checker_on_awkward_data():
    """The package's host mirror of Workload.compute_stats (used for workloads
    given as Request lists) against the checker's statement of it: models with
    no good request, a single good request, unequal counts that tie, a window
    that the warm-up cuts on both sides."""
    from mms_b200.workload import Workload
    from oracle import stats
    rng = np.random.default_rng(23)
    names = [f"m{k}" for k in range(9)]
    counts = [0, 1, 5, 5, 40, 129, 129, 700, 3000]          # ties keep first-appearance order
    which = np.concatenate([np.full(c, k, np.int32) for k, c in enumerate(counts)])
    which = which[rng.permutation(len(which))]
    n = len(which)
    arrivals = np.cumsum(rng.gamma(0.5, 0.02, n))
    good = rng.random(n) < 0.7
    good[which == 2] = False                                   # a model without a good request
    good[which == 1] = True                                    # ... and one with exactly one request
    finish = arrivals + np.where(good, rng.gamma(2.0, 0.04, n), 0.0)
    w = Workload.from_arrays(arrivals, which, np.full(n, 0.5), names)
    for warmup in (0.0, 3.0, 12.0):
        with np.errstate(divide="ignore", invalid="ignore"):
            got = w.compute_stats(arrivals, finish, good, warmup)
            per_model, overall = stats.compute_stats(arrivals, which, names, arrivals, finish,
                                                     good, warmup)
        assert [x.name for x in got.per_model_stats] == [p["name"] for p in per_model]
        for x, p in zip(got.per_model_stats, per_model):
            for field in stats.FIELDS:
                a, b = np.float64(getattr(x, field)), np.float64(p[field])
                assert a.tobytes() == b.tobytes() or (np.isnan(a) and np.isnan(b)), (x.name, field)
        assert (got.goodput, got.latency_mean, got.num_requests, got.request_rate) == tuple(overall)
