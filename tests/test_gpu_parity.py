"""CUDA path (through the C ABI) against the CPU checker and the golden files."""
import hashlib

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


@pytest.fixture(scope="module")
def loaded():
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from mms_b200 import _native
    _native.lib()          # raises if the extension was not built: no fallback
    return True


def same_counters(got, g):
    for arr, key in zip(got, ("model_num_requests", "model_num_good", "group_num_requests",
                              "group_num_good")):
        assert np.array_equal(arr, g[key]), key


def test_mixed_kernel_golden(loaded, golden):
    from mms_b200 import simulator
    g = golden("kernel_mixed")
    N = len(g["tstamps"])
    fin = np.empty(N); good = np.empty(N, bool)
    got = simulator.simulate_requests_mixed(fin, good, g["tstamps"], g["model_ids"], g["slos"],
                                            g["m_id2g_id"], g["num_stages"],
                                            g["stage_latency"], N)
    assert fin.tobytes() == g["finish"].tobytes()
    assert np.array_equal(good, g["good"])
    same_counters(got, g)


def test_legacy_kernel_golden(loaded, golden):
    from mms_b200 import simulator
    g = golden("kernel_legacy")
    N = len(g["tstamps"])
    fin = np.empty(N); good = np.empty(N, bool)
    got = simulator.simulate_requests(fin, good, g["tstamps"], g["model_ids"], g["slos"],
                                      g["m_id2g_id"], g["group_max_latency"],
                                      g["group_sum_latency"], N)
    assert fin.tobytes() == g["finish"].tobytes()
    assert np.array_equal(good, g["good"])
    same_counters(got, g)


def test_fixed_pipeline_case_full_size(loaded, golden):
    from mms_b200 import cases, simulator
    g = golden("case_fixed_pipeline")
    case = cases.fixed_pipeline_case()
    w = case.workload
    names = [d.name for d in case.model_datas]
    profs = [d.profiling_result for d in case.model_datas]
    mids, slos = simulator.workload_arrays(w, names)
    out = simulator.approximate_one_case_one_placement(case.placements[0], names, profs, mids,
                                                       slos, w.arrivals)
    assert sha(out[1]) == str(g["finish_sha256"])
    assert sha(out[2].astype(np.uint8)) == str(g["good_sha256"])
    same_counters(out[3:], g)


def test_evaluator_scores_golden(loaded, golden):
    from mms_b200 import cases
    from mms_b200.placement import PlacementEvaluator
    g = golden("case_candidates")
    case = cases.candidate_batch_case(num_candidates=int(g["num_candidates"]),
                                      duration=float(g["duration"]))
    ev = PlacementEvaluator(case.model_datas, case.cluster_env, case.workload,
                            "fast_simulator", False)
    scores = ev.get_scores(case.placements)
    assert np.array(scores).tobytes() == g["scores"].tobytes()      # bit-exact fp64
    stats = ev.get_stats(case.placements)
    for b, (goodput, per_model, group_req, full) in enumerate(stats):
        assert goodput == g["goodput"][b]
        assert full.latency_mean == g["latency_mean"][b]
        assert np.array_equal(np.array(per_model), g["model_goodput"][b])
        assert np.array_equal(np.array(group_req), g["group_num_requests"][b, :len(group_req)])
        assert isinstance(group_req, tuple)


def test_evaluator_against_cpu_checker_hour_trace(loaded):
    """Full-length trace (about 180 k requests), 96 candidates: every reduced
    output equals the checker's."""
    from mms_b200 import cases
    from mms_b200.placement import PlacementEvaluator
    from mms_b200.simulator import workload_arrays
    from oracle import tables
    case = cases.candidate_batch_case(num_candidates=96, placement_seed=5)
    ev = PlacementEvaluator(case.model_datas, case.cluster_env, case.workload)
    enc, res = ev.evaluate(case.placements)
    scores = ev.scores_from(enc, res)
    names = [d.name for d in case.model_datas]
    profs = [d.profiling_result for d in case.model_datas]
    mids, slos = workload_arrays(case.workload, names)
    for b in range(0, 96, 5):
        p = case.placements[b]
        fin, good, mreq, mgood, greq, _ = tables.one_placement(p, profs, mids, slos,
                                                               case.workload.arrivals)
        assert scores[b] == tables.score(p, fin, good, case.workload.arrivals), b
        assert np.array_equal(res.model_num_good[b], mgood)
        assert np.array_equal(res.model_num_requests[b], mreq)
        assert np.array_equal(res.group_num_requests[b, :len(greq)], greq)
        assert res.good_total[b] == np.count_nonzero(good)


@pytest.mark.parametrize("n", [0, 1, 7, 8, 9, 129, 1001])
def test_short_and_ragged_traces(loaded, n):
    from mms_b200 import simulator
    from oracle import cpu
    rng = np.random.RandomState(n)
    M, G, S = 5, 3, 2
    ts = np.cumsum(rng.gamma(0.5, 0.05, size=n))
    mid = rng.randint(-1, M, size=n).astype(np.int32)
    slo = np.full(n, 0.3, np.float32)
    m2g = np.array([[0, 1, -1], [1, -1, -1], [2, 0, 1], [-1, -1, -1], [0, -1, -1]], np.int32)
    ns = np.array([2, 1, 2], np.int32)
    lat = rng.uniform(0.01, 0.08, size=(M, G, S)).astype(np.float32)
    lat[1, 1, :] = lat[0, 1, :] = 0.05          # equal clocks on ties
    fin = np.empty(n); good = np.empty(n, bool)
    efin = np.empty(n); egood = np.empty(n, bool)
    got = simulator.simulate_requests_mixed(fin, good, ts, mid, slo, m2g, ns, lat, n)
    exp = cpu.simulate_requests_mixed(efin, egood, ts, mid, slo, m2g, ns, lat, n)
    assert fin.tobytes() == efin.tobytes()
    assert np.array_equal(good, egood)
    for a, b in zip(got, exp):
        assert np.array_equal(a, b)


@pytest.mark.parametrize("chunk,run_in,rounds,cap,crowded", [
    (-1, 0, 0, 0, False), (1024, 2048, 0, 0, False), (4096, 1, 0, 0, False),
    (2048, 64, 2, 1, False), (8192, 2048, 6, 2, False), (8192, 16, 1, 1, False),
    (0, 0, 0, 0, False), (0, 0, 16, 3, False),
    # with the hint, more than 48 failing chunks are repaired 32 to a warp
    (4096, 1, 0, 0, True), (2048, 64, 2, 1, True), (3072, 8, 16, 0, True)])
def test_results_do_not_depend_on_chunking(loaded, chunk, run_in, rounds, cap, crowded):
    """Speculative chunks are kept only when provably equivalent, so any cut of
    the trace — even a run-in of one request, which makes nearly every chunk
    wrong and re-simulated — gives the sequential results bit for bit, whether
    the repairs run one chunk to a warp or 32."""
    from mms_b200 import cases, engine
    from mms_b200.placement import PlacementEvaluator
    from mms_b200.simulator import workload_arrays
    from oracle import tables
    case = cases.candidate_batch_case(num_candidates=40, duration=900.0, placement_seed=9)
    ev = PlacementEvaluator(case.model_datas, case.cluster_env, case.workload,
                            options=engine.sim_options(chunk, run_in, rounds, cap))
    enc = engine.encode_placements(case.placements, ev.table, len(ev.model_names))
    res, _, _ = engine.run_batch(ev.trace, enc, ev.table, per_request=True, group_good=True,
                                 options=ev.options, crowded=crowded)
    names = [d.name for d in case.model_datas]
    profs = [d.profiling_result for d in case.model_datas]
    mids, slos = workload_arrays(case.workload, names)
    arr = case.workload.arrivals
    if chunk == 4096:
        assert res.resimulated.sum() > (48 if crowded else 0)   # the repair path really ran
    for b, p in enumerate(case.placements):
        fin, good, mreq, mgood, greq, ggood = tables.one_placement(p, profs, mids, slos, arr)
        assert res.finish[b].tobytes() == fin.tobytes(), (b, chunk)
        assert np.array_equal(res.good[b], good)
        assert np.array_equal(res.model_num_good[b], mgood)
        assert np.array_equal(res.group_num_requests[b, :len(greq)], greq)
        assert np.array_equal(res.group_num_good[b, :len(ggood)], ggood)
        assert res.latency_sum[b] == float(np.add.reduce(fin - arr))


@pytest.mark.parametrize("cap", [1, 2])
@pytest.mark.parametrize("rounds", [1, 2, 4])
def test_capped_repairs_under_sustained_overload(loaded, cap, rounds):
    """Repairs that are cut off after `cap` segments per round and resumed —
    or started over, when the chunk before them changed in the same round —
    on a trace that keeps a few groups busy without a break for whole
    segments while the others heal: every cut gives the sequential result.
    Short chunks of three segments after a run-in of 64 requests make nearly
    every boundary fail; with mirrors and without."""
    from mms_b200 import cases, engine
    from mms_b200.placement import PlacementEvaluator
    from mms_b200.simulator import workload_arrays
    from oracle import tables
    case = cases.candidate_batch_case(num_candidates=24, duration=240.0, placement_seed=21,
                                      total_rate=170.0, cv=2.0)
    ev = PlacementEvaluator(case.model_datas, case.cluster_env, case.workload,
                            options=engine.sim_options(3072, 64, rounds, cap))
    enc = engine.encode_placements(case.placements, ev.table, len(ev.model_names))
    names = [d.name for d in case.model_datas]
    profs = [d.profiling_result for d in case.model_datas]
    mids, slos = workload_arrays(case.workload, names)
    arr = case.workload.arrivals
    want = [tables.one_placement(p, profs, mids, slos, arr) for p in case.placements]
    overloaded = np.mean([np.mean(w[1]) for w in want])
    assert 0.2 < overloaded < 0.9                  # a good part of the requests is dropped
    for mirrors in (False, True):
        res, _, _ = engine.run_batch(ev.trace, enc, ev.table, group_good=True,
                                     options=ev.options, mirrors=mirrors)
        assert res.resimulated.sum() > 24          # the repair path really ran
        for b, (fin, good, mreq, mgood, greq, ggood) in enumerate(want):
            assert res.good_total[b] == np.count_nonzero(good), (b, mirrors)
            assert res.latency_sum[b] == float(np.add.reduce(fin - arr)), (b, mirrors)
            assert np.array_equal(res.model_num_good[b], mgood), (b, mirrors)
            assert np.array_equal(res.group_num_requests[b, :len(greq)], greq), (b, mirrors)
            assert np.array_equal(res.group_num_good[b, :len(ggood)], ggood), (b, mirrors)


def test_contested_bit_of_group_info_is_not_trusted(loaded):
    """group_info bit 16 (the group serves a model with several replicas) is
    derived on the device: a caller that leaves it clear gets the same
    results as one that sets it."""
    from mms_b200 import cases, engine
    from mms_b200.placement import PlacementEvaluator
    case = cases.candidate_batch_case(num_candidates=64, duration=600.0, placement_seed=4)
    ev = PlacementEvaluator(case.model_datas, case.cluster_env, case.workload,
                            options=engine.sim_options(4096, 256))
    enc = engine.encode_placements(case.placements, ev.table, len(ev.model_names))
    with_bit, _, _ = engine.run_batch(ev.trace, enc, ev.table, group_good=True,
                                      options=ev.options, mirrors=False)
    assert np.any(enc.group_info & 0x10000)
    enc.group_info = enc.group_info & ~np.uint32(0x10000)
    without, _, _ = engine.run_batch(ev.trace, enc, ev.table, group_good=True,
                                     options=ev.options, mirrors=False)
    for name in ("good_total", "latency_sum", "model_num_good", "group_num_requests",
                 "group_num_good"):
        assert getattr(with_bit, name).tobytes() == getattr(without, name).tobytes(), name


def test_unsorted_trace_falls_back_to_one_chunk(loaded):
    from mms_b200 import simulator
    from oracle import cpu
    rng = np.random.RandomState(3)
    n, M, G, S = 20000, 6, 4, 2
    ts = np.cumsum(rng.gamma(0.5, 0.02, size=n))
    ts[5000:5010] = ts[5000:5010][::-1]          # arrivals out of order
    mid = rng.randint(-1, M, size=n).astype(np.int32)
    slo = np.full(n, 0.4, np.float32)
    m2g = np.full((M, G), -1, np.int32)
    for m in range(M):
        m2g[m, :2] = np.sort(rng.choice(G, 2, replace=False))
    ns = np.array([2, 1, 2, 1], np.int32)
    lat = rng.uniform(0.01, 0.05, size=(M, G, S)).astype(np.float32)
    fin = np.empty(n); good = np.empty(n, bool)
    efin = np.empty(n); egood = np.empty(n, bool)
    simulator.set_chunking(1024, 16)
    try:
        got = simulator.simulate_requests_mixed(fin, good, ts, mid, slo, m2g, ns, lat, n)
    finally:
        simulator.set_chunking()
    exp = cpu.simulate_requests_mixed(efin, egood, ts, mid, slo, m2g, ns, lat, n)
    assert fin.tobytes() == efin.tobytes()
    assert np.array_equal(good, egood)
    for a, b in zip(got, exp):
        assert np.array_equal(a, b)


def test_batching_kernel_golden(loaded, golden):
    from mms_b200 import simulator
    g = golden("kernel_batching")
    N = len(g["tstamps"])
    fin = np.empty(N); good = np.empty(N, bool)
    simulator.batchsize_config[:] = [int(x) for x in g["batchsize_config"]]
    try:
        got = simulator.simulate_requests_mixed_batching(
            fin, good, g["tstamps"], g["model_ids"], g["slos"], g["m_id2g_id"], g["g_id2m_id"],
            g["num_stages"], g["stage_latency"], N)
    finally:
        simulator.batchsize_config[:] = [1, 2, 4, 8, 16]
    assert fin.tobytes() == g["finish"].tobytes()
    assert np.array_equal(good, g["good"])
    same_counters(got, g)


@pytest.mark.parametrize("copies", [32, 45])
def test_batching_kernel_golden_32_to_a_warp(loaded, golden, copies):
    """The same fixture (unknown models, a model without replica, +inf
    latencies, replicated models) as a batch of identical candidates, which
    takes the kernel that runs 32 candidates per warp: every copy — also in a
    warp that is only partly filled — equals the reference's output."""
    from mms_b200 import engine
    g = golden("kernel_batching")
    N = len(g["tstamps"])
    lat = np.ascontiguousarray(g["stage_latency"], np.float32)
    M, G, S, NB = lat.shape
    trace = engine.DeviceTrace(g["tstamps"], g["model_ids"], g["slos"], M)
    off, rep, info, T = engine.encode_dense(g["m_id2g_id"], g["num_stages"], M)
    tile = lambda x: np.ascontiguousarray(np.tile(x, (copies, 1)))
    res = engine.launch_batching(trace, copies, M, G, rep.shape[1], T, S, G, tile(off), tile(rep),
                                 tile(info), lat, 0, [int(x) for x in g["batchsize_config"]])
    for b in (0, 1, 31, copies - 1):
        assert res.finish[b].tobytes() == g["finish"].tobytes(), b
        assert np.array_equal(res.good[b], g["good"])
        assert np.array_equal(res.model_num_requests[b], g["model_num_requests"])
        assert np.array_equal(res.model_num_good[b], g["model_num_good"])
        assert np.array_equal(res.group_num_requests[b], g["group_num_requests"])
        assert np.array_equal(res.group_num_good[b], g["group_num_good"])


def test_batching_heap_overflow_is_reported_and_retried(loaded):
    """A pending-event heap that is too small is reported per candidate, and
    the default capacity is raised and the run repeated when it overflows."""
    from mms_b200 import cases, engine
    from mms_b200.simulator import workload_arrays
    case = cases.candidate_batch_case(num_candidates=32, duration=120.0, batching=True,
                                      placement_seed=2, total_rate=200.0)
    names = [d.name for d in case.model_datas]
    profs = [d.profiling_result for d in case.model_datas]
    mids, slos = workload_arrays(case.workload, names)
    trace = engine.DeviceTrace(case.workload.arrivals, mids, slos, len(names))
    table = engine.LatencyTable(profs, [1, 2, 4, 8])
    enc = engine.encode_placements(case.placements, table, len(names))
    with pytest.raises(RuntimeError, match="heap overflow"):
        engine.run_batch_batching(trace, enc, table, heap_capacity=2)
    engine.run_batch_batching(trace, enc, table)            # default capacity: fine


def test_batching_candidates_golden(loaded, golden):
    from mms_b200 import cases, engine
    from mms_b200.simulator import workload_arrays
    g = golden("case_candidates_batching")
    case = cases.candidate_batch_case(num_candidates=int(g["num_candidates"]),
                                      duration=float(g["duration"]), batching=True)
    names = [d.name for d in case.model_datas]
    profs = [d.profiling_result for d in case.model_datas]
    mids, slos = workload_arrays(case.workload, names)
    trace = engine.DeviceTrace(case.workload.arrivals, mids, slos, len(names))
    table = engine.LatencyTable(profs, [1, 2, 4, 8])
    enc = engine.encode_placements(case.placements, table, len(names))
    res = engine.run_batch_batching(trace, enc, table)
    for b in range(enc.B):
        G = int(enc.num_groups[b])
        assert res.finish[b].tobytes() == g["finish"][b].tobytes(), b
        assert np.array_equal(res.good[b], g["good"][b])
        assert np.array_equal(res.model_num_requests[b], g["model_num_requests"][b])
        assert np.array_equal(res.model_num_good[b], g["model_num_good"][b])
        assert np.array_equal(res.group_num_requests[b, :G], g["group_num_requests"][b, :G])
        assert np.array_equal(res.group_num_good[b, :G], g["group_num_good"][b, :G])
        assert res.latency_sum[b] == float(np.add.reduce(g["finish"][b] - case.workload.arrivals))
        assert res.good_total[b] == int(g["good"][b].sum())


def test_batching_against_cpu_checker_long(loaded):
    """A 20-minute trace, 64 candidates: every per-request output equals the
    checker's pure restatement of the Python reference."""
    from mms_b200 import cases, engine
    from mms_b200.simulator import workload_arrays
    from oracle import tables
    case = cases.candidate_batch_case(num_candidates=64, duration=1200.0, batching=True,
                                      placement_seed=4)
    names = [d.name for d in case.model_datas]
    profs = [d.profiling_result for d in case.model_datas]
    mids, slos = workload_arrays(case.workload, names)
    arr = case.workload.arrivals
    trace = engine.DeviceTrace(arr, mids, slos, len(names))
    table = engine.LatencyTable(profs, [1, 2, 4, 8])
    enc = engine.encode_placements(case.placements, table, len(names))
    res = engine.run_batch_batching(trace, enc, table)
    for b in range(0, 64, 3):
        fin, good, mreq, mgood, greq, ggood = tables.one_placement(
            case.placements[b], profs, mids, slos, arr, batchsize_config=(1, 2, 4, 8))
        assert res.finish[b].tobytes() == fin.tobytes(), b
        assert np.array_equal(res.good[b], good)
        assert np.array_equal(res.model_num_requests[b], mreq)
        assert np.array_equal(res.group_num_requests[b, :len(greq)], greq)
        assert np.array_equal(res.group_num_good[b, :len(ggood)], ggood)
        assert res.latency_sum[b] == float(np.add.reduce(fin - arr))
        assert res.good_total[b] == np.count_nonzero(good)
    assert res.resimulated is not None and res.resimulated.shape == (64,)


@pytest.mark.parametrize("total_rate,cv", [(150.0, 4.0), (400.0, 1.0), (20.0, 8.0)])
def test_batching_time_cut_under_load(loaded, total_rate, cv):
    """The batching path is cut in time too.  Under overload requests queue
    across chunk boundaries (their outputs travel through the carry lists or
    the chunk is re-simulated); every per-request output must still equal the
    checker's."""
    from mms_b200 import cases, engine
    from mms_b200.simulator import workload_arrays
    from oracle import tables
    case = cases.candidate_batch_case(num_candidates=40, duration=60000.0 / total_rate,
                                      batching=True, placement_seed=6, total_rate=total_rate, cv=cv)
    names = [d.name for d in case.model_datas]
    profs = [d.profiling_result for d in case.model_datas]
    mids, slos = workload_arrays(case.workload, names)
    arr = case.workload.arrivals
    assert len(arr) > 40000                               # long enough to be cut
    trace = engine.DeviceTrace(arr, mids, slos, len(names))
    table = engine.LatencyTable(profs, [1, 2, 4, 8])
    enc = engine.encode_placements(case.placements, table, len(names))
    res = engine.run_batch_batching(trace, enc, table)
    for b in range(0, 40, 3):
        fin, good, mreq, mgood, greq, ggood = tables.one_placement(
            case.placements[b], profs, mids, slos, arr, batchsize_config=(1, 2, 4, 8))
        assert res.finish[b].tobytes() == fin.tobytes(), b
        assert np.array_equal(res.good[b], good)
        assert np.array_equal(res.model_num_requests[b], mreq)
        assert np.array_equal(res.model_num_good[b], mgood)
        assert np.array_equal(res.group_num_requests[b, :len(greq)], greq)
        assert np.array_equal(res.group_num_good[b, :len(ggood)], ggood)
        assert res.latency_sum[b] == float(np.add.reduce(fin - arr))


def test_batching_unsorted_trace_is_not_cut(loaded):
    """Arrival times that go backwards: the batching path falls back to one
    chunk and still equals the checker."""
    from mms_b200 import cases, engine
    from mms_b200.simulator import workload_arrays
    from oracle import tables
    case = cases.candidate_batch_case(num_candidates=6, duration=500.0, batching=True,
                                      placement_seed=8)
    names = [d.name for d in case.model_datas]
    profs = [d.profiling_result for d in case.model_datas]
    mids, slos = workload_arrays(case.workload, names)
    arr = case.workload.arrivals.copy()
    arr[15000], arr[15001] = arr[15001], arr[15000] + 0.0     # one inversion
    assert arr[15000] > arr[15001]
    trace = engine.DeviceTrace(arr, mids, slos, len(names))
    table = engine.LatencyTable(profs, [1, 2, 4, 8])
    enc = engine.encode_placements(case.placements, table, len(names))
    res = engine.run_batch_batching(trace, enc, table)
    for b in range(6):
        fin, good, mreq, mgood, greq, ggood = tables.one_placement(
            case.placements[b], profs, mids, slos, arr, batchsize_config=(1, 2, 4, 8))
        assert res.finish[b].tobytes() == fin.tobytes(), b
        assert np.array_equal(res.good[b], good)
        assert np.array_equal(res.group_num_requests[b, :len(greq)], greq)


@pytest.mark.parametrize("chunk,run_in", [(2048, 256), (4096, 2048), (0, 0)])
def test_twin_groups_keep_exact_counters(loaded, chunk, run_in):
    """Placements full of interchangeable groups (same config, same models):
    speculative chunks may come out with twins' roles swapped; counters per
    group must still be the reference's."""
    from mms_b200 import cases, engine
    from mms_b200.placement import ModelPlacement, PlacementEvaluator
    from mms_b200.profiling import ParallelConfig
    from mms_b200.simulator import workload_arrays
    from oracle import tables
    case = cases.candidate_batch_case(num_candidates=1, duration=1500.0, num_models=8,
                                      num_devices=16, total_rate=40.0, cv=3.0)
    c1, c2, c4 = (ParallelConfig(1, 1, p) for p in (1, 2, 4))
    sols = [
        ModelPlacement([c1] * 8 + [c2] * 4, [[0, 3]] * 4 + [[1, 4]] * 4 + [[2, 5, 6]] * 2 + [[7, 2]] * 2),
        ModelPlacement([c2] * 8, [[0, 1, 3, 4, 6, 7]] * 8),
        ModelPlacement([c4, c4, c2, c2, c1, c1, c1, c1],
                       [[2, 5, 0], [2, 5, 0], [1, 3], [1, 3], [4], [4], [6, 7], [7, 6]]),
        ModelPlacement([c1] * 16, [[0]] * 3 + [[1]] * 3 + [[3, 4]] * 5 + [[6, 7, 0]] * 5),
    ]
    ev = PlacementEvaluator(case.model_datas, case.cluster_env, case.workload,
                            options=engine.sim_options(chunk, run_in))
    enc = engine.encode_placements(sols, ev.table, len(ev.model_names))
    res, _, _ = engine.run_batch(ev.trace, enc, ev.table, per_request=True, group_good=True,
                                 options=ev.options)
    names = [d.name for d in case.model_datas]
    profs = [d.profiling_result for d in case.model_datas]
    mids, slos = workload_arrays(case.workload, names)
    arr = case.workload.arrivals
    assert len(arr) > 30000
    for b, p in enumerate(sols):
        fin, good, mreq, mgood, greq, ggood = tables.one_placement(p, profs, mids, slos, arr)
        assert res.finish[b].tobytes() == fin.tobytes(), b
        assert np.array_equal(res.good[b], good)
        assert np.array_equal(res.model_num_good[b], mgood)
        assert np.array_equal(res.group_num_requests[b, :len(greq)], greq), b
        assert np.array_equal(res.group_num_good[b, :len(ggood)], ggood), b
        assert res.latency_sum[b] == float(np.add.reduce(fin - arr))


@pytest.mark.parametrize("chunk,run_in,rounds,cap", [
    (0, 0, 0, 0), (4096, 512, 0, 0), (2048, 16, 2, 1), (4096, 2048, 1, 0), (8192, 1, 16, 2)])
def test_mirror_candidates_change_nothing_but_speed(loaded, chunk, run_in, rounds, cap):
    """Placements with interchangeable groups get a mirror candidate whose
    speculative chunks start with those groups exchanged; a chunk is taken
    from whichever run continues the chain.  Every reduced output must equal
    the run without mirrors and the checker, for any cut of the trace."""
    from mms_b200 import cases, engine
    from mms_b200.placement import ModelPlacement, PlacementEvaluator
    from mms_b200.profiling import ParallelConfig
    from mms_b200.simulator import workload_arrays
    from oracle import tables
    case = cases.candidate_batch_case(num_candidates=24, duration=1500.0, num_models=8,
                                      num_devices=16, total_rate=40.0, cv=3.0, placement_seed=4)
    c1, c2, c4 = (ParallelConfig(1, 1, p) for p in (1, 2, 4))
    sols = list(case.placements) + [
        ModelPlacement([c1] * 8 + [c2] * 4, [[0, 3]] * 4 + [[1, 4]] * 4 + [[2, 5, 6]] * 2 + [[7, 2]] * 2),
        ModelPlacement([c2] * 8, [[0, 1, 3, 4, 6, 7]] * 2 + [[2, 5]] * 2 + [[0, 1]] * 2 + [[3, 4], [6, 7]]),
        ModelPlacement([c4, c4, c2, c2, c1, c1, c1, c1],
                       [[2, 5, 0], [2, 5, 0], [1, 3], [1, 3], [4], [4], [6, 7], [7, 6]]),
        ModelPlacement([c1] * 16, [[0]] * 3 + [[1]] * 3 + [[3, 4]] * 5 + [[6, 7, 0]] * 5),
        ModelPlacement([c2, c2, c4, c4, c4], [[0, 1, 2], [0, 1, 2], [3, 4, 5, 6, 7], [5], [5]]),
    ]
    ev = PlacementEvaluator(case.model_datas, case.cluster_env, case.workload,
                            options=engine.sim_options(chunk, run_in, rounds, cap))
    enc = engine.encode_placements(sols, ev.table, len(ev.model_names))
    ext = enc.with_mirrors()
    assert ext is not None and len(ext[3]) >= enc.B + 4      # most hand-made ones get mirrors
    with_m, _, _ = engine.run_batch(ev.trace, enc, ev.table, group_good=True, options=ev.options)
    without, _, _ = engine.run_batch(ev.trace, enc, ev.table, group_good=True, options=ev.options,
                                     mirrors=False)
    for name in ("model_num_requests", "model_num_good", "group_num_requests", "group_num_good",
                 "good_total", "latency_sum"):
        a, b = getattr(with_m, name), getattr(without, name)
        assert a.shape == b.shape and a.tobytes() == b.tobytes(), name
    names = [d.name for d in case.model_datas]
    profs = [d.profiling_result for d in case.model_datas]
    mids, slos = workload_arrays(case.workload, names)
    arr = case.workload.arrivals
    for b in range(len(sols) - 5, len(sols)):
        fin, good, mreq, mgood, greq, ggood = tables.one_placement(sols[b], profs, mids, slos, arr)
        assert np.array_equal(with_m.model_num_good[b], mgood), b
        assert np.array_equal(with_m.group_num_requests[b, :len(greq)], greq), b
        assert np.array_equal(with_m.group_num_good[b, :len(ggood)], ggood), b
        assert with_m.latency_sum[b] == float(np.add.reduce(fin - arr))


def test_mirrors_are_refused_with_per_request_outputs(loaded):
    """Per-request outputs come from one run per candidate: the library
    rejects the combination instead of returning rows from two runs."""
    import ctypes
    from mms_b200 import _native as nat
    fake = ctypes.c_void_p(256)             # the size query reads no table
    cands = nat.Placements(4, 2, 1, 1, 1, 1, 1, 3, None, None, None, None, 0, fake, fake)
    opts = nat.SimOptions(0, 0, 0, 0)
    L = nat.lib()
    assert L.mms_sim_workspace_bytes(100000, ctypes.byref(cands), ctypes.byref(opts), 0) > 0
    assert L.mms_sim_workspace_bytes(100000, ctypes.byref(cands), ctypes.byref(opts),
                                     nat.FLAG_PER_REQUEST) == 0
    cands.partner = None                    # mirrors without a partner list
    assert L.mms_sim_workspace_bytes(100000, ctypes.byref(cands), ctypes.byref(opts), 0) == 0


def test_pipelined_evaluation_equals_one_launch(loaded):
    """A long candidate list is encoded and launched in parts on separate
    streams; scores and counters equal those of one launch."""
    from mms_b200 import cases
    from mms_b200.placement import PlacementEvaluator
    case = cases.candidate_batch_case(num_candidates=1700, duration=200.0, placement_seed=3)
    ev = PlacementEvaluator(case.model_datas, case.cluster_env, case.workload)
    ev.pipeline_min_part, ev.pipeline_parts = 400, 4
    enc4, res4 = ev.evaluate(case.placements)
    assert len(enc4.parts) == 4 and enc4.B == 1700
    scores4 = ev.scores_from(enc4, res4)
    ev.pipeline_parts = 1
    enc1, res1 = ev.evaluate(case.placements)
    assert scores4 == ev.scores_from(enc1, res1)
    G = res1.group_num_requests.shape[1]
    assert np.array_equal(res4.model_num_good, res1.model_num_good)
    assert np.array_equal(res4.group_num_requests[:, :G], res1.group_num_requests)
    assert np.array_equal(enc4.num_groups, enc1.num_groups)
    assert ev.get_scores(case.placements[:5]) == scores4[:5]
    # the defaults: two unequal parts, placements with mirrors launched apart inside each
    ev2 = PlacementEvaluator(case.model_datas, case.cluster_env, case.workload)
    enc2, res2 = ev2.evaluate(case.placements)
    assert [e.B for e in enc2.parts] == [638, 1062]
    assert ev2.scores_from(enc2, res2) == scores4
    assert np.array_equal(res2.model_num_good, res1.model_num_good)


def test_trace_sweep_one_placement_many_traces(loaded):
    """Every candidate simulates a trace of its own (request-major trace
    batch, shorter traces padded): goodput, per-model counts and group
    counts of each trace equal the checker's on that trace alone."""
    from mms_b200 import cases
    from mms_b200.placement import ModelPlacement, TraceSweep
    from mms_b200.profiling import ParallelConfig
    from mms_b200.simulator import workload_arrays
    from mms_b200.workload import eps
    from oracle import tables
    base = cases.candidate_batch_case(num_candidates=3, duration=10.0, num_models=8,
                                      num_devices=16, total_rate=30.0)
    datas = base.model_datas
    c1, c2, c4 = (ParallelConfig(1, 1, p) for p in (1, 2, 4))
    placements = [base.placements[1],
                  ModelPlacement([c4, c4, c2, c2, c1, c1, c1, c1],
                                 [[2, 5, 0], [2, 5, 0], [1, 3], [1, 3], [4], [4], [6, 7], [7, 6]])]
    workloads = []
    for t in range(37):                                   # not a multiple of 32
        scale, cv = (0.5, 1.0, 2.0, 4.0)[t % 4], (1.0, 2.0, 4.0, 8.0)[(t // 4) % 4]
        scaled = [type(d)(d.name, d.slo, d.rate * scale, cv, d.profiling_result) for d in datas]
        workloads.append(cases.merged_gamma_trace(scaled, 500.0 / scale ** 0.5, base_seed=100 * t))
    names = [d.name for d in datas]
    profs = [d.profiling_result for d in datas]
    lengths = {len(w.arrivals) for w in workloads}
    assert len(lengths) > 10 and max(lengths) > 2 * 8192       # ragged, and long enough to be cut
    for p in placements:
        got = TraceSweep(datas, base.cluster_env, p, batch=32).evaluate(workloads)
        assert len(got) == len(workloads)
        for t, w in enumerate(workloads):
            mids, slos = workload_arrays(w, names)
            fin, good, mreq, mgood, greq, _ = tables.one_placement(p, profs, mids, slos, w.arrivals)
            goodput, per_model, group_req = got[t]
            assert goodput == np.mean(good), t
            assert np.array_equal(per_model, mgood / (mreq + eps)), t
            assert np.array_equal(np.array(group_req), greq), t
        # everything uploaded first from pageable memory, then launched: the same results as
        # the groups launched as they arrive through the staging buffers (the default)
        plain = TraceSweep(datas, base.cluster_env, p, batch=32)
        plain.eager = False
        again = plain.evaluate(workloads)
        for a, b in zip(got, again):
            assert a[0] == b[0] and np.array_equal(a[1], b[1]) and a[2] == b[2]


def test_split_launch_equals_one_launch(loaded, monkeypatch):
    """Placements with mirror candidates go into a launch of their own beside
    the rest (two streams); every output equals the single launch's, in the
    order of the batch."""
    from mms_b200 import cases, engine
    from mms_b200.placement import PlacementEvaluator
    monkeypatch.setattr(engine, "SPLIT_MIN_HARD", 4)
    monkeypatch.setattr(engine, "SPLIT_MIN_EASY", 16)
    case = cases.candidate_batch_case(num_candidates=300, duration=400.0, placement_seed=11)
    ev = PlacementEvaluator(case.model_datas, case.cluster_env, case.workload)
    enc = engine.encode_placements(case.placements, ev.table, len(ev.model_names))
    batch = engine.ResidentBatch(ev.trace, enc, ev.table, group_good=True)
    assert len(batch.jobs) == 2 and len(batch.index[0]) >= 4
    assert sorted(np.concatenate(batch.index).tolist()) == list(range(300))
    first, _ = batch.launch().results()
    again, _ = batch.launch().results()          # a resident batch can be launched repeatedly
    batch.release()
    one, _, _ = engine.run_batch(ev.trace, enc, ev.table, group_good=True, split=False)
    for name in ("model_num_requests", "model_num_good", "group_num_requests", "group_num_good",
                 "good_total", "latency_sum", "status"):
        assert getattr(first, name).tobytes() == getattr(one, name).tobytes(), name
        assert getattr(again, name).tobytes() == getattr(one, name).tobytes(), name


def test_plain_placement_through_approximate_one_case(loaded, golden):
    """approximate_one_case with a single ModelPlacement
    (controller.py:341-344) and fast_stats, on the fixed 4 x pp2 case at full
    size: the StatsResult carries what the reference computed."""
    from functools import partial
    from mms_b200 import cases, simulator
    g = golden("case_fixed_pipeline")
    case = cases.fixed_pipeline_case()
    w = case.workload
    w.cached_data = None

    def register_models(controller):
        for d in case.model_datas:
            controller.register_model.remote(d.name, partial(object, d.profiling_result))

    serving = (register_models, lambda start=0: w, lambda controller: case.placements[0])
    stats, placement = simulator.approximate_one_case(serving, fast_stats=True)
    assert placement is case.placements[0]
    assert stats.goodput == float(g["goodput"])
    assert stats.latency_mean == float(g["latency_mean"])
    assert stats.num_requests == int(g["num_requests"])
    assert isinstance(stats.group_num_requests, tuple)
    assert np.array_equal(np.array(stats.group_num_requests), g["group_num_requests"])
    mreq, mgood = g["model_num_requests"], g["model_num_good"]
    for i, pm in enumerate(stats.per_model_stats):
        assert pm.num_requests == mreq[i]
        assert pm.goodput == mgood[i] / (mreq[i] + 1e-6)
    # the second call takes the cached arrays (controller.py:323-327), same result
    again, _ = simulator.approximate_one_case(serving, fast_stats=True)
    assert again.goodput == stats.goodput and again.latency_mean == stats.latency_mean


@pytest.mark.parametrize("fast", [True, False])
def test_placement_schedule_through_approximate_one_case(loaded, golden, fast):
    """approximate_one_case on a ModelPlacementWithReplacement, with the
    reference's ServingCase closures: every field of the StatsResult equals
    what the reference returned, for fast_stats and for compute_stats."""
    from functools import partial
    from mms_b200 import cases, simulator
    from mms_b200.placement import ModelPlacementWithReplacement
    g = golden("case_replacement")
    datas, env, w, starts, pls = cases.replacement_case()
    schedule = ModelPlacementWithReplacement(list(starts), pls)

    def register_models(controller):
        for d in datas:
            controller.register_model.remote(d.name, partial(object, d.profiling_result))

    case = (register_models, lambda start=0: w, lambda controller: schedule)
    stats, placement = simulator.approximate_one_case(case, fast_stats=fast)
    assert placement is schedule
    tag = "fast" if fast else "full"
    assert stats.goodput == float(g[f"{tag}_goodput"])
    assert stats.latency_mean == float(g[f"{tag}_latency_mean"])
    assert stats.num_requests == int(g[f"{tag}_num_requests"])
    assert stats.request_rate == float(g[f"{tag}_request_rate"])
    assert isinstance(stats.group_num_requests, tuple)
    assert np.array_equal(np.array(stats.group_num_requests), g[f"{tag}_group_num_requests"])
    pm = stats.per_model_stats
    for field in ("num_requests", "goodput", "throughput", "latency_mean", "latency_std",
                  "latency_p90", "latency_p99"):
        got = np.array([getattr(x, field) for x in pm], np.float64)
        assert np.array_equal(got, g[f"{tag}_model_{field}"].astype(np.float64)), field


def test_many_groups_use_wide_decision_records(loaded):
    """More than 126 groups: the per-request decision records are 16 bits
    wide; counters and outputs still equal the checker's."""
    from mms_b200 import cases, engine
    from mms_b200.placement import ModelPlacement, PlacementEvaluator
    from mms_b200.profiling import ParallelConfig
    from mms_b200.simulator import workload_arrays
    from oracle import tables
    base = cases.candidate_batch_case(num_candidates=1, duration=400.0, num_models=8,
                                      num_devices=16, total_rate=60.0)
    rng = np.random.RandomState(5)
    c1, c2 = ParallelConfig(1, 1, 1), ParallelConfig(1, 1, 2)
    sols = []
    for n_groups in (127, 150, 200):
        configs = [c1 if rng.rand() < 0.9 else c2 for _ in range(n_groups)]
        models = [sorted(rng.choice(8, size=rng.randint(1, 3), replace=False).tolist())
                  for _ in range(n_groups)]
        sols.append(ModelPlacement(configs, models))
    ev = PlacementEvaluator(base.model_datas, base.cluster_env, base.workload)
    enc = engine.encode_placements(sols, ev.table, len(ev.model_names))
    assert enc.G == 200
    res, _, _ = engine.run_batch(ev.trace, enc, ev.table, per_request=True, group_good=True)
    names = [d.name for d in base.model_datas]
    profs = [d.profiling_result for d in base.model_datas]
    mids, slos = workload_arrays(base.workload, names)
    arr = base.workload.arrivals
    assert len(arr) > 2 * 8192
    for b, p in enumerate(sols):
        fin, good, mreq, mgood, greq, ggood = tables.one_placement(p, profs, mids, slos, arr)
        assert res.finish[b].tobytes() == fin.tobytes(), b
        assert np.array_equal(res.model_num_good[b], mgood)
        assert np.array_equal(res.group_num_requests[b, :len(greq)], greq)
        assert np.array_equal(res.group_num_good[b, :len(ggood)], ggood)
