"""The entry points around the simulator, checked through the C ABI: the
search's selection step (mms_argmax_scores, np.argmax over get_scores at
alpa_serve/placement_policy/model_parallelism.py:349-351), the device-side
packing of ragged traces (mms_trace_pack), and Workload.compute_stats on the
device (mms_compute_stats, alpa_serve/simulator/workload.py:308-354)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _score(good, lat, rep, N):
    """The score of base_policy.py:225-226 in numpy's fp64, operation for operation."""
    return good / np.float64(N) - lat / np.float64(N) / 10000.0 + rep / 1000000.0


def test_argmax_scores_picks_the_first_maximum_and_accumulates():
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from mms_b200 import _native as nat
    from mms_b200.engine import _ptr, _stream_ptr
    L = nat.lib()
    dev = torch.device("cuda", 0)
    rng = np.random.default_rng(5)
    N = 180715
    for B in (1, 31, 256, 1000, 4097):
        # few distinct values, so that ties are common and the FIRST one has to win
        good = rng.integers(N // 2, N // 2 + 4, B).astype(np.int64)
        lat = rng.integers(0, 3, B).astype(np.float64) * 0.125
        rep = rng.integers(8, 10, B).astype(np.int64)
        want = _score(good.astype(np.float64), lat, rep.astype(np.float64), N)
        d = [torch.from_numpy(x).to(dev) for x in (good, lat, rep)]
        best = torch.zeros(2, dtype=torch.float64, device=dev)
        nat.check(L.mms_argmax_scores(_ptr(d[0]), _ptr(d[1]), _ptr(d[2]), N, B, None, 0, 0,
                                      _ptr(best), _stream_ptr()), "mms_argmax_scores")
        got = best.cpu().numpy()
        assert int(got[1]) == int(np.argmax(want))
        assert got[0].tobytes() == want.max().tobytes()                 # bit-exact fp64

        # a list scored in two calls, the second with an index map and a base:
        # an equal score later in the list must not replace the earlier one
        half = B // 2
        if half == 0:
            continue
        perm = rng.permutation(B - half).astype(np.int64)
        d2 = [torch.from_numpy(np.ascontiguousarray(x[half:][perm])).to(dev)
              for x in (good, lat, rep)]
        d_map = torch.from_numpy(perm).to(dev)
        best.zero_()
        nat.check(L.mms_argmax_scores(_ptr(d[0]), _ptr(d[1]), _ptr(d[2]), N, half, None, 0, 0,
                                      _ptr(best), _stream_ptr()), "mms_argmax_scores")
        nat.check(L.mms_argmax_scores(_ptr(d2[0]), _ptr(d2[1]), _ptr(d2[2]), N, B - half,
                                      _ptr(d_map), half, 1, _ptr(best), _stream_ptr()),
                  "mms_argmax_scores")
        got = best.cpu().numpy()
        assert int(got[1]) == int(np.argmax(want)), B
        assert got[0].tobytes() == want.max().tobytes()

    # without replica counts the third term is absent
    best = torch.zeros(2, dtype=torch.float64, device=dev)
    nat.check(L.mms_argmax_scores(_ptr(d[0]), _ptr(d[1]), None, N, B, None, 0, 0,
                                  _ptr(best), _stream_ptr()), "mms_argmax_scores")
    want = _score(good.astype(np.float64), lat, np.zeros(B), N)
    assert int(best[1].item()) == int(np.argmax(want))
    assert L.mms_argmax_scores(_ptr(d[0]), _ptr(d[1]), None, N, B, None, 0, 0,
                               None, _stream_ptr()) == -1      # MMS_ERR_ARG


def test_trace_pack_matches_a_host_built_batch():
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from mms_b200 import engine
    rng = np.random.default_rng(9)
    lengths = [0, 1, 31, 32, 33, 1000, 4097, 2500, 64]
    arrivals, mids, slos = [], [], []
    for n in lengths:
        arrivals.append(np.sort(rng.random(n) * 100.0))
        mids.append(rng.integers(0, 7, n).astype(np.int32))
        slos.append((rng.random(n) + 0.5).astype(np.float32))
    tb = engine.DeviceTraceBatch(arrivals, mids, slos, 7)
    N, T = max(lengths), len(lengths)
    assert tuple(tb.arrivals.shape) == (N, T)
    got_a, got_m, got_s = (x.cpu().numpy() for x in (tb.arrivals, tb.model_ids, tb.slos))
    for t, n in enumerate(lengths):
        assert got_a[:n, t].tobytes() == arrivals[t].tobytes()
        assert np.array_equal(got_m[:n, t], mids[t])
        assert got_s[:n, t].tobytes() == slos[t].tobytes()
        # padding: model -1 at the last arrival time (0 for an empty trace)
        assert (got_m[n:, t] == -1).all()
        last = arrivals[t][-1] if n else 0.0
        assert (got_a[n:, t] == last).all()
    # the per-trace histograms count exactly the real requests
    hist = tb.model_hist.cpu().numpy()
    assert hist[-1] == 0
    per = hist[:-1].reshape(T, 8)
    for t, n in enumerate(lengths):
        assert np.array_equal(per[t, :7], np.bincount(mids[t], minlength=7))
        assert per[t, 7] == 0


def _device_stats(arrivals, which, K, finish, good, lo, window):
    import torch
    from mms_b200 import engine
    dev = torch.device("cuda", 0)
    finish = np.ascontiguousarray(np.atleast_2d(finish), np.float64)
    good = np.ascontiguousarray(np.atleast_2d(good)).astype(np.uint8)
    return engine.device_compute_stats(
        torch.from_numpy(np.ascontiguousarray(arrivals, np.float64)).to(dev),
        torch.from_numpy(np.ascontiguousarray(which, np.int32)).to(dev), K,
        torch.from_numpy(finish).to(dev), torch.from_numpy(good).to(dev), lo, window)


def _same_as_checker(st, b, per_model, overall, names, window):
    """Every number of the checker's compute_stats, bit for bit, from the device's arrays."""
    index = {n: k for k, n in enumerate(names)}
    for p in per_model:
        k = index[p["name"]]
        n_good = int(st["num_good"][b, k])
        assert int(st["num_requests"][k]) == p["num_requests"]
        assert np.float64(n_good) / p["num_requests"] == p["goodput"]
        if n_good:
            with np.errstate(divide="ignore"):
                thr = n_good / (st["last_start"][b, k] - st["first_start"][b, k])
            assert thr == p["throughput"]
        for field in ("latency_mean", "latency_std", "latency_p90", "latency_p99"):
            want = np.float64(p[field])
            assert st[field][b, k].tobytes() == want.tobytes(), (p["name"], field)
    assert np.float64(st["good_total"][b]) / window == overall[0]
    assert (st["latency_sum"][b] / window).tobytes() == np.float64(overall[1]).tobytes()


def test_compute_stats_golden(golden):
    """mms_compute_stats on the simulator outputs stored in case_candidates.npz
    against what the reference's Workload.compute_stats returned for them
    (case_stats.npz), in the reference's order of models."""
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from mms_b200 import cases
    from oracle import stats
    g, c = golden("case_stats"), golden("case_candidates")
    w = cases.candidate_batch_case(num_candidates=48, duration=120.0).workload
    n = len(w.arrivals)
    for wi, warmup in enumerate(g["warmups"]):
        lo, hi = stats.window(w.arrivals, float(warmup))
        st = _device_stats(w.arrivals, w.name_index, len(w.names), c["finish_first4"],
                           c["good_first4"], lo, hi - lo)
        assert lo > 0 and hi == n - lo
        for b in range(4):
            tag = f"w{wi}_b{b}"
            per_model = [dict(name=str(name), **{f: g[f"{tag}_{f}"][j] for f in stats.FIELDS})
                         for j, name in enumerate(g[f"{tag}_names"])]
            _same_as_checker(st, b, per_model, g[f"{tag}_overall"], list(w.names), hi - lo)


def test_compute_stats_awkward_counts():
    """Models whose number of good requests sits on every branch of numpy's
    pairwise sum (fewer than 8, up to 128, the first splits), a model with no
    good request, one with a single one, requests of no model, zero latencies;
    windows at the start, in the middle and of one request."""
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from oracle import stats
    rng = np.random.default_rng(17)
    goods = [0, 1, 2, 7, 8, 9, 15, 16, 17, 127, 128, 129, 130, 135, 136, 137, 255, 256, 257, 1000,
             4097, 20011]
    names = [f"m{k}" for k in range(len(goods) + 1)]          # the last name has no request
    which, good = [], []
    for k, n_good in enumerate(goods):
        extra = int(rng.integers(0, 5)) if k else 3           # bad requests of the model
        which += [k] * (n_good + extra)
        good += [True] * n_good + [False] * extra
    which = np.array(which + [-1] * 50, np.int32)             # requests of no model
    good = np.array(good + [True] * 50)
    perm = rng.permutation(len(which))
    which, good = which[perm], good[perm]
    N = len(which)
    arrivals = np.cumsum(rng.gamma(0.3, 0.01, N))
    latency = rng.gamma(2.0, 0.05, N) * rng.choice([1e-3, 1.0, 30.0], N)
    latency[rng.random(N) < 0.01] = 0.0
    finish = arrivals + latency
    finish[~good] = arrivals[~good]
    fin2 = np.stack([finish, arrivals + latency[::-1]])
    good2 = np.stack([good, good[::-1].copy()])
    for lo, window in ((0, N), (N // 7, N - 2 * (N // 7)), (5, 1), (N - 300, 300)):
        st = _device_stats(arrivals, which, len(names), fin2, good2, lo, window)
        for b in range(2):
            a, wh, f, gd = (x[lo:lo + window] for x in (arrivals, which, fin2[b], good2[b]))
            keep = wh >= 0
            with np.errstate(divide="ignore", invalid="ignore"):
                per_model, _ = stats.compute_stats(a[keep], wh[keep], names, a[keep], f[keep],
                                                   gd[keep], 0.0)
                overall = (np.mean(gd), np.mean(f - a))
            _same_as_checker(st, b, per_model, overall, names, window)
            seen = {p["name"] for p in per_model}
            for k, name in enumerate(names):
                if name not in seen:
                    assert st["num_requests"][k] == 0 and st["num_good"][b, k] == 0


def test_compute_stats_full_size_from_device_rows():
    """The one-hour trace: per-request outputs of the simulator stay on the
    GPU, mms_compute_stats reads them there; the checker's numpy statistics of
    the downloaded rows must agree bit for bit.  Then the same through
    approximate_one_case(fast_stats=False)."""
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from functools import partial
    from mms_b200 import cases, engine, simulator
    from mms_b200.simulator import workload_arrays
    from oracle import stats
    case = cases.candidate_batch_case(num_candidates=6)
    w = case.workload
    names = [d.name for d in case.model_datas]
    profs = [d.profiling_result for d in case.model_datas]
    mids, slos = workload_arrays(w, names)
    trace = engine.DeviceTrace(w.arrivals, mids, slos, len(names))
    table = engine.LatencyTable(profs)
    enc = engine.encode_placements(case.placements, table, len(names))
    res, _, _ = engine.run_batch(trace, enc, table, per_request=True, group_good=True,
                                 rows_on_device=True)
    assert res.finish is None and res.finish_device.shape == (6, len(w.arrivals))
    lo, hi = stats.window(w.arrivals, 10.0)
    d_which = torch.from_numpy(np.asarray(w.name_index, np.int32)).to(trace.device)
    st = engine.device_compute_stats(trace.arrivals, d_which, len(w.names), res.finish_device,
                                     res.good_device, lo, hi - lo)
    fin, good = res.finish_device.cpu().numpy(), res.good_device.cpu().numpy().astype(bool)
    for b in range(6):
        per_model, overall = stats.compute_stats(w.arrivals, w.name_index, w.names, w.arrivals,
                                                 fin[b], good[b], 10.0)
        _same_as_checker(st, b, per_model, overall, list(w.names), hi - lo)

    def register_models(controller):
        for d in case.model_datas:
            controller.register_model.remote(d.name, partial(object, d.profiling_result))

    serving = (register_models, lambda start=0: w, lambda controller: case.placements[2])
    got, _ = simulator.approximate_one_case(serving, warmup=10)
    per_model, overall = stats.compute_stats(w.arrivals, w.name_index, w.names, w.arrivals,
                                             fin[2], good[2], 10.0)
    assert [x.name for x in got.per_model_stats] == [p["name"] for p in per_model]
    for x, p in zip(got.per_model_stats, per_model):
        for field in stats.FIELDS:
            assert np.float64(getattr(x, field)).tobytes() == np.float64(p[field]).tobytes(), field
    assert (got.goodput, got.latency_mean, got.num_requests, got.request_rate) == tuple(overall)
    # the per-request arrays of the result are fetched when somebody looks at them
    x = got.per_model_stats[-1]
    pick = (np.asarray(w.name_index)[lo:hi] == list(w.names).index(x.name)) & good[2][lo:hi]
    assert len(x.latency) == int(pick.sum())
    assert np.array_equal(np.asarray(x.latency), (fin[2] - w.arrivals)[lo:hi][pick])
    assert np.array_equal(np.asarray(x.request_starts), np.asarray(w.arrivals)[lo:hi][pick])


def test_pinned_stager_uploads_arrays_and_lazy_arrays():
    """engine.PinnedStager: arrays of awkward sizes, cut into pieces smaller than
    they are, and arrays produced piece by piece (engine.LazyArray) arrive
    unchanged; a second upload reuses the buffers."""
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from mms_b200 import engine
    dev = torch.device("cuda", 0)
    stager = engine.PinnedStager.get(dev, threads=3, piece_bytes=1 << 16)
    rng = np.random.default_rng(2)
    for _ in range(2):
        srcs = [rng.random(n) for n in (1, 8191, 8192, 8193, 100003)]
        ids = rng.integers(0, 50, 70001).astype(np.int32)
        lut = rng.permutation(50).astype(np.int32)
        lazy = engine.LazyArray(len(ids), np.int32,
                                lambda out, lo, hi: np.take(lut, ids[lo:hi], out=out))
        slo64 = rng.random(12345)
        lazy32 = engine.LazyArray(len(slo64), np.float32,
                                  lambda out, lo, hi: np.copyto(out, slo64[lo:hi], casting="same_kind"))
        dsts = [torch.empty(len(a), dtype=torch.float64, device=dev) for a in srcs]
        d_ids = torch.empty(len(ids), dtype=torch.int32, device=dev)
        d_slo = torch.empty(len(slo64), dtype=torch.float32, device=dev)
        stager.upload(list(zip(dsts, srcs)) + [(d_ids, lazy), (d_slo, lazy32)])
        torch.cuda.synchronize()
        for d, a in zip(dsts, srcs):
            assert d.cpu().numpy().tobytes() == a.tobytes()
        assert np.array_equal(d_ids.cpu().numpy(), lut[ids])
        assert d_slo.cpu().numpy().tobytes() == slo64.astype(np.float32).tobytes()
    with pytest.raises(ValueError):
        stager.upload([(torch.empty(3, dtype=torch.float64, device=dev), np.zeros(4))])
