"""Generates the golden fixtures in this directory from the LIVE reference.

Run on a machine that has the reference checkout (see oracle/reference.py):

    python tests/golden/make_golden.py

Every fixture holds seeded inputs together with what the reference's own
code (numba kernels, the pure-Python batching simulator, PlacementEvaluator)
returned for them.  The tests compare the CPU checker and the CUDA path
against these files; nothing at test time needs the reference.
"""
import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from mms_b200 import cases  # noqa: E402
from oracle import reference  # noqa: E402


def digest(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def random_kernel_inputs(seed, N=4000, M=12, G=6, S=4, batch_cols=0):
    """Inputs for the low-level kernels with every awkward feature at once:
    unknown models (-1), a model without replica, groups with 1/2/4 stages,
    +inf latencies, replicated models, near-tied clocks."""
    rng = np.random.RandomState(seed)
    tstamps = np.cumsum(rng.gamma(0.25, 4 * 0.02, size=N))
    model_ids = rng.randint(-1, M, size=N).astype(np.int32)
    slos = rng.choice([0.2, 0.35, 0.5, 1.0], size=N).astype(np.float32)
    num_stages = rng.choice([1, 2, 4], size=G).astype(np.int32)
    num_stages[0] = S
    m2g = np.full((M, G), -1, np.int32)
    for m in range(M - 1):                      # model M-1 stays replica-less
        reps = np.sort(rng.choice(G, size=rng.randint(1, 4), replace=False))
        m2g[m, :len(reps)] = reps
    shape = (M, G, S) if not batch_cols else (M, G, S, batch_cols)
    lat = rng.uniform(0.005, 0.06, size=shape).astype(np.float32)
    if batch_cols:
        lat = np.sort(lat, axis=-1)             # larger batches take longer
    holes = rng.rand(M, G) < 0.08
    lat[holes] = np.float32(np.inf)
    g2m = np.full((G, M), -1, np.int32)
    fill = [0] * G
    for m in range(M):
        for g in m2g[m]:
            if g >= 0:
                g2m[g, fill[g]] = m
                fill[g] += 1
    return tstamps, model_ids, slos, m2g, g2m, num_stages, lat


def main():
    ref = reference.load()
    C = ref.controller

    # ---- low-level kernels -------------------------------------------------
    ts, mid, slo, m2g, g2m, ns, lat = random_kernel_inputs(11)
    N = len(ts)
    fin = np.empty(N); good = np.empty(N, bool)
    cnt = C.simulate_requests_mixed(fin, good, ts, mid, slo, m2g, ns, lat, N)
    np.savez_compressed(os.path.join(HERE, "kernel_mixed.npz"), tstamps=ts, model_ids=mid,
                        slos=slo, m_id2g_id=m2g, num_stages=ns, stage_latency=lat,
                        finish=fin, good=good, model_num_requests=cnt[0],
                        model_num_good=cnt[1], group_num_requests=cnt[2],
                        group_num_good=cnt[3])

    gmax = lat.max(axis=2); gsum = lat.sum(axis=2, dtype=np.float32)
    fin = np.empty(N); good = np.empty(N, bool)
    cnt = C.simulate_requests(fin, good, ts, mid, slo, m2g, gmax, gsum, N)
    np.savez_compressed(os.path.join(HERE, "kernel_legacy.npz"), tstamps=ts, model_ids=mid,
                        slos=slo, m_id2g_id=m2g, group_max_latency=gmax,
                        group_sum_latency=gsum, finish=fin, good=good,
                        model_num_requests=cnt[0], model_num_good=cnt[1],
                        group_num_requests=cnt[2], group_num_good=cnt[3])

    ref.util.batchsize_config[:] = [1, 2, 4, 8]
    ts, mid, slo, m2g, g2m, ns, lat = random_kernel_inputs(12, N=3000, batch_cols=4)
    N = len(ts)
    fin = np.empty(N); good = np.empty(N, bool)
    cnt = C.simulate_requests_mixed_batching(fin, good, ts, mid, slo, m2g, g2m, ns, lat, N)
    np.savez_compressed(os.path.join(HERE, "kernel_batching.npz"), tstamps=ts, model_ids=mid,
                        slos=slo, m_id2g_id=m2g, g_id2m_id=g2m, num_stages=ns,
                        stage_latency=lat, batchsize_config=np.array([1, 2, 4, 8], np.int32),
                        finish=fin, good=good, model_num_requests=cnt[0],
                        model_num_good=cnt[1], group_num_requests=cnt[2],
                        group_num_good=cnt[3])

    # ---- the fixed 4 x pp2 placement, full size ------------------------------
    case = cases.fixed_pipeline_case()
    datas, env, rw, pls = reference.to_reference_case(case)
    names = [d.name for d in datas]; profs = [d.profiling_result for d in datas]
    n2i = {m: i for i, m in enumerate(names)}
    mids = np.array([n2i.get(r.model_name, -1) for r in rw.requests], dtype=np.int32)
    slos = np.array([r.slo for r in rw.requests], dtype=np.float32)
    (start, fin, good, mreq, mgood, greq, ggood) = C.approximate_one_case_one_placement(
        pls[0], names, profs, mids, slos, rw.arrivals)
    ev = ref.base_policy.PlacementEvaluator(datas, env, rw, "fast_simulator", False)
    score = ev.get_scores(pls)[0]
    np.savez_compressed(
        os.path.join(HERE, "case_fixed_pipeline.npz"),
        num_requests=len(start), arrivals_sha256=digest(rw.arrivals),
        model_ids_sha256=digest(mids), finish_sha256=digest(fin),
        good_sha256=digest(good.astype(np.uint8)), finish_head=fin[:2048], good_head=good[:2048],
        model_num_requests=mreq, model_num_good=mgood, group_num_requests=greq,
        group_num_good=ggood, goodput=np.mean(good), latency_mean=np.mean(fin - start),
        score=score)

    # ---- a candidate batch, shrunk (two minutes of the one-hour trace) ------------
    case = cases.candidate_batch_case(num_candidates=48, duration=120.0)
    datas, env, rw, pls = reference.to_reference_case(case)
    ev = ref.base_policy.PlacementEvaluator(datas, env, rw, "fast_simulator", False)
    scores = np.array(ev.get_scores(pls), dtype=np.float64)
    stats = ev.get_stats(pls)
    M = len(datas)
    G = max(len(p.group_configs) for p in pls)
    greq = np.zeros((len(pls), G), np.int32)
    mgood_rate = np.zeros((len(pls), M))
    goodput = np.zeros(len(pls)); lat_mean = np.zeros(len(pls))
    for b, (gp, per_model, group_req, full) in enumerate(stats):
        greq[b, :len(group_req)] = group_req
        mgood_rate[b] = per_model
        goodput[b] = gp
        lat_mean[b] = full.latency_mean
    names = [d.name for d in datas]; profs = [d.profiling_result for d in datas]
    mids, slos = rw.cached_data[0], rw.cached_data[1]
    fins = np.zeros((4, len(rw.arrivals))); goods = np.zeros((4, len(rw.arrivals)), bool)
    for b in range(4):
        out = C.approximate_one_case_one_placement(pls[b], names, profs, mids, slos, rw.arrivals)
        fins[b], goods[b] = out[1], out[2]
    np.savez_compressed(
        os.path.join(HERE, "case_candidates.npz"),
        num_candidates=len(pls), duration=120.0, num_requests=len(rw.arrivals),
        arrivals_sha256=digest(rw.arrivals), scores=scores, goodput=goodput,
        latency_mean=lat_mean, model_goodput=mgood_rate, group_num_requests=greq,
        finish_first4=fins, good_first4=goods)

    # ---- the same with batching (pure-Python reference: keep it small) ------------
    case = cases.candidate_batch_case(num_candidates=12, duration=60.0, batching=True)
    datas, env, rw, pls = reference.to_reference_case(case)
    names = [d.name for d in datas]; profs = [d.profiling_result for d in datas]
    n2i = {m: i for i, m in enumerate(names)}
    mids = np.array([n2i.get(r.model_name, -1) for r in rw.requests], dtype=np.int32)
    slos = np.array([r.slo for r in rw.requests], dtype=np.float32)
    N = len(rw.arrivals)
    fins = np.zeros((len(pls), N)); goods = np.zeros((len(pls), N), bool)
    mgood = np.zeros((len(pls), M), np.int32); mreq = np.zeros((len(pls), M), np.int32)
    G = max(len(p.group_configs) for p in pls)
    greq = np.zeros((len(pls), G), np.int32); ggood = np.zeros((len(pls), G), np.int32)
    for b, p in enumerate(pls):
        out = C.approximate_one_case_one_placement(p, names, profs, mids, slos, rw.arrivals,
                                                   enable_batching=True)
        fins[b], goods[b] = out[1], out[2]
        mreq[b], mgood[b] = out[3], out[4]
        greq[b, :len(out[5])] = out[5]; ggood[b, :len(out[6])] = out[6]
    np.savez_compressed(
        os.path.join(HERE, "case_candidates_batching.npz"),
        num_candidates=len(pls), duration=60.0, num_requests=N,
        arrivals_sha256=digest(rw.arrivals), finish=fins, good=goods,
        model_num_requests=mreq, model_num_good=mgood, group_num_requests=greq,
        group_num_good=ggood)
    # ---- a placement schedule through approximate_one_case ---------------------------
    from functools import partial
    datas0, env0, w0, starts, pls0 = cases.replacement_case()
    case = cases.Case("replacement", datas0, env0, w0, pls0)
    datas, env, rw, pls = reference.to_reference_case(case)
    schedule = ref.base_policy.ModelPlacementWithReplacement(list(starts), pls)

    def register_models(controller):
        for d in datas:
            controller.register_model.remote(d.name, partial(object, d.profiling_result))

    serving_case = ref.util.ServingCase(register_models, lambda start=0: rw,
                                        lambda controller: schedule)
    out = {}
    for tag, fast in (("fast", True), ("full", False)):
        stats, _ = C.approximate_one_case(serving_case, fast_stats=fast)
        pm = stats.per_model_stats
        out.update({
            f"{tag}_goodput": stats.goodput, f"{tag}_latency_mean": stats.latency_mean,
            f"{tag}_num_requests": stats.num_requests, f"{tag}_request_rate": stats.request_rate,
            f"{tag}_group_num_requests": np.array(stats.group_num_requests, np.int64),
            f"{tag}_model_num_requests": np.array([x.num_requests for x in pm], np.int64),
            f"{tag}_model_goodput": np.array([x.goodput for x in pm], np.float64),
            f"{tag}_model_throughput": np.array([x.throughput for x in pm], np.float64),
            f"{tag}_model_latency_mean": np.array([x.latency_mean for x in pm], np.float64),
            f"{tag}_model_latency_std": np.array([x.latency_std for x in pm], np.float64),
            f"{tag}_model_latency_p90": np.array([x.latency_p90 for x in pm], np.float64),
            f"{tag}_model_latency_p99": np.array([x.latency_p99 for x in pm], np.float64)})
    np.savez_compressed(os.path.join(HERE, "case_replacement.npz"),
                        arrivals_sha256=digest(rw.arrivals), num_requests_total=len(rw.arrivals),
                        **out)

    # ---- whole searches: the placements the reference's policies arrive at ----------
    import json
    from mms_b200 import search_cases
    import alpa_serve.placement_policy as RP
    out = {}
    for name, (datas, env, policies) in search_cases.all_cases().items():
        case = cases.Case(name, datas, env, cases.merged_gamma_trace(datas[:1], 1.0, 0), [])
        rdatas, renv, _, _ = reference.to_reference_case(case)
        for pol_name, (cls_name, kwargs) in policies.items():
            policy = getattr(RP, cls_name)(**kwargs)
            placement, _ = policy.solve_placement(rdatas, renv)
            out[f"{name}/{pol_name}"] = {
                "group_configs": [list(map(int, c)) for c in placement.group_configs],
                "group_models": [[int(m) for m in ms] for ms in placement.group_models]}
            print(name, pol_name, out[f"{name}/{pol_name}"]["group_models"])
    with open(os.path.join(HERE, "policies.json"), "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)
    print("golden fixtures written to", HERE)


def loop_cases():
    """The problems the reference's own search loops are run on (here by the
    pure reference, in tests/test_gpu_reference_loops.py by the same loops on
    this package's evaluator): name -> (Case, loop label -> how to run it)."""
    from mms_b200 import search_cases
    datas16, env16, _ = search_cases.all_cases()["mixed-16"]
    from mms_b200.placement import gen_train_workload
    mixed16 = cases.Case("mixed-16", datas16, env16, gen_train_workload(datas16), [])
    big = cases.greedy_search_case(duration=300.0)
    return {"mixed-16": mixed16, "search-64": big}


def run_reference_loops(ref, case_name, rdatas, renv, rw):
    """Runs the reference's own loops (whatever PlacementEvaluator the
    reference modules currently hold) and returns label -> placement."""
    P = ref.profiling.ParallelConfig
    MP = ref.base_policy.ModelPlacement
    out = {}
    if case_name == "mixed-16":
        c4 = P(1, 1, 4)
        start = MP([c4, c4, c4, c4], [[0, 3], [1, 4], [2, 5], []])
        out["on-last-group"] = ref.base_policy.replica_placement_on_last_group(
            start, rdatas, renv, rw, None, 3, 0)
        np.random.seed(7)
        ev = ref.base_policy.PlacementEvaluator(rdatas, renv, rw, "fast_simulator", False)
        seed_sol = MP([c4, c4, c4, c4], [[0, 3, 6], [1, 4, 7], [2, 5, 0], [3, 6, 1]])
        out["evolutionary"] = ref.base_policy.evolutionary_search(
            [seed_sol], rdatas, renv, ev, 2, 0)
    policy = ref.model_parallelism.ModelParallelismSearch(max_op=1)
    out["mp-search-max-op-1"] = policy.solve_placement(rdatas, renv, rw)[0]
    return out


def placement_lists(placement):
    return {"group_configs": [list(map(int, c)) for c in placement.group_configs],
            "group_models": [[int(m) for m in ms] for ms in placement.group_models]}


def reference_loops():
    """reference_loops.json: what replica_placement_on_last_group
    (base_policy.py:482), evolutionary_search (:623) and
    ModelParallelismSearch.solve_placement (model_parallelism.py:411) return
    when they run on the reference's own evaluator."""
    import json
    ref = reference.load()
    out = {}
    for name, case in loop_cases().items():
        rdatas, renv, rw, _ = reference.to_reference_case(case)
        for label, placement in run_reference_loops(ref, name, rdatas, renv, rw).items():
            out[f"{name}/{label}"] = placement_lists(placement)
            print(name, label, out[f"{name}/{label}"]["group_models"])
    with open(os.path.join(HERE, "reference_loops.json"), "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)


STATS_FIELDS = ("num_requests", "goodput", "throughput", "latency_mean", "latency_std",
                "latency_p90", "latency_p99")


def stats_fixture():
    """case_stats.npz: Workload.compute_stats (workload.py:308-354) of the
    reference, with warm-ups of 10 and 25 seconds, on the per-request outputs
    the reference's simulator gave for four placements of the shrunk candidate
    batch (case_candidates.npz holds those outputs)."""
    ref = reference.load()
    case = cases.candidate_batch_case(num_candidates=48, duration=120.0)
    datas, env, rw, pls = reference.to_reference_case(case)
    g = np.load(os.path.join(HERE, "case_candidates.npz"))
    assert digest(rw.arrivals) == str(g["arrivals_sha256"])
    start = np.asarray(rw.arrivals)
    out = {"warmups": np.array([10.0, 25.0])}
    for w, warmup in enumerate(out["warmups"]):
        for b in range(4):
            st = rw.compute_stats(start, g["finish_first4"][b], g["good_first4"][b], float(warmup))
            tag = f"w{w}_b{b}"
            out[f"{tag}_names"] = np.array([x.name for x in st.per_model_stats])
            for field in STATS_FIELDS:
                out[f"{tag}_{field}"] = np.array([getattr(x, field) for x in st.per_model_stats],
                                                 np.float64)
            out[f"{tag}_overall"] = np.array([st.goodput, st.latency_mean, st.num_requests,
                                              st.request_rate], np.float64)
    np.savez_compressed(os.path.join(HERE, "case_stats.npz"), **out)


if __name__ == "__main__":
    if "--only-stats" in sys.argv:
        stats_fixture()
        sys.exit(0)
    if "--only-loops" not in sys.argv:
        main()
        stats_fixture()
    reference_loops()
