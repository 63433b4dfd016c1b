"""Host-side logic that needs no GPU: library exports, encoders, plans."""
import ctypes
import os
import re

import numpy as np
import pytest

from mms_b200 import _native as nat
from mms_b200 import build as mms_build
from mms_b200 import cases, engine
from mms_b200.placement import ModelPlacement
from mms_b200.profiling import ParallelConfig
from oracle import tables

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    mms_build.build()
    lib = ctypes.CDLL(nat.LIB_PATH)
    header = open(os.path.join(ROOT, "include", "mms_sim.h")).read()
    declared = set(re.findall(r"\b(mms_[a-z_0-9]+)\s*\(", header))
    assert declared == set(nat.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), name
    assert nat.lib().mms_abi_version() >= 1


def decode(enc, table, b):
    """Compact tables of candidate b -> the reference's dense tables."""
    G = int(enc.num_groups[b])
    M = enc.M
    info = enc.group_info[b, :G].astype(np.int64)
    slot, ns, contested = info & 0xFF, (info >> 8) & 0xFF, (info >> 16) & 1
    col = np.zeros(G, np.int64)
    m2g = np.full((M, max(G, 1)), -1, np.int32)
    shared = np.zeros(G, np.int64)
    for m in range(M):
        lo, hi = int(enc.model_off[b, m]), int(enc.model_off[b, m + 1])
        ents = enc.model_rep[b, lo:hi].astype(np.int64)
        gs = ents & 0xFF
        assert np.array_equal((ents >> 8) & 0xFF, slot[gs])
        assert np.array_equal((ents >> 16) & 0xFF, ns[gs])
        col[gs] = ents >> 24
        m2g[m, :hi - lo] = gs
        if hi - lo > 1:
            shared[gs] = 1
    assert np.array_equal(shared, contested)
    S = int(ns.max()) if G else 1
    lat = np.zeros((M, G, S), np.float32)
    for g in range(G):
        lat[:, g, :ns[g]] = table.host[:, col[g], :ns[g]]
    # clock slots of consecutive groups tile [0, sum of stages)
    assert np.array_equal(slot, np.cumsum(ns) - ns)
    return m2g, ns.astype(np.int32), lat


def test_encoder_round_trip_on_random_placements():
    case = cases.candidate_batch_case(num_candidates=40, duration=5.0)
    profs = [d.profiling_result for d in case.model_datas]
    table = engine.LatencyTable(profs)
    sols = list(case.placements)
    sols.append(ModelPlacement([ParallelConfig(1, 1, 8)] * 8, [[] for _ in range(8)]))
    sols.append(ModelPlacement([ParallelConfig(1, 2, 4), ParallelConfig(1, 1, 1)],
                               [[3, 1, 2], [1]]))      # unprofiled config -> +inf
    enc = engine.encode_placements(sols, table, len(profs))
    assert enc.B == len(sols)
    for b, p in enumerate(sols):
        m2g, ns, lat = decode(enc, table, b)
        ref_m2g, _, ref_ns, ref_lat = tables.dense_tables(p, profs)
        assert np.array_equal(ns, ref_ns)
        assert np.array_equal(m2g, ref_m2g[:, :m2g.shape[1]])
        for m in range(len(profs)):          # latency of every (model, group) pair in use
            for g in m2g[m][m2g[m] >= 0]:
                assert lat[m, g, :ns[g]].tobytes() == ref_lat[m, g, :ns[g]].tobytes()
        assert enc.num_replicas[b] == sum(len(x) for x in p.group_models)


def test_dense_encoder_matches_batch_encoder():
    case = cases.candidate_batch_case(num_candidates=3, duration=5.0)
    profs = [d.profiling_result for d in case.model_datas]
    for p in case.placements:
        m2g, _, ns, _ = tables.dense_tables(p, profs)
        off, rep, info, T = engine.encode_dense(m2g, ns, len(profs))
        table = engine.LatencyTable(profs)
        enc = engine.encode_placements([p], table, len(profs))
        assert np.array_equal(off[0], enc.model_off[0])
        n = off[0, -1]          # same entries up to the latency column
        assert np.array_equal(rep[0, :n] & 0xFFFFFF, enc.model_rep[0, :n] & 0xFFFFFF)
        assert np.array_equal(info[0], enc.group_info[0, :info.shape[1]])
        assert T == enc.T


def numpy_order_sum(a, leaf_start, merges):
    stack = []
    for leaf in range(len(merges)):
        x = a[leaf_start[leaf]:leaf_start[leaf + 1]]
        n = len(x)
        body = n - n % 8
        p = [0.0] * 8
        for i in range(0, body, 8):
            for j in range(8):
                p[j] = p[j] + x[i + j]
        r = ((p[0] + p[1]) + (p[2] + p[3])) + ((p[4] + p[5]) + (p[6] + p[7]))
        for i in range(body, n):
            r = r + x[i]
        stack.append(r)
        for _ in range(merges[leaf]):
            right = stack.pop()
            stack[-1] = stack[-1] + right
    assert len(stack) == 1
    return stack[0]


def test_sum_plan_reproduces_numpy():
    L = nat.lib()
    for n in (1, 5, 8, 9, 127, 128, 129, 130, 1000, 4097, 57949):
        leaves = L.mms_sum_plan_leaves(n)
        start = np.zeros(leaves + 1, np.int32)
        merges = np.zeros(leaves, np.uint8)
        assert L.mms_sum_plan_fill(n, start.ctypes.data, merges.ctypes.data) == 0
        assert start[0] == 0 and start[-1] == n
        assert np.all(np.diff(start) <= 128) and np.all(start[1:-1] % 8 == 0)
        a = np.random.RandomState(n).gamma(0.3, 1.0, size=n)
        a[::3] = 0.0
        assert numpy_order_sum(a.tolist(), start, merges) == float(np.add.reduce(a))
    assert L.mms_sum_plan_leaves(0) == 0


def test_group_lists_match_reference_tables():
    case = cases.candidate_batch_case(num_candidates=12, duration=5.0, batching=True)
    profs = [d.profiling_result for d in case.model_datas]
    table = engine.LatencyTable(profs, [1, 2, 4, 8])
    enc = engine.encode_placements(case.placements, table, len(profs))
    goff, gmod, gcfg = engine.group_lists(enc.model_off, enc.model_rep, enc.group_info, enc.G)
    for b, p in enumerate(case.placements):
        _, g2m, ns, lat = tables.dense_tables(p, profs, batchsize_config=(1, 2, 4, 8))
        for g in range(len(ns)):
            want = g2m[g][g2m[g] >= 0]
            assert np.array_equal(gmod[b, goff[b, g]:goff[b, g + 1]], want)
            assert (gcfg[b, g] >> 8) & 0xFF == ns[g]
            col = int(gcfg[b, g]) >> 16
            for m in want:
                assert table.host[m, col, :ns[g], :].tobytes() == lat[m, g, :ns[g], :].tobytes()


def test_twin_group_detection_matches_a_plain_search():
    """Interchangeable groups (same parallel config, same set of models) are
    found through hashed model sets; compare with a dictionary of sets.  Every
    permutation of them gets a mirror candidate."""
    from math import factorial
    from mms_b200 import cases, engine
    from mms_b200.placement import ModelPlacement
    from mms_b200.profiling import ParallelConfig
    case = cases.candidate_batch_case(num_candidates=600, duration=5.0, placement_seed=2)
    c1, c2 = ParallelConfig(1, 1, 1), ParallelConfig(1, 1, 2)
    sols = list(case.placements) + [
        ModelPlacement([c1] * 6 + [c2] * 2, [[0, 3], [3, 0], [1], [1], [1], [], [2, 5], [5]]),
        ModelPlacement([c1, c2], [[0], [0]]),
        ModelPlacement([c1, c1], [[], []]),
        ModelPlacement([c1] * 7, [[4]] * 5 + [[2], [2]])]
    table = engine.LatencyTable([d.profiling_result for d in case.model_datas])
    enc = engine.encode_placements(sols, table, len(case.model_datas))
    found = dict(enc.twins)
    expect_mirrors = 0
    for b, p in enumerate(sols):
        classes = {}
        for g, (c, ms) in enumerate(zip(p.group_configs, p.group_models)):
            if len(ms):
                classes.setdefault((c, tuple(sorted(ms))), []).append(g)
        want = sorted(v for v in classes.values() if len(v) >= 2)
        perms = int(np.prod([factorial(len(v)) for v in want])) if want else 1
        if perms - 1 > engine.MAX_MIRRORS:
            want = []                                # too many arrangements: not reported
        assert sorted(found.get(b, [])) == want, b
        expect_mirrors += perms - 1 if want else 0
    assert len(found) >= 4
    assert sorted(found[len(sols) - 4]) == [[0, 1], [2, 3, 4]]
    off, rep, info, partner, swap = enc.with_mirrors()
    assert len(partner) == enc.B + expect_mirrors
    owners = partner[enc.B:]
    assert np.all(np.diff(owners) >= 0)                      # mirrors of one placement are adjacent
    assert len(sols) - 1 not in owners                       # 5! * 2 permutations: none at all
    assert np.count_nonzero(owners == len(sols) - 4) == 2 * 6 - 1
    for b in np.unique(owners):
        assert partner[b] == enc.B + np.flatnonzero(owners == b)[0]
    assert np.all(partner[:enc.B][np.setdiff1d(np.arange(enc.B), owners)] == -1)
    assert np.array_equal(rep[enc.B:], enc.model_rep[owners])
    assert np.all(swap[:enc.B] == engine.NO_SWAP)
    # the exchanges of one placement's mirrors produce distinct arrangements of its groups
    b = len(sols) - 4
    seen = set()
    for w in swap[enc.B:][owners == b].astype(np.uint64):
        word = int(w[0]) | (int(w[1]) << 32)
        arr = list(range(8))
        for k in range(4):
            i, j = (word >> (16 * k)) & 0xFF, (word >> (16 * k + 8)) & 0xFF
            if i != 0xFF:
                arr[i], arr[j] = arr[j], arr[i]
        assert arr != list(range(8))
        for cls in ([0, 1], [2, 3, 4]):
            assert sorted(arr[g] for g in cls) == cls
        seen.add(tuple(arr))
    assert len(seen) == 11


def test_c_flattening_equals_python_flattening():
    """The host helper (csrc/encode_host.c) and the pure-Python passes give the
    encoder the same arrays; bad input raises instead of being encoded."""
    from mms_b200 import _native as nat
    from mms_b200 import cases, engine
    from mms_b200.placement import ModelPlacement
    from mms_b200.profiling import ParallelConfig
    assert nat.host_lib() is not None, "libmms_host.so was not built"
    case = cases.candidate_batch_case(num_candidates=300, duration=5.0, placement_seed=7)
    sols = list(case.placements) + [ModelPlacement([], []),
                                    ModelPlacement((ParallelConfig(1, 1, 2),), ((np.int64(3), 1),))]
    fast = engine._flatten(sols)
    saved, nat._host = nat._host, None
    try:
        slow = engine._flatten(sols)
    finally:
        nat._host = saved
    for a, b in zip(fast, slow):
        assert a.dtype == b.dtype and np.array_equal(a, b)
    with pytest.raises(ValueError):
        engine._flatten([ModelPlacement([ParallelConfig(1, 1, 1)], [[0], [1]])])
    with pytest.raises(TypeError):
        engine._flatten([ModelPlacement(["pp2"], [[0]])])
    with pytest.raises(AttributeError):
        engine._flatten([object()])


def test_c_encoder_equals_numpy_encoder():
    """The tables and the classes of interchangeable groups from
    csrc/encode_host.c equal those of the numpy encoder."""
    from mms_b200 import _native as nat
    from mms_b200 import cases, engine
    from mms_b200.placement import ModelPlacement
    from mms_b200.profiling import ParallelConfig
    assert nat.host_lib() is not None, "libmms_host.so was not built"
    case = cases.candidate_batch_case(num_candidates=700, duration=5.0, placement_seed=11)
    c1, c2 = ParallelConfig(1, 1, 1), ParallelConfig(1, 1, 2)
    sols = list(case.placements) + [
        ModelPlacement([c1] * 6 + [c2] * 2, [[0, 3], [3, 0], [1], [1], [1], [], [2, 5], [5]]),
        ModelPlacement([c1, c2], [[0], [0]]), ModelPlacement([], []),
        ModelPlacement([c1, c1], [[], []]),
        ModelPlacement([c2, c1, c2], [[7, 1, 2], [2], [2, 7, 1]])]
    profs = [d.profiling_result for d in case.model_datas]
    for batch in (sols, sols[-3:-2], []):
        ta, tb = engine.LatencyTable(profs), engine.LatencyTable(profs)
        a = engine.encode_placements(batch, ta, len(profs), native=True)
        b = engine.encode_placements(batch, tb, len(profs), native=False)
        assert ta.configs == tb.configs and ta.host.tobytes() == tb.host.tobytes()
        for k in "B M G P T S C".split():
            assert getattr(a, k) == getattr(b, k), k
        for k in "model_off model_rep group_info num_groups num_replicas".split():
            x, y = getattr(a, k), getattr(b, k)
            assert x.dtype == y.dtype and x.shape == y.shape and np.array_equal(x, y), k
        assert ({i: sorted(c) for i, c in a.twins} == {i: sorted(c) for i, c in b.twins})
        assert [i for i, _ in a.twins] == sorted(i for i, _ in a.twins)
    assert dict(a.twins) == {} and len(sols) - 1 in dict(
        engine.encode_placements(sols, engine.LatencyTable(profs), len(profs)).twins)
    with pytest.raises(IndexError):
        engine.encode_placements([ModelPlacement([c1], [[len(profs)]])], engine.LatencyTable(profs),
                                 len(profs))


def test_expansion_of_normalized_placements_equals_add_then_normalize():
    """search._expand inserts into sorted tuples instead of re-sorting every
    candidate; the placements equal add_model(g, m).normalize()
    (base_policy.py:29-35,439-455), in the same order, ties between equal
    groups included."""
    import random
    from mms_b200 import search
    case = cases.greedy_search_case(duration=5.0)
    M = len(case.model_datas)
    budget = case.cluster_env.mem_budget
    starts = search.ModelParallelismSearch(max_op=1).enumerate_group_configs_uneven(case.cluster_env)
    rng = random.Random(5)
    for sol in starts:
        weight = search._weights(sol.group_configs, case.model_datas)
        visited = set()
        for step in range(10):
            group_mem = search._group_mem(sol, weight)
            want, seen = [], set(visited)
            for g, c in enumerate(sol.group_configs):
                for m in range(M):
                    if weight[c][m] + group_mem[g] < budget and m not in sol.group_models[g]:
                        nxt = sol.add_model(g, m).normalize()
                        if nxt.group_models not in seen:
                            seen.add(nxt.group_models)
                            want.append(nxt)
            got = search._expand(sol, weight, M, budget, visited)
            assert step == 0 or search._is_normalized(sol)
            assert [(tuple(p.group_configs), p.group_models) for p in got] == \
                   [(tuple(p.group_configs), p.group_models) for p in want]
            assert visited == seen
            if not got:
                break
            sol = rng.choice(got)


def test_encoder_threads_change_nothing():
    """The table builder cuts a long list into ranges, one thread each; the
    tables and the lists of interchangeable groups are the same as from one
    thread (and as from the numpy encoder)."""
    import ctypes
    from mms_b200 import _native as nat
    from mms_b200 import cases, engine
    H = nat.host_lib()
    if H is None:
        pytest.skip("host helper not built")
    case = cases.candidate_batch_case(num_candidates=3000, duration=30.0)
    profs = [d.profiling_result for d in case.model_datas]
    knob = ctypes.c_int.in_dll(H, "mms_host_threads")
    encs = []
    try:
        for threads in (1, 3, 5):
            knob.value = threads
            table = engine.LatencyTable(profs)
            encs.append(engine.encode_placements(case.placements, table, len(profs)))
    finally:
        knob.value = 0
    table = engine.LatencyTable(profs)
    encs.append(engine.encode_placements(case.placements, table, len(profs), native=False))
    first = encs[0]
    assert len(first.twins) > 50
    for e in encs[1:]:
        assert np.array_equal(e.model_off, first.model_off)
        assert np.array_equal(e.model_rep, first.model_rep)
        assert np.array_equal(e.group_info, first.group_info)
        assert (e.T, e.G, e.P) == (first.T, first.G, first.P)
        # (the numpy encoder lists a placement's classes in another order)
        assert [(b, sorted(list(c) for c in cl)) for b, cl in e.twins] == \
            [(b, sorted(list(c) for c in cl)) for b, cl in first.twins]
    for e in encs[1:3]:
        assert e.twins == first.twins


def test_lazy_trace_arrays_equal_workload_arrays():
    """The piecewise producers the sweep uploads from give the arrays of
    workload_arrays (controller.py:335-336), whatever the piece boundaries."""
    from mms_b200 import cases
    from mms_b200.placement import TraceSweep
    from mms_b200.simulator import workload_arrays
    case = cases.sweep_case(duration=20.0)
    sweep = TraceSweep.__new__(TraceSweep)
    sweep.model_names = tuple(d.name for d in case.model_datas[:-3])      # three unknown models
    w = case.trace(5)
    ids, slos = workload_arrays(w, sweep.model_names)
    lazy_ids, lazy_slos = sweep._lazy_arrays(w)
    assert len(lazy_ids) == len(ids) and (ids == -1).any()
    assert np.array_equal(lazy_ids.materialize(), ids) and lazy_ids.dtype == np.int32
    assert lazy_slos.materialize().tobytes() == slos.tobytes()
    out = np.empty(1000, np.int32)
    lazy_ids.fill(out, 37, 1037)
    assert np.array_equal(out, ids[37:1037])
    out = np.empty(1000, np.float32)
    lazy_slos.fill(out, 37, 1037)
    assert np.array_equal(out, slos[37:1037])
    # all models known and in the workload's order: the ids are the workload's own index
    sweep.model_names = tuple(d.name for d in case.model_datas)
    ids, _ = workload_arrays(w, sweep.model_names)
    assert np.array_equal(sweep._lazy_arrays(w)[0].materialize(), ids) and (ids >= 0).all()


def test_mirror_words_in_batches_equal_one_by_one():
    """The exchange lists of the mirror candidates, formed for all placements of a
    class pattern together, are those of mirror_swaps, in the same order; a
    sub-batch carries its part of them."""
    from mms_b200 import cases, engine
    case = cases.candidate_batch_case(num_candidates=1500, duration=5.0, placement_seed=3)
    profs = [d.profiling_result for d in case.model_datas]
    enc = engine.encode_placements(case.placements, engine.LatencyTable(profs), len(profs))
    counts, words = enc.mirror_table()
    assert len(enc.twins) > 50 and counts.sum() > 50
    at = 0
    for (_, classes), c in zip(enc.twins, counts.tolist()):
        one = engine.mirror_swaps(classes)
        assert [int(w) for w in words[at:at + c]] == one
        at += c
    pick = np.array(sorted({b for b, _ in enc.twins[::3]} | {0, 1, 2}), np.int64)
    sub = enc.take(pick)
    carried = sub._mirror_table
    sub._mirror_table = None
    fresh = sub.mirror_table()
    assert np.array_equal(carried[0], fresh[0]) and np.array_equal(carried[1], fresh[1])
    off, rep, info, partner, swap = enc.with_mirrors()
    assert len(partner) == enc.B + counts.sum() and (partner[enc.B:] >= 0).all()
    owners = partner[enc.B:]
    assert np.array_equal(rep[enc.B:], enc.model_rep[owners])
    firsts = partner[[b for (b, _), c in zip(enc.twins, counts.tolist()) if c]]
    assert np.array_equal(firsts, enc.B + (np.cumsum(counts) - counts)[counts > 0])
