"""Dense placement tables and whole-case evaluation for the CPU checker.

TEST INFRASTRUCTURE ONLY.  Restates the table construction of
alpa_serve/simulator/controller.py:410-503 and the fast statistics of
controller.py:393-403 / base_policy.py:225-226 on top of oracle.cpu.
"""
import numpy as np

from . import cpu

inf = 1e100   # alpa_serve/util.py:23
eps = 1e-6    # alpa_serve/util.py:22


def dense_tables(placement, prof_ress, batchsize_config=None):
    """(m_id2g_id i32[M][G], g_id2m_id i32[G][M], num_stages i32[G],
    stage_latency f32[M][G][S] or f32[M][G][S][NB]) — controller.py:418-476."""
    configs, models = placement.group_configs, placement.group_models
    G, M = len(configs), len(prof_ress)
    m2g = np.full((M, max(G, 1)), -1, np.int32)
    fill = [0] * M
    for g, ms in enumerate(models):
        for m in ms:
            m2g[m][fill[m]] = g
            fill[m] += 1
    g2m = np.full((max(G, 1), max(M, 1)), -1, np.int32)
    gfill = [0] * G
    for m in range(M):
        for g in m2g[m]:
            if g >= 0:
                g2m[g][gfill[g]] = m
                gfill[g] += 1
    num_stages = np.array([c.pp for c in configs], dtype=np.int32)
    S = int(num_stages.max()) if G else 1
    with np.errstate(over="ignore"):
        if batchsize_config is None:
            lat = np.zeros((M, G, S), np.float32)
            for m in range(M):
                for g in range(G):
                    v = prof_ress[m].para_dict.get(configs[g], None)
                    if v:
                        pen = 0.009 * len(v.latency[1])
                        for k in range(num_stages[g]):
                            lat[m][g][k] = v.latency[1][k] * (1 + pen)
                    else:
                        lat[m][g][:] = inf
        else:
            nb = len(batchsize_config)
            lat = np.zeros((M, G, S, nb), np.float32)
            for m in range(M):
                for g in range(G):
                    v = prof_ress[m].para_dict.get(configs[g], None)
                    if v:
                        pen = 0.009 * len(v.latency[1])
                        for k in range(num_stages[g]):
                            for j, bs in enumerate(batchsize_config):
                                lat[m][g][k][j] = v.latency[bs][k] * (1 + pen)
                    else:
                        lat[m][g][:] = inf
    return m2g, g2m, num_stages, lat


def one_placement(placement, prof_ress, model_ids, slos, arrivals, batchsize_config=None):
    """approximate_one_case_one_placement (controller.py:410-503) on the C
    checker.  Returns (finish, good, model_num_requests, model_num_good,
    group_num_requests, group_num_good)."""
    m2g, g2m, ns, lat = dense_tables(placement, prof_ress, batchsize_config)
    N = len(arrivals)
    finish = np.empty(N, np.float64)
    good = np.empty(N, bool)
    if batchsize_config is None:
        c = cpu.simulate_requests_mixed(finish, good, arrivals, model_ids, slos, m2g, ns, lat, N)
    else:
        c = cpu.simulate_requests_mixed_batching(finish, good, arrivals, model_ids, slos, m2g,
                                                 g2m, ns, lat, N, batchsize_config)
    return (finish, good) + tuple(c)


def score(placement, finish, good, arrivals):
    """base_policy.py:225-226 with the fast statistics of controller.py:401-402."""
    n = len(arrivals)
    goodput = np.float64(int(np.count_nonzero(good))) / n
    latency_mean = np.float64(cpu.pairwise_sum(finish - arrivals)) / n
    replicas = sum(len(x) for x in placement.group_models)
    return goodput - latency_mean / 10000 + replicas / 1000000


def dense_tables_batch(placements, prof_ress):
    """dense_tables for a list of placements, stacked and padded to the
    widest: (m2g i32[B][M][G], num_stages i32[B][G] (1 where there is no
    group), lat f32[B][M][G][S] (+inf where there is no group)).  The f32
    latency row of a (model, parallel config) pair is computed once, with the
    operations of controller.py:467-476, and copied to every group that has
    that config."""
    B, M = len(placements), len(prof_ress)
    G = max([len(p.group_configs) for p in placements] + [1])
    S = max([int(c.pp) for p in placements for c in p.group_configs] + [1])
    m2g = np.full((B, M, G), -1, np.int32)
    ns = np.ones((B, G), np.int32)
    lat = np.full((B, M, G, S), np.float32(np.inf), np.float32)
    rows = {}

    def config_rows(c):
        key = tuple(c)
        if key not in rows:
            tab = np.zeros((M, S), np.float32)
            with np.errstate(over="ignore"):
                for m in range(M):
                    v = prof_ress[m].para_dict.get(c, None)
                    if v:
                        pen = 0.009 * len(v.latency[1])
                        for k in range(int(c.pp)):
                            tab[m][k] = v.latency[1][k] * (1 + pen)
                    else:
                        tab[m][:] = inf
            rows[key] = tab
        return rows[key]

    for b, p in enumerate(placements):
        fill = [0] * M
        for g, (c, ms) in enumerate(zip(p.group_configs, p.group_models)):
            ns[b, g] = c.pp
            lat[b, :, g, :] = config_rows(c)
            for m in ms:
                m2g[b, m, fill[m]] = g
                fill[m] += 1
    return m2g, ns, lat


def score_from_sums(placement, good_total, latency_sum, n):
    """base_policy.py:225-226 from the reductions np.mean is made of."""
    goodput = np.float64(int(good_total)) / n
    latency_mean = np.float64(latency_sum) / n
    replicas = sum(len(x) for x in placement.group_models)
    return goodput - latency_mean / 10000 + replicas / 1000000
