"""Workload.compute_stats for the CPU checker.

TEST INFRASTRUCTURE ONLY.  Restates alpa_serve/simulator/workload.py:308-354
on arrays: the reference walks `Request` objects to group the requests by
model name; here `which[i]` is the index of request i's model in `names`.
The arithmetic is the reference's own numpy calls (np.mean, np.std, np.sort,
fancy indexing), so the floating-point results are the reference's bit for
bit.  Pinned against the reference by tests/golden/case_stats.npz.
"""
import numpy as np

FIELDS = ("num_requests", "goodput", "throughput", "latency_mean", "latency_std",
          "latency_p90", "latency_p99")


def window(arrivals, warmup):
    """[first, last) of the requests compute_stats keeps (workload.py:312-318).
    The reference slices [skip:-skip] only when skip > 0."""
    n = len(arrivals)
    if n > 1:
        skip = int(warmup / (arrivals[-1] - arrivals[0]) * n)
        if skip > 0:
            return skip, max(n - skip, skip)
    return 0, n


def compute_stats(arrivals, which, names, start, finish, good, warmup):
    """Returns (per_model, overall): per_model is a list of dicts with FIELDS
    and "name", in the reference's order (names by first appearance inside the
    window, then a stable sort by request count, workload.py:321-326); overall
    is (goodput, latency_mean, num_requests, request_rate) of workload.py:352."""
    start, finish, good = np.asarray(start), np.asarray(finish), np.asarray(good)
    which = np.asarray(which)
    lo, hi = window(np.asarray(arrivals), warmup)
    start, finish, good, which = start[lo:hi], finish[lo:hi], good[lo:hi], which[lo:hi]
    indices = {}
    for i, k in enumerate(which.tolist()):          # dict keeps first-appearance order
        indices.setdefault(k, []).append(i)
    order = sorted(indices.keys(), key=lambda k: len(indices[k]))
    per_model = []
    for k in order:
        idx = np.asarray(indices[k], dtype=np.int32)
        tmp_good = np.asarray(good[idx], dtype=bool)
        tmp_start = start[idx][tmp_good]
        tmp_finish = finish[idx][tmp_good]
        goodput = np.mean(tmp_good)
        if goodput > 0:
            with np.errstate(divide="ignore"):
                throughput = len(tmp_start) / (tmp_start[-1] - tmp_start[0])
            latency = tmp_finish - tmp_start
        else:
            throughput = 0
            latency = [0]
        srt = np.sort(latency)
        per_model.append(dict(
            name=names[k], num_requests=len(idx), goodput=goodput, throughput=throughput,
            latency_mean=np.mean(latency), latency_std=np.std(latency),
            latency_p90=srt[int(0.90 * len(srt))], latency_p99=srt[int(0.99 * len(srt))]))
    overall = (np.mean(good), np.mean(finish - start), len(start),
               len(start) / (start[-1] - start[0]))
    return per_model, overall
