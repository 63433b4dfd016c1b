"""ctypes front end of the C restatement in mms_oracle.c.

TEST INFRASTRUCTURE ONLY (see the header of mms_oracle.c).  The functions
take and return numpy arrays with the shapes and dtypes of the reference's
simulator kernels in alpa_serve/simulator/controller.py.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libmms_oracle.so")
_lib = None

_c_i32p = ctypes.POINTER(ctypes.c_int32)
_c_f32p = ctypes.POINTER(ctypes.c_float)
_c_f64p = ctypes.POINTER(ctypes.c_double)
_c_u8p = ctypes.POINTER(ctypes.c_uint8)
_c_i64p = ctypes.POINTER(ctypes.c_int64)


def build(force=False):
    """Compile mms_oracle.c with the Makefile beside it."""
    src = os.path.join(_HERE, "mms_oracle.c")
    if (force or not os.path.exists(_LIB_PATH)
            or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)):
        subprocess.run(["make", "-C", _HERE, "-B", "libmms_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.orc_pairwise_sum.restype = ctypes.c_double
        _lib.orc_pairwise_sum.argtypes = [_c_f64p, ctypes.c_int64]
        _lib.orc_latency_mean.restype = ctypes.c_double
        _lib.orc_latency_mean.argtypes = [_c_f64p, _c_f64p, ctypes.c_int64]
    return _lib


def _p(a, ty):
    return a.ctypes.data_as(ty)


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _check(rc, what):
    if rc != 0:
        raise RuntimeError(f"oracle {what} failed with code {rc}")


def _row_table(t, rows):
    t = _i32(t)
    if t.ndim != 2 or t.shape[0] != rows:
        raise ValueError("table must be 2-D with one row per model/group")
    if t.shape[1] == 0:
        t = np.full((rows, 1), -1, dtype=np.int32)
    return t


def simulate_requests_mixed(finish, good, tstamps, model_ids, slos, m_id2g_id,
                            num_stages, stage_latency, num_requests):
    """controller.py:561-628.  Fills `finish` (f64) and `good` (bool) in place
    and returns the four int32 counter arrays."""
    stage_latency = np.ascontiguousarray(stage_latency, dtype=np.float32)
    M, G, S = stage_latency.shape
    m2g = _row_table(m_id2g_id, M)
    ns = _i32(num_stages)
    ts = np.ascontiguousarray(tstamps, dtype=np.float64)
    mi = _i32(model_ids)
    sl = np.ascontiguousarray(slos, dtype=np.float32)
    N = int(num_requests)
    fin = np.empty(N, dtype=np.float64)
    gd = np.empty(N, dtype=np.uint8)
    mreq = np.zeros(M, np.int32); mgood = np.zeros(M, np.int32)
    greq = np.zeros(G, np.int32); ggood = np.zeros(G, np.int32)
    rc = lib().orc_simulate_requests_mixed(
        _p(fin, _c_f64p), _p(gd, _c_u8p), _p(ts, _c_f64p), _p(mi, _c_i32p), _p(sl, _c_f32p),
        _p(m2g, _c_i32p), ctypes.c_int(m2g.shape[1]), _p(ns, _c_i32p),
        _p(stage_latency, _c_f32p), ctypes.c_int64(N), ctypes.c_int(M), ctypes.c_int(G),
        ctypes.c_int(S), _p(mreq, _c_i32p), _p(mgood, _c_i32p), _p(greq, _c_i32p),
        _p(ggood, _c_i32p))
    _check(rc, "simulate_requests_mixed")
    finish[:N] = fin
    good[:N] = gd.astype(bool)
    return mreq, mgood, greq, ggood


def simulate_requests(finish, good, tstamps, model_ids, slos, m_id2g_id,
                      group_max_latency, group_sum_latency, num_requests):
    """controller.py:506-558 (one clock per group)."""
    gmax = np.ascontiguousarray(group_max_latency, dtype=np.float32)
    gsum = np.ascontiguousarray(group_sum_latency, dtype=np.float32)
    M, G = gmax.shape
    m2g = _row_table(m_id2g_id, M)
    ts = np.ascontiguousarray(tstamps, dtype=np.float64)
    mi = _i32(model_ids)
    sl = np.ascontiguousarray(slos, dtype=np.float32)
    N = int(num_requests)
    fin = np.empty(N, dtype=np.float64)
    gd = np.empty(N, dtype=np.uint8)
    mreq = np.zeros(M, np.int32); mgood = np.zeros(M, np.int32)
    greq = np.zeros(G, np.int32); ggood = np.zeros(G, np.int32)
    rc = lib().orc_simulate_requests(
        _p(fin, _c_f64p), _p(gd, _c_u8p), _p(ts, _c_f64p), _p(mi, _c_i32p), _p(sl, _c_f32p),
        _p(m2g, _c_i32p), ctypes.c_int(m2g.shape[1]),
        _p(gmax, _c_f32p), _p(gsum, _c_f32p),
        ctypes.c_int64(N), ctypes.c_int(M), ctypes.c_int(G),
        _p(mreq, _c_i32p), _p(mgood, _c_i32p), _p(greq, _c_i32p), _p(ggood, _c_i32p))
    _check(rc, "simulate_requests")
    finish[:N] = fin
    good[:N] = gd.astype(bool)
    return mreq, mgood, greq, ggood


def simulate_requests_mixed_batching(finish, good, tstamps, model_ids, slos, m_id2g_id,
                                     g_id2m_id, num_stages, stage_latency, num_requests,
                                     batchsize_config=(1, 2, 4, 8, 16)):
    """controller.py:630-798.  `batchsize_config` stands for the module global
    alpa_serve.util.batchsize_config that the reference reads."""
    stage_latency = np.ascontiguousarray(stage_latency, dtype=np.float32)
    M, G, S, NB = stage_latency.shape
    bsz = _i32(list(batchsize_config))
    if len(bsz) != NB:
        raise ValueError("stage_latency's last axis must match batchsize_config")
    m2g = _row_table(m_id2g_id, M)
    g2m = _row_table(g_id2m_id, G)
    ns = _i32(num_stages)
    ts = np.ascontiguousarray(tstamps, dtype=np.float64)
    mi = _i32(model_ids)
    sl = np.ascontiguousarray(slos, dtype=np.float32)
    N = int(num_requests)
    fin = np.empty(N, dtype=np.float64)
    gd = np.empty(N, dtype=np.uint8)
    mreq = np.zeros(M, np.int32); mgood = np.zeros(M, np.int32)
    greq = np.zeros(G, np.int32); ggood = np.zeros(G, np.int32)
    rc = lib().orc_simulate_requests_mixed_batching(
        _p(fin, _c_f64p), _p(gd, _c_u8p), _p(ts, _c_f64p), _p(mi, _c_i32p), _p(sl, _c_f32p),
        _p(m2g, _c_i32p), ctypes.c_int(m2g.shape[1]), _p(g2m, _c_i32p),
        ctypes.c_int(g2m.shape[1]), _p(ns, _c_i32p), _p(stage_latency, _c_f32p),
        _p(bsz, _c_i32p), ctypes.c_int(NB),
        ctypes.c_int64(N), ctypes.c_int(M), ctypes.c_int(G), ctypes.c_int(S),
        _p(mreq, _c_i32p), _p(mgood, _c_i32p), _p(greq, _c_i32p), _p(ggood, _c_i32p))
    _check(rc, "simulate_requests_mixed_batching")
    finish[:N] = fin
    good[:N] = gd.astype(bool)
    return mreq, mgood, greq, ggood


def pairwise_sum(a):
    a = np.ascontiguousarray(a, dtype=np.float64)
    return float(lib().orc_pairwise_sum(_p(a, _c_f64p), ctypes.c_int64(a.size)))


def latency_mean(finish, start):
    f = np.ascontiguousarray(finish, dtype=np.float64)
    s = np.ascontiguousarray(start, dtype=np.float64)
    return float(lib().orc_latency_mean(_p(f, _c_f64p), _p(s, _c_f64p), ctypes.c_int64(f.size)))


def score_batch(tstamps, model_ids, slos, m2g, num_stages, lat, nthreads=1):
    """Runs simulate_requests_mixed for B candidates given as the dense tables
    of controller.py:418-476 (m2g [B][M][R], num_stages [B][G], lat
    [B][M][G][S]) on `nthreads` host threads.  Returns (good_total i64[B],
    latency_sum f64[B], model_good i32[B][M], group_req i32[B][G])."""
    ts = np.ascontiguousarray(tstamps, dtype=np.float64)
    mi = _i32(model_ids)
    sl = np.ascontiguousarray(slos, dtype=np.float32)
    m2g = _i32(m2g); ns = _i32(num_stages)
    lat = np.ascontiguousarray(lat, dtype=np.float32)
    B, M, G, S = lat.shape
    R = m2g.shape[2]
    good_total = np.zeros(B, np.int64)
    lat_sum = np.zeros(B, np.float64)
    model_good = np.zeros((B, M), np.int32)
    group_req = np.zeros((B, G), np.int32)
    rc = lib().orc_score_batch(
        _p(ts, _c_f64p), _p(mi, _c_i32p), _p(sl, _c_f32p), ctypes.c_int64(ts.size),
        ctypes.c_int(M), ctypes.c_int(G), ctypes.c_int(S), ctypes.c_int(R),
        _p(m2g, _c_i32p), _p(ns, _c_i32p), _p(lat, _c_f32p), ctypes.c_int64(B),
        ctypes.c_int(int(nthreads)),
        _p(good_total, _c_i64p), _p(lat_sum, _c_f64p), _p(model_good, _c_i32p),
        _p(group_req, _c_i32p))
    _check(rc, "score_batch")
    return good_total, lat_sum, model_good, group_req
