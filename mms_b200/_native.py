"""ctypes binding of libmms_sim.so (the C ABI declared in include/mms_sim.h).

There is no CPU fallback: if the library is missing, or no CUDA device is
present when a compute entry point is called, the call raises.
"""
import ctypes
import os

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
# MMS_B200_LIB names another build of the library (development: comparing two builds)
LIB_PATH = os.environ.get("MMS_B200_LIB") or os.path.join(_PKG_DIR, "libmms_sim.so")

MMS_OK = 0
ERRORS = {
    -1: "MMS_ERR_ARG (bad argument)",
    -2: "MMS_ERR_UNSUPPORTED (shape outside the kernel limits)",
    -3: "MMS_ERR_CUDA (a CUDA call failed)",
    -4: "MMS_ERR_NO_DEVICE",
}

MAX_GROUPS = 255
MAX_SLOTS = 256
MAX_PLACED = 65535
MAX_STAGES = 255
MAX_COLUMNS = 254

STATUS_HEAP_OVERFLOW = 1
STATUS_QUEUE_LEFT = 2
STATUS_BAD_INDEX = 4

FLAG_PER_REQUEST = 1
FLAG_LEGACY_CLOCK = 2
FLAG_NO_GROUP_GOOD = 4
FLAG_CROWDED = 8

STATIC_SCRATCH_BYTES = 32 << 20

PROFILE_STREAM, PROFILE_CHAIN, PROFILE_BATCH_STREAM, PROFILE_BATCH_CHAIN = 0, 1, 2, 3
PROFILE_CALL, PROFILE_BATCH_REPAIR = 4, 5


def profile_begin():
    """Starts recording kernel spans (benchmarks only, see include/mms_sim.h)."""
    check(lib().mms_profile_begin(), "mms_profile_begin")


def profile_end():
    """Stops recording; returns (durations in ms f32[n], tags i32[n]) in call order."""
    import numpy as np
    cap = 2048
    ms = np.zeros(cap, np.float32)
    tags = np.zeros(cap, np.int32)
    n = ctypes.c_int32(0)
    check(lib().mms_profile_end(ctypes.byref(n), ms.ctypes.data, tags.ctypes.data, cap),
          "mms_profile_end")
    k = min(int(n.value), cap)
    return ms[:k], tags[:k]

# Every symbol include/mms_sim.h declares.
EXPORTS = (
    "mms_abi_version", "mms_last_error", "mms_sum_plan_leaves", "mms_sum_plan_fill",
    "mms_trace_model_histogram", "mms_sim_workspace_bytes", "mms_sim_mixed",
    "mms_sim_mixed_static", "mms_trace_next_same_model", "mms_sim_batching_workspace_bytes", "mms_sim_batching",
    "mms_profile_begin", "mms_profile_end", "mms_argmax_scores",
    "mms_trace_pack", "mms_compute_stats_workspace_bytes", "mms_compute_stats",
)

_vp = ctypes.c_void_p


class Trace(ctypes.Structure):
    _fields_ = [("num_requests", ctypes.c_int64), ("arrivals", _vp), ("model_ids", _vp),
                ("slos", _vp), ("num_traces", ctypes.c_int64)]


class Placements(ctypes.Structure):
    _fields_ = [("num_candidates", ctypes.c_int32), ("num_models", ctypes.c_int32),
                ("max_groups", ctypes.c_int32), ("max_placed", ctypes.c_int32),
                ("max_slots", ctypes.c_int32), ("max_stages", ctypes.c_int32),
                ("num_columns", ctypes.c_int32), ("num_scored", ctypes.c_int32),
                ("model_off", _vp), ("model_rep", _vp), ("group_info", _vp), ("latency", _vp),
                ("latency_stride", ctypes.c_int64), ("partner", _vp), ("mirror_swap", _vp)]


class SimOptions(ctypes.Structure):
    _fields_ = [("chunk_requests", ctypes.c_int32), ("warmup_requests", ctypes.c_int32),
                ("repair_rounds", ctypes.c_int32), ("repair_segments", ctypes.c_int32)]


class SumPlan(ctypes.Structure):
    _fields_ = [("num_leaves", ctypes.c_int32), ("reserved", ctypes.c_int32),
                ("leaf_start", _vp), ("leaf_merges", _vp)]


class Workspace(ctypes.Structure):
    _fields_ = [("ptr", _vp), ("bytes", ctypes.c_size_t)]


class Results(ctypes.Structure):
    _fields_ = [("model_num_requests", _vp), ("model_num_good", _vp),
                ("group_num_requests", _vp), ("group_num_good", _vp), ("good_total", _vp),
                ("latency_sum", _vp), ("status", _vp), ("finish", _vp), ("good", _vp),
                ("resimulated", _vp)]


class Batching(ctypes.Structure):
    _fields_ = [("group_off", _vp), ("group_mod", _vp), ("group_cfg", _vp),
                ("num_batch_sizes", ctypes.c_int32), ("heap_capacity", ctypes.c_int32),
                ("batch_sizes", ctypes.c_int32 * 8)]


class StatsOut(ctypes.Structure):
    _fields_ = [("num_requests", _vp), ("num_good", _vp), ("first_start", _vp),
                ("last_start", _vp), ("latency_mean", _vp), ("latency_std", _vp),
                ("latency_p90", _vp), ("latency_p99", _vp), ("good_total", _vp),
                ("latency_sum", _vp)]


_lib = None


_host = False


def host_lib():
    """The host-side helper (csrc/encode_host.c) through ctypes.PyDLL, or None
    when it has not been built; callers then do the same work in Python."""
    global _host
    if _host is False:
        path = os.path.join(os.path.dirname(LIB_PATH), "libmms_host.so")
        _host = None
        if os.path.exists(path):
            H = ctypes.PyDLL(path)
            H.mms_host_scan.restype = ctypes.c_int
            H.mms_host_scan.argtypes = [ctypes.py_object, _vp, _vp]
            H.mms_host_flatten.restype = ctypes.c_int
            H.mms_host_flatten.argtypes = [ctypes.py_object, _vp, _vp, _vp, ctypes.c_int64,
                                           ctypes.c_int64]
            H.mms_host_flatten_once.restype = ctypes.c_int
            H.mms_host_flatten_once.argtypes = [ctypes.py_object] + [_vp] * 5 + [
                ctypes.c_int64, ctypes.c_int64, _vp]
            H.mms_host_configs.restype = ctypes.c_int64
            H.mms_host_configs.argtypes = [_vp, ctypes.c_int64, _vp, ctypes.c_int64, _vp]
            H.mms_host_encode.restype = ctypes.c_int
            H.mms_host_encode.argtypes = [ctypes.c_int64] * 4 + [_vp] * 14 + [ctypes.c_int64]
            _host = H
    return _host


def lib():
    """Loads the extension; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m mms_b200.build` "
            "(there is no CPU fallback)")
    L = ctypes.CDLL(LIB_PATH)
    L.mms_abi_version.restype = ctypes.c_int
    L.mms_last_error.restype = ctypes.c_char_p
    L.mms_sum_plan_leaves.restype = ctypes.c_int32
    L.mms_sum_plan_leaves.argtypes = [ctypes.c_int64]
    L.mms_sum_plan_fill.restype = ctypes.c_int
    L.mms_sum_plan_fill.argtypes = [ctypes.c_int64, _vp, _vp]
    L.mms_trace_model_histogram.restype = ctypes.c_int
    L.mms_trace_model_histogram.argtypes = [ctypes.POINTER(Trace), ctypes.c_int32, _vp, _vp]
    L.mms_profile_begin.restype = ctypes.c_int
    L.mms_profile_end.restype = ctypes.c_int
    L.mms_profile_end.argtypes = [ctypes.POINTER(ctypes.c_int32), _vp, _vp, ctypes.c_int32]
    L.mms_sim_workspace_bytes.restype = ctypes.c_size_t
    L.mms_sim_workspace_bytes.argtypes = [ctypes.c_int64, ctypes.POINTER(Placements),
                                          ctypes.POINTER(SimOptions), ctypes.c_uint32]
    L.mms_sim_mixed.restype = ctypes.c_int
    L.mms_sim_mixed.argtypes = [ctypes.POINTER(Trace), ctypes.POINTER(Placements),
                                ctypes.POINTER(SumPlan), _vp, ctypes.POINTER(SimOptions),
                                ctypes.POINTER(Workspace), ctypes.POINTER(Results),
                                ctypes.c_uint32, _vp]
    L.mms_sim_mixed_static.restype = ctypes.c_int
    L.mms_sim_mixed_static.argtypes = [ctypes.POINTER(Trace), ctypes.POINTER(Placements),
                                       ctypes.POINTER(SumPlan), _vp, ctypes.POINTER(SimOptions),
                                       ctypes.POINTER(Results), ctypes.c_uint32, _vp]
    L.mms_argmax_scores.restype = ctypes.c_int
    L.mms_argmax_scores.argtypes = [_vp, _vp, _vp, ctypes.c_int64, ctypes.c_int32, _vp,
                                    ctypes.c_int64, ctypes.c_int32, _vp, _vp]
    L.mms_trace_pack.restype = ctypes.c_int
    L.mms_trace_pack.argtypes = [_vp, _vp, _vp, _vp, ctypes.c_int64, ctypes.c_int64, _vp, _vp, _vp,
                                 _vp]
    L.mms_trace_next_same_model.restype = ctypes.c_int
    L.mms_trace_next_same_model.argtypes = [ctypes.POINTER(Trace), ctypes.c_int32, _vp, _vp]
    L.mms_sim_batching_workspace_bytes.restype = ctypes.c_size_t
    L.mms_sim_batching_workspace_bytes.argtypes = [ctypes.c_int64, ctypes.POINTER(Placements),
                                                   ctypes.POINTER(Batching)]
    L.mms_sim_batching.restype = ctypes.c_int
    L.mms_sim_batching.argtypes = [ctypes.POINTER(Trace), ctypes.POINTER(Placements),
                                   ctypes.POINTER(Batching), _vp, ctypes.POINTER(SumPlan),
                                   ctypes.POINTER(Workspace), ctypes.POINTER(Results), _vp]
    L.mms_compute_stats_workspace_bytes.restype = ctypes.c_size_t
    L.mms_compute_stats_workspace_bytes.argtypes = [ctypes.c_int64, ctypes.c_int32, ctypes.c_int32]
    L.mms_compute_stats.restype = ctypes.c_int
    L.mms_compute_stats.argtypes = [_vp, _vp, ctypes.c_int32, _vp, _vp, ctypes.c_int64,
                                    ctypes.c_int32, ctypes.c_int64, ctypes.c_int64,
                                    ctypes.POINTER(Workspace), ctypes.POINTER(StatsOut), _vp]
    _lib = L
    return L


def check(rc, what):
    if rc != MMS_OK:
        msg = ERRORS.get(rc, f"code {rc}")
        detail = lib().mms_last_error().decode(errors="replace")
        raise RuntimeError(f"{what}: {msg}" + (f" [{detail}]" if detail and rc == -3 else ""))
