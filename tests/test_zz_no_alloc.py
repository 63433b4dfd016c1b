"""mms_sim_mixed_static: the entry point for hosts that cannot allocate.

Collected last on purpose (file name), so a run that stops at the first
failure has already exercised everything else.  The check is against
mms_sim_mixed itself, through the C ABI, bit for bit, on two calls in a row:
the second call finds the scratch array full of the first call's data, with
a different batch and a different chunking.
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _call(entry, trace, enc, table, opts, per_request):
    """Runs one of the two entry points on `enc`; returns the outputs as numpy."""
    import torch
    from mms_b200 import _native as nat
    from mms_b200.engine import _ptr, _stream_ptr
    L = nat.lib()
    dev = trace.device
    B, M, G, N = enc.B, enc.M, enc.G, trace.num_requests
    t = {k: torch.from_numpy(v).to(dev) for k, v in
         dict(off=enc.model_off, rep=enc.model_rep, info=enc.group_info).items()}
    lat = table.device(dev)
    cands = nat.Placements(B, M, G, enc.P, enc.T, enc.S, enc.C, 0, _ptr(t["off"]), _ptr(t["rep"]),
                           _ptr(t["info"]), _ptr(lat), 0)
    i32 = dict(dtype=torch.int32, device=dev)
    o = dict(mreq=torch.full((B, M), -7, **i32), mgood=torch.full((B, M), -7, **i32),
             greq=torch.full((B, G), -7, **i32), ggood=torch.full((B, G), -7, **i32),
             total=torch.full((B,), -7, dtype=torch.int64, device=dev),
             lsum=torch.full((B,), -7.0, dtype=torch.float64, device=dev),
             status=torch.zeros(B, **i32), redo=torch.zeros(B, **i32),
             fin=torch.zeros((B, N), dtype=torch.float64, device=dev),
             good=torch.zeros((B, N), dtype=torch.uint8, device=dev))
    flags = nat.FLAG_PER_REQUEST if per_request else 0      # group_num_good is wanted
    out = nat.Results(_ptr(o["mreq"]), _ptr(o["mgood"]), _ptr(o["greq"]), _ptr(o["ggood"]),
                      _ptr(o["total"]), _ptr(o["lsum"]), _ptr(o["status"]),
                      _ptr(o["fin"]) if per_request else None,
                      _ptr(o["good"]) if per_request else None, _ptr(o["redo"]))
    tr, plan = trace.c_trace(), trace.c_plan()
    if entry == "static":
        rc = L.mms_sim_mixed_static(ctypes.byref(tr), ctypes.byref(cands), ctypes.byref(plan),
                                    _ptr(trace.model_hist), ctypes.byref(opts), ctypes.byref(out),
                                    flags, _stream_ptr())
    else:
        need = L.mms_sim_workspace_bytes(N, ctypes.byref(cands), ctypes.byref(opts), flags)
        ws_t = torch.empty(need, dtype=torch.uint8, device=dev)
        ws = nat.Workspace(_ptr(ws_t), need)
        rc = L.mms_sim_mixed(ctypes.byref(tr), ctypes.byref(cands), ctypes.byref(plan),
                             _ptr(trace.model_hist), ctypes.byref(opts), ctypes.byref(ws),
                             ctypes.byref(out), flags, _stream_ptr())
    torch.cuda.synchronize()
    return rc, {k: v.cpu().numpy() for k, v in o.items()}


def test_static_scratch_entry_point_matches_workspace_entry_point():
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from mms_b200 import _native as nat
    from mms_b200 import cases, engine
    from mms_b200.simulator import workload_arrays

    case = cases.candidate_batch_case(num_candidates=48, duration=600.0, placement_seed=21)
    names = [d.name for d in case.model_datas]
    profs = [d.profiling_result for d in case.model_datas]
    mids, slos = workload_arrays(case.workload, names)
    trace = engine.DeviceTrace(case.workload.arrivals, mids, slos, len(names))
    table = engine.LatencyTable(profs)

    # two calls in a row: a chunked score-only batch, then a smaller batch with
    # per-request outputs and another cut of the trace
    rounds = [(case.placements[:32], engine.sim_options(4096, 1024), False),
              (case.placements[32:], engine.sim_options(8192, 512), True)]
    for sols, opts, per_request in rounds:
        enc = engine.encode_placements(sols, table, len(names))
        rc_s, got = _call("static", trace, enc, table, opts, per_request)
        rc_w, want = _call("workspace", trace, enc, table, opts, per_request)
        assert rc_s == 0 and rc_w == 0
        assert not got["status"].any() and not want["status"].any()
        for key in ("mreq", "mgood", "greq", "ggood", "total", "redo"):
            assert np.array_equal(got[key], want[key]), key
        assert got["lsum"].tobytes() == want["lsum"].tobytes()          # bit-exact fp64
        assert got["total"].min() > 0
        if per_request:
            assert got["fin"].tobytes() == want["fin"].tobytes()
            assert np.array_equal(got["good"], want["good"])

    # a shape that needs more scratch than the built-in array is refused, loudly
    big = engine.encode_placements(case.placements * 40, table, len(names))
    rc, _ = _call("static", trace, big, table, engine.sim_options(), False)
    assert rc == -2                                                     # MMS_ERR_UNSUPPORTED
    msg = nat.lib().mms_last_error().decode()
    assert "scratch" in msg and str(nat.STATIC_SCRATCH_BYTES) in msg
