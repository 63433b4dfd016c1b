"""Imports the live reference (alpa_serve) for differential tests and for
timing the reference's own code.

TEST INFRASTRUCTURE ONLY.  The reference is looked for, in this order, in the
directory the MMS_REFERENCE_DIR environment variable names, in a checkout
called `reference` beside this repository, and in `oracle/_ref` — a private,
git-ignored copy of the reference's Python package that `make -C oracle ref`
makes on a machine that has the checkout, so that it travels to machines
that do not (a GPU box) together with the built libraries.  The package
`mms_b200` never imports this module.
`ray` and `matplotlib`, which the reference imports at module level but does
not use on the simulator path, are replaced by the import-only stubs in
oracle/stubs.
"""
import os
import sys
import warnings

_HERE = os.path.dirname(os.path.abspath(__file__))
_mods = None


def reference_dir():
    cands = [os.environ.get("MMS_REFERENCE_DIR"),
             os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference"),
             os.path.join(_HERE, "_ref")]
    for c in cands:
        if c and os.path.isdir(os.path.join(c, "alpa_serve")):
            return c
    return None


def available():
    return reference_dir() is not None


def build_copy():
    """`make -C oracle ref` when a checkout is at hand (the private copy under
    oracle/_ref); returns the directory the reference will be imported from,
    or None."""
    import subprocess
    here_copy = os.path.join(_HERE, "_ref")
    for c in (os.environ.get("MMS_REFERENCE_DIR"),
              os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")):
        if c and os.path.isdir(os.path.join(c, "alpa_serve")):
            subprocess.run(["make", "-C", _HERE, "ref", f"MMS_REFERENCE_DIR={c}"], check=True,
                           stdout=subprocess.DEVNULL)
            return here_copy
    return reference_dir()


def load():
    """Returns a namespace with the reference's simulator, placement and
    workload modules."""
    global _mods
    if _mods is not None:
        return _mods
    ref = reference_dir()
    if ref is None:
        raise RuntimeError("reference checkout not found (set MMS_REFERENCE_DIR)")
    stubs = os.path.join(_HERE, "stubs")
    for p in (stubs, ref):
        if p not in sys.path:
            sys.path.insert(0, p)
    warnings.filterwarnings("ignore", message="overflow encountered in cast")
    import alpa_serve.util as util
    import alpa_serve.profiling as profiling
    import alpa_serve.simulator.workload as workload
    import alpa_serve.simulator.controller as controller
    import alpa_serve.placement_policy.base_policy as base_policy
    import alpa_serve.placement_policy.model_parallelism as model_parallelism
    import alpa_serve.placement_policy.selective_replication as selective_replication

    class NS:
        pass
    ns = NS()
    ns.util, ns.profiling, ns.workload = util, profiling, workload
    ns.controller, ns.base_policy = controller, base_policy
    ns.model_parallelism, ns.selective_replication = model_parallelism, selective_replication
    _mods = ns
    return ns


def to_reference_case(case):
    """Re-expresses a mms_b200.cases.Case with the reference's own classes, so
    that the reference code runs on exactly the same numbers."""
    ref = load()
    P = ref.profiling

    def prof(p):
        return P.ProfilingResult(p.model_name, {
            P.ParallelConfig(*c): P.LatencyMemData(dict(v.latency), dict(v.act_mem),
                                                   list(v.weight_mem))
            for c, v in p.para_dict.items()}, p.preprocess_cpu, p.postprocess_cpu)

    cache = {}
    datas = []
    for d in case.model_datas:
        key = id(d.profiling_result)
        if key not in cache:
            cache[key] = prof(d.profiling_result)
        datas.append(ref.base_policy.ModelData(d.name, d.slo, d.rate, d.cv, cache[key]))
    env = ref.base_policy.ClusterEnv(case.cluster_env.num_devices, case.cluster_env.mem_budget,
                                     case.cluster_env.num_devices_per_node)
    w = case.workload
    reqs = [ref.workload.Request(w.names[k], None, None if s != s else float(s), i, {})
            for i, (k, s) in enumerate(zip(w.name_index.tolist(), w.request_slo.tolist()))]
    rw = ref.workload.Workload(w.arrivals, reqs)
    placements = [ref.base_policy.ModelPlacement(
        [P.ParallelConfig(*c) for c in p.group_configs], [list(ms) for ms in p.group_models])
        for p in case.placements]
    return datas, env, rw, placements
