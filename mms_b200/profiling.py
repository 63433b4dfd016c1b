"""Latency and memory tables of a model, keyed by parallel configuration.

Host-side mirror of the containers in alpa_serve/profiling.py:14-68 that the
simulator reads (`para_dict[config].latency[batch_size]` is the list of
per-stage latencies, `weight_mem` the per-stage weight bytes).  The classes
are duck-type compatible with the reference's: a reference ProfilingResult
can be passed wherever one of these is expected, and ParallelConfig compares
and hashes like the reference's namedtuple.
"""
from collections import namedtuple
import dataclasses
from typing import Any, Dict, List

GB = 1 << 30     # alpa_serve/util.py:21

# (data parallel, operator parallel, pipeline parallel) — profiling.py:14
ParallelConfig = namedtuple("ParallelConfig", ("dp", "op", "pp"))


@dataclasses.dataclass
class LatencyMemData:
    """profiling.py:16-41."""
    latency: Dict[int, List[float]]
    act_mem: Dict[int, List[float]]
    weight_mem: List[float]
    metadata: Any = None


@dataclasses.dataclass
class ProfilingResult:
    """profiling.py:44-68."""
    model_name: str
    para_dict: Dict[ParallelConfig, LatencyMemData]
    preprocess_cpu: float = 0.0
    postprocess_cpu: float = 0.0


def synthetic_profile(name: str, single_device_latency: float, weight_bytes: float,
                      pipeline_degrees=(1, 2, 4, 8), stage_overhead: float = 0.05,
                      batch_sizes=(1,), batch_slope: float = 0.2) -> ProfilingResult:
    """A made-up profile: at pipeline degree p every stage takes
    L/p * (1 + stage_overhead*(p-1)) seconds at batch size 1 and
    l(b) = l(1) * (1 - batch_slope + batch_slope*b) at batch size b; the
    weights are split evenly over the stages."""
    para = {}
    for p in pipeline_degrees:
        l1 = single_device_latency / p * (1 + stage_overhead * (p - 1))
        latency = {int(b): [l1 * ((1 - batch_slope) + batch_slope * b)] * p if b != 1
                   else [l1] * p for b in batch_sizes}
        para[ParallelConfig(1, 1, p)] = LatencyMemData(
            latency=latency, act_mem={int(b): [0.0] * p for b in batch_sizes},
            weight_mem=[weight_bytes / p] * p)
    return ProfilingResult(name, para)


def test_profile_2gb_100ms() -> ProfilingResult:
    """The toy profile the reference's placement tests use
    (load_test_prof_result("test-2GB-100ms"), profiling.py:276-315): 2 GB of
    weights, 100 ms on one device, 2x51 ms on two, 4x26 ms on four."""
    stages = {1: [0.100], 2: [0.051, 0.051], 4: [0.026, 0.026, 0.026, 0.026]}
    para = {}
    for p, lat in stages.items():
        para[ParallelConfig(1, 1, p)] = LatencyMemData(
            latency={1: list(lat)}, act_mem={1: [0.0] * p}, weight_mem=[2 * GB / p] * p)
    return ProfilingResult("test-2GB-100ms", para)
