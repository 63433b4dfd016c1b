"""Small search problems used by the parity tests of the placement searches
(the golden placements come from running the reference's own policies on
them; see tests/golden/make_golden.py)."""
from .cases import mixed_models
from .placement import ClusterEnv, ModelData
from .profiling import GB, test_profile_2gb_100ms


def all_cases():
    """name -> (model_datas, cluster_env, {label: (policy class name, kwargs)})."""
    toy = test_profile_2gb_100ms()
    out = {}
    # the three toy problems of the reference's tests/serve/test_placement_policy.py
    out["toy-replication"] = (
        [ModelData(f"m{i}", 1, 5, 1, toy) for i in range(4)], ClusterEnv(4, 4.5 * GB),
        {"sr-greedy": ("SelectiveReplicationGreedy", {}),
         "sr-search": ("SelectiveReplicationSearch", {}),
         "mp-greedy-2": ("ModelParallelismGreedy", {"group_size": 2})})
    out["toy-search"] = (
        [ModelData(f"m{i}", 0.4, 4, 8, toy) for i in range(4)], ClusterEnv(4, 2.5 * GB),
        {"mp-search": ("ModelParallelismSearch", {})})
    # a mid-size mixed problem: 16 devices, 8 models in three size classes
    mid = mixed_models(num_models=8, total_rate=30.0, cv=3.0)
    out["mixed-16"] = (
        mid, ClusterEnv(16, 13 * GB),
        {"sr-greedy": ("SelectiveReplicationGreedy", {}),
         "mp-greedy-2": ("ModelParallelismGreedy", {"group_size": 2}),
         "mp-greedy-4": ("ModelParallelismGreedy", {"group_size": 4}),
         "mp-search": ("ModelParallelismSearch", {})})
    return out
