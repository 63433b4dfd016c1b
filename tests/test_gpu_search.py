"""Placement searches on the GPU evaluator against the placements the
reference's own policies produce (tests/golden/policies.json)."""
import json
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "policies.json")


@pytest.fixture(scope="module")
def golden_placements():
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    with open(GOLDEN) as f:
        return json.load(f)


def as_lists(placement):
    return ([list(map(int, c)) for c in placement.group_configs],
            [[int(m) for m in ms] for ms in placement.group_models])


@pytest.mark.parametrize("case_name", ["toy-replication", "toy-search", "mixed-16"])
def test_policies_arrive_at_the_reference_placements(golden_placements, case_name):
    from mms_b200 import search, search_cases
    datas, env, policies = search_cases.all_cases()[case_name]
    for label, (cls_name, kwargs) in policies.items():
        policy = getattr(search, cls_name)(**kwargs)
        placement, _ = policy.solve_placement(datas, env)
        configs, models = as_lists(placement)
        want = golden_placements[f"{case_name}/{label}"]
        assert configs == want["group_configs"], (case_name, label)
        assert models == want["group_models"], (case_name, label)
        placement.verify(datas, env)


def test_lockstep_beam_search_equals_one_search_at_a_time(golden_placements):
    from mms_b200 import search, search_cases
    from mms_b200.placement import ModelPlacement, PlacementEvaluator, gen_train_workload
    from mms_b200.profiling import ParallelConfig
    datas, env, _ = search_cases.all_cases()["mixed-16"]
    workload = gen_train_workload(datas)
    ev = PlacementEvaluator(datas, env, workload)
    starts = [ModelPlacement([ParallelConfig(1, 1, p)] * (env.num_devices // p),
                             [[] for _ in range(env.num_devices // p)]) for p in (2, 4, 8)]
    layers = []
    together = search.beam_search_lockstep(starts, datas, env, ev, 2,
                                           on_layer=lambda n, s: layers.append(n))
    alone = [search.replica_placement_beam_search(s, datas, env, workload, ev, 2) for s in starts]
    assert [as_lists(p) for p in together] == [as_lists(p) for p in alone]
    assert max(layers) > 30          # layers really were batched across the searches


def test_place_models_drives_a_controller(golden_placements):
    from mms_b200 import search, search_cases
    from mms_b200.simulator import DummyController
    datas, env, _ = search_cases.all_cases()["toy-replication"]
    calls = []

    class Recorder(DummyController):
        def create_replica(self, name, group, configs):
            calls.append((name, group))
    placement = search.ModelParallelismGreedy(group_size=2).place_models(Recorder(), env, datas)
    assert len(calls) == sum(len(ms) for ms in placement.group_models)
