"""The reference's OWN search loops, unchanged, on this package's evaluator.

`replica_placement_on_last_group` (alpa_serve/placement_policy/base_policy.py:
482-570), `evolutionary_search` (:623-715) and
`ModelParallelismSearch.solve_placement` (model_parallelism.py:411-456) are
imported from the reference, the one name they construct evaluators from —
`PlacementEvaluator` — is pointed at `mms_b200.placement.PlacementEvaluator`,
and they are run on the reference's own `ModelPlacement` / `ModelData` /
`Workload` objects.  The placements they return must be the ones the same
loops return on the reference's evaluator (tests/golden/reference_loops.json,
written by tests/golden/make_golden.py).  Needs the reference importable:
a checkout, or the private copy `make -C oracle ref` leaves under oracle/_ref.
"""
import importlib.util
import json
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def _make_golden_module():
    spec = importlib.util.spec_from_file_location(
        "make_golden", os.path.join(HERE, "golden", "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="module")
def setup():
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from oracle import reference
    if not reference.available():
        pytest.skip("the reference is not importable here: no checkout and no oracle/_ref copy "
                    "(make -C oracle ref)")
    with open(os.path.join(HERE, "golden", "reference_loops.json")) as f:
        want = json.load(f)
    return reference, reference.load(), _make_golden_module(), want


@pytest.mark.parametrize("case_name", ["mixed-16", "search-64"])
def test_reference_loops_run_unchanged_on_the_gpu_evaluator(setup, monkeypatch, case_name):
    reference, ref, gold, want = setup
    from mms_b200.placement import PlacementEvaluator
    made = []

    class Counting(PlacementEvaluator):
        def __init__(self, *args, **kwargs):
            super().__init__(*args, **kwargs)
            made.append(self)

    monkeypatch.setattr(ref.base_policy, "PlacementEvaluator", Counting)
    monkeypatch.setattr(ref.model_parallelism, "PlacementEvaluator", Counting)
    case = gold.loop_cases()[case_name]
    rdatas, renv, rw, _ = reference.to_reference_case(case)
    got = gold.run_reference_loops(ref, case_name, rdatas, renv, rw)
    assert made, "the reference's loops did not build their evaluator from the patched name"
    for label, placement in got.items():
        assert type(placement).__module__.startswith("alpa_serve."), type(placement)
        assert gold.placement_lists(placement) == want[f"{case_name}/{label}"], (case_name, label)
        placement.verify(rdatas, renv)


def test_lockstep_search_arrives_at_the_reference_placement_on_64_devices(setup):
    """This package's restated search (all partitions advanced in lockstep)
    against the placement the reference's ModelParallelismSearch returns for
    64 devices and 56 models."""
    reference, ref, gold, want = setup
    from mms_b200 import search
    case = gold.loop_cases()["search-64"]
    placement, _ = search.ModelParallelismSearch(max_op=1).solve_placement(
        case.model_datas, case.cluster_env, case.workload)
    assert gold.placement_lists(placement) == want["search-64/mp-search-max-op-1"]
