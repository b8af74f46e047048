"""The oracle's cost model must reproduce what the reference itself computed (golden JSON made by
running the reference, tests/golden/make_golden.py) and the known answers in the reference's own
tests (EDM-IR/tests/analysis_test.py:27, :52-58) and demo (EDM-IR/examples/synthetic_demo.py)."""
import json
import os

import pytest

from oracle import cost_model


def _load(golden_dir, name):
    with open(os.path.join(golden_dir, name)) as f:
        return json.load(f)


def _as_lists(g):
    nodes = [{"id": n["id"], "op": n["op"], "start": n["start"], "end": n["end"]} for n in g["nodes"]]
    edges = [(s, d) for s, d, _ in g["edges"]]
    return nodes, edges


def test_analysis_golden(golden_dir):
    data = _load(golden_dir, "analysis_golden.json")
    assert len(data) >= 5
    for name, g in data.items():
        nodes, edges = _as_lists(g)
        ex = cost_model.exposure(nodes, edges)
        want = g["expect"]
        assert ex["critical_path"] == want["critical_path"], name
        for key in ("critical_path_us", "phase_time_us", "total_comm_us", "exposed_comm_us",
                    "total_data_movement_us", "exposed_data_movement_us", "ecr", "edmr"):
            assert ex[key] == want[key], (name, key)


def test_reference_known_answers(golden_dir):
    data = _load(golden_dir, "analysis_golden.json")
    # EDM-IR/tests/analysis_test.py:27
    assert cost_model.phase_duration(_as_lists(data["test_phase_boundaries"])[0]) == 50.0
    # EDM-IR/tests/analysis_test.py:52-58
    ex = cost_model.exposure(*_as_lists(data["test_ecr_edmr"]))
    assert (ex["phase_time_us"], ex["total_comm_us"], ex["exposed_comm_us"]) == (100.0, 10.0, 10.0)
    assert (ex["total_data_movement_us"], ex["exposed_data_movement_us"]) == (30.0, 30.0)
    assert ex["ecr"] == pytest.approx(0.1) and ex["edmr"] == pytest.approx(0.3)
    # demo graphs: hidden (92, ecr 0), exposed (117, ecr 0.214), harmful (117, edmr 0.154)
    for name, cp, ecr, edmr in (("demo_hidden_communication", 92.0, 0.0, 0.0),
                                ("demo_exposed_communication", 117.0, 0.214, None),
                                ("demo_harmful_overlap", 117.0, None, 0.154)):
        ex = cost_model.exposure(*_as_lists(data[name]))
        assert ex["critical_path_us"] == cp
        if ecr is not None:
            assert round(ex["ecr"], 3) == ecr
        if edmr is not None:
            assert round(ex["edmr"], 3) == edmr


def test_selector_golden(golden_dir):
    data = _load(golden_dir, "selector_golden.json")
    cand = data["candidates"]
    assert len(data["cases"]) >= 400
    for case in data["cases"]:
        params = dict(zip(data["param_order"], case["p"]))
        chosen, costs = cost_model.select_schedule(params, cand)
        assert chosen == case["chosen"], params
        for got, want in zip(costs, case["costs"]):
            assert [got["makespan"], got["exposed_comm"], got["total_comm"]] == want, params


def test_pipeline_example():
    # two-stage pipeline: GEMM 8000, transfer 4000, alpha 300, split 100
    p = {"gemm_total": 8000, "comm_bytes": 4000, "alpha": 300, "beta_num": 1, "beta_den": 1,
         "split_overhead": 100, "comm_first": 0}
    chosen, costs = cost_model.select_schedule(p, [1, 2, 4, 8])
    assert [c["makespan"] for c in costs] == [12300, 10500, 9700, 9600]
    assert [c["exposed_comm"] for c in costs] == [4300, 2300, 1300, 800]
    assert chosen == 3
