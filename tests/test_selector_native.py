"""The native (C ABI) selector must return, bit for bit, the makespans, exposed-communication
sums and chosen index the reference's evaluator produced for the same candidates."""
import json
import os

from edmir_b200 import selector
from edmir_b200.ir.analysis import analyze_exposure


def test_native_selector_matches_reference_golden(native_lib, golden_dir):
    with open(os.path.join(golden_dir, "selector_golden.json")) as f:
        data = json.load(f)
    cand = data["candidates"]
    for case in data["cases"]:
        p = selector.CostParams(**dict(zip(data["param_order"], case["p"])))
        chosen, costs = selector.select(p, cand)
        assert chosen == case["chosen"], p
        got = [[c.makespan, c.exposed_comm, c.total_comm] for c in costs]
        assert got == case["costs"], p


def test_native_selector_matches_graph_evaluator(native_lib):
    # the same candidates as EDM graphs, scored by the analysis pass of the ir package
    for comm_first in (0, 1):
        p = selector.CostParams(gemm_total=294_000, comm_bytes=117_440_512, alpha=2_000, beta_num=1000,
                                beta_den=770, split_overhead=1_500, comm_first=comm_first)
        chosen, costs = selector.select(p, (1, 2, 4, 8, 16))
        for i, c in enumerate(costs):
            g = selector.candidate_graph(p, c.chunks, "ag_gemm" if comm_first else "gemm_rs", world=8,
                                         tp_rank=0, schedule_index=i)
            ex = analyze_exposure(g)
            assert (ex.critical_path_us, ex.exposed_comm_us, ex.total_comm_us) == \
                (c.makespan, c.exposed_comm, c.total_comm)
            assert len(g.uops) == 2 * c.chunks + 2
        assert costs[chosen].makespan == min(c.makespan for c in costs)


def test_pipeline_example_native(native_lib):
    p = selector.CostParams(8000, 4000, 300, 1, 1, 100, 0)
    chosen, costs = selector.select(p, (1, 2, 4, 8))
    assert [c.makespan for c in costs] == [12300, 10500, 9700, 9600]
    assert [c.exposed_comm for c in costs] == [4300, 2300, 1300, 800]
    assert chosen == 3
    # ties go to the lowest index
    flat = selector.CostParams(1000, 0, 0, 1, 1, 0, 0)
    assert selector.select(flat, (1, 2, 4))[0] == 0


def test_selector_rejects_bad_input(native_lib):
    import pytest

    with pytest.raises(ValueError):
        selector.schedule_cost(selector.CostParams(1, 1, 0, 1, 0, 0, 0), 2)   # beta_den == 0
    with pytest.raises(ValueError):
        selector.schedule_cost(selector.CostParams(1, 1, 0, 1, 1, 0, 0), 0)   # zero chunks
