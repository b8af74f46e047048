"""EDM graphs survive a trip through JSON: same records, same edge order, same analyses."""
import json

import pytest

from edmir_b200 import graph_json, lowering
from edmir_b200.ir import EDMBuilder, MovementDesc, TensorDesc, buffer_ref
from edmir_b200.ir import ops as irops
from edmir_b200.ir.analysis import analyze_critical_path, analyze_exposure


def _same_analysis(a, b):
    ca, cb = analyze_critical_path(a), analyze_critical_path(b)
    assert ca.path == cb.path and ca.duration_us == cb.duration_us
    ea, eb = analyze_exposure(a), analyze_exposure(b)
    assert ea == eb


def test_schedule_candidates_round_trip(native_lib):
    spec = lowering.TPLinearSpec("gemm_rs", M=8192, N=8192, K=3584, world=8)
    sel = lowering.select_schedule(spec, tp_rank=3)
    for g in sel.graphs:
        text = graph_json.dumps(g)
        back = graph_json.loads(text)
        assert list(back.uops) == list(g.uops)
        assert all(back.uops[i] == g.uops[i] for i in g.uops)
        assert [(e.src, e.dst, e.kind, e.attrs) for e in back.edges] == [(e.src, e.dst, e.kind, e.attrs) for e in g.edges]
        _same_analysis(g, back)
        assert graph_json.dumps(back) == text


def test_measured_graph_and_descriptors_round_trip(tmp_path):
    spec = lowering.TPLinearSpec("ag_gemm", M=8192, N=1280, K=8192, world=8)
    g = lowering.measured_graph(spec, lowering.Schedule(index=1, chunks=2, transport="ce"), total_us=355.0, gemm_only_us=130.0, tp_rank=0,
                                device="B200", iteration=4)
    b = EDMBuilder(default_phase="decode")
    u = b.uop(irops.MOVEMENT_COPY, "kv.transfer", 0.0, 18.0,
              tensor=TensorDesc(name="kv", kind="buffer", shape=(2, "seq", None), dtype="bf16", size_bytes=1 << 20),
              movement=MovementDesc(kind="copy", backend="nvlink", size_bytes=1 << 20, group="tp",
                                    group_ranks=(0, 1), src_ranks=(0,), dst_ranks=(1,)),
              reads=(buffer_ref("kv", "read", "gpu0"),), writes=(buffer_ref("kv", "write", "gpu1"),),
              attrs={"chunk": 0}, raw_events=("memcpy#1",))
    for graph in (g, b.build()):
        path = tmp_path / "g.json"
        graph_json.save(graph, str(path))
        back = graph_json.load(str(path))
        assert all(back.uops[i] == graph.uops[i] for i in graph.uops)
        _same_analysis(graph, back)
    assert isinstance(back.uops[u.id].movement.group_ranks, tuple)
    assert back.uops[u.id].tensor.shape == (2, "seq", None)


def test_bad_documents_are_refused():
    with pytest.raises(ValueError):
        graph_json.from_dict({"format": "something else", "uops": [], "edges": []})
    doc = {"format": graph_json.FORMAT, "uops": [{"id": 0, "op": "compute.gemm", "name": "x", "start_us": 0.0,
                                                  "end_us": 1.0, "colour": "red"}], "edges": []}
    with pytest.raises(ValueError):
        graph_json.from_dict(doc)
    doc["uops"][0].pop("colour")
    doc["edges"] = [{"src": 0, "dst": 7, "kind": "data.dependency"}]
    with pytest.raises(KeyError):
        graph_json.from_dict(json.loads(json.dumps(doc)))
