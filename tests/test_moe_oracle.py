"""The MoE oracle's integer conventions and the host-side helpers (no GPU)."""
import numpy as np

from edmir_b200 import moe
from edmir_b200.ir.analysis import analyze_exposure
from oracle import moe as oracle


def test_top2_ties_go_to_the_lower_index_and_weights_are_a_softmax():
    lg = np.array([[1.0, 3.0, 3.0, 0.0], [0.5, 0.5, 0.5, 0.5], [-1.0, -2.0, 4.0, 4.5]])
    idx, w = oracle.top2(lg)
    assert idx.tolist() == [[1, 2], [0, 1], [3, 2]]
    assert np.allclose(w.sum(axis=1), 1.0) and np.allclose(w[0], [0.5, 0.5])
    assert np.isclose(w[2, 0], 1.0 / (1.0 + np.exp(-0.5)))


def test_slots_order_pairs_by_rank_token_choice():
    idx = [np.array([[0, 1], [1, 0], [1, 2]]), np.array([[1, 0], [2, 1]])]
    rows, counts = oracle.slots(idx, 3)
    assert counts.tolist() == [[2, 3, 1], [1, 2, 1]]
    assert rows[0].tolist() == [[0, 0], [1, 1], [2, 0]]
    assert rows[1].tolist() == [[3, 2], [1, 4]]   # after rank 0's 3 rows for expert 1, 2 for expert 0, 1 for expert 2


def test_layer_is_the_weighted_sum_of_the_selected_experts():
    rng = np.random.default_rng(0)
    x = [rng.standard_normal((5, 8))]
    lg = [rng.standard_normal((5, 4))]
    w1 = [rng.standard_normal((12, 8)) * 0.3 for _ in range(4)]
    w2 = [rng.standard_normal((8, 6)) * 0.3 for _ in range(4)]
    out = oracle.moe_layer(x, lg, w1, w2)[0]
    idx, w = oracle.top2(lg[0])
    for t in range(5):
        want = sum(w[t, k] * oracle.expert_ffn(x[0][t:t + 1], w1[idx[t, k]], w2[idx[t, k]])[0] for k in range(2))
        assert np.allclose(out[t], want)


def test_work_and_graph_helpers():
    # the layer of the configuration list: 4096 tokens per rank, hidden 4096, ffn 14336, 8 ranks
    assert moe.layer_flops(4096, 4096, 14336) == 2.0 * 4096 * 2 * 4096 * 14336 * 3
    assert moe.dispatch_bytes(4096, 4096, 8) == 4096 * 2 * 4096 * 2 * 7 / 8
    g = moe.measured_graph(4096, 4096, 14336, 8, 8, total_us=2400.0, ep_rank=5)
    ex = analyze_exposure(g)
    assert ex.phase_time_us == 2400.0 and ex.total_comm_us > 0
    ops = [u.op for u in g.uops.values()]
    assert ops.count("comm.all_to_all") == 2 and "compute.mlp" in ops
    assert all(u.ep_rank == 5 for u in g.uops.values() if u.op != "phase.begin" and u.op != "phase.end")
