"""Expert-parallel MoE layer against the float64 oracle, ranks emulated on one GPU: routing
(selected experts, slots) must match exactly, outputs within the bf16 tolerance."""
import numpy as np
import pytest
import torch

from edmir_b200 import moe, symm
from oracle import moe as oracle
from oracle import tp_linear as tpo

pytestmark = pytest.mark.gpu
BF16_TOL = 1e-2


def _rand(shape, scale, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g, dtype=torch.float32) * scale).to(torch.bfloat16)


@pytest.mark.parametrize("world,T,H,F,E", [(1, 256, 256, 512, 8), (2, 256, 256, 512, 8), (4, 384, 512, 768, 8),
                                           (2, 1000, 256, 264, 4), (4, 64, 128, 256, 16)])
def test_moe_layer_matches_oracle(cuda_clean, world, T, H, F, E):
    e_local = E // world
    g = symm.EmulatedGroup(world, moe.window_bytes(T, H, E, world), 1 << 20)
    try:
        w1_e = [_rand((2 * F, H), 0.05, 100 + e) for e in range(E)]
        w2_e = [_rand((H, F), 0.05, 200 + e) for e in range(E)]
        w1 = [torch.cat(w1_e[r * e_local:(r + 1) * e_local]).cuda() for r in range(world)]
        w2 = [torch.cat(w2_e[r * e_local:(r + 1) * e_local]).cuda() for r in range(world)]
        ws = [moe.MoEWorkspace(T, H, F, E, world) for _ in range(world)]
        outs = [torch.empty(T, H, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
        for call in range(3):  # new tokens every call; both halves of the window get used
            x = [_rand((T, H), 1.0, 300 + 10 * call + r) for r in range(world)]
            lg = [oracle.router_logits(T, E, 400 + 10 * call + r) for r in range(world)]
            torch.cuda.synchronize()
            g.poison()
            for o in outs:
                o.fill_(float("nan"))
            moe.moe_forward_emulated(g, ws, [t.cuda() for t in x], [torch.from_numpy(l).cuda() for l in lg], w1, w2, outs)
            torch.cuda.synchronize()
            idx_want = [oracle.top2(l)[0] for l in lg]
            rows_want, counts = oracle.slots(idx_want, E)
            base = np.cumsum(counts, axis=0) - counts
            for r in range(world):
                idx = ws[r].topk_idx.cpu().numpy()
                assert np.array_equal(idx, idx_want[r]), (call, r)
                # slot within (rank, expert) + rows of lower ranks = the row in the expert's buffer
                row = ws[r].slot.cpu().numpy() + base[r][idx]
                assert np.array_equal(row, rows_want[r]), (call, r)
                wt = ws[r].topk_weight.cpu().numpy()
                assert np.allclose(wt, oracle.top2(lg[r])[1], rtol=1e-4, atol=1e-6)
            want = oracle.moe_layer([t.float().numpy() for t in x], lg, [w.float().numpy() for w in w1_e],
                                    [w.float().numpy() for w in w2_e])
            for r in range(world):
                assert tpo.rel_l2(outs[r].float().cpu().numpy(), want[r]) <= BF16_TOL, (call, r)
    finally:
        torch.cuda.synchronize()
        g.close()


def test_moe_skewed_router_sends_most_rows_to_one_expert(cuda_clean):
    # a strongly biased router: one expert receives nearly every token (its buffer is sized for all of them)
    world, T, H, F, E = 2, 512, 256, 256, 4
    g = symm.EmulatedGroup(world, moe.window_bytes(T, H, E, world), 1 << 20)
    try:
        w1_e = [_rand((2 * F, H), 0.05, 500 + e) for e in range(E)]
        w2_e = [_rand((H, F), 0.05, 600 + e) for e in range(E)]
        w1 = [torch.cat(w1_e[r * 2:(r + 1) * 2]).cuda() for r in range(world)]
        w2 = [torch.cat(w2_e[r * 2:(r + 1) * 2]).cuda() for r in range(world)]
        ws = [moe.MoEWorkspace(T, H, F, E, world) for _ in range(world)]
        x = [_rand((T, H), 1.0, 700 + r) for r in range(world)]
        lg = [oracle.router_logits(T, E, 800 + r) for r in range(world)]
        for l in lg:
            l[:, 3] += 6.0
        outs = [torch.zeros(T, H, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
        moe.moe_forward_emulated(g, ws, [t.cuda() for t in x], [torch.from_numpy(l).cuda() for l in lg], w1, w2, outs)
        torch.cuda.synchronize()
        assert (ws[0].topk_idx[:, 0] == 3).float().mean().item() > 0.95
        want = oracle.moe_layer([t.float().numpy() for t in x], lg, [w.float().numpy() for w in w1_e],
                                [w.float().numpy() for w in w2_e])
        for r in range(world):
            assert tpo.rel_l2(outs[r].float().cpu().numpy(), want[r]) <= BF16_TOL, r
    finally:
        torch.cuda.synchronize()
        g.close()


def test_moe_shape_checks(cuda_clean):
    with pytest.raises(ValueError):
        moe.window_bytes(64, 128, 6, 4)          # experts not divisible by ranks
    g = symm.EmulatedGroup(2, 1 << 20, 1 << 20)  # window far too small
    try:
        T, H, F, E = 256, 256, 256, 4
        ws = [moe.MoEWorkspace(T, H, F, E, 2) for _ in range(2)]
        x = [torch.zeros(T, H, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
        lg = [torch.zeros(T, E, device="cuda") for _ in range(2)]
        w1 = [torch.zeros(2 * 2 * F, H, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
        w2 = [torch.zeros(2 * H, F, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
        from edmir_b200 import _lib
        with pytest.raises(_lib.EdmError) as err:
            moe.moe_forward_emulated(g, ws, x, lg, w1, w2, [torch.empty_like(t) for t in x])
        assert err.value.code == _lib.EDM_ERR_CAPACITY
    finally:
        g.close()
