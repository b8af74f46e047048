"""Parity of the fused tensor-parallel launches against the CPU oracle, with the ranks of a
group emulated inside ONE cooperative launch on a single GPU (each rank gets 1/W of the SMs,
its own symmetric window and flags).  The protocol -- tile pushes into the owner's window,
flag words, epoch/parity reuse across calls, chunked shard pushes -- is the one the multi-GPU
path runs; only the peer pointers differ.

Repeated calls draw new inputs every time and the windows, gather buffers and outputs are filled
with NaN before each launch: a slot read before its sender wrote it, or a flag left over from the
previous call, would show in the result instead of reproducing the previous call's numbers.
"""
import numpy as np
import pytest
import torch

from edmir_b200 import _lib, linear, symm
from edmir_b200.schedule import Schedule
from oracle import tp_linear as oracle

pytestmark = pytest.mark.gpu

BF16_TOL = 1e-2
FP32_TOL = 1e-5


def _rand(shape, scale, dtype, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g, dtype=torch.float32) * scale).to(dtype)


@pytest.fixture()
def group_factory():
    made = []

    def make(world, window=96 << 20, heap=64 << 20):
        g = symm.EmulatedGroup(world, window, heap)
        made.append(g)
        return g

    yield make
    torch.cuda.synchronize()
    for g in made:
        g.close()


def _np(t):
    return t.float().cpu().numpy()


def _poison(group, outs):
    """NaN everywhere a launch is about to write: windows / gather buffers of every rank and the
    outputs (all launches of the previous call have finished)."""
    torch.cuda.synchronize()
    group.poison()
    for o in outs:
        o.fill_(float("nan"))
    torch.cuda.synchronize()


@pytest.mark.parametrize("world,M,N,K", [(2, 512, 512, 256), (2, 256, 1032, 72), (4, 2048, 1024, 512),
                                         (4, 512, 264, 1000)])
def test_gemm_reduce_scatter(cuda_clean, group_factory, world, M, N, K):
    g = group_factory(world)
    outs = [torch.zeros(M // world, N, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    for call in range(3):  # repeated calls walk both window parities and advance the epoch
        a = [_rand((M, K), 1.0, torch.bfloat16, 100 + 10 * call + r) for r in range(world)]
        b = [_rand((N, K), 0.02, torch.bfloat16, 200 + 10 * call + r) for r in range(world)]
        want = oracle.gemm_reduce_scatter([_np(x) for x in a], [_np(x) for x in b])
        _poison(g, outs)
        g.run("gemm_rs", [x.cuda() for x in a], [x.cuda() for x in b], outs)
        torch.cuda.synchronize()
        for r in range(world):
            assert oracle.rel_l2(_np(outs[r]), want[r]) <= BF16_TOL, (call, r)


@pytest.mark.parametrize("world,M,N,K", [(2, 256, 1024, 512), (2, 1, 4096, 1792), (4, 1000, 1032, 264),
                                         (4, 16, 4096, 3584), (3, 384, 520, 128)])
def test_gemm_all_reduce_bf16(cuda_clean, group_factory, world, M, N, K):
    g = group_factory(world)
    outs = [ctx.empty((M, N), torch.bfloat16) for ctx in g.ranks]
    for call in range(3):
        a = [_rand((M, K), 1.0, torch.bfloat16, 300 + 10 * call + r) for r in range(world)]
        b = [_rand((N, K), 0.02, torch.bfloat16, 400 + 10 * call + r) for r in range(world)]
        want = oracle.gemm_all_reduce([_np(x) for x in a], [_np(x) for x in b])[0]
        _poison(g, outs)
        g.run("gemm_ar", [x.cuda() for x in a], [x.cuda() for x in b], outs)
        torch.cuda.synchronize()
        for r in range(world):
            assert oracle.rel_l2(_np(outs[r]), want) <= BF16_TOL, (call, r)
        for r in range(1, world):  # every rank must hold the same bits
            assert torch.equal(outs[r], outs[0])


def test_config1_all_reduce_fp32(cuda_clean, group_factory):
    # world 2, per-rank A[256,512] and B[512,1024] ~N(0,1) from seed 0, output = sum_r A_r @ B_r
    g = group_factory(2)
    a_sh, b_sh = oracle.config1_inputs()
    want = oracle.config1_output(a_sh, b_sh)
    a_d = [torch.from_numpy(a).cuda() for a in a_sh]
    b_d = [torch.from_numpy(np.ascontiguousarray(b.T)).cuda() for b in b_sh]
    outs = [ctx.empty((256, 1024), torch.float32) for ctx in g.ranks]
    for call in range(2):
        _poison(g, outs)
        g.run("gemm_ar", a_d, b_d, outs)
        torch.cuda.synchronize()
        for r in range(2):
            assert oracle.rel_l2(outs[r].cpu().numpy(), want) <= FP32_TOL, (call, r)
        assert torch.equal(outs[0], outs[1])


ONE_SHOT = Schedule(one_shot=True)


@pytest.mark.parametrize("world,M,N,K", [(2, 1, 4096, 1792), (2, 64, 4096, 1792), (4, 16, 4096, 3584),
                                         (3, 128, 520, 264), (4, 300, 1032, 512)])
def test_one_shot_all_reduce_bf16(cuda_clean, group_factory, world, M, N, K):
    # plain GEMM into the window, then every rank adds up all partials itself: outputs need not be
    # symmetric, every rank holds the same bits, and those are exactly the fp32 sum in rank order
    # of the ranks' bf16 GEMM results
    g = group_factory(world)
    outs = [torch.empty(M, N, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    for call in range(4):  # both window banks twice
        a = [_rand((M, K), 1.0, torch.bfloat16, 1300 + 10 * call + r) for r in range(world)]
        b = [_rand((N, K), 0.02, torch.bfloat16, 1400 + 10 * call + r) for r in range(world)]
        want = oracle.gemm_all_reduce([_np(x) for x in a], [_np(x) for x in b])[0]
        a_d, b_d = [x.cuda() for x in a], [x.cuda() for x in b]
        _poison(g, outs)
        g.run("gemm_ar", a_d, b_d, outs, schedule=ONE_SHOT)
        torch.cuda.synchronize()
        acc = torch.zeros(M, N, dtype=torch.float32, device="cuda")
        for r in range(world):
            acc += linear.gemm(a_d[r], b_d[r]).float()
        for r in range(world):
            assert oracle.rel_l2(_np(outs[r]), want) <= BF16_TOL, (call, r)
            assert torch.equal(outs[r], acc.to(torch.bfloat16)), (call, r)
    assert linear.status()[0] == 0


def test_one_shot_all_reduce_fp32_and_strided_output(cuda_clean, group_factory):
    g = group_factory(2)
    a_sh, b_sh = oracle.config1_inputs()
    want = oracle.config1_output(a_sh, b_sh)
    a_d = [torch.from_numpy(a).cuda() for a in a_sh]
    b_d = [torch.from_numpy(np.ascontiguousarray(b.T)).cuda() for b in b_sh]
    wide = [torch.zeros(256, 1024 + 64, dtype=torch.float32, device="cuda") for _ in range(2)]
    outs = [w[:, :1024] for w in wide]  # row stride larger than the width
    for call in range(2):
        g.poison()
        for w in wide:
            w.fill_(7.0)
        g.run("gemm_ar", a_d, b_d, outs, schedule=ONE_SHOT)
        torch.cuda.synchronize()
        for r in range(2):
            assert oracle.rel_l2(outs[r].cpu().numpy(), want) <= FP32_TOL, (call, r)
            assert torch.all(wide[r][:, 1024:] == 7.0)  # nothing written past the row's end
        assert torch.equal(outs[0], outs[1])


def test_one_shot_and_fused_all_reduce_alternate_on_one_context(cuda_clean, group_factory):
    # both kinds share the window banks and flag words of the context, call after call
    world, N, K = 4, 2048, 512
    g = group_factory(world)
    for step, (M, sched) in enumerate([(16, ONE_SHOT), (256, None), (16, ONE_SHOT), (16, ONE_SHOT), (48, None),
                                       (128, ONE_SHOT)]):
        a = [_rand((M, K), 1.0, torch.bfloat16, 1500 + 10 * step + r) for r in range(world)]
        b = [_rand((N, K), 0.02, torch.bfloat16, 1600 + 10 * step + r) for r in range(world)]
        want = oracle.gemm_all_reduce([_np(x) for x in a], [_np(x) for x in b])[0]
        outs = [ctx.empty((M, N), torch.bfloat16) for ctx in g.ranks]
        _poison(g, outs)
        g.run("gemm_ar", [x.cuda() for x in a], [x.cuda() for x in b], outs, schedule=sched)
        torch.cuda.synchronize()
        for r in range(world):
            assert oracle.rel_l2(_np(outs[r]), want) <= BF16_TOL, (step, r)
        for ctx in g.ranks:
            ctx.reset_heap()


def test_one_shot_rejects_what_it_cannot_run(cuda_clean):
    g = symm.EmulatedGroup(2, 1 << 20, 1 << 20)
    try:
        a = [torch.zeros(64, 64, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
        b = [torch.zeros(8192, 64, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
        outs = [torch.zeros(64, 8192, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
        with pytest.raises(_lib.EdmError) as err:   # the partial (1 MiB) does not fit half of the window
            g.run("gemm_ar", a, b, outs, schedule=ONE_SHOT)
        assert err.value.code == _lib.EDM_ERR_CAPACITY
        b4 = [torch.zeros(36, 64, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
        o4 = [torch.zeros(64, 36, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
        with pytest.raises(ValueError):             # rows are not whole 16-byte vectors
            g.run("gemm_ar", a, b4, o4, schedule=ONE_SHOT)
        with pytest.raises(ValueError):
            g.ranks[0]._call("gemm_rs", a[0], b[0], torch.zeros(32, 8192, dtype=torch.bfloat16, device="cuda"), ONE_SHOT)
    finally:
        g.close()


def test_one_shot_missing_peer_times_out_and_context_survives(group_factory):
    # rank 0 of a 2-rank group runs alone: its peer's flag never comes, the bounded wait gives up with
    # its own status code and nothing is added up
    assert torch.cuda.is_available()
    linear.clear_status()
    g = group_factory(2)
    a = _rand((16, 256), 1.0, torch.bfloat16, 41).cuda()
    b = _rand((512, 256), 0.02, torch.bfloat16, 42).cuda()
    out = torch.full((16, 512), 3.0, dtype=torch.bfloat16, device="cuda")
    linear.set_timeout_ms(50)
    try:
        g.ranks[0].gemm_ar(a, b, out, schedule=ONE_SHOT)
        st = linear.status()
    finally:
        linear.set_timeout_ms(2000)
        linear.clear_status()
    assert st[0] == 11, st[:8]
    assert torch.all(out == 3.0)
    got = linear.gemm(a, b)
    assert oracle.rel_l2(_np(got), oracle.gemm(_np(a), _np(b))) <= BF16_TOL
    assert linear.status()[0] == 0


AG_SCHEDULES = {
    "sm": dict(transport="sm"),                                    # push warps inside every GEMM CTA
    "ce": dict(transport="ce"),                                    # copy engines only
    "striped": dict(transport="cs"),                               # copy engines, a stream per chunk
    "pushers": dict(transport="sm", pusher_ctas=4),                # CTAs that only push
    "hybrid": dict(transport="hybrid", pusher_ctas=2, ce_peers=1, side_streams=1),  # farthest peer by copy engine
}


@pytest.mark.parametrize("how", sorted(AG_SCHEDULES))
@pytest.mark.parametrize("world,M,N,K,chunks", [(2, 512, 512, 256, 2), (4, 2048, 768, 512, 4), (4, 256, 768, 512, 1),
                                                (2, 1024, 264, 1000, 3), (4, 4096, 512, 1024, 8),
                                                (2, 2048, 1280, 2048, 2),   # 40 tiles on 37 pairs: tail cut in 8
                                                (2, 1024, 512, 4096, 2),    # 8 tiles on 37 pairs: every tile cut in 4
                                                (3, 384, 520, 136, 2)])     # shards shorter than a row block, odd world
def test_all_gather_gemm(cuda_clean, group_factory, world, M, N, K, chunks, how):
    g = group_factory(world)
    sched = Schedule(chunks=chunks, **AG_SCHEDULES[how])
    outs = [torch.zeros(M, N, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    for call in range(3):
        x = [_rand((M // world, K), 1.0, torch.bfloat16, 500 + 10 * call + r) for r in range(world)]
        w = [_rand((N, K), 0.02, torch.bfloat16, 600 + 10 * call + r) for r in range(world)]
        want = oracle.all_gather_gemm([_np(t) for t in x], [_np(t) for t in w])
        _poison(g, outs)
        g.run("ag_gemm", [t.cuda() for t in x], [t.cuda() for t in w], outs, schedule=sched)
        torch.cuda.synchronize()
        for r in range(world):
            assert oracle.rel_l2(_np(outs[r]), want[r]) <= BF16_TOL, (call, r)


def test_all_gather_gemm_strided_shard_with_pushers(cuda_clean, group_factory):
    # the shard is a column slice of a wider tensor: the pusher CTAs copy it row by row
    world, M, N, K = 2, 512, 256, 384
    g = group_factory(world)
    wide = [_rand((M // world, K + 128), 1.0, torch.bfloat16, 900 + r).cuda() for r in range(world)]
    x = [t[:, 64:64 + K] for t in wide]
    w = [_rand((N, K), 0.02, torch.bfloat16, 910 + r) for r in range(world)]
    want = oracle.all_gather_gemm([_np(t) for t in x], [_np(t) for t in w])
    outs = [torch.zeros(M, N, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    _poison(g, outs)
    g.run("ag_gemm", x, [t.cuda() for t in w], outs, schedule=Schedule(chunks=2, transport="sm", pusher_ctas=6))
    torch.cuda.synchronize()
    for r in range(world):
        assert oracle.rel_l2(_np(outs[r]), want[r]) <= BF16_TOL, r


def test_super_tile_raster_gives_the_same_bits(cuda_clean, group_factory):
    # the tile walk only changes the order of the tiles, never their values
    world, M, N, K = 2, 2048, 1536, 512
    g = group_factory(world)
    x = [_rand((M // world, K), 1.0, torch.bfloat16, 920 + r).cuda() for r in range(world)]
    w = [_rand((N, K), 0.02, torch.bfloat16, 930 + r).cuda() for r in range(world)]
    base = [torch.zeros(M, N, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    g.run("ag_gemm", x, w, base, schedule=Schedule(transport="sm", pusher_ctas=2))
    for rows, cols in ((2, 3), (4, 2), (3, 1)):
        outs = [torch.zeros(M, N, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
        _poison(g, outs)
        g.run("ag_gemm", x, w, outs, schedule=Schedule(transport="sm", pusher_ctas=2, band_rows=rows, band_cols=cols))
        torch.cuda.synchronize()
        for r in range(world):
            assert torch.equal(outs[r], base[r]), (rows, cols, r)


def test_pusher_count_is_checked(cuda_clean, group_factory):
    g = group_factory(2)
    x = [torch.zeros(128, 64, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    w = [torch.zeros(256, 64, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    outs = [torch.zeros(256, 256, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    with pytest.raises(ValueError):  # no CTA would be left for the tiles
        g.run("ag_gemm", x, w, outs, schedule=Schedule(transport="sm", pusher_ctas=4096))
    with pytest.raises(ValueError):  # more copy-engine peers than peers
        g.run("ag_gemm", x, w, outs, schedule=Schedule(transport="hybrid", pusher_ctas=2, ce_peers=2))


# ---------------------------------------------------------------- full-size cases, bit-exact
# One-hot activations make every product a selection of weight rows, exact in bf16, so the
# benchmark-sized launches can be checked bit for bit without a slow float64 GEMM: the fused
# reduction must equal the fp32 sum of the W selected rows in rank order, rounded once.
def _one_hot(rows, K, seed):
    gen = torch.Generator(device="cpu").manual_seed(seed)
    pick = torch.randint(0, K, (rows,), generator=gen)
    a = torch.zeros(rows, K, dtype=torch.bfloat16)
    a[torch.arange(rows), pick] = 1.0
    return a.cuda(), pick.cuda()


def _selected_sum(b_list, picks):
    total = None
    for b, pick in zip(b_list, picks):  # rank order, fp32, like the reducer
        part = b[:, pick].t().float()
        total = part if total is None else total + part
    return total.to(torch.bfloat16)


# per-rank extents of the benchmark configurations (world <= 4: what one GPU can emulate)
FULL_ROW_PARALLEL = [
    ("gemm_rs", 4, 8192, 8192, 1024),    # 70B o_proj
    ("gemm_rs", 2, 8192, 8192, 3584),    # 70B down_proj
    ("gemm_ar", 4, 8192, 4096, 3584),    # 8B down_proj + all-reduce at TP=4
    ("gemm_ar", 2, 1024, 4096, 7168),
    ("gemm_ar", 4, 128, 4096, 3584),
    ("gemm_ar", 2, 16, 4096, 7168),
    ("gemm_ar", 4, 1, 4096, 3584),
]


@pytest.mark.parametrize("op,world,M,N,K", FULL_ROW_PARALLEL)
def test_full_size_row_parallel_one_hot(cuda_clean, op, world, M, N, K):
    g = symm.EmulatedGroup(world, 2 * (M * N * 2 + (1 << 20)), world and (M * N * 2 + (1 << 20)))
    try:
        a, picks = zip(*[_one_hot(M, K, 40 + r) for r in range(world)])
        b = [_rand((N, K), 0.02, torch.bfloat16, 50 + r).cuda() for r in range(world)]
        want = _selected_sum(b, picks)
        if op == "gemm_rs":
            outs = [torch.empty(M // world, N, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
        else:
            outs = [ctx.empty((M, N), torch.bfloat16) for ctx in g.ranks]
        for call in range(2):
            _poison(g, outs)
            g.run(op, list(a), b, outs)
            torch.cuda.synchronize()
            for r in range(world):
                ref = want[r * (M // world):(r + 1) * (M // world)] if op == "gemm_rs" else want
                assert torch.equal(outs[r], ref), (call, r)
    finally:
        torch.cuda.synchronize()
        g.close()


FULL_ALL_GATHER = [
    (4, 8192, 1280, 8192, dict(transport="sm", pusher_ctas=8, chunks=4)),   # 70B qkv
    (4, 8192, 1280, 8192, dict(transport="ce", chunks=2)),
    (2, 8192, 7168, 8192, dict(transport="hybrid", pusher_ctas=4, ce_peers=1, chunks=2)),  # 70B gate_up
    (4, 8192, 7168, 4096, dict(transport="sm", pusher_ctas=4, chunks=1)),   # 8B gate_up at TP=4
]


@pytest.mark.parametrize("world,M,N,K,how", FULL_ALL_GATHER)
def test_full_size_all_gather_one_hot(cuda_clean, world, M, N, K, how):
    g = symm.EmulatedGroup(world, 2 * (M * K * 2 + (1 << 20)), 1 << 20)
    try:
        x, picks = zip(*[_one_hot(M // world, K, 60 + r) for r in range(world)])
        pick = torch.cat(picks)
        w = [_rand((N, K), 0.02, torch.bfloat16, 70 + r).cuda() for r in range(world)]
        outs = [torch.empty(M, N, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
        for call in range(2):
            _poison(g, outs)
            g.run("ag_gemm", list(x), w, outs, schedule=Schedule(**how))
            torch.cuda.synchronize()
            for r in range(world):
                assert torch.equal(outs[r], w[r][:, pick].t()), (call, r)
    finally:
        torch.cuda.synchronize()
        g.close()


def test_mixed_ops_share_one_context(cuda_clean, group_factory):
    # different ops and shapes back to back on the same windows and flag words
    world = 2
    g = group_factory(world)
    for step, (op, M, N, K) in enumerate([("gemm_rs", 512, 512, 128), ("ag_gemm", 512, 256, 256),
                                          ("gemm_ar", 130, 520, 72), ("gemm_rs", 256, 1024, 64),
                                          ("ag_gemm", 256, 512, 64), ("gemm_ar", 512, 512, 128)]):
        if op == "ag_gemm":
            a = [_rand((M // world, K), 1.0, torch.bfloat16, 700 + 10 * step + r) for r in range(world)]
        else:
            a = [_rand((M, K), 1.0, torch.bfloat16, 700 + 10 * step + r) for r in range(world)]
        b = [_rand((N, K), 0.02, torch.bfloat16, 800 + 10 * step + r) for r in range(world)]
        fn = {"gemm_rs": oracle.gemm_reduce_scatter, "gemm_ar": oracle.gemm_all_reduce,
              "ag_gemm": oracle.all_gather_gemm}[op]
        want = fn([_np(t) for t in a], [_np(t) for t in b])
        if op == "gemm_ar":
            outs = [ctx.empty((M, N), torch.bfloat16) for ctx in g.ranks]
        elif op == "gemm_rs":
            outs = [torch.zeros(M // world, N, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
        else:
            outs = [torch.zeros(M, N, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
        g.run(op, [t.cuda() for t in a], [t.cuda() for t in b], outs)
        torch.cuda.synchronize()
        for r in range(world):
            assert oracle.rel_l2(_np(outs[r]), want[r]) <= BF16_TOL, (step, op, r)


def test_one_hot_reduce_scatter_is_bit_exact(cuda_clean, group_factory):
    # one-hot rows on rank 0 and zeros elsewhere: the reduced rows must equal rows of B_0 exactly
    world, M, N, K = 2, 1024, 512, 256
    g = group_factory(world)
    gen = torch.Generator(device="cpu").manual_seed(21)
    pick = torch.randint(0, K, (M,), generator=gen)
    a0 = torch.zeros(M, K, dtype=torch.bfloat16)
    a0[torch.arange(M), pick] = 1.0
    a = [a0.cuda(), torch.zeros(M, K, dtype=torch.bfloat16, device="cuda")]
    b = [_rand((N, K), 0.02, torch.bfloat16, 22 + r).cuda() for r in range(world)]
    outs = [torch.zeros(M // world, N, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    g.run("gemm_rs", a, b, outs)
    torch.cuda.synchronize()
    full = b[0][:, pick.cuda()].t().contiguous()
    for r in range(world):
        assert torch.equal(outs[r], full[r * (M // world):(r + 1) * (M // world)])


def test_all_reduce_output_must_be_symmetric(cuda_clean, group_factory):
    g = group_factory(2)
    a = [torch.zeros(128, 64, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    b = [torch.zeros(256, 64, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    outs = [torch.zeros(128, 256, dtype=torch.bfloat16, device="cuda") for _ in range(2)]  # not from ctx.empty
    with pytest.raises(_lib.EdmError) as err:
        g.run("gemm_ar", a, b, outs)
    assert err.value.code == _lib.EDM_ERR_NOT_SYMMETRIC


def test_window_capacity_is_checked(cuda_clean):
    g = symm.EmulatedGroup(2, 1 << 20, 1 << 20)
    try:
        a = [torch.zeros(1024, 64, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
        b = [torch.zeros(1024, 64, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
        outs = [torch.zeros(512, 1024, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
        with pytest.raises(_lib.EdmError) as err:
            g.run("gemm_rs", a, b, outs)
        assert err.value.code == _lib.EDM_ERR_CAPACITY
    finally:
        g.close()


def test_missing_peer_times_out_and_context_survives(group_factory):
    # failure detection without faulting the GPU: rank 0 of a 2-rank group is launched alone, so
    # the partial tiles it waits for never arrive.  The bounded wait must expire, the status word
    # must say which wait it was, and the device must stay usable.
    assert torch.cuda.is_available()
    linear.clear_status()
    g = group_factory(2)
    M, N, K = 256, 256, 64
    a = _rand((M, K), 1.0, torch.bfloat16, 31).cuda()
    b = _rand((N, K), 0.02, torch.bfloat16, 32).cuda()
    out = torch.zeros(M // 2, N, dtype=torch.bfloat16, device="cuda")
    linear.set_timeout_ms(50)
    try:
        g.ranks[0].gemm_rs(a, b, out)   # its peer never runs
        st = linear.status()
    finally:
        linear.set_timeout_ms(2000)
        linear.clear_status()
    assert st[0] == 5, st[:8]           # a peer's partial tile never arrived
    # the context is intact: a plain GEMM afterwards is correct
    got = linear.gemm(a, b)
    assert oracle.rel_l2(_np(got), oracle.gemm(_np(a), _np(b))) <= BF16_TOL
    assert linear.status()[0] == 0


def test_missing_shard_stops_every_role_and_context_survives(group_factory):
    # the same for all-gather + GEMM with long K loops: rank 0 waits for a shard nobody pushes.  When
    # the wait runs out every role must stop issuing loads, MMAs and copies (not run through its
    # remaining tiles unthrottled), so the launch ends with only a pipeline's worth in flight.
    assert torch.cuda.is_available()
    linear.clear_status()
    g = group_factory(2)
    M, N, K = 1024, 1024, 2048
    x = _rand((M // 2, K), 1.0, torch.bfloat16, 33).cuda()
    w = _rand((N, K), 0.02, torch.bfloat16, 34).cuda()
    out = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
    linear.set_timeout_ms(50)
    try:
        g.ranks[0].ag_gemm(x, w, out, schedule=Schedule(transport="sm", pusher_ctas=4, chunks=2))  # its peer never runs
        st = linear.status()
    finally:
        linear.set_timeout_ms(2000)
        linear.clear_status()
    # the role that started waiting first reports: the producer for the shard's chunk flag (7), or
    # the MMA / epilogue warps that were already waiting for what the producer would have loaded
    assert st[0] in (1, 3, 7), st[:8]
    assert _lib.load().edm_status_check() == _lib.EDM_OK   # re-armed
    # rows of the own shard were finished before the wait: they are correct; the device works on
    want = oracle.gemm(_np(x), _np(w))
    assert oracle.rel_l2(_np(out[:M // 2]), want) <= BF16_TOL
    got = linear.gemm(x, w)
    assert oracle.rel_l2(_np(got), want) <= BF16_TOL
    assert linear.status()[0] == 0
