"""GPU parity for the small-step form of the decode attention: one thread-block cluster per (token,
kv head), the history cut into one range per warp of the cluster, split-K merge inside the launch
(every warp sends its partial to the blocks that own the heads, through the cluster's shared memory;
decode_tma_kernel with CLUSTER).  The host planner chooses it
(pkv_decode_plan.cluster); results must match the CPU checker exactly as the ordinary form does."""
import numpy as np
import pytest

from tests.gpu_util import Case, check_case, from_device, rel_errors, to_device

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _cluster_form_on(monkeypatch):
    """The cluster form is the default for small steps; PKV_DECODE_CLUSTER=0 (read at every planning call)
    switches it off, so make sure the environment does not."""
    monkeypatch.delenv("PKV_DECODE_CLUSTER", raising=False)


def _nb(ctx, bs):
    return sum((c + 1 + bs - 1) // bs for c in ctx) + 16


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("mode", ["host_plan", "fused_append"])
@pytest.mark.parametrize("shape", [
    # q_heads, kv_heads, block_size, contexts (positions of the one new token per sequence)
    (14, 2, 16, [300, 700, 1100, 1500, 1900, 2047, 256, 999]),        # 16 pairs: clusters of 8, up to 32 ranges
    (32, 4, 16, [64, 65, 127, 128, 129, 1023, 1024, 1025] * 4),        # 128 pairs: clusters of 3
    (8, 8, 32, [33, 200, 511]),                                        # one query head per kv head, block 32
    (16, 2, 16, [31, 32, 33, 63, 64, 95, 96, 97, 255, 256, 257]),      # range edges on slab boundaries
    (14, 2, 16, [200 + 37 * i for i in range(40)]),                    # 80 pairs: 5 blocks would fit, clusters of 4
    (14, 2, 16, [150 + 3 * i for i in range(100)]),                    # 200 pairs: clusters of 2
])
def test_cluster_form_matches_checker(pkv, orc, torch_cuda, dtype, mode, shape):
    qh, kvh, bs, ctx = shape
    case = Case(orc, dtype, qh, kvh, 64, bs, _nb(ctx, bs), ctx, [1] * len(ctx), 77, pkv)
    want = case.expected(orc)
    before = pkv.lib().pkv_debug_cluster_launches()
    d = case.run_gpu(pkv, torch_cuda, mode)
    assert d["plan"].plan.cluster >= 2, "the planner was expected to choose the cluster form for this step"
    assert pkv.lib().pkv_debug_cluster_launches() == before + 1, "the launch fell back to the ordinary form"
    check_case(case, pkv, torch_cuda, orc, mode)
    del want


def test_cluster_form_agrees_with_ordinary_form(pkv, orc, torch_cuda):
    """Same step through both forms (the caller may clear pkv_decode_plan.cluster): the outputs agree to
    rounding of the 16-bit result (the keys are grouped differently), both within tolerance of the checker."""
    ctx = [int(x) for x in np.random.default_rng(5).integers(256, 2049, size=40)]
    case = Case(orc, "bf16", 14, 2, 64, 16, _nb(ctx, 16), ctx, [1] * len(ctx), 11, pkv)
    _, _, want = case.expected(orc)
    d = case.upload(torch_cuda)
    pkv.launch_store_kv(d["k"], d["v"], d["slots"], d["kc"], d["vc"], case.N, case.kvh * case.hd)
    args = (d["q"], d["kc"], d["vc"], d["block_tables"], d["table_offset"], d["token_seq"], d["token_pos"])
    plan = pkv.DecodePlan(case.N, case.qh, case.kvh, case.hd).build_host(case.idx.token_pos)
    assert plan.plan.cluster >= 2
    out_c = torch_cuda.zeros_like(d["out"])
    plan.attention(*args, out_c, case.bs, case.scale)
    plan.plan.cluster = 0
    out_o = torch_cuda.zeros_like(d["out"])
    plan.attention(*args, out_o, case.bs, case.scale)
    torch_cuda.cuda.synchronize()
    _, got_c = from_device(torch_cuda, orc, out_c, "bf16")
    _, got_o = from_device(torch_cuda, orc, out_o, "bf16")
    assert np.abs(got_c - got_o).max() <= 2e-2 * np.abs(want).max()
    assert np.abs(got_c - want.reshape(got_c.shape)).max() <= 2e-2 * np.abs(want).max()
    assert pkv.debug_device_flags() == 0


def test_planner_keeps_the_ordinary_form_for_large_or_long_steps(pkv, torch_cuda, monkeypatch):
    """More (token, kv head) pairs than can each have a resident cluster, or histories too long for a
    cluster's warps: the plan says 0 and the ordinary split-K launch runs.  Likewise without the switch."""
    many = pkv.DecodePlan(256, 32, 4, 64).build_host(np.full(256, 1000, dtype=np.int32))
    assert many.plan.cluster == 0
    long_ctx = pkv.DecodePlan(8, 32, 4, 64).build_host(np.full(8, 20000, dtype=np.int32))
    assert long_ctx.plan.cluster == 0
    wide = pkv.DecodePlan(8, 32, 2, 64).build_host(np.full(8, 1000, dtype=np.int32))   # 16 query heads per kv head
    assert wide.plan.cluster == 0
    small = pkv.DecodePlan(8, 32, 4, 64).build_host(np.full(8, 1000, dtype=np.int32))
    assert small.plan.cluster == 8
    monkeypatch.setenv("PKV_DECODE_CLUSTER", "0")
    off = pkv.DecodePlan(8, 32, 4, 64).build_host(np.full(8, 1000, dtype=np.int32))
    assert off.plan.cluster == 0


def test_configuration_2_at_full_size_through_clusters(pkv, orc, torch_cuda, workloads):
    """Configuration 2 (64 sequences, contexts 256..2,048, 14 query / 2 kv heads, bf16): the step the
    cluster form is meant for, with the append inside the launch, at full size."""
    w = workloads.make("cfg2", layers=1)
    ctx = [int(c) for c in w.ctx]
    case = Case(orc, "bf16", w.q_heads, w.kv_heads, w.head_dim, w.block_size, w.num_blocks, ctx, [1] * len(ctx), 1235, pkv)
    before = pkv.lib().pkv_debug_cluster_launches()
    d = case.run_gpu(pkv, torch_cuda, "fused_append")
    assert d["plan"].plan.cluster == 3
    assert pkv.lib().pkv_debug_cluster_launches() == before + 1, "the launch fell back to the ordinary form"
    check_case(case, pkv, torch_cuda, orc, "fused_append")


def test_captured_cluster_launch_replays_over_later_steps(pkv, orc, torch_cuda):
    """A cluster-form launch captured into a CUDA graph reads no plan, only the step's index arrays: replayed
    over later steps of the same token count (every sequence a few keys longer, some across a block
    boundary, the arrays rewritten in place) it must give those steps' results."""
    torch = torch_cuda
    qh, kvh, bs, nb = 14, 2, 16, 1024
    base = [300, 705, 1100, 1513, 1900, 2040, 256, 999, 47, 1290]
    cases = [Case(orc, "bf16", qh, kvh, 64, bs, nb, [c + 9 * s for c in base], [1] * len(base), 5, pkv) for s in range(3)]
    N = cases[0].N
    d = cases[0].upload(torch)
    tab_len = max(c.idx.block_tables.size for c in cases)
    d["block_tables"] = torch.zeros(tab_len, dtype=torch.int32, device="cuda")
    plan = pkv.DecodePlan(N, qh, kvh, 64).build_host(cases[0].idx.token_pos)
    assert plan.plan.cluster >= 2
    args = lambda: (d["q"], d["k"], d["v"], d["slots"], d["kc"], d["vc"], d["block_tables"], d["table_offset"],
                    d["token_seq"], d["token_pos"], d["out"], bs, cases[0].scale)
    i32 = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).cuda()

    def load(case):
        for name in ("kc", "vc", "q", "k", "v"):
            d[name].copy_(to_device(torch, getattr(case, name + "_bits"), "bf16"))
        d["block_tables"][:case.idx.block_tables.size].copy_(i32(case.idx.block_tables))
        for name in ("slots", "token_seq", "token_pos", "table_offset"):
            d[name].copy_(i32(getattr(case.idx, name)))
        d["out"].zero_()

    load(cases[0])
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        plan.append_attention(*args())                    # warm-up outside the capture
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    before = pkv.lib().pkv_debug_cluster_launches()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        plan.append_attention(*args())
    assert pkv.lib().pkv_debug_cluster_launches() == before + 1
    for step, case in enumerate(cases):
        load(case)
        plan.build_host(case.idx.token_pos)               # what a serving loop does every step; the captured launch ignores it
        torch.cuda.synchronize()
        g.replay()
        torch.cuda.synchronize()
        want_kc, want_vc, want = case.expected(orc)
        kcb, _ = from_device(torch, orc, d["kc"], "bf16")
        assert np.array_equal(kcb, want_kc), f"step {step}: K pool differs from the reference append"
        _, got = from_device(torch, orc, d["out"], "bf16")
        e_ref, e_row = rel_errors(got.reshape(N * qh, 64), want.reshape(N * qh, 64))
        assert e_row <= 2e-2, (step, e_ref, e_row)
    assert pkv.debug_device_flags() == 0


@pytest.mark.parametrize("seed", range(12))
def test_cluster_form_on_random_small_steps(pkv, orc, torch_cuda, seed):
    """Seeded random small steps -- 1 to 110 sequences, 1 to 8 query heads per kv head, 1 to 8 kv heads,
    block 16 or 32, histories of 1 to 3,000 keys, with and without the append inside the launch -- through
    whichever form the planner picks (the cluster form for most), against the CPU checker."""
    rng = np.random.default_rng(1000 + seed)
    kvh = int(rng.choice([1, 2, 4, 8]))
    group = int(rng.integers(1, 9))
    bs = int(rng.choice([16, 32]))
    n = int(rng.integers(1, max(2, 220 // kvh // 2)))
    top = int(rng.choice([40, 300, 1200, 3000]))
    ctx = [int(x) for x in rng.integers(0, top, size=n)]
    dtype = "bf16" if seed % 2 == 0 else "f16"
    mode = "fused_append" if seed % 3 else "host_plan"
    case = Case(orc, dtype, group * kvh, kvh, 64, bs, _nb(ctx, bs), ctx, [1] * n, 4000 + seed, pkv)
    check_case(case, pkv, torch_cuda, orc, mode)
