"""GPU parity for the shared-prefix-aware decode plan (pkv_decode_plan_host_shared): sequences whose
tables start with the same blocks have that range read once per group of up to four tokens; the
result must still be the CPU checker's attention for every token, within the tolerance of the KV dtype."""
import numpy as np
import pytest

from tests.gpu_util import Case, check_case, from_device, rel_errors

pytestmark = pytest.mark.gpu


def shared_case(orc, pkv, dtype, qh, kvh, clusters, loners, bs=16, seed=0, hd=64):
    """clusters: [(n_members, shared_blocks, (lo, hi) own context beyond the shared part)]."""
    rng = np.random.default_rng(seed)
    ctx, share, s = [], [], 0
    for n, nsh, (lo, hi) in clusters:
        members = list(range(s, s + n))
        for _ in members:
            ctx.append(nsh * bs + int(rng.integers(lo, hi + 1)))
        share.append((members, nsh))
        s += n
    for lo, hi in loners:
        ctx.append(int(rng.integers(lo, hi + 1)))
    order = rng.permutation(len(ctx))                       # clusters interleaved in the packed order
    ctx = [ctx[i] for i in order]
    inv = np.argsort(order)
    share = [([int(inv[m]) for m in members], nsh) for members, nsh in share]
    nb = sum((c + 1 + bs - 1) // bs for c in ctx) + 64
    return Case(orc, dtype, qh, kvh, hd, bs, nb, ctx, [1] * len(ctx), 900 + seed, pkv, share=share)


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("heads", [(32, 4), (14, 2), (8, 8)])
def test_shared_prefix_plan_matches_checker(pkv, orc, torch_cuda, dtype, heads):
    qh, kvh = heads
    case = shared_case(orc, pkv, dtype, qh, kvh,
                       clusters=[(9, 32, (1, 300)), (4, 4, (0, 40)), (2, 130, (5, 700)), (5, 17, (16, 16)), (3, 40, (1, 3))],
                       loners=[(1, 50), (200, 900), (64, 64), (3000, 3000)], seed=heads[0])
    check_case(case, pkv, torch_cuda, orc, "shared_plan")


def test_shared_units_are_planned_and_agree_with_the_ordinary_plan(pkv, orc, torch_cuda):
    case = shared_case(orc, pkv, "bf16", 32, 4, clusters=[(16, 32, (32, 256)), (7, 64, (1, 100))], loners=[(10, 2000)] * 5, seed=5)
    d_shared = case.run_gpu(pkv, torch_cuda, "shared_plan")
    assert d_shared["plan"].n_shared_units > 0
    _, got_shared = from_device(torch_cuda, orc, d_shared["out"], "bf16")
    d_plain = case.run_gpu(pkv, torch_cuda, "host_plan")
    assert d_plain["plan"].n_shared_units == 0
    _, got_plain = from_device(torch_cuda, orc, d_plain["out"], "bf16")
    e_ref, e_row = rel_errors(got_shared.reshape(-1, 64), got_plain.reshape(-1, 64))
    assert e_ref <= 1e-2 and e_row <= 2e-2          # the same keys grouped differently: bf16 output rounding apart
    assert pkv.debug_device_flags() == 0


def test_without_shared_prefixes_the_plan_is_the_ordinary_one(pkv, orc, torch_cuda):
    case = shared_case(orc, pkv, "bf16", 32, 4, clusters=[], loners=[(100, 3000)] * 24, seed=6)
    d1 = case.run_gpu(pkv, torch_cuda, "shared_plan")
    assert d1["plan"].n_shared_units == 0
    a = d1["out"].view(torch_cuda.int16).cpu().numpy().copy()
    d2 = case.run_gpu(pkv, torch_cuda, "host_plan")
    assert np.array_equal(a, d2["out"].view(torch_cuda.int16).cpu().numpy())


def test_geometries_the_shared_units_do_not_cover_fall_back(pkv, orc, torch_cuda):
    case = shared_case(orc, pkv, "bf16", 8, 2, clusters=[(6, 16, (10, 200))], loners=[(50, 500)], seed=7, hd=128)
    d = case.run_gpu(pkv, torch_cuda, "shared_plan")
    assert d["plan"].n_shared_units == 0
    check_case(case, pkv, torch_cuda, orc, "shared_plan")
    case32 = shared_case(orc, pkv, "f32", 14, 2, clusters=[(6, 16, (10, 200))], loners=[(50, 500)], seed=8)
    with pytest.raises(pkv.PkvError):               # fp32 K/V cannot take a plan with shared units: said, not run
        case32.run_gpu(pkv, torch_cuda, "shared_plan")


def test_prefill_chunks_in_the_same_step_are_left_alone(pkv, orc, torch_cuda):
    """A mixed step: decode tokens of a shared-prefix cluster plus a sequence that brings a 40-token chunk."""
    rng = np.random.default_rng(11)
    bs, nsh = 16, 24
    ctx = [nsh * bs + int(rng.integers(1, 200)) for _ in range(6)] + [nsh * bs + 7, 333]
    new = [1] * 6 + [40, 1]
    nb = sum((c + n + bs - 1) // bs for c, n in zip(ctx, new)) + 8
    case = Case(orc, "bf16", 14, 2, 64, bs, nb, ctx, new, 77, pkv, share=[(list(range(7)), nsh)])
    d = case.run_gpu(pkv, torch_cuda, "shared_plan")
    assert d["plan"].n_shared_units > 0
    check_case(case, pkv, torch_cuda, orc, "shared_plan")


def test_cfg5_at_full_size(pkv, orc, torch_cuda, workloads):
    w = workloads.make("cfg5")
    case = Case.__new__(Case)
    S = w.n_seqs
    share = [(list(range(S)), w.shared_prefix_blocks)]
    case = Case(orc, "bf16", w.q_heads, w.kv_heads, w.head_dim, w.block_size, w.num_blocks,
                [int(c) for c in w.ctx], [1] * S, w.seed, pkv, share=share)
    d = case.run_gpu(pkv, torch_cuda, "shared_plan")
    assert d["plan"].n_shared_units >= (S // 4) * 1
    check_case(case, pkv, torch_cuda, orc, "shared_plan")


def test_default_threshold_keeps_small_prefixes_on_the_ordinary_plan(pkv, orc, torch_cuda):
    """A 512-key prefix shared by 16 sequences saves 6 MB of reads per layer: not worth a launch."""
    case = shared_case(orc, pkv, "bf16", 32, 4, clusters=[(16, 32, (32, 256))], loners=[], seed=9)
    plan = pkv.DecodePlan(case.N, 32, 4, 64)
    plan.build_host_shared(case.idx, 16)
    assert plan.n_shared_units == 0
    plan.build_host_shared(case.idx, 16, min_saved_bytes=0)
    assert plan.n_shared_units > 0
