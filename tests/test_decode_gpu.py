"""GPU parity: K/V append + paged decode attention through the C ABI against the CPU
checker.  Cache contents must match bit for bit; attention within 1e-5 (fp32 KV) or
2e-2 (bf16 / f16 KV, inputs cast the reference's way) max relative error.

Each case is aimed at a plausible wrong kernel that naive tests would pass (slot taken
from the position instead of the table, head % group instead of head / group, off-by-one
on pos, reading the whole last block, position taken from the index in the step, wrong
table_offset with several sequences per step)."""
import os

import numpy as np
import pytest

from tests.gpu_util import Case, TOL, check_case, from_device, rel_errors, to_device

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
MODES = ["direct", "split", "host_plan", "device_plan"]


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16"])
def test_cfg1_qwen_layer(pkv, orc, torch_cuda, workloads, dtype, mode):
    """Configuration 1: 14 query / 2 kv heads, head_dim 64, 8 sequences with contexts
    U[64,512], block 16 in a 4,096-block shuffled pool, one appended token per sequence."""
    w = workloads.make("cfg1")
    case = Case(orc, dtype, w.q_heads, w.kv_heads, w.head_dim, w.block_size, w.num_blocks,
                [int(c) for c in w.ctx], [1] * w.n_seqs, seed=w.seed, pkv=pkv)
    check_case(case, pkv, torch_cuda, orc, mode)


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_every_position_across_three_blocks(pkv, orc, torch_cuda, dtype):
    """pos = 0 .. 3*bs: first token, every partial last-block length, exact block boundaries."""
    bs = 16
    ctx = list(range(0, 3 * bs + 1))
    case = Case(orc, dtype, 14, 2, 64, bs, 256, ctx, [1] * len(ctx), seed=5, pkv=pkv)
    for mode in ("direct", "split"):
        check_case(case, pkv, torch_cuda, orc, mode)


@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16"])
def test_mixed_step_chunks_and_decodes_share_tables(pkv, orc, torch_cuda, dtype):
    """Prefill chunks that start mid-block next to decode tokens: several tokens per sequence
    (token_seq / table_offset indirection) and positions that are not the index in the step;
    chunk tokens attend K/V appended by earlier tokens of the same step."""
    ctx = [33, 5, 16, 0, 100, 47]
    new = [1, 9, 1, 20, 37, 1]
    case = Case(orc, dtype, 32, 4, 64, 16, 64, ctx, new, seed=6, pkv=pkv)
    for mode in MODES:
        check_case(case, pkv, torch_cuda, orc, mode)


GEOMETRIES = [
    # q_heads, kv_heads, head_dim, block_size
    (14, 2, 64, 16),    # Qwen2.5-0.5B, group 7
    (32, 4, 64, 16),    # TinyLlama, group 8
    (8, 8, 64, 16),     # multi-head attention, group 1
    (32, 2, 64, 16),    # group 16: the widest the tensor-core path takes
    (40, 2, 64, 8),     # group 20: falls to the SIMT path, three head batches
    (8, 2, 128, 16),    # head_dim 128
    (8, 2, 128, 32),
    (6, 3, 80, 16),     # head_dim that is neither 64 nor 128
    (4, 1, 256, 8),
    (14, 2, 64, 4),     # small blocks
    (14, 2, 64, 1),
    (14, 2, 64, 128),   # one block covers many tiles
    (12, 4, 64, 12),    # block size that is not a power of two
    (5, 5, 24, 5),
]


@pytest.mark.parametrize("geom", GEOMETRIES, ids=lambda g: "q%d_kv%d_d%d_bs%d" % g)
@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16"])
def test_geometries(pkv, orc, torch_cuda, geom, dtype):
    qh, kvh, hd, bs = geom
    ctx = [0, 1, bs - 1, bs, 2 * bs + 3, 130, 517, 64, 63, 255]
    nb = sum((c + 1 + bs - 1) // bs for c in ctx) + 37
    case = Case(orc, dtype, qh, kvh, hd, bs, nb, ctx, [1] * len(ctx), seed=7, pkv=pkv)
    for mode in ("direct", "host_plan"):
        check_case(case, pkv, torch_cuda, orc, mode)


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_long_and_skewed_contexts_exercise_split_k(pkv, orc, torch_cuda, dtype):
    """Contexts from 1 to 8,192 in one step (the 64x skew of configuration 3): many chunks per
    long sequence merged by the last-arriving block, single-chunk sequences written directly."""
    ctx = [8191, 1, 4096, 700, 8192, 130, 2049, 64, 5000, 3]
    bs = 16
    nb = sum((c + 1 + bs - 1) // bs for c in ctx) + 11
    case = Case(orc, dtype, 32, 4, 64, bs, nb, ctx, [1] * len(ctx), seed=8, pkv=pkv)
    for mode in ("split", "host_plan", "device_plan", "direct"):
        check_case(case, pkv, torch_cuda, orc, mode)


def test_plan_is_reusable_across_layers(pkv, orc, torch_cuda):
    """One plan, many attention calls (one per layer in a decode step): the arrival counters
    must come back to zero after every call, and different pools must give different results."""
    torch = torch_cuda
    ctx = [3000, 20, 1500, 999, 4000, 257]
    case = Case(orc, "bf16", 14, 2, 64, 16, 1024, ctx, [1] * len(ctx), seed=9, pkv=pkv)
    _, _, want = case.expected(orc)
    for planner in ("host_plan", "device_plan"):
        d = case.run_gpu(pkv, torch, planner)
        plan = d["plan"]
        args = (d["q"], d["kc"], d["vc"], d["block_tables"], d["table_offset"], d["token_seq"], d["token_pos"])
        outs = []
        for layer in range(4):
            out = torch.zeros_like(d["out"])
            plan.attention(*args, out, case.bs, case.scale)
            outs.append(out)
        torch.cuda.synchronize()
        for out in outs:
            _, got = from_device(torch, orc, out, "bf16")
            e_ref, e_row = rel_errors(got.reshape(-1, 64), want.reshape(-1, 64))
            assert e_row <= TOL["bf16"]
            assert torch.equal(out, outs[0])      # same inputs, same plan: bit-identical every time


@pytest.mark.parametrize("name", ["attn_qwen_f32", "attn_tiny_f32"])
@pytest.mark.parametrize("mode", ["direct", "split"])
def test_golden_fixture_from_compiled_reference(pkv, orc, torch_cuda, name, mode):
    """Inputs and expected outputs committed under tests/golden/ (produced by the reference's
    own code): append must reproduce the cache bit for bit, attention within 1e-5."""
    torch = torch_cuda
    g = np.load(os.path.join(GOLD, name + ".npz"))
    qh, kvh, hd, bs, nb = (int(x) for x in g["geometry"])
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    kc, vc = dev(g["k_cache"]), dev(g["v_cache"])
    N = int(g["token_pos"].shape[0])
    pkv.launch_store_kv(dev(g["k"]), dev(g["v"]), dev(g["slots"]), kc, vc, N, kvh * hd)
    want_kc, want_vc = g["k_cache"].copy(), g["v_cache"].copy()
    orc.append(g["k"], g["v"], g["slots"], want_kc, want_vc)
    assert np.array_equal(kc.cpu().numpy().view(np.uint32), want_kc.view(np.uint32))
    assert np.array_equal(vc.cpu().numpy().view(np.uint32), want_vc.view(np.uint32))
    out = torch.zeros((N, qh * hd), dtype=torch.float32, device="cuda")
    ws = pkv.alloc_decode_workspace(N, qh, kvh, hd) if mode == "split" else None
    pkv.launch_attention_decode(dev(g["q"]), kc, vc, dev(g["block_tables"]), dev(g["table_offset"]),
                                dev(g["token_seq"]), dev(g["token_pos"]), out, N, qh, kvh, hd, bs,
                                float(g["scale"]), workspace=ws)
    torch.cuda.synchronize()
    e_ref, e_row = rel_errors(out.cpu().numpy().reshape(-1, hd), g["out"].reshape(-1, hd))
    assert e_ref <= 1e-5 and e_row <= 1e-5, (e_ref, e_row)


def test_relocation_invariance_at_full_size(pkv, orc, torch_cuda, workloads):
    """Configuration 3 at its full size (256 sequences, contexts log-uniform to 8,192, 65,536-block
    pool, one layer): the result may depend on what is stored, never on where.  Moving every
    block to a different physical id (and rewriting the tables) must leave the output
    bit-identical; a sample of tokens is also checked against the CPU checker, and constant
    V rows must come back as that constant."""
    torch = torch_cuda
    w = workloads.make("cfg3", layers=1)
    bs, kv_dim = w.block_size, w.kv_dim
    g = torch.Generator(device="cuda").manual_seed(33)
    kc = torch.randn((w.num_blocks * bs, kv_dim), generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    vc = torch.randn((w.num_blocks * bs, kv_dim), generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    tabs, pos, _ = w.step_tokens()
    idx = pkv.pack_step(tabs, pos, bs)
    N = idx.n_tokens
    i32 = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).cuda()
    q = torch.randn((N, w.q_heads * w.head_dim), generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    k = torch.randn((N, kv_dim), generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    v = torch.randn((N, kv_dim), generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    d_pos, d_seq = i32(idx.token_pos), i32(idx.token_seq)

    def run(kc_, vc_, tables, offs, slots):
        pkv.launch_store_kv(k, v, i32(slots), kc_, vc_, N, kv_dim)
        plan = pkv.DecodePlan(N, w.q_heads, w.kv_heads, w.head_dim).build_host(idx.token_pos)
        out = torch.zeros((N, w.q_heads * w.head_dim), dtype=torch.bfloat16, device="cuda")
        plan.attention(q, kc_, vc_, i32(tables), i32(offs), d_seq, d_pos, out, bs, w.scale)
        torch.cuda.synchronize()
        return out

    out_a = run(kc, vc, idx.block_tables, idx.table_offset, idx.slots)
    # append round trip: every new row is where slot() says, bit for bit
    assert torch.equal(kc[i32(idx.slots).long()], k) and torch.equal(vc[i32(idx.slots).long()], v)

    # relocate: physical block b moves to perm[b]
    perm = np.random.default_rng(3).permutation(w.num_blocks).astype(np.int64)
    inv = torch.from_numpy(np.argsort(perm)).cuda()
    kc_b = kc.view(w.num_blocks, bs * kv_dim)[inv].contiguous().view(-1, kv_dim)
    vc_b = vc.view(w.num_blocks, bs * kv_dim)[inv].contiguous().view(-1, kv_dim)
    tables_b = perm[idx.block_tables].astype(np.int32)
    slots_b = (perm[idx.slots // bs] * bs + idx.slots % bs).astype(np.int32)
    out_b = run(kc_b, vc_b, tables_b, idx.table_offset, slots_b)
    assert torch.equal(out_a, out_b)

    # a sample of tokens (longest, shortest, a few in between) against the CPU checker
    order = np.argsort(idx.token_pos)
    sample = np.unique(np.concatenate([order[:3], order[-3:], order[::41]]))
    kc_h = orc.from_bf16_bits(kc.view(torch.int16).cpu().numpy().view(np.uint16))
    vc_h = orc.from_bf16_bits(vc.view(torch.int16).cpu().numpy().view(np.uint16))
    q_h = orc.from_bf16_bits(q.view(torch.int16).cpu().numpy().view(np.uint16))
    want = orc.paged_attention(q_h[sample], kc_h, vc_h, idx.block_tables, idx.table_offset, idx.token_seq[sample],
                               idx.token_pos[sample], w.q_heads, w.kv_heads, w.head_dim, bs, w.scale, threads=8)
    got = orc.from_bf16_bits(out_a.view(torch.int16).cpu().numpy().view(np.uint16))[sample]
    e_ref, e_row = rel_errors(got.reshape(-1, w.head_dim), want.reshape(-1, w.head_dim))
    assert e_ref <= TOL["bf16"] and e_row <= TOL["bf16"], (e_ref, e_row)
    del kc_h, vc_h

    # softmax weights sum to one: constant V rows come back unchanged
    vc.fill_(0.75)
    v.fill_(0.75)
    out_c = run(kc, vc, idx.block_tables, idx.table_offset, idx.slots)
    assert torch.allclose(out_c.float(), torch.full_like(out_c, 0.75, dtype=torch.float32), rtol=0, atol=0.75 * 2 ** -7)


def test_pool_size_in_the_plan_bounds_the_tensor_maps(pkv, orc, torch_cuda):
    """pkv_decode_plan.num_blocks: with the pool size known the kernels' tensor maps end at the pool.
    Same step, same bits as with the unbounded maps; and a table entry beyond the pool reads zeros
    (a finite output) instead of whatever lies behind the pool."""
    torch = torch_cuda
    ctx = [700, 15, 3000, 64]
    case = Case(orc, "bf16", 14, 2, 64, 16, 256, ctx, [1] * len(ctx), seed=21, pkv=pkv)
    d = case.run_gpu(pkv, torch, "host_plan")
    want = d["out"].clone()
    args = (d["q"], d["kc"], d["vc"], d["block_tables"], d["table_offset"], d["token_seq"], d["token_pos"])
    plan = pkv.DecodePlan(case.N, case.qh, case.kvh, case.hd, num_blocks=case.nb).build_host(case.idx.token_pos)
    assert plan.plan.num_blocks == case.nb
    out = torch.zeros_like(want)
    plan.attention(*args, out, case.bs, case.scale)
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int16), want.view(torch.int16))
    bad = d["block_tables"].clone()
    bad[3] = case.nb + 5                                    # a block id past the end of the pool
    plan.attention(d["q"], d["kc"], d["vc"], bad, *args[4:], out, case.bs, case.scale)
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all() and pkv.debug_device_flags() == 0
