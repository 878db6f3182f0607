"""GPU parity for paged (chunked) prefill attention on the tcgen05 tensor cores.

The reference has no prefill kernel; what the result must agree with is
ref::paged_attention_head applied to every (token, head) of the chunk
(include/engine/ops.h:87-111), i.e. the CPU checker run with one packed token per
chunk position.  K/V of the chunk are appended first, as the reference orders
store_kv before attention, so tokens of a chunk attend to earlier tokens of the
same chunk.  Tolerance 2e-2 (16-bit KV, inputs cast the reference's way)."""
import numpy as np
import pytest

from tests.gpu_util import Case, TOL, from_device, rel_errors

pytestmark = pytest.mark.gpu


def run_prefill(pkv, torch, case, d=None):
    d = d or case.upload(torch)
    kv_dim = case.kvh * case.hd
    pkv.launch_store_kv(d["k"], d["v"], d["slots"], d["kc"], d["vc"], case.N, kv_dim)
    i32 = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).cuda()
    q_len = np.asarray(case.seq_new, dtype=np.int32)
    q_start = np.concatenate([[0], np.cumsum(q_len)[:-1]]).astype(np.int32)
    ctx = np.asarray(case.seq_ctx, dtype=np.int32)
    pkv.launch_attention_prefill(d["q"], d["kc"], d["vc"], d["block_tables"], d["table_offset"], i32(q_start), i32(q_len),
                                 i32(ctx), d["out"], case.N, len(q_len), int(q_len.max()), case.qh, case.kvh, case.hd,
                                 case.bs, case.nb, case.scale)
    torch.cuda.synchronize()
    assert pkv.debug_device_flags() == 0, "a kernel gave up on a bounded wait"
    return d


def make_case(orc, pkv, dtype, qh, kvh, bs, ctx, new, seed):
    nb = sum((c + n + bs - 1) // bs for c, n in zip(ctx, new)) + 19
    case = Case(orc, dtype, qh, kvh, 64, bs, nb, ctx, new, seed=seed, pkv=pkv)
    case.seq_ctx, case.seq_new = list(ctx), list(new)
    return case


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("shape", [
    # q_heads, kv_heads, block_size, cached context per sequence, new tokens per sequence
    (14, 2, 16, [0], [128]),                       # one full tile, no history: pure causal
    (14, 2, 16, [0, 37, 200], [128, 70, 300]),     # ragged chunks, chunk starting mid-block, several tiles
    (32, 4, 16, [511, 5, 1000, 0], [1, 129, 257, 16]),   # a decode-sized chunk, tile boundaries +1
    (8, 8, 32, [100, 0], [200, 90]),               # no GQA, larger blocks
    (4, 1, 128, [300], [260]),                     # one block spans a whole key tile
])
def test_prefill_matches_checker(pkv, orc, torch_cuda, dtype, shape):
    qh, kvh, bs, ctx, new = shape
    case = make_case(orc, pkv, dtype, qh, kvh, bs, ctx, new, seed=21)
    _, _, want = case.expected(orc, threads=8)
    d = run_prefill(pkv, torch_cuda, case)
    _, got = from_device(torch_cuda, orc, d["out"], dtype)
    assert np.isfinite(got).all()
    e_ref, e_row = rel_errors(got.reshape(-1, 64), want.reshape(-1, 64))
    assert e_ref <= TOL[dtype] and e_row <= TOL[dtype], (e_ref, e_row)


def test_prefill_agrees_with_decode_kernel_on_the_same_step(pkv, orc, torch_cuda):
    """The same packed step through the reference's route (every chunk token through the decode
    launcher) and through the prefill kernel."""
    torch = torch_cuda
    case = make_case(orc, pkv, "bf16", 14, 2, 16, [64, 700, 3], [256, 140, 33], seed=22)
    d1 = case.run_gpu(pkv, torch, "split")
    out_decode = d1["out"].clone()
    d2 = run_prefill(pkv, torch, case)
    a = out_decode.float().cpu().numpy().reshape(-1, 64)
    b = d2["out"].float().cpu().numpy().reshape(-1, 64)
    e_ref, e_row = rel_errors(b, a)
    assert e_row <= 2e-2, (e_ref, e_row)


def test_prefill_unsupported_geometry_is_an_error_not_a_trap(pkv, torch_cuda):
    torch = torch_cuda
    z = torch.zeros((4, 128 * 8), device="cuda", dtype=torch.bfloat16)
    i = torch.zeros(4, device="cuda", dtype=torch.int32)
    pool = torch.zeros((64, 128 * 2), device="cuda", dtype=torch.bfloat16)
    with pytest.raises(pkv.PkvError):   # head_dim 128
        pkv.launch_attention_prefill(z, pool, pool, i, i, i, i, i, z, 4, 1, 4, 8, 2, 128, 16, 4, 0.1)
    with pytest.raises(pkv.PkvError):   # block_size 8
        pkv.launch_attention_prefill(z, pool, pool, i, i, i, i, i, z, 4, 1, 4, 16, 4, 64, 8, 8, 0.1)


def test_cfg4_chunked_prefill_sampled_at_full_size(pkv, orc, torch_cuda, workloads):
    """Configuration 4 at full size (32 sequences, cached context U[0,1536], 512-token chunk, Qwen shapes,
    bf16, shuffled tables): a sample of chunk tokens against the CPU checker, and causality: changing
    K/V rows of LATER positions must not change earlier tokens' outputs."""
    torch = torch_cuda
    w = workloads.make("cfg4")
    ctx, new = [int(c) for c in w.ctx], [int(n) for n in w.new]
    case = Case(orc, "bf16", w.q_heads, w.kv_heads, w.head_dim, w.block_size, w.num_blocks, ctx, new, seed=w.seed, pkv=pkv)
    case.seq_ctx, case.seq_new = ctx, new
    d = run_prefill(pkv, torch, case)
    _, got = from_device(torch, orc, d["out"], "bf16")
    rng = np.random.default_rng(0)
    starts = np.concatenate([[0], np.cumsum(new)[:-1]])
    sample = np.unique(np.concatenate([starts, starts + np.asarray(new) - 1, starts + 127, starts + 128,
                                       rng.integers(0, case.N, size=40)]))
    kc, vc = case.kc.copy(), case.vc.copy()
    orc.append(case.k, case.v, case.idx.slots, kc, vc)
    want = orc.paged_attention(case.q[sample], kc, vc, case.idx.block_tables, case.idx.table_offset,
                               case.idx.token_seq[sample], case.idx.token_pos[sample], case.qh, case.kvh, case.hd,
                               case.bs, case.scale, threads=8)
    e_ref, e_row = rel_errors(got[sample].reshape(-1, 64), want.reshape(-1, 64))
    assert e_ref <= TOL["bf16"] and e_row <= TOL["bf16"], (e_ref, e_row)
    # causality: poison the K/V rows of the last 128 chunk tokens of every sequence (one whole query tile, so
    # that no earlier token shares a thread block with a poisoned one), rerun without the append: every
    # earlier token must come out bit-identical
    out_before = d["out"].clone()
    later = np.concatenate([np.arange(s + n - 128, s + n) for s, n in zip(starts, new)])
    slots = torch.from_numpy(case.idx.slots[later].astype(np.int64)).cuda()
    kc_saved, vc_saved = d["kc"].clone(), d["vc"].clone()
    d["kc"][slots] = 7.0
    d["vc"][slots] = -3.0
    i32 = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).cuda()
    pkv.launch_attention_prefill(d["q"], d["kc"], d["vc"], d["block_tables"], d["table_offset"], i32(starts),
                                 i32(new), i32(ctx), d["out"], case.N, len(new), 512, case.qh, case.kvh, case.hd,
                                 case.bs, case.nb, case.scale)
    torch.cuda.synchronize()
    earlier = torch.from_numpy(np.setdiff1d(np.arange(case.N), later)).cuda()
    assert torch.equal(d["out"][earlier], out_before[earlier])
    # ... and within a tile too: poison positions 450.. of every chunk; tokens 384..449 share a block with
    # poisoned tokens (the lazy rescale may pick other reference maxima there), so they are compared by value
    later2 = np.concatenate([np.arange(s + 450, s + n) for s, n in zip(starts, new)])
    slots2 = torch.from_numpy(case.idx.slots[later2].astype(np.int64)).cuda()
    d["kc"].copy_(kc_saved)
    d["vc"].copy_(vc_saved)
    d["kc"][slots2] = 9.0
    d["vc"][slots2] = 5.0
    pkv.launch_attention_prefill(d["q"], d["kc"], d["vc"], d["block_tables"], d["table_offset"], i32(starts),
                                 i32(new), i32(ctx), d["out"], case.N, len(new), 512, case.qh, case.kvh, case.hd,
                                 case.bs, case.nb, case.scale)
    torch.cuda.synchronize()
    mid = torch.from_numpy(np.concatenate([np.arange(s + 384, s + 450) for s in starts])).cuda()
    a = d["out"][mid].float().cpu().numpy().reshape(-1, 64)
    b = out_before[mid].float().cpu().numpy().reshape(-1, 64)
    assert rel_errors(a, b)[1] <= 2e-2


def test_more_items_than_resident_blocks_and_empty_tile_slots(pkv, orc, torch_cuda):
    """The kernel's blocks are persistent and take (sequence, tile, head) items from a ticket counter:
    here 300 short sequences x 8 heads x 3 tile slots (max_q_len 300, most chunks far shorter, so most
    slots are empty) give 7,200 tickets for 296 blocks."""
    rng = np.random.default_rng(31)
    S = 300
    ctx = [int(x) for x in rng.integers(0, 200, size=S)]
    new = [int(x) for x in rng.integers(1, 140, size=S)]
    new[17], new[255] = 300, 257
    case = make_case(orc, pkv, "bf16", 8, 2, 16, ctx, new, seed=23)
    _, _, want = case.expected(orc, threads=8)
    d = run_prefill(pkv, torch_cuda, case)
    _, got = from_device(torch_cuda, orc, d["out"], "bf16")
    assert np.isfinite(got).all()
    e_ref, e_row = rel_errors(got.reshape(-1, 64), want.reshape(-1, 64))
    assert e_ref <= TOL["bf16"] and e_row <= TOL["bf16"], (e_ref, e_row)


def test_launches_in_a_row_and_on_two_streams_keep_their_ticket_counters_apart(pkv, orc, torch_cuda):
    """70 launches in a row (the pool of ticket counters has 64 slots and every launch must leave its
    slot at zero), then two different steps launched on two streams at once."""
    torch = torch_cuda
    a = make_case(orc, pkv, "bf16", 14, 2, 16, [0, 300, 77], [200, 129, 64], seed=24)
    b = make_case(orc, pkv, "bf16", 8, 8, 16, [50, 0], [150, 260], seed=25)
    wants = [c.expected(orc, threads=8)[2] for c in (a, b)]
    da = run_prefill(pkv, torch, a)
    first = da["out"].clone()
    for _ in range(70):
        da["out"].zero_()
        run_prefill(pkv, torch, a, d=da)
        assert torch.equal(first, da["out"])
    db = b.upload(torch)
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    torch.cuda.synchronize()
    for case, d, st in ((a, da, streams[0]), (b, db, streams[1])):
        d["out"].zero_()
        with torch.cuda.stream(st):
            for _ in range(5):
                run_prefill_async(pkv, torch, case, d)
    torch.cuda.synchronize()
    assert pkv.debug_device_flags() == 0
    for case, d, want in ((a, da, wants[0]), (b, db, wants[1])):
        _, got = from_device(torch, orc, d["out"], "bf16")
        e_ref, e_row = rel_errors(got.reshape(-1, 64), want.reshape(-1, 64))
        assert e_ref <= TOL["bf16"] and e_row <= TOL["bf16"], (e_ref, e_row)


def run_prefill_async(pkv, torch, case, d):
    """run_prefill without the synchronisation, on the current stream."""
    i32 = lambda x: torch.from_numpy(np.ascontiguousarray(x, dtype=np.int32)).cuda()
    if "pf_idx" not in d:
        q_len = np.asarray(case.seq_new, dtype=np.int32)
        d["pf_idx"] = (i32(np.concatenate([[0], np.cumsum(q_len)[:-1]])), i32(q_len), i32(np.asarray(case.seq_ctx)), int(q_len.max()), len(q_len))
        torch.cuda.synchronize()
    qs, ql, cl, mx, ns = d["pf_idx"]
    pkv.launch_store_kv(d["k"], d["v"], d["slots"], d["kc"], d["vc"], case.N, case.kvh * case.hd)
    pkv.launch_attention_prefill(d["q"], d["kc"], d["vc"], d["block_tables"], d["table_offset"], qs, ql, cl, d["out"], case.N, ns, mx,
                                 case.qh, case.kvh, case.hd, case.bs, case.nb, case.scale)
