"""Mixed steps through pkv_mixed_attn_*: prefill chunks and decode tokens in one call, split on the
device into runs for the tensor-core prefill kernel and tokens for the decode kernels.  The result
must be what ref::paged_attention_head gives for every packed token (include/engine/ops.h:87-111),
however the step is split."""
import numpy as np
import pytest

from tests.gpu_util import Case, TOL, from_device, rel_errors

pytestmark = pytest.mark.gpu


def run_mixed(case, pkv, torch, orc, min_run=0, num_blocks=0, workspace=True):
    want_kc, want_vc, want = case.expected(orc)
    d = case.upload(torch)
    pkv.launch_store_kv(d["k"], d["v"], d["slots"], d["kc"], d["vc"], case.N, case.kvh * case.hd)
    n = pkv.mixed_workspace_bytes(case.N, case.qh, case.kvh, case.hd)
    ws = torch.empty(n, dtype=torch.uint8, device="cuda")
    ws.fill_(0xCD)                                  # the call must not rely on a cleared workspace
    pkv.launch_attention_mixed(d["q"], d["kc"], d["vc"], d["block_tables"], d["table_offset"], d["token_seq"], d["token_pos"],
                               d["out"], case.N, case.qh, case.kvh, case.hd, case.bs, case.scale, ws,
                               num_blocks=num_blocks, min_run=min_run)
    torch.cuda.synchronize()
    assert pkv.debug_device_flags() == 0
    kcb, _ = from_device(torch, orc, d["kc"], case.dtype)
    assert np.array_equal(kcb, want_kc)
    _, got = from_device(torch, orc, d["out"], case.dtype)
    assert np.isfinite(got).all()
    e_ref, e_row = rel_errors(got.reshape(-1, case.hd), want.reshape(-1, case.hd))
    assert e_ref <= TOL[case.dtype] and e_row <= TOL[case.dtype], (e_ref, e_row)
    return d, ws


def make(orc, pkv, dtype, qh, kvh, bs, ctx, new, seed):
    nb = sum((c + n + bs - 1) // bs for c, n in zip(ctx, new)) + 8
    return Case(orc, dtype, qh, kvh, 64, bs, nb, ctx, new, seed, pkv), nb


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("kind", ["mixed", "decode_only", "prefill_only", "edges"])
def test_mixed_step_matches_checker(pkv, orc, torch_cuda, dtype, kind):
    rng = np.random.default_rng(abs(hash(kind)) % 997)
    if kind == "mixed":
        ctx = [37, 200, 0, 90] + [int(x) for x in rng.integers(1, 3000, size=20)]
        new = [300, 300, 129, 5] + [1] * 20
    elif kind == "decode_only":          # the router runs and finds no chunk: an empty prefill launch
        ctx = [int(x) for x in rng.integers(1, 5000, size=40)]
        new = [1] * 40
    elif kind == "prefill_only":         # no decode token at all: an empty decode plan
        ctx = [0, 511, 1000]
        new = [257, 128, 16]
    else:                                # run lengths around the threshold and around the 128-row tile
        ctx = [5, 6, 7, 8, 100, 9, 10]
        new = [15, 16, 17, 127, 128, 129, 1]
    case, nb = make(orc, pkv, dtype, 14, 2, 16, ctx, new, 77)
    run_mixed(case, pkv, torch_cuda, orc, num_blocks=nb if kind == "mixed" else 0)


def test_threshold_and_geometry_choices(pkv, orc, torch_cuda):
    ctx, new = [40, 300, 2000, 17], [64, 33, 1, 1]
    case, _ = make(orc, pkv, "bf16", 32, 4, 32, ctx, new, 5)      # TinyLlama heads, block 32
    for min_run in (1, 16, 40, 1000):                              # everything / both / one / no run goes to the prefill kernel
        run_mixed(case, pkv, torch_cuda, orc, min_run=min_run)
    case, _ = make(orc, pkv, "bf16", 14, 2, 8, ctx, new, 6)       # block 8: the prefill kernel does not run it
    run_mixed(case, pkv, torch_cuda, orc)


def test_a_sequence_that_appears_in_two_runs(pkv, orc, torch_cuda):
    """Not a step llm-engine's scheduler builds (one slice per sequence), but well defined: two
    separate stretches of one sequence's tokens are two runs, each causal over all earlier keys."""
    bs = 16
    rng = np.random.default_rng(9)
    table = rng.permutation(64).astype(np.int32)[:20]
    other = rng.permutation(64).astype(np.int32)[20:30] + 64
    tok_tabs = [table] * 40 + [other] * 3 + [table] * 30
    tok_pos = list(range(10, 50)) + [100, 101, 102] + list(range(200, 230))
    case = Case(orc, "bf16", 14, 2, 64, bs, 160, [320, 160], [0, 0], 1, pkv)     # pools only; the step is set below
    case.idx = pkv.pack_step(tok_tabs, tok_pos, bs)
    case.N = case.idx.n_tokens
    from tests.gpu_util import cast_like_reference
    f = lambda *s: rng.standard_normal(s, dtype=np.float32)
    case.q_bits, case.q = cast_like_reference(orc, f(case.N, 14 * 64), "bf16")
    case.k_bits, case.k = cast_like_reference(orc, f(case.N, 2 * 64), "bf16")
    case.v_bits, case.v = cast_like_reference(orc, f(case.N, 2 * 64), "bf16")
    run_mixed(case, pkv, torch_cuda, orc)


def test_configuration_4_through_the_mixed_entry_point_equals_the_prefill_call(pkv, orc, torch_cuda, workloads):
    """Configuration 4 at full size (32 sequences, 512-token chunks over 0..1,536 cached tokens, 16,384 packed
    rows) handed over the way llm-engine hands a step over: token_seq / token_pos only.  The router must find the
    32 chunks and give the prefill kernel the records a caller of pkv_prefill_attn_* would have passed, so the two
    outputs agree bit for bit; a sample of rows is checked against the CPU checker."""
    torch = torch_cuda
    w = workloads.make("cfg4", layers=1)
    bs, kv_dim, H = w.block_size, w.kv_dim, w.q_heads * w.head_dim
    tabs, pos, _ = w.step_tokens()
    idx = pkv.pack_step(tabs, pos, bs)
    N = idx.n_tokens
    g = torch.Generator(device="cuda").manual_seed(5)
    rnd = lambda *s: torch.randn(s, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    kc, vc, q = rnd(w.num_blocks * bs, kv_dim), rnd(w.num_blocks * bs, kv_dim), rnd(N, H)
    i32 = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).cuda()
    d_tab, d_off, d_seq, d_pos = i32(idx.block_tables), i32(idx.table_offset), i32(idx.token_seq), i32(idx.token_pos)
    q_len = w.new.astype(np.int32)
    q_start = np.concatenate([[0], np.cumsum(q_len)[:-1]]).astype(np.int32)
    direct = torch.zeros((N, H), dtype=torch.bfloat16, device="cuda")
    pkv.launch_attention_prefill(q, kc, vc, d_tab, d_off, i32(q_start), i32(q_len), i32(w.ctx.astype(np.int32)), direct, N,
                                 w.n_seqs, int(q_len.max()), w.q_heads, w.kv_heads, w.head_dim, bs, w.num_blocks, w.scale)
    routed = torch.zeros_like(direct)
    ws = torch.empty(pkv.mixed_workspace_bytes(N, w.q_heads, w.kv_heads, w.head_dim), dtype=torch.uint8, device="cuda")
    pkv.launch_attention_mixed(q, kc, vc, d_tab, d_off, d_seq, d_pos, routed, N, w.q_heads, w.kv_heads, w.head_dim, bs,
                               w.scale, ws, num_blocks=w.num_blocks)
    torch.cuda.synchronize()
    assert pkv.debug_device_flags() == 0
    assert torch.equal(direct.view(torch.int16), routed.view(torch.int16))
    sample = np.unique(np.concatenate([np.arange(0, N, 997), [0, 511, 512, N - 1]]))
    bits = lambda t: orc.from_bf16_bits(t.view(torch.int16).cpu().numpy().view(np.uint16))
    want = orc.paged_attention(bits(q)[sample], bits(kc), bits(vc), idx.block_tables, idx.table_offset, idx.token_seq[sample],
                               idx.token_pos[sample], w.q_heads, w.kv_heads, w.head_dim, bs, w.scale, threads=8)
    e_ref, e_row = rel_errors(bits(routed)[sample].reshape(-1, 64), want.reshape(-1, 64))
    assert e_ref <= TOL["bf16"] and e_row <= TOL["bf16"], (e_ref, e_row)
