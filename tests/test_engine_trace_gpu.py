"""The golden engine trace replayed through the product path on a GPU.  Every step the reference's own
Scheduler built for a small serving run (chunked prefill, decode, prefix-cache hits, five preemptions with
recompute; 320 steps, 3,829 tokens) goes through the calls llm-engine's forward pass makes for one layer --
pack the step, append K/V, attention over every packed token in ONE call (pkv_mixed_attn_*, which routes the
prefill chunks to the tensor-core kernel on the device) -- on pools that live across all the steps.  K, V and q
rows are functions of a position's content, so a recomputed or shared position must reproduce what was there.
Checked: attention of every step against the CPU checker on the host mirror of the pools, and the pools bit
for bit at the end."""
import numpy as np
import pytest

from tests.engine_trace_util import EngineTrace, rows_from_keys
from tests.gpu_util import TOL, cast_like_reference, from_device, rel_errors, to_device

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
def test_engine_trace_through_the_mixed_entry_point(pkv, orc, torch_cuda, dtype):
    torch = torch_cuda
    tr = EngineTrace()
    qh, kvh, hd, bs = 14, 2, 64, tr.bs
    kv_dim, H = kvh * hd, qh * hd
    slots_total = tr.num_blocks * bs
    scale = float(np.float32(1.0) / np.sqrt(np.float32(hd)))
    kc_bits = np.zeros((slots_total, kv_dim), dtype=np.uint16)
    vc_bits = np.zeros_like(kc_bits)
    kc_val = np.zeros((slots_total, kv_dim), dtype=np.float32)
    vc_val = np.zeros_like(kc_val)
    d_kc, d_vc = to_device(torch, kc_bits, dtype), to_device(torch, vc_bits, dtype)
    ws = torch.empty(pkv.mixed_workspace_bytes(tr.budget, qh, kvh, hd), dtype=torch.uint8, device="cuda")
    i32 = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).cuda()
    worst = (0.0, 0.0)
    routed_chunks = 0
    for s in range(len(tr.steps)):
        tabs, pos, sid, keys = tr.packed(s)
        idx = pkv.pack_step(tabs, pos, bs, tok_keys=sid.tolist())
        N = idx.n_tokens
        k_bits, k_val = cast_like_reference(orc, rows_from_keys(keys, kv_dim, 1), dtype)
        v_bits, v_val = cast_like_reference(orc, rows_from_keys(keys, kv_dim, 2), dtype)
        q_bits, q_val = cast_like_reference(orc, rows_from_keys(keys, H, 3), dtype)
        orc.append(k_val, v_val, idx.slots, kc_val, vc_val)
        orc.append(k_bits, v_bits, idx.slots, kc_bits, vc_bits)
        want = orc.paged_attention(q_val, kc_val, vc_val, idx.block_tables, idx.table_offset, idx.token_seq, idx.token_pos,
                                   qh, kvh, hd, bs, scale, threads=4)
        d_q, d_k, d_v = to_device(torch, q_bits, dtype), to_device(torch, k_bits, dtype), to_device(torch, v_bits, dtype)
        out = torch.zeros((N, H), dtype=d_q.dtype, device="cuda")
        pkv.launch_store_kv(d_k, d_v, i32(idx.slots), d_kc, d_vc, N, kv_dim)
        pkv.launch_attention_mixed(d_q, d_kc, d_vc, i32(idx.block_tables), i32(idx.table_offset), i32(idx.token_seq),
                                   i32(idx.token_pos), out, N, qh, kvh, hd, bs, scale, ws, num_blocks=tr.num_blocks)
        _, got = from_device(torch, orc, out, dtype)
        assert np.isfinite(got).all(), s
        e_ref, e_row = rel_errors(got.reshape(-1, hd), want.reshape(-1, hd))
        assert e_ref <= TOL[dtype] and e_row <= TOL[dtype], (s, e_ref, e_row)
        worst = (max(worst[0], e_ref), max(worst[1], e_row))
        routed_chunks += sum(1 for _, _, ln, _ in tr.steps[s] if ln >= 16)
    assert pkv.debug_device_flags() == 0
    got_kc, _ = from_device(torch, orc, d_kc, dtype)
    got_vc, _ = from_device(torch, orc, d_vc, dtype)
    assert np.array_equal(got_kc, kc_bits) and np.array_equal(got_vc, vc_bits), "pools differ from the reference appends"
    assert routed_chunks >= 20
    print(f"engine trace {dtype}: 320 steps, worst rel err {worst[0]:.2e} / {worst[1]:.2e}, {routed_chunks} chunks through the prefill kernel")
