"""GPU parity for the fused RoPE + K/V append: q rotated in place, rotated k and v written to their
slots, against the CPU checker's rope_inplace followed by the append.  fp32 must match bit for bit
(products rounded separately on both sides); 16-bit types must equal the fp32 result rounded once with
the reference's own cast."""
import numpy as np
import pytest

from tests.gpu_util import cast_like_reference, from_device, to_device

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("geom", [
    # q_heads, kv_heads, head_dim, n_tokens
    (14, 2, 64, 64),      # Qwen2.5-0.5B decode step
    (32, 4, 64, 300),     # TinyLlama, a prefill-sized step
    (8, 2, 128, 33),
    (6, 3, 40, 17),       # head_dim whose half is not a multiple of the vector width (element-wise path)
    (4, 4, 6, 5),
])
def test_rope_append_matches_checker(pkv, orc, torch_cuda, dtype, geom):
    torch = torch_cuda
    qh, kvh, hd, N = geom
    rng = np.random.default_rng(qh * 100 + hd)
    kv_dim, slots_total, max_pos = kvh * hd, 4096, 9000
    cos, sin = orc.rope_tables(hd, max_pos, 10000.0)
    pos = rng.integers(0, max_pos, size=N).astype(np.int32)
    pos[:3] = [0, 1, max_pos - 1]
    slots = rng.permutation(slots_total)[:N].astype(np.int32)
    f = lambda *shape: rng.standard_normal(shape, dtype=np.float32)
    q_bits, q32 = cast_like_reference(orc, f(N, qh * hd), dtype)
    k_bits, k32 = cast_like_reference(orc, f(N, kv_dim), dtype)
    v_bits, v32 = cast_like_reference(orc, f(N, kv_dim), dtype)
    kc_bits, _ = cast_like_reference(orc, f(slots_total, kv_dim), dtype)
    vc_bits, _ = cast_like_reference(orc, f(slots_total, kv_dim), dtype)
    # expected: fp32 rotation of the (widened) inputs, rounded once to the element type, then the append
    want_q, _ = cast_like_reference(orc, orc.rope(q32, qh, hd, pos, cos, sin), dtype)
    want_k, _ = cast_like_reference(orc, orc.rope(k32, kvh, hd, pos, cos, sin), dtype)
    want_kc, want_vc = kc_bits.copy(), vc_bits.copy()
    orc.append(want_k, v_bits, slots, want_kc, want_vc)

    d_q, d_k, d_v = (to_device(torch, a, dtype) for a in (q_bits, k_bits, v_bits))
    d_kc, d_vc = to_device(torch, kc_bits, dtype), to_device(torch, vc_bits, dtype)
    pkv.launch_rope_store_kv(d_q, d_k, d_v, torch.from_numpy(pos).cuda(), torch.from_numpy(cos).cuda(),
                             torch.from_numpy(sin).cuda(), torch.from_numpy(slots).cuda(), d_kc, d_vc, N, qh, kvh, hd)
    torch.cuda.synchronize()
    view = (lambda a: np.ascontiguousarray(a).view(np.uint32)) if dtype == "f32" else (lambda a: a)
    got_q, _ = from_device(torch, orc, d_q, dtype)
    got_kc, _ = from_device(torch, orc, d_kc, dtype)
    got_vc, _ = from_device(torch, orc, d_vc, dtype)
    got_k, _ = from_device(torch, orc, d_k, dtype)
    assert np.array_equal(view(got_q), view(want_q)), "rotated q differs"
    assert np.array_equal(view(got_kc), view(want_kc)), "K pool differs"
    assert np.array_equal(view(got_vc), view(want_vc)), "V pool differs"
    assert np.array_equal(view(got_k), view(k_bits)), "k input must be left as it was"


def test_rope_append_then_attention_equals_separate_steps(pkv, orc, torch_cuda):
    """Fused path vs. rotating on the host and using the plain append: identical pools, identical attention."""
    torch = torch_cuda
    from tests.gpu_util import Case
    case = Case(orc, "bf16", 14, 2, 64, 16, 128, [40, 3, 77], [1, 5, 1], seed=3, pkv=pkv)
    cos, sin = orc.rope_tables(64, 256, 10000.0)
    d = case.upload(torch)
    pos = case.idx.token_pos
    pkv.launch_rope_store_kv(d["q"], d["k"], d["v"], d["token_pos"], torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda(),
                             d["slots"], d["kc"], d["vc"], case.N, case.qh, case.kvh, case.hd)
    ws = pkv.alloc_decode_workspace(case.N, case.qh, case.kvh, case.hd)
    pkv.launch_attention_decode(d["q"], d["kc"], d["vc"], d["block_tables"], d["table_offset"], d["token_seq"],
                                d["token_pos"], d["out"], case.N, case.qh, case.kvh, case.hd, case.bs, case.scale, workspace=ws)
    torch.cuda.synchronize()
    # host: rotate, cast, then the ordinary case machinery
    qb, qf = cast_like_reference(orc, orc.rope(case.q, case.qh, 64, pos, cos, sin), "bf16")
    kb, kf = cast_like_reference(orc, orc.rope(case.k, case.kvh, 64, pos, cos, sin), "bf16")
    case.q_bits, case.q, case.k_bits, case.k = qb, qf, kb, kf
    _, _, want = case.expected(orc)
    from tests.gpu_util import rel_errors
    _, got = from_device(torch, orc, d["out"], "bf16")
    assert rel_errors(got.reshape(-1, 64), want.reshape(-1, 64))[1] <= 2e-2
