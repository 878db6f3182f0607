"""The decode entry point that brings its own scratch, for callers that cannot allocate a
workspace (an engine that has already given all free HBM to its block pool, or a per-token
loop that must not hit cudaMalloc's device synchronisation).

Called through the C ABI twice in a row -- the second call on different inputs, reusing the
same built-in area -- and compared both with the ordinary entry point fed a caller-owned
workspace and with the CPU checker, within the 2e-2 the bf16 parity tests use.  Collected last on purpose (file name), so a run
that stops at the first failure has already run every other test; it also passes alone in a
fresh process."""
import ctypes as C

import numpy as np
import pytest

from tests.gpu_util import Case, TOL, from_device, rel_errors

pytestmark = pytest.mark.gpu


def _call(pkv, torch, name, d, case, extra):
    fn = getattr(pkv.lib(), name)
    st = fn(d["q"].data_ptr(), d["kc"].data_ptr(), d["vc"].data_ptr(), d["block_tables"].data_ptr(),
            d["table_offset"].data_ptr(), d["token_seq"].data_ptr(), d["token_pos"].data_ptr(), d["out"].data_ptr(),
            case.N, case.qh, case.kvh, case.hd, case.bs, C.c_float(case.scale), *extra,
            torch.cuda.current_stream().cuda_stream)
    assert st == 0, pkv.lib().pkv_last_error()


def test_builtin_scratch_matches_caller_workspace_on_two_calls(pkv, orc, torch_cuda):
    torch = torch_cuda
    # long and short contexts in one step, so tokens are split and the scratch really is used
    for seed, ctx in ((31, [4100, 3, 900, 2049, 17, 640]), (32, [1500, 7000, 64, 1, 333, 2600, 90])):
        case = Case(orc, "bf16", 32, 4, 64, 16, 2048, ctx, [1] * len(ctx), seed=seed, pkv=pkv)
        d = case.upload(torch)
        pkv.launch_store_kv(d["k"], d["v"], d["slots"], d["kc"], d["vc"], case.N, case.kvh * case.hd)
        ws = pkv.alloc_decode_workspace(case.N, case.qh, case.kvh, case.hd)
        _call(pkv, torch, "pkv_decode_attn_bf16", d, case, (ws.data_ptr(), ws.numel()))
        torch.cuda.synchronize()
        want = d["out"].clone()
        d["out"].zero_()
        _call(pkv, torch, "pkv_decode_attn_bf16_builtin_scratch", d, case, ())
        torch.cuda.synchronize()
        assert pkv.debug_device_flags() == 0
        _, a = from_device(torch, orc, d["out"], "bf16")
        _, b = from_device(torch, orc, want, "bf16")
        assert np.isfinite(a).all()
        e_ref, e_row = rel_errors(a.reshape(-1, 64), b.reshape(-1, 64))
        assert e_ref <= TOL["bf16"] and e_row <= TOL["bf16"], (seed, e_ref, e_row)
        # and against the CPU checker itself, not only against the library's other entry point
        _, _, want_cpu = case.expected(orc)
        e_ref, e_row = rel_errors(a.reshape(-1, 64), want_cpu.reshape(-1, 64))
        assert e_ref <= TOL["bf16"] and e_row <= TOL["bf16"], (seed, "checker", e_ref, e_row)


def test_builtin_scratch_rejects_steps_beyond_its_size(pkv, torch_cuda):
    one = 0x1000
    st = pkv.lib().pkv_decode_attn_bf16_builtin_scratch(one, one, one, one, one, one, one, one, 4000000, 64, 8, 128, 16,
                                                       C.c_float(0.1), None)
    assert st == pkv._lib.PKV_E_WORKSPACE
    msg = pkv.lib().pkv_last_error().decode()
    assert "built-in area holds" in msg and "33554432" in msg
