"""llm-engine's own launcher symbols, run with data.  engine::launch_store_kv and
engine::launch_attention_decode[_gqa] are called by their C++ names (through
tests/support/shim_harness.cpp) on f16 tensors, the reference's CUDA dtype, in the call order of
src/model/cuda/cuda_model.cu:366-377, and checked against the CPU checker: pools bit for bit,
attention within 2e-2.  Covered: a fragmented mixed step (prefill chunks that start in mid-block
plus decode tokens, which the launcher must route to the tensor-core prefill kernel and the decode
kernels respectively), steps that make the launchers' scratch grow twice, the same without scratch
(PKV_SHIM_NO_WORKSPACE=1, in a child process), and the mapping of refusals to exceptions."""
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from tests.gpu_util import Case, TOL, from_device, rel_errors   # noqa: E402
from tests.shim_util import build_harness, call_layer            # noqa: E402

pytestmark = pytest.mark.gpu

QH, KVH, HD, BS = 14, 2, 64, 16      # Qwen2.5-0.5B attention shapes


def mixed_case(orc, pkv, seed=11):
    """Prefill slices first, then decode tokens (include/engine/sequence.h:74-89): two 300-token chunks
    whose cached contexts end in mid-block, one 5-token slice (below the router's threshold: decode
    path), then 20 decode tokens with contexts from 1 to 3,000."""
    rng = np.random.default_rng(seed)
    ctx = [37, 200, 90] + [int(x) for x in rng.integers(1, 3000, size=20)]
    new = [300, 300, 5] + [1] * 20
    nb = sum((c + n + BS - 1) // BS for c, n in zip(ctx, new)) + 8
    return Case(orc, "f16", QH, KVH, HD, BS, nb, ctx, new, seed, pkv)


def check_through_launchers(H, case, pkv, torch, orc, use_gqa):
    want_kc, want_vc, want = case.expected(orc)
    d = case.upload(torch)
    code, msg = call_layer(H, d, case, use_gqa=use_gqa)
    assert code == 0, msg
    torch.cuda.synchronize()
    kcb, _ = from_device(torch, orc, d["kc"], "f16")
    vcb, _ = from_device(torch, orc, d["vc"], "f16")
    assert np.array_equal(kcb, want_kc) and np.array_equal(vcb, want_vc), "pools differ from the reference append"
    _, got = from_device(torch, orc, d["out"], "f16")
    assert np.isfinite(got).all()
    assert pkv.debug_device_flags() == 0
    e_ref, e_row = rel_errors(got.reshape(-1, HD), want.reshape(-1, HD))
    assert e_ref <= TOL["f16"] and e_row <= TOL["f16"], (e_ref, e_row)
    return e_ref, e_row


@pytest.fixture(scope="module")
def harness(pkv, tmp_path_factory):
    return build_harness(tmp_path_factory.mktemp("shim"))


@pytest.mark.parametrize("use_gqa", [False, True])
def test_mixed_step_through_the_launchers(pkv, orc, torch_cuda, harness, use_gqa):
    check_through_launchers(harness, mixed_case(orc, pkv), pkv, torch_cuda, orc, use_gqa)


def test_scratch_grows_twice_and_results_stay_right(pkv, orc, torch_cuda, harness):
    """Three steps on one device, each needing more than 1.5 times the scratch of everything before it
    (the launchers allocate half as much again as they are asked for): 8 decode tokens with 8 kv heads,
    then 60 tokens with histories up to 9,000 keys on Qwen's 14 / 2 heads (split-K partials), then a step
    with a 1,500-token chunk on 28 query heads over one kv head.  Nothing is freed or synchronised in
    between, and every step must still match the checker."""
    rng = np.random.default_rng(5)
    steps = [
        (8, 8, [int(x) for x in rng.integers(1, 200, size=8)], [1] * 8),
        (14, 2, [9000, 6000] + [int(x) for x in rng.integers(1, 2500, size=58)], [1] * 60),
        (28, 1, [700, 33] + [int(x) for x in rng.integers(1, 800, size=30)], [1500, 40] + [1] * 30),
    ]
    need = [pkv.mixed_workspace_bytes(sum(n), qh, kvh, HD) for qh, kvh, _, n in steps]
    assert need[0] * 1.5 < need[1] and need[1] * 1.5 < need[2], need
    for i, (qh, kvh, ctx, new) in enumerate(steps):
        nb = sum((c + n + BS - 1) // BS for c, n in zip(ctx, new)) + 8
        case = Case(orc, "f16", qh, kvh, HD, BS, nb, ctx, new, 100 + i, pkv)
        check_through_launchers(harness, case, pkv, torch_cuda, orc, use_gqa=bool(i & 1))


def test_without_scratch_in_a_child_process(pkv, orc, torch_cuda):
    """PKV_SHIM_NO_WORKSPACE=1 is read once per process: a child runs the mixed step with it."""
    env = dict(os.environ, PKV_SHIM_NO_WORKSPACE="1")
    r = subprocess.run([sys.executable, os.path.abspath(__file__)], cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "mixed step without scratch: ok" in r.stdout


def test_refusals_become_exceptions_and_nothing_is_enqueued(pkv, orc, torch_cuda, harness):
    torch = torch_cuda
    case = Case(orc, "f16", QH, KVH, HD, BS, 64, [50, 60], [1, 1], 3, pkv)
    d = case.upload(torch)
    before = d["out"].clone()
    case.kvh = 4                                   # 14 query heads over 4 kv heads: the reference launcher throws too
    code, msg = call_layer(harness, d, case, do_store=False)   # (src/kernels/attention_decode_gqa.cu:212-214)
    case.kvh = KVH
    assert code == 1 and "multiple" in msg and "launch_attention_decode" in msg
    # a recorded give-up of an earlier launch surfaces once, as an exception, and then clears
    pkv.lib().pkv_debug_set_reported_flags(2)
    code, msg = call_layer(harness, d, case)
    assert code == 1 and "gave up" in msg and "0x2" in msg
    torch.cuda.synchronize()
    assert torch.equal(before.view(torch.int16), d["out"].view(torch.int16))
    code, msg = call_layer(harness, d, case)
    assert code == 0, msg
    torch.cuda.synchronize()
    assert pkv.debug_device_flags() == 0


if __name__ == "__main__":
    import importlib
    import tempfile

    import torch

    import oracle
    pkv_mod = importlib.import_module("llm-engine_b200")
    orc_ = oracle.load_orc()
    with tempfile.TemporaryDirectory() as tmp:
        H_ = build_harness(tmp)
        check_through_launchers(H_, mixed_case(orc_, pkv_mod), pkv_mod, torch, orc_, use_gqa=False)
    print("mixed step without scratch: ok")
