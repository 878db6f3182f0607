"""GPU parity for the append fused into the decode attention (pkv_append_decode_attn_planned_*): the
pools must end up byte-identical to the reference append and the attention within the tolerance of
the KV dtype, exactly as with the two separate calls."""
import numpy as np
import pytest

from tests.gpu_util import Case, check_case

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("shape", [
    # q_heads, kv_heads, head_dim, block_size, contexts
    (14, 2, 64, 16, "uniform"),      # Qwen shapes (configurations 1, 2)
    (32, 4, 64, 16, "loguniform"),   # TinyLlama shapes (configuration 3): long histories are split
    (16, 2, 128, 16, "uniform"),     # head_dim 128: two boxes per row
    (32, 2, 64, 32, "edges"),        # 16 heads per kv head, block 32, positions on block and slab edges
])
def test_fused_append_matches_checker(pkv, orc, torch_cuda, dtype, shape):
    qh, kvh, hd, bs, kind = shape
    rng = np.random.default_rng(hash(shape) % 1000)
    if kind == "uniform":
        ctx = [int(x) for x in rng.integers(64, 2049, size=48)]
    elif kind == "loguniform":
        ctx = [int(x) for x in np.exp(rng.uniform(np.log(128), np.log(8192), size=64))]
    else:
        ctx = [0, 1, 15, 16, 17, 31, 32, 33, 63, 64, 255, 256, 257, 1023, 1024, 4095, 4096]
    nb = sum((c + 1 + bs - 1) // bs for c in ctx) + 16
    case = Case(orc, dtype, qh, kvh, hd, bs, nb, ctx, [1] * len(ctx), 321, pkv)
    check_case(case, pkv, torch_cuda, orc, "fused_append")


def test_fused_append_refuses_what_it_cannot_run(pkv, orc, torch_cuda):
    """block_size 8 does not run on the TMA kernel: the call says so and enqueues nothing."""
    case = Case(orc, "bf16", 14, 2, 64, 8, 256, [100, 200], [1, 1], 5, pkv)
    d = case.upload(torch_cuda)
    before = d["kc"].view(torch_cuda.int16).clone()
    with pytest.raises(pkv.PkvError, match="TMA kernel"):
        case.run_gpu(pkv, torch_cuda, "fused_append", d=d)
    torch_cuda.cuda.synchronize()
    assert torch_cuda.equal(before, d["kc"].view(torch_cuda.int16))
    check_case(case, pkv, torch_cuda, orc, "host_plan")          # the two separate calls do run it


def test_configuration_2_at_full_size(pkv, orc, torch_cuda, workloads):
    """Configuration 2 as BASELINE words it, one layer of it: 64 sequences with contexts uniform in
    256..2,048 (the workload's own seeded draw), 14 query / 2 kv heads of 64, bf16, block 16, a
    16,384-block pool dealt in shuffled order.  This is the configuration that takes the append inside
    the attention launch by default; the two separate calls are checked on the same step."""
    w = workloads.make("cfg2", layers=1)
    assert w.n_seqs == 64 and w.ctx.min() >= 256 and w.ctx.max() <= 2048 and w.num_blocks == 16384
    ctx = [int(c) for c in w.ctx]
    case = Case(orc, "bf16", w.q_heads, w.kv_heads, w.head_dim, w.block_size, w.num_blocks, ctx, [1] * len(ctx), 1235, pkv)
    for mode in ("fused_append", "host_plan"):
        e_ref, e_row = check_case(case, pkv, torch_cuda, orc, mode)
        assert e_row <= 2e-2
