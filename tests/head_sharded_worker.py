"""Worker of tests/test_head_sharded_gpu.py: one process per GPU (torchrun).  Every rank builds the
same seeded step, keeps the K/V pools and the query columns of its own heads only, runs the
head-sharded decode call, and checks the FULL output it ends up with against the CPU checker."""
import importlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    import torch
    import torch.distributed as dist
    import oracle
    from tests.gpu_util import Case, TOL, from_device, rel_errors, to_device
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("gloo")                      # carries 64-byte handles and barriers only
    pkv = importlib.import_module("llm-engine_b200")
    sharding = importlib.import_module("llm-engine_b200.sharding")
    orc = oracle.load_orc()
    qh, kvh, hd, bs = 32, 4, 64, 16
    rng = np.random.default_rng(3)
    ctx = [int(x) for x in rng.integers(1, 3000, size=40)] + [5000, 17, 64]
    for dtype in ("bf16", "f16"):
        case = Case(orc, dtype, qh, kvh, hd, bs, 8192, ctx, [1] * len(ctx), 4242, pkv)
        _, _, want = case.expected(orc)
        q0, ql, kv0, kvl = sharding.head_slices(qh, kvh, world, rank)
        cols = lambda a, h0, n: np.ascontiguousarray(a[:, h0 * hd:(h0 + n) * hd])
        d = {name: to_device(torch, cols(getattr(case, name + "_bits"), kv0, kvl), dtype) for name in ("kc", "vc", "k", "v")}
        d["q"] = to_device(torch, cols(case.q_bits, q0, ql), dtype)
        i32 = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(dev)
        idx = [i32(case.idx.block_tables), i32(case.idx.table_offset), i32(case.idx.token_seq), i32(case.idx.token_pos)]
        pkv.launch_store_kv(d["k"], d["v"], i32(case.idx.slots), d["kc"], d["vc"], case.N, kvl * hd)
        plan = pkv.DecodePlan(case.N, ql, kvl, hd, device=dev).build_host(case.idx.token_pos)
        # The exchange lives in the merge kernel, so the peer call always takes the split-K form; ask the
        # local call for the same (a step this small would otherwise run as thread-block clusters, which
        # groups the keys differently and rounds differently).
        plan.plan.cluster = 0
        # this rank's own columns are what the ordinary call computes for the same heads, bit for bit
        local = torch.zeros((case.N, ql * hd), dtype=d["q"].dtype, device=dev)
        plan.attention(d["q"], d["kc"], d["vc"], *idx, local, bs, case.scale)
        torch.cuda.synchronize()
        # Both ways of numbering the calls: counted on the device (epoch argument 0, the form a CUDA
        # graph replays) and passed by the host as a growing epoch.  A fresh set of buffers each, since
        # the flags of one form would satisfy the other's first waits.
        for device_epoch in (True, False):
            ex = sharding.HeadShardedExchange(case.N, qh, hd, d["q"].dtype, dist, dev)
            for rep in range(3):                          # the flags are reused from call to call
                ex.out.zero_()
                torch.cuda.synchronize()
                dist.barrier()                            # every rank's buffer is cleared before anybody stores into it
                out = ex.attention(plan, d["q"], d["kc"], d["vc"], *idx, bs, case.scale, device_epoch=device_epoch)
                torch.cuda.synchronize()
                _, got = from_device(torch, orc, out, dtype)
                e_ref, e_row = rel_errors(got.reshape(case.N * qh, hd), want.reshape(case.N * qh, hd))
                assert e_ref <= TOL[dtype] and e_row <= TOL[dtype], (rank, dtype, device_epoch, rep, e_ref, e_row)
                assert torch.equal(local.view(torch.int16), out[:, q0 * hd:(q0 + ql) * hd].contiguous().view(torch.int16)), \
                    (rank, dtype, device_epoch, rep, "own columns differ from the ordinary call")
                dist.barrier()                            # nobody overwrites a buffer a peer is still checking
            assert pkv.debug_device_flags() == 0
            ex.close()
        print(f"rank {rank}: {dtype}: full output within {TOL[dtype]} of the checker, own columns bit-identical to the "
              f"ordinary call, device-counted and host-passed epochs, 3 calls each", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    print(f"rank {rank}: head-sharded decode matches the checker on all {world} ranks", flush=True)


if __name__ == "__main__":
    main()
