"""Host-side multi-GPU logic on CPU: sequence dealing, and the cross-rank reduction with a
world_size-2 gloo group (the GPU benchmark uses the same code over NCCL)."""
import importlib
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_dealing_partitions_the_batch_and_balances_bytes(pkv, workloads):
    sh = importlib.import_module("llm-engine_b200.sharding")
    w = workloads.make("cfg3")
    for world in (1, 2, 4, 8):
        for policy in ("round_robin", "balanced"):
            parts = [sh.deal_sequences(w.ctx, world, r, policy) for r in range(world)]
            allidx = np.sort(np.concatenate(parts))
            assert np.array_equal(allidx, np.arange(w.n_seqs))
        loads = [int((w.ctx[sh.deal_sequences(w.ctx, world, r, "balanced")] + 1).sum()) for r in range(world)]
        assert max(loads) - min(loads) <= int(w.ctx.max()) + 1
    assert sh.rank_seed(1237, 3) != sh.rank_seed(1237, 2)


WORKER = r'''
import importlib, os, sys
sys.path.insert(0, sys.argv[1])
import torch, torch.distributed as dist
sh = importlib.import_module("llm-engine_b200.sharding")
wl = importlib.import_module("llm-engine_b200.workloads")
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
w = wl.make("cfg3", seed=sh.rank_seed(1237, rank), n_seqs=16, num_blocks=16384)
tokens, ms = sh.reduce_step(float(w.n_seqs), 10.0 + 5.0 * rank, dist, None)
mine = sh.deal_sequences(wl.make("cfg3").ctx, world, rank)
cnt = torch.tensor([float(mine.size)], dtype=torch.float64)
dist.all_reduce(cnt)
if rank == 0:
    print("RESULT", tokens, ms, int(cnt.item()), flush=True)
dist.destroy_process_group()
'''


def test_two_rank_reduction_over_gloo(pkv, tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29533", str(script), ROOT]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=env)
    assert r.returncode == 0, r.stdout + r.stderr
    line = [l for l in r.stdout.splitlines() if l.startswith("RESULT")][0].split()
    assert float(line[1]) == 32.0      # tokens summed over both ranks
    assert float(line[2]) == 15.0      # the slower rank's time
    assert int(line[3]) == 256         # every sequence of the shared batch owned exactly once


def test_head_slices_partition_the_heads():
    import importlib
    sh = importlib.import_module("llm-engine_b200.sharding")
    for qh, kvh, world in ((32, 4, 2), (32, 4, 4), (14, 2, 2), (8, 8, 8)):
        seen_q, seen_kv = [], []
        for r in range(world):
            q0, ql, kv0, kvl = sh.head_slices(qh, kvh, world, r)
            assert ql * kvh == qh * kvl                       # whole GQA groups
            seen_q += list(range(q0, q0 + ql)); seen_kv += list(range(kv0, kv0 + kvl))
        assert seen_q == list(range(qh)) and seen_kv == list(range(kvh))
    import pytest
    with pytest.raises(ValueError):
        sh.head_slices(14, 2, 4, 0)
