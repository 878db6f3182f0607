"""Host-side pieces of bench.py that the GPU never sees: the CPU arm must build the same step as the
product arm without importing the product, and the strong-scaling deal must cover the batch once."""
import importlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def test_cpu_arm_packs_the_step_like_the_library(pkv):
    """bench.pack_step_numpy restates CudaModel::upload_step_indices (src/model/cuda/cuda_model.cu:453-473)
    in numpy so that `bench.py --impl reference` loads nothing of the product; it must give the integers
    pkv_step_pack gives, on every configuration."""
    import bench
    wl = bench.load_workloads_standalone()
    for name in ("cfg1", "cfg2", "cfg3", "cfg4", "cfg5"):
        w = wl.make(name)
        a = bench.pack_step_numpy(w)
        tabs, pos, _ = w.step_tokens()
        b = pkv.pack_step(tabs, pos, w.block_size)
        for key in ("slots", "token_seq", "token_pos", "block_tables", "table_offset"):
            assert np.array_equal(a[key], getattr(b, key)), (name, key)
        assert a["n_tokens"] == b.n_tokens


def test_strong_scaling_deal_is_a_partition_with_even_bytes(pkv):
    sharding = importlib.import_module("llm-engine_b200.sharding")
    wl = importlib.import_module("llm-engine_b200.workloads")
    w = wl.make("cfg3")
    for world in (2, 4, 8):
        owned = [sharding.deal_sequences(w.ctx, world, r, "balanced") for r in range(world)]
        assert sorted(np.concatenate(owned).tolist()) == list(range(w.n_seqs))
        loads = [int((w.ctx[o] + 1).sum()) for o in owned]
        assert max(loads) - min(loads) <= int(w.ctx.max()) // 64      # within a sixty-fourth of the longest context
