"""Head-sharded decode variant on two and on four GPUs of one box: the exchange fused into the merge
kernel (peer stores over NVLink, bounded flag wait) must leave the checker's output on every rank."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("world", [2, 4])
def test_every_rank_ends_with_the_full_output(torch_cuda, world):
    n = torch_cuda.cuda.device_count()
    if n < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29533 + world), os.path.join(ROOT, "tests", "head_sharded_worker.py")]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("matches the checker") == world
