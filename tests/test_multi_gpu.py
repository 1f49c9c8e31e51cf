"""The tensor-parallel path on real GPUs: runs tests/tp_worker.py under torchrun on every visible GPU count of 2, 4, 8
(skipped on a single-GPU box; the host logic of N > 1 is covered on CPU by tests/test_tp_cpu.py).  The worker checks
the push all-reduce against NCCL and an exact fp32 sum, the fused multiply + all-reduce against the separate one bit
for bit and against the fp64 oracle of the unsharded layer, eager and from a replayed CUDA graph."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tensor_parallel_ranks(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs, {torch.cuda.device_count()} visible")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    port = 29700 + (os.getpid() + 7 * world) % 200
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(ROOT, "tests", "tp_worker.py")]
    res = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    tail = (res.stdout + res.stderr)[-4000:]
    assert res.returncode == 0 and "tp_worker ok" in res.stdout, tail
