"""Tensor-parallel parity on as many GPUs as the box has (2, 4, 8); skipped on a single GPU."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _ngpus() -> int:
    import torch
    return torch.cuda.device_count()


@pytest.mark.parametrize("n,batch", [(2, 1), (2, 2), (4, 1), (4, 3), (8, 1), (8, 2)])
def test_tensor_parallel_matches_oracle(n, batch):
    """batch 1: the reduce runs in the next projection's prologue; batch >= 2: in the norm+quantise launch."""
    if _ngpus() < n:
        pytest.skip(f"needs {n} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", str(29500 + n), os.path.join(ROOT, "tests", "tp_worker.py"), "24", str(batch)]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert f"TP{n} OK" in out.stdout
