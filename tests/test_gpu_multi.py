"""Multi-GPU checks (skipped unless at least two GPUs are visible): the fused peer-memory engine against NCCL."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_engine_matches_nccl_engine_on_two_gpus():
    worker = os.path.join(os.path.dirname(__file__), "multi_gpu_worker.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                          "--master-port", "29611", worker], capture_output=True, text=True, timeout=900, env=env)
    assert "MULTI_GPU_ENGINE_OK" in out.stdout, out.stdout[-3000:] + out.stderr[-3000:]
