"""Multi-GPU checks (run as child processes, one per GPU; skipped with fewer than two GPUs)."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _torchrun(script: str, nproc: int, port: int, timeout: int = 600):
    env = dict(os.environ, PYTHONPATH=f"{ROOT}:{ROOT / 'tests'}", MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1", "--master-port", str(port), script]
    res = subprocess.run(cmd, cwd=str(ROOT), env=env, capture_output=True, text=True, timeout=timeout)
    assert res.returncode == 0, res.stdout[-4000:] + res.stderr[-4000:]
    return res.stdout


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tensor_parallel_decoder_two_gpus():
    out = _torchrun(str(ROOT / "tests" / "multi_gpu_tp_worker.py"), 2, 29571)
    assert "TP_OK" in out


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_expert_parallel_moe_two_gpus():
    out = _torchrun(str(ROOT / "tests" / "multi_gpu_ep_worker.py"), 2, 29573)
    assert "EP_OK" in out


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_sharded_parameters_two_gpus():
    out = _torchrun(str(ROOT / "tests" / "multi_gpu_zero3_worker.py"), 2, 29575)
    assert "ZERO3_OK" in out
