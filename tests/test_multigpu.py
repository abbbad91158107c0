"""Launches the multi-GPU worker under torchrun when at least two GPUs are visible."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def test_fused_collectives_and_tp_engine():
    n = min(torch.cuda.device_count(), 8)
    n = 1 << (n.bit_length() - 1)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                        "--master-addr", "127.0.0.1", "--master-port", "29611",
                        os.path.join(root, "tests", "mgpu_worker.py")],
                       capture_output=True, text=True, timeout=600, env=env, cwd=root)
    assert r.returncode == 0 and "MGPU_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_tensor_parallel_serving_stack():
    """Scheduler + control channel + one worker per GPU + engine backend (fused all-reduce workspace,
    sequence-parallel prefill): what ``launch --gpus N -- serve`` assembles, on real GPUs."""
    n = min(torch.cuda.device_count(), 8)
    n = 1 << (n.bit_length() - 1)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                        "--master-addr", "127.0.0.1", "--master-port", "29631",
                        os.path.join(root, "tests", "mgpu_serve.py")],
                       capture_output=True, text=True, timeout=600, env=env, cwd=root)
    assert r.returncode == 0 and "MGPU_SERVE_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
