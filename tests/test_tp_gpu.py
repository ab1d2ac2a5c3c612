"""Tensor-parallel fused kernels on real GPUs (2 ranks, one process per GPU). See workers/tp_worker.py."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(world, env_extra=None, port=29541):
    env = dict(os.environ)
    env.update({"NCCL_NVLS_ENABLE": "0"})
    env.update(env_extra or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "workers", "tp_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=150)
    assert r.returncode == 0 and "TP_WORKER_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tp2_fused():
    _run(2)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tp2_nccl_baseline_mode():
    _run(2, {"SKEIN_COMM": "nccl"}, port=29542)


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")
def test_tp4_fused():
    _run(4, port=29543)
