"""Fused tensor-parallel path on 2 GPUs of one box (child processes under torchrun)."""

import os
import subprocess
import sys

import pytest

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def test_tp2_forward_and_engine_match_single_gpu():
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29517", os.path.join(here, "tp_worker.py")]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=280)
    tail = (proc.stdout + proc.stderr)[-3000:]
    assert proc.returncode == 0, tail
    assert "TP_OK" in proc.stdout, tail
