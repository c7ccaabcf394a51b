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


def test_tp2_rank_leaves_between_steps_and_the_other_learns_on_the_host():
    """No GPU is faulted: the leaving rank has nothing in flight, NVLS and multicast are off,
    and the surviving rank finds out from the store before it launches its next step."""
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1", DASER_TP_HEALTH_TIMEOUT="3")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29519", os.path.join(here, "tp_leave_worker.py")]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=200, env=env)
    tail = (proc.stdout + proc.stderr)[-3000:]
    assert proc.returncode == 0, tail
    if "TP_LEAVE_SKIPPED" in proc.stdout:
        pytest.skip("symmetric buffers carry a multicast mapping on this box")
    assert "TP_LEAVE_OK" in proc.stdout, tail


def test_pp2_pipeline_stages_match_a_single_gpu():
    """Two pipeline stages of the native engine (NCCL point-to-point hand-over, per-stage store
    files, multi-part commits) produce the tokens of the whole model on one GPU."""
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29521", os.path.join(here, "pp_worker.py")]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=280)
    tail = (proc.stdout + proc.stderr)[-3000:]
    assert proc.returncode == 0, tail
    assert "PP_OK" in proc.stdout, tail
