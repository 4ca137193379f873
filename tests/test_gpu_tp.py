"""Tensor-parallel decode on two GPUs (skipped on a single-GPU box; the multi-rank arithmetic
itself is also covered on one GPU by test_gpu_tp_folded.py). The ranks are launched with
torchrun, as a deployment would; the check itself is tests/tp_check.py: all ranks decode the
same tokens, the exchanged token is the argmax of the gathered logits, logits agree with the
single-GPU fused decoder (rel-L2 <= 1e-2) and with the reference's real-mode logits
(rel-L2 <= 2e-2), for every all-reduce route (folded into the GEMVs, eager and graphed; the
separate peer-memory kernel; NCCL)."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_two_gpu_decode_matches_single_gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29533", os.path.join(here, "tp_check.py")]
    done = subprocess.run(cmd, capture_output=True, text=True, timeout=170, env=env)
    assert "TP_CHECK_OK" in done.stdout, done.stdout[-2000:] + done.stderr[-2000:]
