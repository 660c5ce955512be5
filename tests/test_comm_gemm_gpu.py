"""Fused all-gather->GEMM and GEMM->reduce-scatter on 2 GPUs against fp32 references."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def test_fused_collective_gemms_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29547", os.path.join(HERE, "_comm_gemm_worker.py")]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout[-1500:] + out.stderr[-3000:]
    res = [json.loads(l[7:]) for l in out.stdout.splitlines() if l.startswith("RESULT ")]
    assert len(res) == 2
    for r in res:
        assert r["err"] == 0, r
        assert r["ag_err"] < 2e-2 and r["rs_err"] < 2e-2 and r["rs_tn_err"] < 2e-2, r
        assert r["rs_b2b_err"] < 2e-2, r      # six calls in a row, no host barrier, ranks out of step
