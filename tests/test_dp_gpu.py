"""Fused data-parallel step on 2 GPUs == single-device training on the whole batch."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(world, graph):
    env = dict(os.environ, MIMIR_TEST_GRAPH="1" if graph else "0", NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", "29533", os.path.join(HERE, "_dp_worker.py")]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    return [json.loads(l[7:]) for l in out.stdout.splitlines() if l.startswith("RESULT ")]


@pytest.mark.parametrize("graph", [False, True])
def test_dp2_matches_single_device(graph):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    res = _run(2, graph)
    assert len(res) == 2
    for r in res:
        assert r["err"] == 0
        assert r["identical"], "replicas diverged"
        assert r["restore_exact"], "a data-parallel checkpoint did not restore bit for bit"
        assert r["resume_max_diff"] < 1e-3 and r["resume_frac_diff"] < 0.02, r
        assert r["err2"] == 0
    r0 = [r for r in res if r["rank"] == 0][0]
    for a, b in zip(r0["losses"], r0["single"]):
        assert abs(a - b) < 3e-2, (r0["losses"], r0["single"])
    assert r0["losses"][-1] < r0["losses"][0]
    assert r0["max_param_diff"] < 2e-2


def test_bounded_peer_wait_reports_timeout():
    """A wait on a flag that nothing sets ends by itself and sets the error word."""
    from mimir_b200 import _native
    from mimir_b200.ops._util import check_error_word
    lib = _native.lib()
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    check_error_word()
    lib.mimir_peer_wait_probe(flag.data_ptr(), 1, 200, status.data_ptr(),
                              torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert status.item() == 2
    assert check_error_word() & 8
    # and a satisfied wait returns at once without touching the word
    flag.fill_(1)
    lib.mimir_peer_wait_probe(flag.data_ptr(), 1, 200, status.data_ptr(),
                              torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert status.item() == 1
    assert check_error_word() == 0
