"""Sharded training on CPU ranks (gloo): every strategy must match one device, and the
collective counts must be the ones the layouts call for (train/sharded_test.go:84-274)."""
import json
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(strategy, world=4, port=29561):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "_mesh_worker.py"), strategy]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=240)
    assert out.returncode == 0, out.stdout[-1500:] + out.stderr[-3000:]
    res = [json.loads(l[7:]) for l in out.stdout.splitlines() if l.startswith("RESULT ")]
    assert len(res) == world
    return res


@pytest.mark.parametrize("strategy,port", [("dp", 29561), ("tp", 29562), ("fsdp", 29563), ("dpxtp", 29564),
                                            ("fsdpxtp", 29565)])
def test_sharded_matches_one_device(strategy, port):
    res = _run(strategy, 4, port)
    for r in res:
        assert r["diff"] < 2e-5, r
        for a, b in zip(r["losses"], r["ref_losses"]):
            assert abs(a - b) < 2e-4, r
    r = res[0]
    if strategy == "dp":
        assert r["fwd"] == {"ar": 0, "ag": 0, "rs": 0}
        assert r["step"]["ar"] == r["params"] + 1 and r["step"]["ag"] == 0  # gradients + the loss
    if strategy == "tp":
        assert r["fwd"] == {"ar": 2, "ag": 0, "rs": 0}  # attention out + MLP down of a GPT-2 block
    if strategy == "fsdp":
        assert r["fwd"]["ar"] == 0 and r["fwd"]["ag"] > 0 and r["fwd"]["rs"] == 0
        assert r["step"]["ag"] == r["step"]["rs"]  # gathered once, gradient scattered once per sharded tensor


def test_tensor_shard_unshard_and_relayout():
    res = _run("layouts", 4, 29566)
    assert all(r["ok"] for r in res), res
