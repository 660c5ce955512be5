"""The partitioner on CPU ranks (gloo): a model with an embedding, layer norms, attention over split
heads, reshapes that carry a split and a loss over a ``P("data")`` batch, sharded by the layout rules
alone.  Every strategy must match one device, and the collectives must be the ones the reference's
contract names (train/sharded_test.go:84-274): dp = no collective in the forward pass, all-reduces in
the step; tp = one all-reduce per row-parallel layer in the forward pass; fsdp = one all-gather per
parameter forward, and a step of `params` all-gathers + `params` reduce-scatters + 1 all-reduce."""
import json
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(strategy, world=4, port=29581):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "_spmd_worker.py"), strategy]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=240)
    assert out.returncode == 0, out.stdout[-1500:] + out.stderr[-3000:]
    res = [json.loads(l[7:]) for l in out.stdout.splitlines() if l.startswith("RESULT ")]
    assert len(res) == world
    return res


@pytest.mark.parametrize("strategy,port", [("dp", 29581), ("tp", 29582), ("fsdp", 29583), ("dpxtp", 29584),
                                            ("fsdpxtp", 29585)])
def test_partitioned_model_matches_one_device(strategy, port):
    res = _run(strategy, 4, port)
    for r in res:
        assert r["fdiff"] < 2e-5, r
        assert r["diff"] < 2e-5, r
        for a, b in zip(r["losses"], r["ref_losses"]):
            assert abs(a - b) < 2e-4, r
        assert r["analysed"] <= 1, r          # three steps, one analysis: later steps reuse it by structure
    r = res[0]
    if strategy == "dp":
        assert r["fwd"] == {"ar": 0, "ag": 0, "rs": 0}
        assert r["out_layout"][0] == "data"
        assert r["step"] == {"ar": r["params"] + 1, "ag": 0, "rs": 0}        # every gradient + the loss
    if strategy == "tp":
        assert r["fwd"] == {"ar": 2, "ag": 0, "rs": 0}                       # attention out + MLP down
    if strategy == "fsdp":
        assert r["fwd"] == {"ar": 0, "ag": r["params"], "rs": 0}
        assert r["step"] == {"ar": 1, "ag": r["params"], "rs": r["params"]}  # backward reuses the gathered weights


def test_fit_sharded_equals_fit_on_one_device():
    res = _run("fit", 4, 29586)
    for r in res:
        assert r["diff"] < 5e-5, r
        for a, b in zip(r["l1"], r["l2"]):
            assert abs(a - b) < 2e-4, r
