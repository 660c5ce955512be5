"""Graph sections written by the reference itself run here and give its expected outputs.

The nine sample models the reference ships (exported from PyTorch and ONNX, and a quantized Llama
converted from GGUF, each with an ``expected.json`` produced by the exporting framework) are decoded
by ``io/mmfg.py`` and run by the graph interpreter; tolerances are the reference's own
(io/mim/mim_test.go:141-260, session_test.go:28-100)."""
import base64
import json
import os

import numpy as np
import pytest
import torch

from _refdir import reference_dir

REF = reference_dir()
pytestmark = pytest.mark.skipif(REF is None, reason="no checkout of the reference (MIMIR_REFERENCE_DIR)")
DT = {"f32": np.float32, "i64": np.int64, "i32": np.int32, "f16": np.float16, "bool": np.bool_}


def _dec(t, default="f32"):
    a = np.frombuffer(base64.b64decode(t["data"]), dtype=DT[t.get("dtype", default)]).reshape(t["shape"])
    return torch.from_numpy(a.copy())


def _near(got, want, tol):
    got, want = got.float().reshape(-1), want.float().reshape(-1)
    assert got.shape == want.shape
    scale = max(want.abs().max().item(), 1e-30)
    err = (got - want).abs().max().item() / scale
    assert err <= tol, f"relative error {err} above {tol}"


def _models(kind):
    base = os.path.join(REF, "io", "mim", "testdata", kind)
    with open(os.path.join(base, "expected.json")) as f:
        return base, json.load(f)


@pytest.mark.parametrize("name", ["tiny-cnn", "audio", "tiny-gpt", "tiny-llama", "tiny-llama-kv"])
def test_pytorch_exports_match_pytorch(name):
    import mimir_b200.tensor as T
    from mimir_b200.io import mim
    T.set_default_device(T.CPU())
    base, exp = _models("pytorch")
    model = [m for m in exp["models"] if m["name"] == name][0]
    m = mim.open(os.path.join(base, model["mim"]))
    # the key-value cache model keeps its cache from one run to the next: a session
    runner = m.new_session() if name.endswith("-kv") else m
    for run in model["runs"]:
        out = runner.run({k: _dec(v) for k, v in run["inputs"].items()})
        assert set(out) == set(run["outputs"])
        for k, v in run["outputs"].items():
            _near(out[k].data(), _dec(v), exp["tolerance"])


def test_onnx_conversion_matches_onnxruntime():
    import mimir_b200.tensor as T
    from mimir_b200.io import mim
    T.set_default_device(T.CPU())
    base, exp = _models("onnx")
    m = mim.open(os.path.join(base, exp["mim"]))
    for run in exp["runs"]:
        out = m.run({k: _dec(v) for k, v in run["inputs"].items()})
        for k, v in run["outputs"].items():
            _near(out[k].data(), _dec(v), exp["tolerance"])


@pytest.mark.parametrize("name,tol,use_abs", [("exact", 2e-5, False), ("f16-cache", 1e-3, False), ("a8", 1.5, True)])
def test_quantized_llama_graphs_match_the_float64_oracle(name, tol, use_abs):
    """Prompt logits and eight greedy steps of the Q4_K_M Llama graphs: weights decoded and products in
    float32 ("exact"), an fp16 cache, and activations rounded to 8 bits as llama.cpp does ("a8", held to
    1.5 x llama.cpp's own distance from the oracle)."""
    import mimir_b200.tensor as T
    from mimir_b200.io import mim
    T.set_default_device(T.CPU())
    base, e = _models("llama")
    flo = lambda s: torch.from_numpy(np.frombuffer(base64.b64decode(s), dtype=np.float32).copy())  # noqa: E731
    m = mim.open(os.path.join(base, f"tiny-q4km-{name}.mim"))
    s = m.new_session()

    def step(ids, pos):
        out = s.run({"tokens": torch.tensor([ids], dtype=torch.int32),
                     "positions": torch.tensor([list(range(pos, pos + len(ids)))], dtype=torch.int32)})
        return out["logits"].data().float().reshape(-1)

    def compare(got, want):
        _near(got, want, tol * e["llama_cpp_max_diff"] / max(want.abs().max().item(), 1e-30) if use_abs else tol)
    allv = step(e["prompt_ids"], 0)
    compare(allv, flo(e["prompt_logits"]))
    logits, pos = allv[-e["vocab"]:], len(e["prompt_ids"])
    for i, want in enumerate(e["greedy"]):
        compare(logits, flo(e["greedy_logits"][i]))
        if not use_abs:
            assert int(logits.argmax()) == want, f"step {i}"
        logits = step([want], pos)
        pos += 1
