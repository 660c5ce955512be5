"""The host decoder over quantized weights against the float model (reference: llm/decode_test.go:
the recorded CPU decode step equals ``Logits`` with caches)."""
import os

import pytest
import torch

import mimir_b200.tensor as T
from mimir_b200 import llm, nn
from mimir_b200.io import mim
from mimir_b200.ops import quant as Q
from mimir_b200.ops import quant_cpu


def _model(arch="llama", embed=256, hidden=512):
    nn.manual_seed(1)
    c = llm.Config(arch=arch, vocab=96, context=48, embed=embed, hidden=hidden, layers=2, heads=4, kv_heads=2, head_dim=embed // 4,
                   rope_dim=embed // 4, rope_base=10000.0)
    return llm.Model(c)


@pytest.mark.parametrize("arch", ["llama", "qwen2"])
def test_float_weights_exact_mode_equals_the_model_with_caches(arch):
    m = _model(arch)
    dec = llm.CPUDecoder.from_model(m, batch=2, cap=16, mode="exact", float_as="f32")
    toks = torch.randint(0, 96, (2, 7))
    caches = m.new_caches(2, 16)
    for t in range(7):
        want = m.logits(T.from_torch(toks[:, t:t + 1]), caches).data()[:, 0]
        got = dec.step(toks[:, t])
        assert torch.allclose(got, want, atol=2e-4, rtol=1e-4), t
    assert dec.len == 7
    dec.reset()
    assert torch.allclose(dec.prefill(toks), want, atol=2e-4, rtol=1e-4)              # all positions in one pass
    dec.reset()
    assert torch.allclose(dec.prefill(toks, chunk=3), want, atol=2e-4, rtol=1e-4)     # chunks of 3, 3 and 1 positions
    assert dec.len == 7


def _quantized_file(tmp_path, m):
    """The model's file with every projection as Q8_0 blocks and the rest float."""
    tensors = {}
    for n, p in m._file_tensors():
        w = p._data
        if w.dim() == 2 and n != "token_embd.weight":
            tensors[n] = mim.QuantizedTensor(Q.Q8_0, w.shape, Q.quantize_q8_0(w).reshape(-1))
        else:
            tensors[n] = w
    path = os.path.join(tmp_path, "q.mim")
    mim.write_tensors(path, tensors, metadata=m.cfg.metadata())
    return path


def test_quantized_file_stays_quantized_and_matches_the_dequantised_model(tmp_path):
    m = _model()
    path = _quantized_file(tmp_path, m)
    ref = llm.Model.load(path)                                   # dequantises at load
    dec = llm.CPUDecoder.load(path, cap=16, mode="exact", float_as="f32")
    float_bytes = sum(p._data.numel() * 4 for _, p in m._file_tensors())
    assert dec.weight_bytes() < 0.5 * float_bytes               # blocks, not floats (the embedding stays float here)
    assert dec.layers[0]["qkv"] is not None and dec.layers[0]["gate_up"] is not None       # fused rows
    toks = torch.randint(0, 96, (1, 6))
    caches = ref.new_caches(1, 16)
    for t in range(6):
        want = ref.logits(T.from_torch(toks[:, t:t + 1]), caches).data()[:, 0]
        got = dec.step(toks[:, t])
        assert torch.allclose(got, want, atol=5e-4, rtol=1e-3), t
    if quant_cpu.has_int8():
        fast = llm.CPUDecoder.load(path, cap=16, mode="int8", float_as="f32")
        a, b = dec.generate(toks, 0), fast.generate(toks, 0)     # prefill only
        dec.reset(), fast.reset()
        la, lb = dec.prefill(toks), fast.prefill(toks)
        assert float((la - lb).abs().max()) < 3e-2 * float(la.abs().max())
        assert a.shape == b.shape == (1, 0)


def test_mixed_encodings_fall_back_to_separate_products_and_generate_is_greedy(tmp_path):
    m = _model()
    tensors = {n: p._data for n, p in m._file_tensors()}
    w = tensors["blk.0.attn_v.weight"]
    blocks = torch.zeros(w.numel() // 256, 210, dtype=torch.uint8)          # an all-zero Q6_K matrix beside float q and k
    tensors["blk.0.attn_v.weight"] = mim.QuantizedTensor(Q.Q6_K, w.shape, blocks.reshape(-1))
    dec = llm.CPUDecoder(m.cfg, tensors, cap=24, mode="exact", float_as="f32")
    assert dec.layers[0]["qkv"] is None and dec.layers[1]["qkv"] is not None
    prompt = torch.randint(0, 96, (1, 4))
    out = dec.generate(prompt, 5)
    assert out.shape == (1, 5) and dec.len == 4 + 5
    dec.reset()
    again = dec.generate(prompt, 5)
    assert torch.equal(out, again)
    drawn = llm.CPUDecoder(m.cfg, tensors, cap=24, mode="exact", float_as="f32").generate(prompt, 3, llm.Sampler(temperature=0.0))
    assert torch.equal(drawn, out[:, :3])
    with pytest.raises(IndexError):
        dec.generate(prompt, 40)


@pytest.mark.parametrize("mode,tol", [("exact", 2e-5), ("int8", None)])
def test_reference_q4_k_m_sample_prompt_logits_and_greedy_steps(mode, tol):
    """The reference's tiny Q4_K_M Llama (Q4_K projections and embedding, Q6_K output head) with its
    float64 oracle: logits after every prompt token, then eight greedy steps.  The int8 path is held to
    1.5 x the distance llama.cpp itself has from that oracle, like the reference's own a8 variant."""
    import base64
    import json

    import numpy as np
    from tests._refdir import reference_dir
    root = reference_dir()
    base = os.path.join(root or "", "io", "mim", "testdata", "llama")
    if not os.path.exists(os.path.join(base, "expected.json")):
        pytest.skip("reference samples not present")
    if mode == "int8" and not quant_cpu.has_int8():
        pytest.skip("this CPU has no AVX-512 VNNI")
    e = json.load(open(os.path.join(base, "expected.json")))
    flo = lambda s: torch.from_numpy(np.frombuffer(base64.b64decode(s), dtype=np.float32).copy())  # noqa: E731
    dec = llm.CPUDecoder.load(os.path.join(base, "tiny-q4km-exact.mim"), cap=32, mode=mode)
    assert dec.embed.code == Q.Q4_K and dec.head.code == Q.Q6_K and dec.layers[0]["qkv"].code == Q.Q4_K

    def near(got, want):
        if tol is not None:
            assert float((got - want).abs().max()) <= tol * max(float(want.abs().max()), 1.0), float((got - want).abs().max())
        else:
            assert float((got - want).abs().max()) <= 1.5 * e["llama_cpp_max_diff"]
    want_all = flo(e["prompt_logits"]).view(len(e["prompt_ids"]), e["vocab"])
    for t, tok in enumerate(e["prompt_ids"]):
        logits = dec.step(torch.tensor([tok]))[0]
        near(logits, want_all[t])
    for i, want in enumerate(e["greedy"]):
        near(logits, flo(e["greedy_logits"][i]))
        if tol is not None:
            assert int(logits.argmax()) == want, i
        logits = dec.step(torch.tensor([want]))[0]


def test_a_long_prompt_runs_on_expanded_weights_and_agrees_with_the_exact_products(tmp_path):
    """Chunks of 32 activation rows or more expand each quantized matrix to bfloat16 once and multiply there;
    the logits stay within bfloat16's precision of the exact products, and shorter chunks are untouched."""
    m = _model()
    path = _quantized_file(tmp_path, m)
    exact = llm.CPUDecoder.load(path, cap=48, mode="exact", float_as="f32")
    fast = llm.CPUDecoder.load(path, cap=48, mode="auto", float_as="f32")
    toks = torch.randint(0, 96, (1, 40), generator=torch.Generator().manual_seed(0))
    want = exact.prefill(toks)
    got = fast.prefill(toks)                                     # one chunk of 40 rows: the expanded path
    assert fast.len == 40 and float((got - want).abs().max()) < 3e-2 * float(want.abs().max())
    assert got.argmax(-1).equal(want.argmax(-1))
    nxt = want.argmax(-1)
    assert float((fast.step(nxt) - exact.step(nxt)).abs().max()) < 3e-2 * float(want.abs().max())     # the cache it filled decodes on
    w = quant_cpu.dequant_bf16(Q.Q8_0, fast.layers[0]["o"].data, fast.layers[0]["o"].n, fast.layers[0]["o"].k)
    full = Q.dequantize_raw(Q.Q8_0, fast.layers[0]["o"].data, w.numel()).view(w.shape)
    assert torch.equal(w, full.bfloat16())                       # round to nearest even, bit for bit
    with pytest.raises(ValueError):
        quant_cpu.dequant_bf16(Q.Q8_0, fast.layers[0]["o"].data, 4, 4, torch.empty(3, dtype=torch.bfloat16))


@pytest.mark.parametrize("arch", ["llama", "qwen2"])
@pytest.mark.parametrize("mode", ["exact", "int8"])
def test_the_native_layer_routine_equals_the_tensor_op_path(tmp_path, arch, mode):
    """Single-token steps over block-encoded weights run one native call per layer (normalisations, rotary
    positions, cache append, attention, SwiGLU and residuals included); the tensor-op path that prompts use is
    its oracle, for both rotary orders, with and without projection biases, and after a chunked prompt."""
    if mode == "int8" and not quant_cpu.has_int8():
        pytest.skip("no VNNI on this CPU")
    m = _model(arch)
    path = _quantized_file(tmp_path, m)
    fused = llm.CPUDecoder.load(path, batch=2, cap=24, mode=mode, float_as="f32")
    plain = llm.CPUDecoder.load(path, batch=2, cap=24, mode=mode, float_as="f32", fused_layers=False)
    assert fused.fused_layers and not plain.fused_layers
    assert (fused.layers[0]["qkv_bias"] is not None) == (arch == "qwen2")
    toks = torch.randint(0, 96, (2, 12), generator=torch.Generator().manual_seed(3))
    fused.prefill(toks[:, :5]), plain.prefill(toks[:, :5])
    for t in range(5, 12):
        got, want = fused.step(toks[:, t]), plain.step(toks[:, t])
        assert torch.allclose(got, want, atol=2e-4, rtol=1e-4), t
    assert fused.len == plain.len == 12
    assert torch.allclose(fused.kc, plain.kc, atol=1e-5) and torch.allclose(fused.vc, plain.vc, atol=1e-5)
    with pytest.raises(IndexError):
        for _ in range(13):
            fused.step(toks[:, 0])
