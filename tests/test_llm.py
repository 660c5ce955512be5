"""LLM loader, KV-cache decoding, tokenizers, sampler, LoRA (reference: llm/llm_test.go,
examples/llama/tokenizer_test.go, llama_test.go)."""
import os

import pytest
import torch

import mimir_b200.tensor as T
from mimir_b200 import llm, nn, optim
from mimir_b200.io import mim


def _tiny(arch="llama"):
    nn.manual_seed(0)
    c = llm.Config(arch=arch, vocab=50, context=32, embed=32, hidden=64, layers=2, heads=4, kv_heads=2, head_dim=8,
                   rope_dim=8, rope_base=10000.0)
    return llm.Model(c)


@pytest.mark.parametrize("arch", ["llama", "qwen2"])
def test_save_load_and_cached_decoding_matches_full_forward(tmp_path, arch):
    m = _tiny(arch)
    p = os.path.join(tmp_path, "m.mim")
    m.save(p)
    m2 = llm.Model.load(p)
    assert m2.cfg == m.cfg
    toks = torch.randint(0, 50, (1, 9))
    full = m.logits(T.from_torch(toks)).data()
    assert torch.allclose(m2.logits(T.from_torch(toks)).data(), full, atol=1e-5)
    caches = m.new_caches(1, 16)
    a = m.logits(T.from_torch(toks[:, :5]), caches).data()
    steps = [m.logits(T.from_torch(toks[:, i:i + 1]), caches).data() for i in range(5, 9)]
    assert torch.allclose(torch.cat([a] + steps, 1), full, atol=1e-4)


def test_config_errors():
    with pytest.raises(T.ErrUnsupported):
        llm.Config.from_metadata({"general.architecture": "gptj"})
    with pytest.raises(T.ErrShape) as e:
        llm.Config.from_metadata({"general.architecture": "llama", "llama.embedding_length": 32, "llama.block_count": 2,
                                  "llama.attention.head_count": 3, "llama.attention.head_count_kv": 2})
    assert "feed_forward_length" in str(e.value) and "3 heads" in str(e.value)


def test_loss_score_embedding_and_quantized_file(tmp_path):
    m = _tiny()
    seqs = [[1, 2, 3, 4, 5], [6, 7, 8]]
    learn = [[False, False, True, True, True], [False, True, True]]
    l_all, l_some = float(m.loss(seqs).data()), float(m.loss(seqs, learn).data())
    s_loss, right, total = m.score(seqs, learn)
    assert total == 5 and abs(s_loss - l_some) < 1e-5 and l_all != l_some and 0 <= right <= 5
    e = m.embedding([1, 2, 3])
    assert e.shape == (32,) and abs(float(e.norm()) - 1) < 1e-5
    with pytest.raises(T.ErrShape):
        m.loss([[1]])
    with pytest.raises(T.ErrIndex):
        m.loss([[1, 99]])
    # a file whose projections are Q8_0 loads by dequantising them
    from mimir_b200.ops.quant import Q8_0, quantize_q8_0
    tensors = {n: p._data for n, p in m._file_tensors()}
    w = tensors["blk.0.ffn_up.weight"]
    tensors["blk.0.ffn_up.weight"] = mim.QuantizedTensor(Q8_0, w.shape, quantize_q8_0(w).reshape(-1))
    p = os.path.join(tmp_path, "q.mim")
    mim.write_tensors(p, tensors, metadata=m.cfg.metadata())
    mq = llm.Model.load(p)
    assert (mq.blocks[0].up.weight._data - w).abs().max() < 0.01 * w.abs().max() + 1e-3


def test_lora_trains_only_adapters_and_round_trips(tmp_path):
    m = _tiny()
    base = m.logits(T.from_torch(torch.tensor([[1, 2, 3]]))).data().clone()
    m.add_lora(rank=2, alpha=4.0, targets=("q", "v"))
    ad = m.adapters()
    assert len(ad) == 2 * 2 * 2 and all(p.trainable for p in ad)
    assert torch.allclose(m.logits(T.from_torch(torch.tensor([[1, 2, 3]]))).data(), base, atol=1e-6)   # B starts at zero
    opt = optim.Adam(ad, lr=1e-2)
    frozen = m.blocks[0].q.base.weight._data.clone()
    first = None
    for _ in range(15):
        loss = m.loss([[1, 2, 3, 4, 5, 6]])
        for p in ad:
            p.zero_grad()
        T.backward(loss)
        first = first or float(loss.data())
        last = float(loss.data())
        opt.step()
    assert last < first and torch.equal(m.blocks[0].q.base.weight._data, frozen)
    p = os.path.join(tmp_path, "a.mim")
    m.write_adapter(p, base="tiny", name="t")
    m2 = _tiny()
    m2.read_adapter(p)
    x = T.from_torch(torch.tensor([[1, 2, 3, 4]]))
    assert torch.allclose(m2.logits(x).data(), m.logits(x).data(), atol=1e-5)
    w = m.tp_weights()
    assert w["blk.0.qkv"].shape == (4 * 8 + 2 * 2 * 8, 32) and w["blk.1.gate_up"].shape == (128, 32)


def test_sentencepiece_and_bpe_tokenizers():
    toks = ["<unk>", "<s>", "</s>"] + [f"<0x{b:02X}>" for b in range(256)] + ["▁", "h", "e", "l", "o", "▁h", "he", "ll", "▁he", "llo", "▁hello", "▁w", "or", "ld"]
    scores = [0.0] * 259 + [-1, -2, -2, -2, -2, -3, -4, -5, -1.5, -4.5, -0.5, -6, -7, -8]
    types = [2, 3, 3] + [6] * 256 + [1] * 14
    sp = llm.tokenizer_from_metadata({"tokenizer.ggml.model": "llama", "tokenizer.ggml.tokens": toks, "tokenizer.ggml.scores": scores,
                                      "tokenizer.ggml.token_type": types, "tokenizer.ggml.bos_token_id": 1, "tokenizer.ggml.eos_token_id": 2})
    ids = sp.encode("hello hello")
    assert ids == [1, toks.index("▁hello"), toks.index("▁hello")]
    assert sp.decode(ids) == "hello hello"
    z = sp.encode("hé", bos=False)     # é is not in the vocabulary: two UTF-8 byte tokens
    assert z[:1] == [toks.index("▁h")] and z[1:] == [3 + 0xC3, 3 + 0xA9] and sp.decode(z) == "hé"

    b2u = llm.tokenizer._byte_table()
    sym = lambda s: "".join(b2u[b] for b in s.encode())  # noqa: E731
    vocab = [b2u[b] for b in range(256)] + [sym("he"), sym("ll"), sym("hell"), sym(" w"), "<|eot|>"]
    merges = [f"{sym('h')} {sym('e')}", f"{sym('l')} {sym('l')}", f"{sym('he')} {sym('ll')}", f"{sym(' ')} {sym('w')}"]
    bpe = llm.tokenizer_from_metadata({"tokenizer.ggml.model": "gpt2", "tokenizer.ggml.tokens": vocab, "tokenizer.ggml.merges": merges})
    ids = bpe.encode("hello w<|eot|>é")
    assert ids[:3] == [258, vocab.index(sym("o")), 259] and ids[3] == 260 and len(ids) == 6
    assert bpe.decode(ids) == "hello w<|eot|>é"


def test_sampler_filters_and_generate():
    lg = torch.tensor([2.0, 1.0, 0.5, -1.0, -3.0])
    assert llm.Sampler(temperature=0).sample(lg) == 0
    p = llm.Sampler(temperature=1.0, top_k=3, top_p=1.0).distribution(lg)
    assert (p[3:] == 0).all() and abs(float(p.sum()) - 1) < 1e-6
    p = llm.Sampler(temperature=1.0, top_k=0, top_p=0.6).distribution(lg)
    assert (p > 0).sum() == 1 + int(torch.softmax(lg, 0)[0] < 0.6)
    p = llm.Sampler(temperature=1.0, top_k=0, top_p=1.0, repeat_penalty=2.0).distribution(lg, history=[0])
    assert p[0] < torch.softmax(lg, 0)[0]
    s1 = [llm.Sampler(seed=3).sample(lg) for _ in range(1)]
    assert s1 == [llm.Sampler(seed=3).sample(lg)]
    m = _tiny()
    out = llm.generate(m, [1, 2, 3], 6)
    full = [1, 2, 3]
    for _ in range(6):
        full.append(int(m.logits(T.from_torch(torch.tensor([full]))).data()[0, -1].argmax()))
    assert out == full[3:]
