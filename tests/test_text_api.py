"""Vocabularies built from texts, the tokenizer's id interface, and a text classifier that hides padding,
learns, and swaps heads (reference: text/tokenizer.go, text/bert.go and their tests)."""
import torch

import mimir_b200.tensor as T
from mimir_b200 import nn, optim, text


TEXTS = ["Where is my order?", "My order never arrived.", "I love this product!", "The product works great, thanks.",
         "Refund my order please.", "Great quality, love it."]


def test_built_vocabulary_reads_every_word_without_unknowns():
    vocab = text.build_vocab(TEXTS, 80)
    tok = text.WordPiece(vocab)
    assert len(vocab) <= 80 and vocab[:5] == ["[PAD]", "[UNK]", "[CLS]", "[SEP]", "[MASK]"] and tok.size == len(vocab)
    for t in TEXTS:
        assert "[UNK]" not in tok.tokenize(t)
    assert "order" in vocab and tok.tokenize("orders")[0] in ("order", "o")      # read whole or in pieces
    ids = tok.encode_ids("Where is my order?", 12)
    assert len(ids) == 12 and ids[0] == tok.id("[CLS]") and ids[-1] == tok.pad_id and tok.id("[SEP]") in ids
    assert len(tok.encode_ids(" ".join(TEXTS), 8)) == 8 and tok.encode_ids(" ".join(TEXTS), 8)[-1] == tok.id("[SEP]")
    assert tok.token(tok.id("order")) == "order" and tok.token(10 ** 6) == "[UNK]" and tok.id("zebra") == tok.id("[UNK]")
    assert text.WordPiece(tok.vocab()).encode_ids(TEXTS[0], 12) == ids
    plain = text.WordPiece(["a", "b"])
    assert plain.size == 7 and plain.pad_id == 2                                   # missing special tokens go at the end


def test_classifier_hides_padding_learns_and_swaps_heads():
    nn.manual_seed(0)
    tok = text.WordPiece(text.build_vocab(TEXTS, 120))
    cfg = text.BertConfig(vocab=tok.size, dim=32, layers=1, heads=2, hidden=64, max_positions=16, dropout=0.0)
    m = text.TextClassifier(cfg, 2, pad_id=tok.pad_id).eval()
    short = torch.tensor([tok.encode_ids(TEXTS[0], 10)])
    longer = torch.tensor([tok.encode_ids(TEXTS[0], 16)])
    assert torch.allclose(m.features(T.tensor(short)).data(), m.features(T.tensor(longer)).data(), atol=1e-5)
    assert m.encode(T.tensor(longer)).shape == (1, 16, 32) and m.width == 32
    x = torch.tensor([tok.encode_ids(t, 16) for t in TEXTS])
    y = torch.tensor([0, 0, 1, 1, 0, 1])                                          # orders against praise
    m.train()
    opt = optim.Adam(m.parameters(), lr=3e-3)
    for _ in range(60):
        nn.loss.cross_entropy(m(T.tensor(x)), T.tensor(y)).backward()
        opt.step()
        opt.zero_grad()
    m.eval()
    assert (m(T.tensor(x)).data().argmax(1) == y).all()
    m.set_head(4)
    assert m(T.tensor(x)).shape == (6, 4) and len(m.head_parameters()) == 2
    try:
        m(T.tensor(torch.zeros(1, 40, dtype=torch.int64)))
        raise AssertionError("expected ValueError")
    except ValueError:
        pass
    assert text.BertConfig.base().dim == 768 and text.BertConfig.mini().layers == 4 and text.BertConfig.small().dim == 128
