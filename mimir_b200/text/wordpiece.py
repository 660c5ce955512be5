"""WordPiece tokenizer (reference: text/wordpiece.go): basic tokenisation (lower-casing, accent
stripping, punctuation splitting, CJK spacing) then greedy longest-match-first sub-words with the
``##`` continuation prefix."""
from __future__ import annotations

import unicodedata


class WordPiece:
    def __init__(self, vocab, lower: bool = True, unk="[UNK]", cls="[CLS]", sep="[SEP]", pad="[PAD]", mask="[MASK]",
                 max_chars: int = 100):
        self.tokens = list(vocab)
        have = set(self.tokens)
        for special in (pad, unk, cls, sep, mask):          # the special tokens a vocabulary lacks are added at the end
            if special not in have:
                self.tokens.append(special)
                have.add(special)
        self.ids = {t: i for i, t in enumerate(self.tokens)}
        self.lower, self.unk, self.cls, self.sep, self.pad, self.mask, self.max_chars = lower, unk, cls, sep, pad, mask, max_chars

    # -- the vocabulary
    @property
    def size(self) -> int:
        return len(self.tokens)

    def vocab(self) -> list:
        """The tokens in id order, to save and read back."""
        return list(self.tokens)

    def id(self, token: str) -> int:
        return self.ids.get(token, self.ids[self.unk])

    def token(self, i: int) -> str:
        return self.tokens[i] if 0 <= i < len(self.tokens) else self.unk

    @property
    def pad_id(self) -> int:
        return self.ids[self.pad]

    def encode_ids(self, text: str, length: int) -> list:
        """The ids of [CLS], the text's tokens and [SEP], cut or padded with [PAD] to ``length``: one input
        row of a BERT."""
        return self.encode(text, max_len=length)[0]

    @staticmethod
    def from_file(path: str, **kw) -> "WordPiece":
        with open(path, encoding="utf-8") as f:
            return WordPiece([l.rstrip("\n") for l in f], **kw)

    @staticmethod
    def _is_punct(ch: str) -> bool:
        cp = ord(ch)
        return (33 <= cp <= 47 or 58 <= cp <= 64 or 91 <= cp <= 96 or 123 <= cp <= 126
                or unicodedata.category(ch).startswith("P"))

    @staticmethod
    def _is_cjk(cp: int) -> bool:
        return (0x4E00 <= cp <= 0x9FFF or 0x3400 <= cp <= 0x4DBF or 0x20000 <= cp <= 0x2A6DF
                or 0xF900 <= cp <= 0xFAFF or 0x2F800 <= cp <= 0x2FA1F)

    def basic(self, text: str) -> list:
        out, word = [], []

        def flush():
            if word:
                out.append("".join(word))
                word.clear()
        if self.lower:
            text = "".join(c for c in unicodedata.normalize("NFD", text.lower()) if unicodedata.category(c) != "Mn")
        for ch in text:
            cp = ord(ch)
            if cp == 0 or cp == 0xFFFD or (unicodedata.category(ch).startswith("C") and ch not in "\t\n\r"):
                continue
            if ch.isspace():
                flush()
            elif self._is_punct(ch) or self._is_cjk(cp):
                flush()
                out.append(ch)
            else:
                word.append(ch)
        flush()
        return out

    def word_pieces(self, word: str) -> list:
        if len(word) > self.max_chars:
            return [self.unk]
        pieces, start = [], 0
        while start < len(word):
            end, cur = len(word), None
            while start < end:
                sub = ("##" if start else "") + word[start:end]
                if sub in self.ids:
                    cur = sub
                    break
                end -= 1
            if cur is None:
                return [self.unk]
            pieces.append(cur)
            start = end
        return pieces

    def tokenize(self, text: str) -> list:
        return [p for w in self.basic(text) for p in self.word_pieces(w)]

    def encode(self, text: str, pair: str | None = None, max_len: int | None = None):
        """``(ids, type_ids, attention_mask)`` with [CLS] / [SEP], truncated and padded to ``max_len``."""
        a = self.tokenize(text)
        b = self.tokenize(pair) if pair is not None else []
        if max_len is not None:
            budget = max_len - 2 - (1 if b else 0)
            while len(a) + len(b) > budget:
                (a if len(a) >= len(b) else b).pop()
        toks = [self.cls] + a + [self.sep] + (b + [self.sep] if b else [])
        types = [0] * (len(a) + 2) + [1] * (len(b) + 1 if b else 0)
        ids = [self.ids.get(t, self.ids.get(self.unk, 0)) for t in toks]
        mask = [1] * len(ids)
        if max_len is not None:
            padn = max_len - len(ids)
            ids += [self.ids.get(self.pad, 0)] * padn
            types += [0] * padn
            mask += [0] * padn
        return ids, types, mask

    def decode(self, ids) -> str:
        words = []
        for i in ids:
            t = self.tokens[i]
            if t in (self.cls, self.sep, self.pad):
                continue
            if t.startswith("##") and words:
                words[-1] += t[2:]
            else:
                words.append(t)
        return " ".join(words)


def build_vocab(texts, size: int, lower: bool = True) -> list:
    """A vocabulary of at most ``size`` tokens for a BERT taught from scratch on ``texts``: the special
    tokens, every character the texts hold (alone and as a word piece), then the most common words and the
    most common word endings until ``size`` is reached.  Every word of the texts is then read whole or in
    pieces and none is [UNK]."""
    basic = WordPiece([], lower=lower)
    words: dict = {}
    for t in texts:
        for w in basic.basic(t):
            words[w] = words.get(w, 0) + 1
    out = list(basic.tokens)
    seen = set(out)

    def add(tok):
        if tok not in seen and len(out) < size:
            out.append(tok)
            seen.add(tok)
    chars = sorted({c for w in words for c in w})
    for c in chars:
        add(c)
    for c in chars:
        add("##" + c)
    endings: dict = {}
    for w, n in words.items():
        for k in range(1, len(w)):
            e = "##" + w[k:]
            endings[e] = endings.get(e, 0) + n
    by_count = lambda d: [k for k, _ in sorted(d.items(), key=lambda kv: (-kv[1], kv[0]))]  # noqa: E731
    ws, es = by_count({w: n for w, n in words.items() if len(w) > 1}), by_count({e: n for e, n in endings.items() if len(e) > 3})
    for i in range(max(len(ws), len(es))):                 # words and endings in turn, the most common first
        if i < len(ws):
            add(ws[i])
        if i < len(es):
            add(es[i])
        if len(out) >= size:
            break
    return out
