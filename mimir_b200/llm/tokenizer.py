"""Tokenizers built from a model file's ``tokenizer.ggml.*`` metadata (reference:
examples/llama/tokenizer.go, pretokenize.go): SentencePiece-style ("llama": highest-score
pair merging over UTF-8 characters with byte fallback) and byte-level BPE ("gpt2": regex
pre-tokenisation, byte-to-unicode table, ranked merges)."""
from __future__ import annotations

import heapq


def from_metadata(md: dict):
    kind = md.get("tokenizer.ggml.model")
    tokens = md.get("tokenizer.ggml.tokens")
    if tokens is None:
        raise KeyError("no tokenizer.ggml.tokens in the metadata")
    common = dict(bos=md.get("tokenizer.ggml.bos_token_id"), eos=md.get("tokenizer.ggml.eos_token_id"),
                  add_bos=md.get("tokenizer.ggml.add_bos_token", kind == "llama"))
    if kind == "llama":
        return SentencePiece(tokens, md.get("tokenizer.ggml.scores"), md.get("tokenizer.ggml.token_type"), **common)
    if kind == "gpt2":
        return BytePairs(tokens, md.get("tokenizer.ggml.merges", []), pre=md.get("tokenizer.ggml.pre", "gpt2"), **common)
    raise ValueError(f"tokenizer model {kind!r} not supported")


class SentencePiece:
    BYTE = 6  # token type of <0xNN> byte tokens

    def __init__(self, tokens, scores=None, types=None, bos=None, eos=None, add_bos=True, add_space_prefix=True):
        self.tokens = list(tokens)
        self.scores = list(scores) if scores is not None else [0.0] * len(self.tokens)
        self.ids = {t: i for i, t in enumerate(self.tokens)}
        self.bos, self.eos, self.add_bos, self.add_space_prefix = bos, eos, add_bos, add_space_prefix
        self.bytes = {}
        for i, t in enumerate(self.tokens):
            if len(t) == 6 and t.startswith("<0x") and t.endswith(">") and (types is None or types[i] == self.BYTE):
                self.bytes[int(t[3:5], 16)] = i
        self.unk = self.ids.get("<unk>", 0)

    def encode(self, text: str, bos: bool | None = None) -> list:
        out = [self.bos] if (self.add_bos if bos is None else bos) and self.bos is not None else []
        if not text:
            return out
        text = ("▁" if self.add_space_prefix else "") + text.replace(" ", "▁")
        # doubly linked list of symbols; repeatedly merge the adjacent pair with the highest score
        sym = list(text)
        prev = list(range(-1, len(sym) - 1))
        nxt = list(range(1, len(sym) + 1))
        nxt[-1] = -1
        alive = [True] * len(sym)
        heap = []

        def push(a):
            b = nxt[a]
            if a < 0 or b < 0:
                return
            i = self.ids.get(sym[a] + sym[b])
            if i is not None:
                heapq.heappush(heap, (-self.scores[i], a, sym[a], sym[b]))
        for a in range(len(sym)):
            push(a)
        while heap:
            _, a, sa, sb = heapq.heappop(heap)
            b = nxt[a] if a >= 0 else -1
            if b < 0 or not alive[a] or not alive[b] or sym[a] != sa or sym[b] != sb:
                continue
            sym[a] = sa + sb
            alive[b] = False
            nxt[a] = nxt[b]
            if nxt[b] >= 0:
                prev[nxt[b]] = a
            push(prev[a])
            push(a)
        a = 0
        while a >= 0:
            i = self.ids.get(sym[a])
            if i is not None:
                out.append(i)
            else:
                for byte in sym[a].encode("utf-8"):
                    out.append(self.bytes.get(byte, self.unk))
            a = nxt[a]
        return out

    def decode(self, ids) -> str:
        buf = bytearray()
        for i in ids:
            if i in (self.bos, self.eos):
                continue
            t = self.tokens[i]
            if len(t) == 6 and t.startswith("<0x") and t.endswith(">") and int(t[3:5], 16) in self.bytes and self.bytes[int(t[3:5], 16)] == i:
                buf.append(int(t[3:5], 16))
            else:
                buf += t.replace("▁", " ").encode("utf-8")
        s = buf.decode("utf-8", errors="replace")
        return s[1:] if self.add_space_prefix and s.startswith(" ") else s


def _byte_table():
    bs = list(range(33, 127)) + list(range(161, 173)) + list(range(174, 256))
    cs, n = bs[:], 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return {b: chr(c) for b, c in zip(bs, cs)}


_GPT2_PAT = r"""'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+"""
_LLAMA3_PAT = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+")


class BytePairs:
    def __init__(self, tokens, merges, pre="gpt2", bos=None, eos=None, add_bos=False, special=None):
        import regex
        self.tokens = list(tokens)
        self.ids = {t: i for i, t in enumerate(self.tokens)}
        self.rank = {tuple(m.split(" ", 1)) if isinstance(m, str) else tuple(m): r for r, m in enumerate(merges)}
        self.b2u = _byte_table()
        self.u2b = {u: b for b, u in self.b2u.items()}
        self.pat = regex.compile(_LLAMA3_PAT if pre in ("llama3", "llama-bpe") else _GPT2_PAT)
        self.bos, self.eos, self.add_bos = bos, eos, add_bos
        self.special = sorted(special or [t for t in self.tokens if t.startswith("<|") and t.endswith("|>")], key=len, reverse=True)
        self._cache = {}

    def _bpe(self, word: str) -> list:
        if word in self._cache:
            return self._cache[word]
        parts = list(word)
        while len(parts) > 1:
            best, at = None, -1
            for i in range(len(parts) - 1):
                r = self.rank.get((parts[i], parts[i + 1]))
                if r is not None and (best is None or r < best):
                    best, at = r, i
            if best is None:
                break
            a, b = parts[at], parts[at + 1]
            merged, i = [], 0
            while i < len(parts):
                if i < len(parts) - 1 and parts[i] == a and parts[i + 1] == b:
                    merged.append(a + b)
                    i += 2
                else:
                    merged.append(parts[i])
                    i += 1
            parts = merged
        self._cache[word] = parts
        return parts

    def _plain(self, text: str, out: list) -> None:
        for piece in self.pat.findall(text):
            word = "".join(self.b2u[b] for b in piece.encode("utf-8"))
            for p in self._bpe(word):
                i = self.ids.get(p)
                if i is not None:
                    out.append(i)
                else:   # unknown merge result: fall back to single byte symbols
                    out.extend(self.ids[c] for c in p if c in self.ids)

    def encode(self, text: str, bos: bool | None = None) -> list:
        out = [self.bos] if (self.add_bos if bos is None else bos) and self.bos is not None else []
        pos = 0
        while pos < len(text):
            hit, where = None, len(text)
            for sp in self.special:
                j = text.find(sp, pos)
                if j >= 0 and j < where:
                    hit, where = sp, j
            self._plain(text[pos:where], out)
            if hit is None:
                break
            out.append(self.ids[hit])
            pos = where + len(hit)
        return out

    def decode(self, ids) -> str:
        buf = bytearray()
        for i in ids:
            t = self.tokens[i]
            if t in self.special:
                if i not in (self.bos, self.eos):
                    buf += t.encode("utf-8")
                continue
            for ch in t:
                buf.append(self.u2b.get(ch, ord("?")))
        return buf.decode("utf-8", errors="replace")
