"""Byte-level BPE tokenizer (GPT-2 vocabulary format: ``vocab.json`` + ``merges.txt``).

Text is split into chunks by the GPT-2 pre-tokenization pattern, every chunk is mapped byte by byte onto
printable unicode code points, and adjacent symbols are merged greedily in the order of the merge table.
A ``<pad>`` token is appended after the vocabulary, ``<|endoftext|>`` is the end-of-document token.
Reference: hotspa/tokenizer/tokenizer.py (_GPT2BPETokenizer) and hotspa/tokenizer/gpt2_tokenization.py.
"""
from __future__ import annotations

import json
from functools import lru_cache

try:
    import regex as re
    _PATTERN = r"'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+"
except ImportError:  # pragma: no cover
    import re
    _PATTERN = r"'s|'t|'re|'ve|'m|'ll|'d| ?[A-Za-z]+| ?[0-9]+| ?[^\sA-Za-z0-9]+|\s+(?!\S)|\s+"


@lru_cache()
def byte_to_unicode() -> dict:
    """Reversible map from the 256 byte values to printable unicode characters: printable latin-1 bytes map to
    themselves, the rest are shifted above U+0100 in order."""
    keep = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAC + 1)) + list(range(0xAE, 0xFF + 1))
    table, extra = {}, 0
    for b in range(256):
        if b in keep:
            table[b] = chr(b)
        else:
            table[b] = chr(256 + extra)
            extra += 1
    return table


class GPT2BPETokenizer:
    def __init__(self, vocab_file: str | None = None, merge_file: str | None = None, vocab: dict | None = None,
                 merges: list | None = None, special_tokens=("<pad>",)):
        if vocab is None:
            with open(vocab_file, encoding="utf-8") as f:
                vocab = json.load(f)
        if merges is None:
            with open(merge_file, encoding="utf-8") as f:
                lines = f.read().split("\n")
            merges = [tuple(ln.split()) for ln in lines if ln and not ln.startswith("#version") and len(ln.split()) == 2]
        self.encoder = dict(vocab)
        self.decoder = {v: k for k, v in self.encoder.items()}
        self.ranks = {tuple(m): i for i, m in enumerate(merges)}
        self.b2u = byte_to_unicode()
        self.u2b = {v: k for k, v in self.b2u.items()}
        self.pattern = re.compile(_PATTERN)
        self.special_tokens = {}
        nxt = len(self.encoder)
        for tok in special_tokens:
            self.special_tokens[tok] = nxt
            nxt += 1
        self.special_decoder = {v: k for k, v in self.special_tokens.items()}
        self._cache: dict = {}

    # ---- properties with the reference's names ------------------------------------------------------
    @property
    def vocab_size(self) -> int:
        return len(self.encoder)

    @property
    def vocab(self) -> dict:
        return self.encoder

    @property
    def inv_vocab(self) -> dict:
        return self.decoder

    @property
    def eod(self) -> int:
        return self.encoder.get("<|endoftext|>", len(self.encoder) - 1)

    @property
    def pad(self) -> int:
        return self.special_tokens["<pad>"]

    # ---- BPE ------------------------------------------------------------------------------------------
    def _bpe(self, token: str) -> list:
        if token in self._cache:
            return self._cache[token]
        word = list(token)
        while len(word) > 1:
            best, best_rank = None, None
            for pair in zip(word[:-1], word[1:]):
                r = self.ranks.get(pair)
                if r is not None and (best_rank is None or r < best_rank):
                    best, best_rank = pair, r
            if best is None:
                break
            merged, i = [], 0
            while i < len(word):
                if i < len(word) - 1 and (word[i], word[i + 1]) == best:
                    merged.append(word[i] + word[i + 1])
                    i += 2
                else:
                    merged.append(word[i])
                    i += 1
            word = merged
        self._cache[token] = word
        return word

    def tokenize(self, text: str) -> list:
        ids = []
        for chunk in self.pattern.findall(text):
            mapped = "".join(self.b2u[b] for b in chunk.encode("utf-8"))
            for piece in self._bpe(mapped):
                if piece in self.encoder:
                    ids.append(self.encoder[piece])
                else:                                   # unknown merge result: fall back to its single symbols
                    ids.extend(self.encoder[ch] for ch in piece if ch in self.encoder)
        return ids

    encode = tokenize

    def detokenize(self, token_ids) -> str:
        out = bytearray()
        for t in token_ids:
            t = int(t)
            if t in self.special_decoder:
                out.extend(self.special_decoder[t].encode("utf-8"))
                continue
            for ch in self.decoder.get(t, ""):
                out.append(self.u2b.get(ch, ord("?")))
        return out.decode("utf-8", errors="replace")

    decode = detokenize


def build_tokenizer(args) -> GPT2BPETokenizer:
    """`args` needs ``vocab_file`` and ``merge_file`` (``tokenizer_type`` must be GPT2BPETokenizer when present)."""
    kind = getattr(args, "tokenizer_type", "GPT2BPETokenizer")
    if kind != "GPT2BPETokenizer":
        raise NotImplementedError(f"{kind} tokenizer is not implemented")
    return GPT2BPETokenizer(args.vocab_file, args.merge_file)
