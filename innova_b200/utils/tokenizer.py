"""Tokenizers: byte-level, and a byte-pair-encoding tokenizer with a trainer.

Covers the reference's Tokenizer / BPETokenizer (include/oil/tokenizer.h:10-59,
include/oil/bpe_tokenizer.h:17-216): train on a corpus to a target vocabulary, encode / decode, special
tokens (pad, bos, eos, unk), save / load of the ``<model>.vocab`` sidecar that the inference engine
reads next to a ``.oil`` file (engines/inference/inference.cpp:91-101).
"""
from __future__ import annotations

import json
from collections import Counter
from typing import Dict, Iterable, List, Tuple


class ByteTokenizer:
    """One token per byte (vocabulary 256), the vocabulary of the tiny configuration."""
    vocab_size = 256
    eos_id = None

    def encode(self, text: str) -> List[int]:
        return list(text.encode("utf-8", errors="replace"))

    def decode(self, ids: Iterable[int]) -> str:
        return bytes(int(i) & 255 for i in ids).decode("utf-8", errors="replace")

    def save(self, path: str):
        json.dump({"type": "byte"}, open(path, "w"))


class BPETokenizer:
    """Byte-level BPE: base alphabet = 256 bytes, merges learned greedily by pair frequency."""
    SPECIALS = ["<pad>", "<bos>", "<eos>", "<unk>"]

    def __init__(self):
        self.merges: List[Tuple[int, int]] = []
        self.rank: Dict[Tuple[int, int], int] = {}
        self.pieces: List[bytes] = [bytes([i]) for i in range(256)]
        self.n_special = len(self.SPECIALS)

    @property
    def vocab_size(self) -> int:
        return len(self.pieces) + self.n_special

    @property
    def pad_id(self):
        return len(self.pieces)

    @property
    def bos_id(self):
        return len(self.pieces) + 1

    @property
    def eos_id(self):
        return len(self.pieces) + 2

    def train(self, text: str, vocab_size: int, max_words: int = 200000) -> "BPETokenizer":
        """Learn merges until the vocabulary reaches ``vocab_size`` (specials included)."""
        words = Counter(text.split(" "))
        if len(words) > max_words:
            words = Counter(dict(words.most_common(max_words)))
        seqs = {w: [b for b in (" " + w).encode("utf-8")] for w in words}
        target = max(256, vocab_size - self.n_special)
        while len(self.pieces) < target:
            pairs = Counter()
            for w, s in seqs.items():
                c = words[w]
                for a, b in zip(s, s[1:]):
                    pairs[(a, b)] += c
            if not pairs:
                break
            (a, b), cnt = pairs.most_common(1)[0]
            if cnt < 2:
                break
            new_id = len(self.pieces)
            self.pieces.append(self.pieces[a] + self.pieces[b])
            self.rank[(a, b)] = len(self.merges)
            self.merges.append((a, b))
            for w, s in seqs.items():
                if len(s) < 2:
                    continue
                out, i = [], 0
                while i < len(s):
                    if i + 1 < len(s) and s[i] == a and s[i + 1] == b:
                        out.append(new_id)
                        i += 2
                    else:
                        out.append(s[i])
                        i += 1
                seqs[w] = out
        return self

    def _encode_word(self, bs: bytes) -> List[int]:
        s = list(bs)
        while len(s) > 1:
            best, at = None, -1
            for i, p in enumerate(zip(s, s[1:])):
                r = self.rank.get(p)
                if r is not None and (best is None or r < best):
                    best, at = r, i
            if best is None:
                break
            a, b = self.merges[best]
            s[at:at + 2] = [256 + best]
        return s

    def encode(self, text: str, add_bos: bool = False, add_eos: bool = False) -> List[int]:
        ids: List[int] = [self.bos_id] if add_bos else []
        first = True
        for w in text.split(" "):
            piece = (w if first and not text.startswith(" ") else " " + w)
            first = False
            ids.extend(self._encode_word(piece.encode("utf-8")))
        if add_eos:
            ids.append(self.eos_id)
        return ids

    def decode(self, ids: Iterable[int]) -> str:
        out = b"".join(self.pieces[i] for i in ids if 0 <= int(i) < len(self.pieces))
        return out.decode("utf-8", errors="replace")

    def save(self, path: str):
        json.dump({"type": "bpe", "merges": self.merges}, open(path, "w"))

    @staticmethod
    def load(path: str):
        d = json.load(open(path))
        if d.get("type") == "byte":
            return ByteTokenizer()
        t = BPETokenizer()
        for a, b in d["merges"]:
            t.rank[(a, b)] = len(t.merges)
            t.merges.append((a, b))
            t.pieces.append(t.pieces[a] + t.pieces[b])
        return t


def load_tokenizer(path: str):
    return BPETokenizer.load(path)
