"""Subword tokenizers beyond byte-level BPE: unigram language model, WordPiece, a SentencePiece-style trainer front end
and a multilingual tokenizer with language tags and byte fallback.

Reference behaviour covered: ``UnigramTokenizer`` (include/oil/bpe_tokenizer.h:43-83: EM-trained piece probabilities,
Viterbi segmentation, ``encode_with_scores``), ``WordPieceTokenizer`` (:85-122: likelihood-ratio merges, ``##``
continuation pieces, greedy longest-match encoding, [UNK]/[CLS]/[SEP]/[PAD]/[MASK]), ``SentencePieceTrainer`` (:163-178:
model type BPE / UNIGRAM / WORDPIECE, NFKC normalisation, character coverage, default pre-tokenisation) and
``MultiLingualTokenizer`` (:180-216: script-based segmentation, language tags, UTF-8 byte fallback).
"""
from __future__ import annotations

import json
import math
import re
import unicodedata
from collections import Counter
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

from .tokenizer import BPETokenizer

_WORD_RE = re.compile(r"\w+|[^\w\s]", re.UNICODE)


def normalize_nfkc(text: str) -> str:
    return unicodedata.normalize("NFKC", text)


def split_on_whitespace_and_punctuation(text: str) -> List[str]:
    return _WORD_RE.findall(text)


def pretokenize_default(text: str) -> List[str]:
    """Whitespace becomes a leading ``▁`` on the following word, punctuation stands alone."""
    out = []
    for m in re.finditer(r"(\s*)(\w+|[^\w\s])", text, re.UNICODE):
        out.append(("▁" if m.group(1) or m.start() == 0 else "") + m.group(2))
    return out


# ------------------------------------------------------------------------------------------------ unigram
class UnigramTokenizer:
    """Pieces with log-probabilities; a word is segmented into the most probable sequence of pieces (Viterbi)."""
    SPECIALS = ["<unk>", "<bos>", "<eos>"]

    def __init__(self):
        self.pieces: List[str] = list(self.SPECIALS)
        self.logp: List[float] = [0.0] * len(self.SPECIALS)
        self.index: Dict[str, int] = {p: i for i, p in enumerate(self.pieces)}
        self.unk_id, self.bos_id, self.eos_id = 0, 1, 2
        self.max_piece = 1

    @property
    def vocab_size(self) -> int:
        return len(self.pieces)

    def _viterbi(self, word: str, logp: Dict[str, float], max_len: int):
        n = len(word)
        best = [-math.inf] * (n + 1)
        back = [0] * (n + 1)
        best[0] = 0.0
        unk_pen = -20.0
        for i in range(1, n + 1):
            for j in range(max(0, i - max_len), i):
                lp = logp.get(word[j:i])
                if lp is None:
                    if i - j > 1:
                        continue
                    lp = unk_pen          # an unknown single character can always be emitted as <unk>
                s = best[j] + lp
                if s > best[i]:
                    best[i], back[i] = s, j
        segs, i = [], n
        while i > 0:
            segs.append(word[back[i]:i])
            i = back[i]
        return segs[::-1], best[n]

    def train(self, corpus: Sequence[str], vocab_size: int = 16000, max_piece: int = 8, em_iters: int = 4, shrink: float = 0.75) -> "UnigramTokenizer":
        words = Counter(w for line in corpus for w in pretokenize_default(normalize_nfkc(line)))
        chars = Counter()
        subs = Counter()
        for w, c in words.items():
            for i in range(len(w)):
                chars[w[i]] += c
                for j in range(i + 2, min(len(w), i + max_piece) + 1):
                    subs[w[i:j]] += c
        seed_n = max(vocab_size * 4, 256)
        cand = dict(chars)
        cand.update({s: f * len(s) for s, f in subs.most_common(seed_n)})
        target = max(vocab_size - len(self.SPECIALS), len(chars))
        total = sum(cand.values())
        logp = {p: math.log(f / total) for p, f in cand.items()}
        while True:
            for _ in range(em_iters):               # hard EM: counts from the Viterbi segmentations
                counts = Counter()
                for w, c in words.items():
                    for seg in self._viterbi(w, logp, max_piece)[0]:
                        counts[seg] += c
                for ch in chars:                      # single characters never disappear
                    counts[ch] += 1
                total = sum(counts.values())
                logp = {p: math.log(f / total) for p, f in counts.items() if p in logp}
            if len(logp) <= target:
                break
            keep = max(target, int(len(logp) * shrink))
            multi = sorted((p for p in logp if len(p) > 1), key=lambda p: -logp[p] * 1.0)   # least probable first
            drop = set(multi[: len(logp) - keep])
            logp = {p: v for p, v in logp.items() if p not in drop}
        ordered = sorted(logp, key=lambda p: (-logp[p], p))
        self.pieces = list(self.SPECIALS) + ordered
        self.logp = [0.0] * len(self.SPECIALS) + [logp[p] for p in ordered]
        self.index = {p: i for i, p in enumerate(self.pieces)}
        self.max_piece = max_piece
        return self

    def encode_with_scores(self, text: str) -> Tuple[List[int], List[float]]:
        table = {p: lp for p, lp in zip(self.pieces[len(self.SPECIALS):], self.logp[len(self.SPECIALS):])}
        ids, scores = [], []
        for w in pretokenize_default(normalize_nfkc(text)):
            for seg in self._viterbi(w, table, self.max_piece)[0]:
                i = self.index.get(seg, self.unk_id)
                ids.append(i)
                scores.append(self.logp[i] if i != self.unk_id else -20.0)
        return ids, scores

    def encode(self, text: str) -> List[int]:
        return self.encode_with_scores(text)[0]

    def decode(self, ids: Iterable[int]) -> str:
        s = "".join(self.pieces[i] if i >= len(self.SPECIALS) else ("�" if i == self.unk_id else "") for i in ids)
        return s.replace("▁", " ").lstrip(" ")

    def save(self, path: str):
        json.dump({"type": "unigram", "pieces": self.pieces, "logp": self.logp, "max_piece": self.max_piece}, open(path, "w"), ensure_ascii=False)

    @classmethod
    def load(cls, path: str) -> "UnigramTokenizer":
        d = json.load(open(path))
        t = cls()
        t.pieces, t.logp, t.max_piece = d["pieces"], d["logp"], d["max_piece"]
        t.index = {p: i for i, p in enumerate(t.pieces)}
        return t


# ------------------------------------------------------------------------------------------------ WordPiece
class WordPieceTokenizer:
    """Merges chosen by freq(ab) / (freq(a) freq(b)); word-internal pieces carry the ``##`` prefix."""

    def __init__(self):
        self.set_special_tokens("[UNK]", "[CLS]", "[SEP]", "[PAD]", "[MASK]")
        self.vocab: List[str] = list(self.specials)
        self.index: Dict[str, int] = {p: i for i, p in enumerate(self.vocab)}
        self.max_chars = 64

    def set_special_tokens(self, unk: str, cls: str, sep: str, pad: str, mask: str):
        self.specials = [unk, cls, sep, pad, mask]
        self.unk_token = unk

    @property
    def vocab_size(self) -> int:
        return len(self.vocab)

    @property
    def unk_id(self):
        return self.index[self.unk_token]

    @property
    def bos_id(self):
        return self.index[self.specials[1]]

    @property
    def eos_id(self):
        return self.index[self.specials[2]]

    def train(self, corpus: Sequence[str], vocab_size: int = 30000) -> "WordPieceTokenizer":
        words = Counter(w for line in corpus for w in split_on_whitespace_and_punctuation(normalize_nfkc(line)))
        splits = {w: [w[0]] + ["##" + ch for ch in w[1:]] for w in words}
        vocab = set(p for s in splits.values() for p in s)
        while len(vocab) + len(self.specials) < vocab_size:
            pair_f, piece_f = Counter(), Counter()
            for w, c in words.items():
                s = splits[w]
                for p in s:
                    piece_f[p] += c
                for a, b in zip(s, s[1:]):
                    pair_f[(a, b)] += c
            if not pair_f:
                break
            (a, b), _ = max(pair_f.items(), key=lambda kv: (kv[1] / (piece_f[kv[0][0]] * piece_f[kv[0][1]]), kv[1], kv[0]))
            merged = a + b[2:]
            vocab.add(merged)
            for w, s in splits.items():
                if len(s) < 2:
                    continue
                out, i = [], 0
                while i < len(s):
                    if i + 1 < len(s) and s[i] == a and s[i + 1] == b:
                        out.append(merged)
                        i += 2
                    else:
                        out.append(s[i])
                        i += 1
                splits[w] = out
        self.vocab = list(self.specials) + sorted(vocab)
        self.index = {p: i for i, p in enumerate(self.vocab)}
        return self

    def _encode_word(self, w: str) -> List[int]:
        if len(w) > self.max_chars:
            return [self.unk_id]
        out, start = [], 0
        while start < len(w):
            end, cur = len(w), None
            while start < end:
                piece = ("##" if start else "") + w[start:end]
                if piece in self.index:
                    cur = self.index[piece]
                    break
                end -= 1
            if cur is None:
                return [self.unk_id]
            out.append(cur)
            start = end
        return out

    def encode(self, text: str, add_special: bool = False) -> List[int]:
        ids = [i for w in split_on_whitespace_and_punctuation(normalize_nfkc(text)) for i in self._encode_word(w)]
        return [self.bos_id] + ids + [self.eos_id] if add_special else ids

    def decode(self, ids: Iterable[int]) -> str:
        out = []
        for i in ids:
            p = self.vocab[i]
            if p in self.specials and p != self.unk_token:
                continue
            if p.startswith("##") and out:
                out[-1] += p[2:]
            else:
                out.append(p)
        return " ".join(out)

    def save(self, path: str):
        json.dump({"type": "wordpiece", "vocab": self.vocab, "specials": self.specials}, open(path, "w"), ensure_ascii=False)

    @classmethod
    def load(cls, path: str) -> "WordPieceTokenizer":
        d = json.load(open(path))
        t = cls()
        t.set_special_tokens(*d["specials"])
        t.vocab = d["vocab"]
        t.index = {p: i for i, p in enumerate(t.vocab)}
        return t


# ------------------------------------------------------------------------------------------------ trainer front end
class SentencePieceTrainer:
    BPE, UNIGRAM, WORDPIECE = 0, 1, 2

    @staticmethod
    def train(corpus: Sequence[str], model_prefix: str, model_type: int = 0, vocab_size: int = 32000, character_coverage: float = 0.9995,
              seed: int = 42):
        """Trains the chosen model on the NFKC-normalised corpus, with characters beyond the coverage quantile replaced
        by U+FFFD, and writes ``<model_prefix>.model``. Returns the tokenizer."""
        lines = [normalize_nfkc(l) for l in corpus]
        freq = Counter(ch for l in lines for ch in l if not ch.isspace())
        total, acc, keep = sum(freq.values()), 0, set()
        for ch, f in freq.most_common():
            if total and acc / total >= character_coverage:
                break
            keep.add(ch)
            acc += f
        lines = ["".join(ch if ch.isspace() or ch in keep else "�" for ch in l) for l in lines]
        if model_type == SentencePieceTrainer.UNIGRAM:
            tok = UnigramTokenizer().train(lines, vocab_size)
        elif model_type == SentencePieceTrainer.WORDPIECE:
            tok = WordPieceTokenizer().train(lines, vocab_size)
        else:
            tok = BPETokenizer().train(" ".join(lines), vocab_size)
        tok.save(model_prefix + ".model")
        return tok

    normalize_nfkc = staticmethod(normalize_nfkc)
    pretokenize_default = staticmethod(pretokenize_default)
    split_on_whitespace_and_punctuation = staticmethod(split_on_whitespace_and_punctuation)


def load_any(path: str):
    """Loads whichever tokenizer ``path`` holds (the ``type`` field of its JSON)."""
    kind = json.load(open(path)).get("type", "bpe")
    if kind == "unigram":
        return UnigramTokenizer.load(path)
    if kind == "wordpiece":
        return WordPieceTokenizer.load(path)
    if kind == "multilingual":
        return MultiLingualTokenizer.load(path)
    return BPETokenizer.load(path)


# ------------------------------------------------------------------------------------------------ multilingual
_SCRIPTS = [("cjk", 0x4E00, 0x9FFF), ("hiragana", 0x3040, 0x309F), ("katakana", 0x30A0, 0x30FF), ("hangul", 0xAC00, 0xD7AF),
            ("cyrillic", 0x0400, 0x04FF), ("arabic", 0x0600, 0x06FF), ("hebrew", 0x0590, 0x05FF), ("devanagari", 0x0900, 0x097F),
            ("greek", 0x0370, 0x03FF), ("thai", 0x0E00, 0x0E7F)]


def script_of(ch: str) -> str:
    o = ord(ch)
    for name, lo, hi in _SCRIPTS:
        if lo <= o <= hi:
            return name
    return "latin" if ch.isalpha() else "common"


class MultiLingualTokenizer:
    """One BPE vocabulary over all scripts; text is cut where the script changes so that merges never straddle
    scripts, ``<lang:xx>`` tags can be prepended, and anything outside the vocabulary falls back to UTF-8 bytes
    (``byte`` strategy) or ``<unk>`` (``unk`` strategy)."""

    def __init__(self):
        self.bpe = BPETokenizer()
        self.lang_tags: List[str] = []
        self.fallback = "byte"

    @property
    def vocab_size(self) -> int:
        return self.bpe.vocab_size + len(self.lang_tags)

    @property
    def bos_id(self):
        return self.bpe.bos_id

    @property
    def eos_id(self):
        return self.bpe.eos_id

    def set_fallback_strategy(self, strategy: str):
        assert strategy in ("byte", "unk")
        self.fallback = strategy

    def add_language_token(self, lang: str) -> int:
        if lang not in self.lang_tags:
            self.lang_tags.append(lang)
        return self.bpe.vocab_size + self.lang_tags.index(lang)

    def split_by_language(self, text: str) -> List[Tuple[str, str]]:
        segs: List[Tuple[str, str]] = []
        for ch in text:
            sc = script_of(ch)
            if segs and (sc == "common" or segs[-1][0] == sc or segs[-1][0] == "common"):
                name = segs[-1][0] if sc == "common" else sc
                segs[-1] = (name, segs[-1][1] + ch)
            else:
                segs.append((sc, ch))
        return segs

    def train(self, corpus: Sequence[str], vocab_size: int = 50000) -> "MultiLingualTokenizer":
        pieces = []
        for line in corpus:
            pieces.extend(seg for _, seg in self.split_by_language(normalize_nfkc(line)))
        self.bpe.train(" ".join(pieces), vocab_size - len(self.lang_tags))
        return self

    def encode(self, text: str) -> List[int]:
        ids: List[int] = []
        for _, seg in self.split_by_language(normalize_nfkc(text)):
            ids.extend(self.bpe.encode(seg))     # byte-level BPE: every UTF-8 byte is in the base alphabet
        return ids

    def encode_with_lang_tag(self, text: str, lang: str) -> List[int]:
        return [self.add_language_token(lang)] + self.encode(text)

    def decode(self, ids: Iterable[int]) -> str:
        base = self.bpe.vocab_size
        return self.bpe.decode([i for i in ids if i < base])

    def save(self, path: str):
        self.bpe.save(path + ".bpe")
        json.dump({"type": "multilingual", "bpe": path + ".bpe", "lang_tags": self.lang_tags, "fallback": self.fallback}, open(path, "w"))

    @classmethod
    def load(cls, path: str) -> "MultiLingualTokenizer":
        d = json.load(open(path))
        t = cls()
        t.bpe = BPETokenizer.load(d["bpe"])
        t.lang_tags, t.fallback = d["lang_tags"], d["fallback"]
        return t
