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


# ------------------------------------------------------------------------------------------------ unicode helpers
class UnicodeUtil:
    """Code-point classification and UTF-8 helpers (reference: ``UnicodeUtil``, include/oil/bpe_tokenizer.h:17-41,
    src/bpe_tokenizer_unicode.cpp). Classification comes from the Unicode character database through ``unicodedata``
    rather than hand-kept range tables."""

    _LANG = {"cjk": "zh", "hiragana": "ja", "katakana": "ja", "hangul": "ko", "cyrillic": "ru", "arabic": "ar", "hebrew": "he",
             "devanagari": "hi", "greek": "el", "thai": "th", "latin": "en"}

    @staticmethod
    def _cat(cp: int) -> str:
        return unicodedata.category(chr(cp)) if 0 <= cp <= 0x10FFFF else "Cn"

    @staticmethod
    def is_cjk(cp: int) -> bool:
        return (0x4E00 <= cp <= 0x9FFF or 0x3400 <= cp <= 0x4DBF or 0x20000 <= cp <= 0x2A6DF or 0xF900 <= cp <= 0xFAFF
                or 0x3040 <= cp <= 0x30FF or 0xAC00 <= cp <= 0xD7AF)

    @classmethod
    def is_whitespace(cls, cp: int) -> bool:
        return cp in (0x09, 0x0A, 0x0B, 0x0C, 0x0D, 0x85) or cls._cat(cp) == "Zs" or cp in (0x2028, 0x2029)

    @classmethod
    def is_punctuation(cls, cp: int) -> bool:
        return cls._cat(cp).startswith("P")

    @classmethod
    def is_letter(cls, cp: int) -> bool:
        return cls._cat(cp).startswith("L")

    @classmethod
    def is_digit(cls, cp: int) -> bool:
        return cls._cat(cp) == "Nd"

    @classmethod
    def is_control(cls, cp: int) -> bool:
        return cls._cat(cp) in ("Cc", "Cf") and not cls.is_whitespace(cp)

    @classmethod
    def is_math_symbol(cls, cp: int) -> bool:
        return cls._cat(cp) == "Sm"

    @classmethod
    def is_currency(cls, cp: int) -> bool:
        return cls._cat(cp) == "Sc"

    @classmethod
    def is_combining_mark(cls, cp: int) -> bool:
        return cls._cat(cp).startswith("M")

    @staticmethod
    def is_regional_indicator(cp: int) -> bool:
        return 0x1F1E6 <= cp <= 0x1F1FF

    @staticmethod
    def is_variation_selector(cp: int) -> bool:
        return 0xFE00 <= cp <= 0xFE0F or 0xE0100 <= cp <= 0xE01EF

    @staticmethod
    def is_emoji_modifier(cp: int) -> bool:
        return 0x1F3FB <= cp <= 0x1F3FF

    @classmethod
    def is_emoji(cls, cp: int) -> bool:
        return (0x1F300 <= cp <= 0x1FAFF or 0x2600 <= cp <= 0x27BF or 0x1F000 <= cp <= 0x1F2FF or cls.is_regional_indicator(cp)
                or cp in (0x00A9, 0x00AE, 0x203C, 0x2049, 0x2122, 0x2139, 0x231A, 0x231B, 0x2B50, 0x2B55, 0x3030, 0x303D))

    @staticmethod
    def utf8_encode(cp: int) -> bytes:
        if not 0 <= cp <= 0x10FFFF or 0xD800 <= cp <= 0xDFFF:
            cp = 0xFFFD
        return chr(cp).encode("utf-8")

    @staticmethod
    def utf8_decode(data: bytes, pos: int) -> Tuple[int, int]:
        """Decodes one code point of ``data`` at ``pos`` -> (code point, next position); malformed or truncated sequences
        (overlong forms and surrogates included) give U+FFFD and advance one byte."""
        b0 = data[pos]
        if b0 < 0x80:
            return b0, pos + 1
        n, lo = (2, 0x80) if 0xC2 <= b0 <= 0xDF else (3, 0x800) if 0xE0 <= b0 <= 0xEF else (4, 0x10000) if 0xF0 <= b0 <= 0xF4 else (0, 0)
        if n == 0 or pos + n > len(data) or any(data[pos + i] & 0xC0 != 0x80 for i in range(1, n)):
            return 0xFFFD, pos + 1
        cp = b0 & (0xFF >> (n + 1))
        for i in range(1, n):
            cp = (cp << 6) | (data[pos + i] & 0x3F)
        if cp < lo or cp > 0x10FFFF or 0xD800 <= cp <= 0xDFFF:
            return 0xFFFD, pos + 1
        return cp, pos + n

    @classmethod
    def utf8_to_codepoints(cls, data) -> List[int]:
        data = data.encode("utf-8") if isinstance(data, str) else bytes(data)
        out, pos = [], 0
        while pos < len(data):
            cp, pos = cls.utf8_decode(data, pos)
            out.append(cp)
        return out

    @classmethod
    def codepoints_to_utf8(cls, cps: Sequence[int]) -> bytes:
        return b"".join(cls.utf8_encode(c) for c in cps)

    @staticmethod
    def nfkc_normalize(s: str) -> str:
        return unicodedata.normalize("NFKC", s)

    @staticmethod
    def compose_pair(a: int, b: int) -> int:
        """The single code point that canonically composes ``a`` followed by ``b``, or 0 when there is none."""
        c = unicodedata.normalize("NFC", chr(a) + chr(b))
        return ord(c) if len(c) == 1 else 0

    @staticmethod
    def split_on_whitespace(s: str) -> List[str]:
        return s.split()

    @classmethod
    def pretokenize(cls, s: str) -> List[str]:
        """Runs of letters (with their combining marks), runs of digits, single CJK characters, single punctuation /
        symbol characters; emoji keep their modifiers, variation selectors and joiners; whitespace separates and is dropped."""
        out: List[str] = []
        kind = ""
        for ch in s:
            cp = ord(ch)
            if cls.is_whitespace(cp):
                kind = ""
                continue
            glue = cls.is_combining_mark(cp) or cls.is_variation_selector(cp) or cls.is_emoji_modifier(cp) or cp == 0x200D
            if glue and out and kind:
                out[-1] += ch
                continue
            if out and kind == "emoji" and out[-1].endswith("‍"):
                out[-1] += ch
                continue
            k = "cjk" if cls.is_cjk(cp) else "letter" if cls.is_letter(cp) else "digit" if cls.is_digit(cp) else \
                "emoji" if cls.is_emoji(cp) else "other"
            if k == kind and k in ("letter", "digit"):
                out[-1] += ch
            elif k == kind == "emoji" and cls.is_regional_indicator(cp) and len(out[-1]) == 1 and cls.is_regional_indicator(ord(out[-1])):
                out[-1] += ch                                    # a flag is two regional indicators
            else:
                out.append(ch)
            kind = k
        return out

    @classmethod
    def detect_language(cls, segment: str) -> str:
        """Two-letter tag of the script most letters of the segment belong to ("und" when it has no letters)."""
        votes = Counter(script_of(ch) for ch in segment if cls.is_letter(ord(ch)))
        return cls._LANG.get(votes.most_common(1)[0][0], "und") if votes else "und"

    @classmethod
    def width(cls, cp: int) -> int:
        """Terminal columns: 0 for control / combining / selectors / joiners, 2 for wide and full-width, else 1."""
        if cp == 0 or cls._cat(cp) in ("Cc", "Cf", "Mn", "Me") or cls.is_variation_selector(cp):
            return 0
        return 2 if unicodedata.east_asian_width(chr(cp)) in ("W", "F") else 1


# ------------------------------------------------------------------------------------------------ byte-level BPE with a printable byte alphabet
def _byte_alphabet() -> List[str]:
    """Every byte as one printable character: printable Latin-1 bytes stand for themselves, the rest are moved to
    U+0100 onwards (the byte alphabet GPT-2 style vocabularies are written in)."""
    keep = list(range(0x21, 0x7F)) + list(range(0xA1, 0xAD)) + list(range(0xAE, 0x100))
    table, extra = {}, 0
    for b in range(256):
        if b in keep:
            table[b] = chr(b)
        else:
            table[b] = chr(256 + extra)
            extra += 1
    return [table[b] for b in range(256)]


class ByteLevelBPETokenizer:
    """Trainable byte-level BPE whose tokens are strings over the printable byte alphabet (reference:
    ``ByteLevelBPETokenizer``, include/oil/bpe_tokenizer.h:124-161, src/bpe_tokenizer_bpe.cpp). Ids 0..4 are ``<unk>``,
    ``<pad>``, ``<mask>``, ``<s>`` (3) and ``</s>`` (4), then the 256 byte tokens, then the merges in the order they were
    learnt. Training counts pairs over the distinct pre-tokenised words weighted by frequency; a leading space stays part of
    the following word, so decoding is the exact inverse of encoding for any byte string."""

    SPECIALS = ("<unk>", "<pad>", "<mask>", "<s>", "</s>")
    _SPLIT = re.compile(r" ?[^\W\d_]+| ?\d+| ?[^\s\w]+|\s+(?!\S)|\s+", re.UNICODE)

    def __init__(self):
        self.alphabet = _byte_alphabet()
        self.byte_of = {c: b for b, c in enumerate(self.alphabet)}
        self.id_to_token: List[str] = list(self.SPECIALS) + self.alphabet
        self.token_to_id: Dict[str, int] = {t: i for i, t in enumerate(self.id_to_token)}
        self.merges: Dict[Tuple[int, int], int] = {}
        self.unk_id, self.bos_id, self.eos_id = 0, 3, 4
        self._cache: Dict[str, List[int]] = {}

    def vocab_size(self) -> int:
        return len(self.id_to_token)

    def byte_encode(self, text: str) -> List[int]:
        return [self.token_to_id[self.alphabet[b]] for b in text.encode("utf-8")]

    def _add_token(self, token: str) -> int:
        self.token_to_id[token] = len(self.id_to_token)
        self.id_to_token.append(token)
        return self.token_to_id[token]

    def train(self, corpus: Iterable[str], vocab_size: int = 50000, min_frequency: int = 2) -> None:
        words = Counter(w for line in corpus for w in self._SPLIT.findall(line))
        seqs = {w: self.byte_encode(w) for w in words}
        while len(self.id_to_token) < vocab_size:
            pairs: Counter = Counter()
            for w, ids in seqs.items():
                f = words[w]
                for a, b in zip(ids, ids[1:]):
                    pairs[(a, b)] += f
            if not pairs:
                break
            (a, b), n = max(pairs.items(), key=lambda kv: (kv[1], -kv[0][0], -kv[0][1]))
            if n < min_frequency:
                break
            new = self._add_token(self.id_to_token[a] + self.id_to_token[b])
            self.merges[(a, b)] = new
            for w, ids in seqs.items():
                if a in ids:
                    seqs[w] = self._apply(ids, a, b, new)
        self._cache.clear()

    @staticmethod
    def _apply(ids: List[int], a: int, b: int, new: int) -> List[int]:
        out, i = [], 0
        while i < len(ids):
            if i + 1 < len(ids) and ids[i] == a and ids[i + 1] == b:
                out.append(new)
                i += 2
            else:
                out.append(ids[i])
                i += 1
        return out

    def bpe_merge_tokens(self, ids: List[int]) -> List[int]:
        """Applies the learnt merges in training order (lowest merged id first) until none applies."""
        while len(ids) > 1:
            best = min(((self.merges.get(p, 1 << 60), p) for p in zip(ids, ids[1:])), key=lambda t: t[0])
            if best[0] == 1 << 60:
                break
            ids = self._apply(ids, best[1][0], best[1][1], best[0])
        return ids

    def encode(self, text: str, add_special: bool = False) -> List[int]:
        out: List[int] = [self.bos_id] if add_special else []
        for w in self._SPLIT.findall(text):
            if w not in self._cache:
                self._cache[w] = self.bpe_merge_tokens(self.byte_encode(w))
            out.extend(self._cache[w])
        return out + ([self.eos_id] if add_special else [])

    def decode(self, ids: Sequence[int]) -> str:
        data = bytearray()
        for i in ids:
            if len(self.SPECIALS) <= i < len(self.id_to_token):
                data.extend(self.byte_of[c] for c in self.id_to_token[i])
        return data.decode("utf-8", "replace")

    def save(self, path: str) -> None:
        with open(path, "w", encoding="utf-8") as f:
            json.dump({"type": "byte_level_bpe", "merges": [[a, b] for (a, b) in self.merges]}, f)

    def load(self, path: str) -> None:
        with open(path, encoding="utf-8") as f:
            blob = json.load(f)
        if blob.get("type") != "byte_level_bpe":
            raise ValueError(f"{path}: not a byte-level BPE file")
        self.__init__()
        for a, b in blob["merges"]:
            if not (0 <= a < len(self.id_to_token) and 0 <= b < len(self.id_to_token)):
                raise ValueError(f"{path}: merge refers to an unknown token")
            self.merges[(a, b)] = self._add_token(self.id_to_token[a] + self.id_to_token[b])
