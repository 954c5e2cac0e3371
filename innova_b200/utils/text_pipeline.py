"""Text cleaning, the three-stage text -> token-batch pipeline, a sharded streaming loader and a MinHash-style n-gram
de-duplication filter (include/oil/dataloader.h:18-146, include/oil/mmap_dataloader.h:47-90).

``TextPreprocessor``: lower-casing, accent removal, HTML / URL / e-mail / PII removal, whitespace normalisation, length
filter, exact and fuzzy (character-shingle Jaccard) de-duplication, a script-based language guess.
``DataPipeline``: stage 1 clean, stage 2 tokenize, stage 3 pack into ``[batch, seq]`` int64 tensors; extra named stages can be
appended. ``DataLoader``: a text file streamed as shuffled, rank-sharded token windows with next-token labels.
``MinHashDedup``: fingerprints of token n-grams in a bounded filter; ``is_duplicate`` answers from ``num_hashes`` probes.
Host-side code: the tensors it yields are what the trainers copy to the GPU from pinned memory.
"""
from __future__ import annotations

import html
import random
import re
import unicodedata
from collections import OrderedDict, deque
from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence, Tuple

import numpy as np
import torch

_URL = re.compile(r"(?:https?://|ftp://|www\.)[^\s<>\"']+", re.I)
_EMAIL = re.compile(r"[A-Za-z0-9._%+-]+@[A-Za-z0-9.-]+\.[A-Za-z]{2,}")
_TAG = re.compile(r"<(script|style)\b.*?</\1\s*>|<!--.*?-->|<[^>]+>", re.S | re.I)
_PII = [re.compile(r"\b\d{3}-\d{2}-\d{4}\b"),                                   # US social security number
        re.compile(r"\b(?:\d[ -]?){13,16}\b"),                                   # payment card number
        re.compile(r"(?<!\w)(?:\+?\d{1,3}[ .-]?)?(?:\(\d{2,4}\)[ .-]?)?\d{3}[ .-]\d{3,4}(?:[ .-]\d{2,4})?(?!\w)"),  # phone number
        re.compile(r"\b(?:\d{1,3}\.){3}\d{1,3}\b")]                             # IPv4 address


class TextPreprocessor:
    def __init__(self):
        self.lowercase = self.remove_accents = self.strip_html = self.remove_urls = self.remove_emails = False
        self.normalize_whitespace = self.remove_pii = True
        self.deduplicate_ = False
        self.fuzzy_threshold = 0.95
        self.min_length, self.max_length = 0, -1

    # the reference's setter surface
    def set_lowercase(self, v: bool): self.lowercase = v
    def set_accent_removal(self, v: bool): self.remove_accents = v
    def set_html_stripping(self, v: bool): self.strip_html = v
    def set_url_removal(self, v: bool): self.remove_urls = v
    def set_email_removal(self, v: bool): self.remove_emails = v
    def set_whitespace_normalization(self, v: bool): self.normalize_whitespace = v
    def set_pii_removal(self, v: bool): self.remove_pii = v
    def set_deduplication(self, v: bool): self.deduplicate_ = v
    def set_fuzzy_dedup_threshold(self, t: float): self.fuzzy_threshold = t
    def set_min_length(self, n: int): self.min_length = n
    def set_max_length(self, n: int): self.max_length = n

    def process(self, text: str) -> str:
        """The cleaned text, or "" when it falls outside the length limits."""
        if self.strip_html:
            text = html.unescape(_TAG.sub(" ", text))
        if self.remove_urls:
            text = _URL.sub(" ", text)
        if self.remove_emails:
            text = _EMAIL.sub(" ", text)
        if self.remove_pii:
            for pat in _PII:
                text = pat.sub("[REDACTED]", text)
        if self.remove_accents:
            text = "".join(c for c in unicodedata.normalize("NFKD", text) if not unicodedata.combining(c))
        if self.lowercase:
            text = text.lower()
        if self.normalize_whitespace:
            text = re.sub(r"[ \t\f\v ]+", " ", text)
            text = re.sub(r" ?\n ?", "\n", text)
            text = re.sub(r"\n{3,}", "\n\n", text).strip()
        if len(text) < self.min_length:
            return ""
        if self.max_length >= 0 and len(text) > self.max_length:
            text = text[: self.max_length]
        return text

    def process_batch(self, texts: Sequence[str]) -> List[str]:
        out = [t for t in (self.process(x) for x in texts) if t]
        return self.deduplicate(out) if self.deduplicate_ else out

    @staticmethod
    def detect_language(text: str) -> str:
        """A guess from the Unicode scripts of the letters ("en" for Latin text with a common English word, "latin" otherwise)."""
        counts = {"latin": 0, "cyrillic": 0, "cjk": 0, "arabic": 0, "devanagari": 0, "greek": 0, "hebrew": 0, "hangul": 0, "kana": 0}
        for ch in text:
            o = ord(ch)
            if ch.isascii() and ch.isalpha() or 0x00C0 <= o <= 0x024F:
                counts["latin"] += 1
            elif 0x0400 <= o <= 0x04FF:
                counts["cyrillic"] += 1
            elif 0x4E00 <= o <= 0x9FFF:
                counts["cjk"] += 1
            elif 0x3040 <= o <= 0x30FF:
                counts["kana"] += 1
            elif 0xAC00 <= o <= 0xD7AF:
                counts["hangul"] += 1
            elif 0x0600 <= o <= 0x06FF:
                counts["arabic"] += 1
            elif 0x0900 <= o <= 0x097F:
                counts["devanagari"] += 1
            elif 0x0370 <= o <= 0x03FF:
                counts["greek"] += 1
            elif 0x0590 <= o <= 0x05FF:
                counts["hebrew"] += 1
        best = max(counts, key=counts.get)
        if counts[best] == 0:
            return "unknown"
        if counts["kana"] > 0 and best in ("cjk", "kana"):
            return "ja"
        code = {"cyrillic": "ru", "cjk": "zh", "arabic": "ar", "devanagari": "hi", "greek": "el", "hebrew": "he", "hangul": "ko"}.get(best)
        if code:
            return code
        words = set(re.findall(r"[a-z']+", text.lower()))
        return "en" if words & {"the", "and", "is", "of", "to", "in", "that", "it", "for", "with", "this", "are", "was"} else "latin"

    @staticmethod
    def _shingles(s: str, n: int = 5) -> set:
        s = re.sub(r"\s+", " ", s.lower()).strip()
        return {s[i:i + n] for i in range(max(1, len(s) - n + 1))}

    def fuzzy_similarity(self, a: str, b: str) -> float:
        """Jaccard similarity of the two texts' 5-character shingles."""
        sa, sb = self._shingles(a), self._shingles(b)
        return len(sa & sb) / len(sa | sb) if sa or sb else 1.0

    def deduplicate(self, texts: Sequence[str]) -> List[str]:
        """Drops exact repeats, then texts whose similarity to an already kept text reaches the fuzzy threshold."""
        kept: List[str] = []
        kept_sh: List[set] = []
        seen = set()
        for t in texts:
            if t in seen:
                continue
            seen.add(t)
            sh = self._shingles(t)
            if self.fuzzy_threshold < 1.0 and any(len(sh & k) / max(1, len(sh | k)) >= self.fuzzy_threshold for k in kept_sh):
                continue
            kept.append(t)
            kept_sh.append(sh)
        return kept

    def process_with_metadata(self, texts: Sequence[str]) -> Tuple[List[str], List[str], List[int]]:
        out = self.process_batch(texts)
        return out, [self.detect_language(t) for t in out], [len(t) for t in out]


class DataPipeline:
    def __init__(self):
        self.preprocessor: Optional[TextPreprocessor] = None
        self.tokenizer = None
        self.batch_size, self.seq_length, self.num_workers = 32, 2048, 1
        self.total_processed = 0
        self.custom_stages: List[Tuple[str, Callable[[List[torch.Tensor]], List[torch.Tensor]]]] = []

    def add_stage(self, name: str, fn: Callable[[List[torch.Tensor]], List[torch.Tensor]]):
        """A named stage run on the list of batch tensors after packing."""
        self.custom_stages.append((name, fn))

    def set_preprocessor(self, p: TextPreprocessor): self.preprocessor = p
    def set_tokenizer(self, t): self.tokenizer = t
    def set_batch_size(self, n: int): self.batch_size = n
    def set_seq_length(self, n: int): self.seq_length = n
    def set_num_workers(self, n: int): self.num_workers = n

    def clear_pipeline(self):
        self.custom_stages.clear()
        self.total_processed = 0

    def run_stage1(self, raw_texts: Sequence[str]) -> List[str]:
        return self.preprocessor.process_batch(raw_texts) if self.preprocessor is not None else [t for t in raw_texts if t]

    def run_stage2(self, preprocessed: Sequence[str]) -> List[List[int]]:
        if self.tokenizer is None:
            return [list(t.encode("utf-8")) for t in preprocessed]
        if self.num_workers > 1 and len(preprocessed) > 1:
            from concurrent.futures import ThreadPoolExecutor
            with ThreadPoolExecutor(self.num_workers) as ex:
                return list(ex.map(self.tokenizer.encode, preprocessed))
        return [self.tokenizer.encode(t) for t in preprocessed]

    def run_stage3(self, tokenized: Sequence[Sequence[int]]) -> List[torch.Tensor]:
        """Documents are concatenated into one stream and cut into [batch, seq] blocks (the last partial block is dropped)."""
        stream = np.fromiter((tok for doc in tokenized for tok in doc), dtype=np.int64)
        per = self.batch_size * self.seq_length
        n = stream.size // per
        return [torch.from_numpy(stream[i * per:(i + 1) * per].copy()).view(self.batch_size, self.seq_length) for i in range(n)]

    def process_texts(self, texts: Sequence[str]) -> List[torch.Tensor]:
        batches = self.run_stage3(self.run_stage2(self.run_stage1(texts)))
        for _, fn in self.custom_stages:
            batches = fn(batches)
        self.total_processed += len(texts)
        return batches

    def process_file(self, path: str) -> List[torch.Tensor]:
        with open(path, "r", encoding="utf-8", errors="replace") as f:
            docs = [d for d in re.split(r"\n\s*\n", f.read()) if d.strip()]
        return self.process_texts(docs)


@dataclass
class DataLoaderConfig:
    data_path: str = ""
    batch_size: int = 8
    seq_length: int = 2048
    shuffle_buffer: int = 10000
    num_epochs: int = 1
    num_workers: int = 1
    seed: int = 42
    drop_last: bool = True
    world_size: int = 1
    rank: int = 0


class DataLoader:
    """Windows of ``seq_length + 1`` tokens cut from the tokenised file; rank r takes windows r, r + world, ...; a shuffle
    buffer of ``shuffle_buffer`` windows decorrelates neighbours; ``num_epochs`` passes, reshuffled per epoch."""

    def __init__(self, cfg: DataLoaderConfig, tokenizer=None):
        self.config, self.tokenizer = cfg, tokenizer
        with open(cfg.data_path, "rb") as f:
            raw = f.read()
        ids = tokenizer.encode(raw.decode("utf-8", "replace")) if tokenizer is not None else list(raw)
        self.tokens = torch.tensor(ids, dtype=torch.int64)
        L = cfg.seq_length
        n_windows = max(0, (self.tokens.numel() - 1) // L)
        self.windows = list(range(cfg.rank, n_windows, max(1, cfg.world_size)))
        self.reset()

    def _epoch_order(self, epoch: int) -> List[int]:
        rng = random.Random(self.config.seed * 1000003 + epoch)
        buf: deque = deque()
        out: List[int] = []
        for w in self.windows:                      # streaming shuffle: a bounded buffer, one random eviction per arrival
            buf.append(w)
            if len(buf) > max(1, self.config.shuffle_buffer):
                i = rng.randrange(len(buf))
                buf[i], buf[-1] = buf[-1], buf[i]
                out.append(buf.pop())
        rest = list(buf)
        rng.shuffle(rest)
        return out + rest

    def reset(self):
        self.batch_index = 0
        self.order = [w for e in range(max(1, self.config.num_epochs)) for w in self._epoch_order(e)]

    def num_batches(self) -> int:
        b = self.config.batch_size
        return len(self.order) // b if self.config.drop_last else -(-len(self.order) // b)

    def has_next(self) -> bool:
        return self.batch_index < self.num_batches()

    def next_batch_with_labels(self) -> Tuple[torch.Tensor, torch.Tensor]:
        if not self.has_next():
            raise StopIteration
        b, L = self.config.batch_size, self.config.seq_length
        ws = self.order[self.batch_index * b:(self.batch_index + 1) * b]
        self.batch_index += 1
        rows = torch.stack([self.tokens[w * L:w * L + L + 1] for w in ws])
        return rows[:, :-1].contiguous(), rows[:, 1:].contiguous()

    def next_batch(self) -> torch.Tensor:
        return self.next_batch_with_labels()[0]

    def __iter__(self):
        while self.has_next():
            yield self.next_batch_with_labels()


class MinHashDedup:
    """Bounded filter over token n-grams. An n-gram's ``num_hashes`` 64-bit fingerprints (one multiply-xorshift family per
    hash) are looked up in / inserted into an LRU-bounded set; it counts as a duplicate when at least 90 % of them are
    present, which tolerates the evictions of a full filter without calling unseen n-grams duplicates."""

    def __init__(self, ngram_size: int = 4, num_hashes: int = 128, max_capacity: int = 1_000_000):
        self.ngram_size, self.num_hashes, self.max_capacity = ngram_size, num_hashes, max_capacity
        rng = np.random.default_rng(0x4D48)
        self._mul = rng.integers(1, 1 << 62, num_hashes, dtype=np.uint64) | np.uint64(1)
        self._add = rng.integers(0, 1 << 62, num_hashes, dtype=np.uint64)
        self._seen: "OrderedDict[int, None]" = OrderedDict()
        self.total_checked = self.duplicates_found = 0

    def _fingerprints(self, tokens: Sequence[int]) -> np.ndarray:
        h = np.uint64(1469598103934665603)
        with np.errstate(over="ignore"):
            for t in tokens[: self.ngram_size]:
                h = (h ^ np.uint64(int(t) & 0xFFFFFFFFFFFFFFFF)) * np.uint64(1099511628211)
            f = h * self._mul + self._add
            f ^= f >> np.uint64(29)
            f *= np.uint64(0xBF58476D1CE4E5B9)
            f ^= f >> np.uint64(32)
        return f

    def is_duplicate(self, tokens: Sequence[int]) -> bool:
        self.total_checked += 1
        fp = self._fingerprints(tokens)
        hits = sum(1 for v in fp.tolist() if v in self._seen)
        dup = hits >= 0.9 * self.num_hashes
        self.duplicates_found += dup
        return dup

    def insert(self, tokens: Sequence[int]):
        for v in self._fingerprints(tokens).tolist():
            self._seen[v] = None
            self._seen.move_to_end(v)
        while len(self._seen) > self.max_capacity:
            self._seen.popitem(last=False)

    def filter_stream(self, ids: Sequence[int]) -> List[int]:
        """Tokens of ``ids`` with every n-gram window that was seen before cut out (first occurrences stay)."""
        n, out, i = self.ngram_size, [], 0
        while i < len(ids):
            gram = ids[i:i + n]
            if len(gram) == n and self.is_duplicate(gram):
                i += n
                continue
            if len(gram) == n:
                self.insert(gram)
            out.append(ids[i])
            i += 1
        return out

    def clear(self):
        self._seen.clear()
        self.total_checked = self.duplicates_found = 0

    def duplicate_rate(self) -> float:
        return self.duplicates_found / self.total_checked if self.total_checked else 0.0


# ------------------------------------------------------------------------------------------------ memory-mapped and streaming text loaders
@dataclass
class MmapDataLoaderConfig:
    batch_size: int = 8
    seq_length: int = 2048
    shuffle_buffer: int = 100000          # sequences are drawn at random from up to this many buffered tokens' worth
    mmap_window: int = 1024 * 1024        # bytes of text tokenised per refill
    dedup_enabled: bool = True
    ngram_size: int = 4
    seed: int = 42
    drop_last: bool = True
    num_workers: int = 1
    max_seen_ngrams: int = 4_000_000


def _cut_at_boundary(buf, start: int, end: int, limit: int) -> int:
    """Moves ``end`` back to just after the last whitespace byte of [start, end) when the window does not reach ``limit``
    (the end of the data), so that neither a word nor a UTF-8 sequence is split; falls back to a character boundary."""
    if end >= limit:
        return limit
    for i in range(end, max(start, end - 4096), -1):
        if buf[i - 1] in b" \n\t\r":
            return i
    while end > start and (buf[end] & 0xC0) == 0x80:
        end -= 1
    return end


class MmapDataLoader:
    """Batches straight from a memory-mapped text file (reference: ``MmapDataLoader``, include/oil/mmap_dataloader.h:94-160,
    src/tensor_view.cpp:100-260): a window of the file is tokenised per refill, n-grams seen before are dropped, and batches
    of ``batch_size`` x ``seq_length`` ids are cut from the token buffer; ``next_batch_with_labels`` returns the next-token
    targets too. The file is never read whole.

    The n-gram filter is exact and vectorised: every n-gram of a window gets a 64-bit polynomial hash in one numpy pass, a
    token is dropped when the n-gram starting at it was seen in an earlier window or earlier in this one, and the bounded set
    of seen hashes is a sorted array probed with ``searchsorted`` (the reference probes a MinHash filter once per token)."""

    def __init__(self, file_path: str, tokenizer, cfg: Optional[MmapDataLoaderConfig] = None):
        import mmap
        self.cfg = cfg or MmapDataLoaderConfig()
        self.tokenizer = tokenizer
        self._file = open(file_path, "rb")
        self._size = self._file.seek(0, 2)
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ) if self._size else b""
        self._rng = np.random.default_rng(self.cfg.seed)
        self.reset()

    def reset(self) -> None:
        self._offset, self.total_tokens, self.tokens_dropped = 0, 0, 0
        self._buffer = np.zeros(0, dtype=np.int64)
        self._seen = np.zeros(0, dtype=np.uint64)
        self._pool: List[np.ndarray] = []

    def close(self) -> None:
        if self._size:
            self._map.close()
        self._file.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # -- refill
    def tokenize_window(self, start: int, length: int) -> np.ndarray:
        text = bytes(self._map[start: start + length]).decode("utf-8", "replace")
        return np.asarray(self.tokenizer.encode(text), dtype=np.int64)

    def _dedup(self, tokens: np.ndarray) -> np.ndarray:
        n = self.cfg.ngram_size
        if tokens.size < n:
            return tokens
        win = np.lib.stride_tricks.sliding_window_view(tokens.astype(np.uint64), n)
        h = np.full(win.shape[0], 1469598103934665603, dtype=np.uint64)
        with np.errstate(over="ignore"):
            for k in range(n):
                h = (h ^ win[:, k]) * np.uint64(1099511628211)
        pos = np.searchsorted(self._seen, h)
        earlier = (pos < self._seen.size) & (self._seen[np.minimum(pos, max(0, self._seen.size - 1))] == h) if self._seen.size else \
            np.zeros(h.size, dtype=bool)
        _, first = np.unique(h, return_index=True)
        repeat = np.ones(h.size, dtype=bool)
        repeat[first] = False
        drop = earlier | repeat
        merged = np.union1d(self._seen, h)
        self._seen = merged[-self.cfg.max_seen_ngrams:] if merged.size > self.cfg.max_seen_ngrams else merged
        keep = np.ones(tokens.size, dtype=bool)
        keep[: h.size] = ~drop
        self.tokens_dropped += int(drop.sum())
        return tokens[keep]

    def refill_buffer(self) -> bool:
        if self._offset >= self._size:
            return False
        end = _cut_at_boundary(self._map, self._offset, min(self._size, self._offset + self.cfg.mmap_window), self._size)
        if end <= self._offset:
            end = min(self._size, self._offset + self.cfg.mmap_window)
        tokens = self.tokenize_window(self._offset, end - self._offset)
        self._offset = end
        if self.cfg.dedup_enabled:
            tokens = self._dedup(tokens)
        self._buffer = np.concatenate([self._buffer, tokens])
        self.total_tokens += int(tokens.size)
        return True

    # -- batches
    def _need(self, extra: int) -> int:
        return self.cfg.batch_size * self.cfg.seq_length + extra

    def has_next(self) -> bool:
        return self._buffer.size >= self._need(1) or self._offset < self._size or len(self._pool) >= self.cfg.batch_size

    def num_batches(self) -> int:
        """Batches worth of tokens read so far (the file's total is only known once it has been read through)."""
        return self.total_tokens // (self.cfg.batch_size * self.cfg.seq_length)

    def _take(self, extra: int) -> Optional[np.ndarray]:
        """``batch_size`` rows of ``seq_length + extra`` tokens as a 2-D array (row r + 1 of an unshuffled batch starts where
        row r's inputs end). With a shuffle buffer the rows are drawn at random from a pool of up to
        ``shuffle_buffer // seq_length`` buffered rows, each cut whole from the stream with its own label token."""
        S, B = self.cfg.seq_length, self.cfg.batch_size
        if self.cfg.shuffle_buffer > 0:
            want = max(B, self.cfg.shuffle_buffer // S)
            while len(self._pool) < want:
                while self._buffer.size < S + 1 and self.refill_buffer():
                    pass
                if self._buffer.size < S + 1:
                    break
                self._pool.append(self._buffer[: S + 1].copy())
                self._buffer = self._buffer[S:]
            if len(self._pool) < B:
                if self.cfg.drop_last or not self._pool:
                    self._pool.clear()
                    return None
                rows = self._pool + [np.zeros(S + 1, dtype=np.int64)] * (B - len(self._pool))
                self._pool = []
                return np.stack(rows)[:, : S + extra]
            pick = sorted(self._rng.choice(len(self._pool), B, replace=False).tolist(), reverse=True)
            rows = [self._pool.pop(i) for i in pick]
            return np.stack(rows[::-1])[:, : S + extra]
        need = B * S + extra
        while self._buffer.size < need and self.refill_buffer():
            pass
        if self._buffer.size < need:
            if self.cfg.drop_last or self._buffer.size <= extra:
                self._buffer = self._buffer[:0]
                return None
            flat = np.zeros(need, dtype=np.int64)
            flat[: self._buffer.size] = self._buffer
            self._buffer = self._buffer[:0]
        else:
            flat = self._buffer[:need]
            self._buffer = self._buffer[B * S:]
        return np.stack([flat[r * S: r * S + S + extra] for r in range(B)])

    def next_batch(self) -> Optional[torch.Tensor]:
        rows = self._take(0)
        return None if rows is None else torch.from_numpy(np.ascontiguousarray(rows))

    def next_batch_with_labels(self) -> Optional[Tuple[torch.Tensor, torch.Tensor]]:
        rows = self._take(1)
        if rows is None:
            return None
        t = torch.from_numpy(np.ascontiguousarray(rows))
        return t[:, :-1].contiguous(), t[:, 1:].contiguous()


class StreamingDataLoader:
    """Sequential batches from a text file read 1 MiB at a time through a rolling token buffer (reference:
    ``StreamingDataLoader``, include/oil/trainer.h:193-213): ``next_batch`` returns (ids, labels) or None at the end; the
    file is tokenised incrementally and never held whole."""

    def __init__(self, tokenizer, data_path: str, batch_size: int, seq_length: int, chunk_bytes: int = 1 << 20):
        self.tokenizer, self.path = tokenizer, data_path
        self._batch_size, self._seq_length, self.chunk_bytes = batch_size, seq_length, chunk_bytes
        self._file = open(data_path, "rb")
        self.reset()

    def batch_size(self) -> int:
        return self._batch_size

    def seq_length(self) -> int:
        return self._seq_length

    def num_batches(self) -> int:
        return self._served

    def reset(self) -> None:
        self._file.seek(0)
        self._buffer: List[int] = []
        self._carry = b""
        self._eof, self._served = False, 0

    def close(self) -> None:
        self._file.close()

    def fill_buffer(self) -> None:
        data = self._file.read(self.chunk_bytes)
        if not data:
            self._eof = True
            data, self._carry = self._carry, b""
        else:
            data = self._carry + data
            cut = _cut_at_boundary(data + b" ", 0, len(data), len(data) + 1)
            data, self._carry = data[:cut], data[cut:]
        if data:
            self._buffer.extend(self.tokenizer.encode(data.decode("utf-8", "replace")))

    def next_batch(self) -> Optional[Tuple[torch.Tensor, torch.Tensor]]:
        need = self._batch_size * self._seq_length + 1
        while len(self._buffer) < need and not self._eof:
            self.fill_buffer()
        if len(self._buffer) < need:
            return None
        flat = torch.tensor(self._buffer[:need], dtype=torch.long)
        del self._buffer[: need - 1]
        self._served += 1
        B, S = self._batch_size, self._seq_length
        return flat[:-1].view(B, S), flat[1:].view(B, S)
