"""Synthetic text tasks, a difficulty curriculum, tokenizer evaluation and Parquet shard reading.

Reference behaviour covered (include/oil/data_gen.h:14-128, include/oil/parquet_streamer.h:9-36): ``DataGenerator`` (random
strings / words / sentences / integer sequences, arithmetic problems, copy / reverse / n-gram tasks), ``CurriculumGenerator``
(stages of rising difficulty, promotion when the reported accuracy stays above a threshold), ``TokenizerEvaluator``
(compression ratio, round-trip accuracy, vocabulary coverage and utilisation, character error rate, bytes per token)
and ``ParquetReader`` (token batches out of a text or token column of Parquet shards; here through ``pyarrow`` instead
of a hand-written page decoder).
"""
from __future__ import annotations

import random
import string
from collections import Counter
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import torch

_SYLL = ["ka", "lo", "mi", "re", "tu", "sa", "ne", "vo", "di", "pu", "an", "el", "or", "is", "um"]


class DataGenerator:
    def __init__(self, seed: int = 42):
        self.rng = random.Random(seed)

    def random_string(self, length: int, include_digits: bool = True) -> str:
        alphabet = string.ascii_lowercase + (string.digits if include_digits else "")
        return "".join(self.rng.choice(alphabet) for _ in range(length))

    def random_word(self) -> str:
        return "".join(self.rng.choice(_SYLL) for _ in range(self.rng.randint(1, 4)))

    def random_sentence(self, words: int) -> str:
        s = " ".join(self.random_word() for _ in range(max(1, words)))
        return s[0].upper() + s[1:] + "."

    def random_sequence(self, length: int, max_val: int = 100) -> List[int]:
        return [self.rng.randint(0, max_val - 1) for _ in range(length)]

    @staticmethod
    def compute_arithmetic(a: int, b: int, op: str) -> int:
        if op == "+":
            return a + b
        if op == "-":
            return a - b
        if op == "*":
            return a * b
        if op == "/":
            return a // b if b else 0
        raise ValueError(f"unknown operator {op!r}")

    def format_arithmetic_problem(self, a: int, b: int, op: str) -> str:
        return f"{a} {op} {b} = {self.compute_arithmetic(a, b, op)}"

    def arithmetic_task(self, n: int, max_operand: int = 99, ops: str = "+-*") -> List[str]:
        return [self.format_arithmetic_problem(self.rng.randint(0, max_operand), self.rng.randint(0, max_operand), self.rng.choice(ops))
                for _ in range(n)]

    def copy_task(self, n: int, length: int = 8) -> List[str]:
        out = []
        for _ in range(n):
            s = self.random_string(length, False)
            out.append(f"copy: {s} -> {s}")
        return out

    def reverse_task(self, n: int, length: int = 8) -> List[str]:
        out = []
        for _ in range(n):
            s = self.random_string(length, False)
            out.append(f"reverse: {s} -> {s[::-1]}")
        return out

    def ngram_task(self, n: int, order: int = 2, length: int = 32, alphabet: str = "abcdefgh") -> List[str]:
        """Strings from a random order-``order`` Markov chain (each context has one strongly preferred successor)."""
        table: Dict[str, str] = {}
        out = []
        for _ in range(n):
            s = "".join(self.rng.choice(alphabet) for _ in range(order))
            while len(s) < length:
                ctx = s[-order:]
                fav = table.setdefault(ctx, self.rng.choice(alphabet))
                s += fav if self.rng.random() < 0.8 else self.rng.choice(alphabet)
            out.append(s)
        return out

    def passes_task_weight(self, cumulative_weight: float) -> bool:
        return self.rng.random() < cumulative_weight


@dataclass
class CurriculumStage:
    name: str
    difficulty: int
    generator_fn: Callable[[int], List[str]]
    promote_accuracy: float = 0.9
    min_batches: int = 1


class CurriculumGenerator:
    """Serves batches from the current stage; ``report_accuracy`` feeds a short moving window and the generator moves to the
    next stage once the window's mean reaches the stage's threshold (and ``min_batches`` were served)."""

    def __init__(self, seed: int = 42, window: int = 3):
        self.stages: List[CurriculumStage] = []
        self.idx, self.window = 0, window
        self._acc: List[float] = []
        self._served = 0
        self.progress_fn: Optional[Callable[[str, int, float], None]] = None
        self.gen = DataGenerator(seed)

    def add_stage(self, stage: CurriculumStage):
        self.stages.append(stage)
        self.stages.sort(key=lambda s: s.difficulty)

    def set_progress_fn(self, fn):
        self.progress_fn = fn

    def current_stage_name(self) -> str:
        return self.stages[min(self.idx, len(self.stages) - 1)].name if self.stages else ""

    def current_difficulty(self) -> int:
        return self.stages[min(self.idx, len(self.stages) - 1)].difficulty if self.stages else 0

    def is_complete(self) -> bool:
        return self.idx >= len(self.stages)

    def generate_next_batch(self, batch_size: int) -> List[str]:
        st = self.stages[min(self.idx, len(self.stages) - 1)]
        self._served += 1
        return st.generator_fn(batch_size)

    def should_promote(self) -> bool:
        if self.is_complete() or not self._acc:
            return False
        st = self.stages[self.idx]
        recent = self._acc[-self.window:]
        return self._served >= st.min_batches and len(recent) >= min(self.window, st.min_batches) and sum(recent) / len(recent) >= st.promote_accuracy

    def report_accuracy(self, accuracy: float):
        self._acc.append(accuracy)
        if self.progress_fn is not None:
            self.progress_fn(self.current_stage_name(), self.current_difficulty(), accuracy)
        if self.should_promote():
            self.idx += 1
            self._acc, self._served = [], 0

    @classmethod
    def default(cls, seed: int = 42) -> "CurriculumGenerator":
        c = cls(seed)
        g = c.gen
        c.add_stage(CurriculumStage("copy", 1, lambda n: g.copy_task(n, 4)))
        c.add_stage(CurriculumStage("reverse", 2, lambda n: g.reverse_task(n, 6)))
        c.add_stage(CurriculumStage("ngram", 3, lambda n: g.ngram_task(n)))
        c.add_stage(CurriculumStage("arithmetic", 4, lambda n: g.arithmetic_task(n)))
        return c


def _edit_distance(a: str, b: str) -> int:
    prev = list(range(len(b) + 1))
    for i, ca in enumerate(a, 1):
        cur = [i]
        for j, cb in enumerate(b, 1):
            cur.append(min(prev[j] + 1, cur[j - 1] + 1, prev[j - 1] + (ca != cb)))
        prev = cur
    return prev[-1]


@dataclass
class EvaluationReport:
    compression_ratio: float = 0.0
    re_encoding_accuracy: float = 0.0
    vocabulary_coverage: float = 0.0
    average_token_length: float = 0.0
    vocabulary_utilization: float = 0.0
    reconstruction_fidelity: float = 0.0
    byte_efficiency: float = 0.0
    documents: int = 0


class TokenizerEvaluator:
    """Works with any tokenizer that has ``encode(str) -> ids``, ``decode(ids) -> str`` and ``vocab_size``."""

    def __init__(self, tokenizer):
        self.tok = tokenizer

    def encode_with_check(self, text: str) -> List[int]:
        ids = list(self.tok.encode(text))
        V = self.tok.vocab_size
        if any(i < 0 or i >= V for i in ids):
            raise ValueError("token id outside the vocabulary")
        return ids

    def compression_ratio(self, text: str) -> float:
        """UTF-8 bytes per token."""
        n = len(self.encode_with_check(text))
        return len(text.encode("utf-8")) / n if n else 0.0

    def re_encoding_accuracy(self, text: str) -> float:
        """Share of positions at which encode(decode(encode(text))) repeats encode(text)."""
        a = self.encode_with_check(text)
        b = list(self.tok.encode(self.tok.decode(a)))
        if not a:
            return 1.0
        return sum(x == y for x, y in zip(a, b)) / max(len(a), len(b))

    def vocabulary_coverage(self, corpus: str) -> float:
        """Share of the corpus' distinct characters that survive a round trip."""
        chars = set(corpus)
        if not chars:
            return 1.0
        return sum(self.tok.decode(self.tok.encode(c)) == c for c in chars) / len(chars)

    def average_token_length(self, corpus: str) -> float:
        n = len(self.encode_with_check(corpus))
        return len(corpus) / n if n else 0.0

    def vocabulary_utilization(self, corpus: str) -> float:
        return len(set(self.encode_with_check(corpus))) / max(1, self.tok.vocab_size)

    @staticmethod
    def character_error_rate(original: str, reconstructed: str) -> float:
        return _edit_distance(original, reconstructed) / max(1, len(original))

    def reconstruction_fidelity(self, text: str) -> float:
        return 1.0 - min(1.0, self.character_error_rate(text, self.tok.decode(self.encode_with_check(text))))

    def byte_efficiency(self, text: str) -> float:
        """Bytes of text per byte of token ids when an id is stored in the fewest whole bytes the vocabulary allows."""
        n = len(self.encode_with_check(text))
        width = max(1, ((self.tok.vocab_size - 1).bit_length() + 7) // 8)
        return len(text.encode("utf-8")) / (n * width) if n else 0.0

    def evaluate(self, corpus: Sequence[str]) -> EvaluationReport:
        docs = [d for d in corpus if d]
        if not docs:
            return EvaluationReport()
        joined = "\n".join(docs)
        mean = lambda f: sum(f(d) for d in docs) / len(docs)
        return EvaluationReport(mean(self.compression_ratio), mean(self.re_encoding_accuracy), self.vocabulary_coverage(joined),
                                self.average_token_length(joined), self.vocabulary_utilization(joined), mean(self.reconstruction_fidelity),
                                mean(self.byte_efficiency), len(docs))

    @staticmethod
    def report_string(r: EvaluationReport) -> str:
        return (f"docs {r.documents}  bytes/token {r.compression_ratio:.2f}  chars/token {r.average_token_length:.2f}  round-trip "
                f"{100 * r.re_encoding_accuracy:.1f}%  fidelity {100 * r.reconstruction_fidelity:.1f}%  coverage {100 * r.vocabulary_coverage:.1f}%  "
                f"vocab used {100 * r.vocabulary_utilization:.1f}%  byte efficiency {r.byte_efficiency:.2f}")


@dataclass
class ParquetShard:
    path: str
    num_rows: int = 0
    num_tokens: int = 0


class ParquetReader:
    """Streams token ids out of Parquet shards row group by row group. ``column`` holds either text (tokenised with
    ``tokenizer``) or lists of token ids. ``next_batch(max_tokens)`` returns up to that many ids (int64 tensor), carrying the
    remainder of a row over to the next call; an empty tensor marks the end."""

    def __init__(self, column: str = "text", tokenizer=None, eos_id: Optional[int] = None):
        self.column, self.tokenizer, self.eos_id = column, tokenizer, eos_id
        self._file = None
        self.shard: Optional[ParquetShard] = None
        self.reset_counters()

    def reset_counters(self):
        self.total_tokens = self.rows_read = 0
        self._group = 0
        self._carry: List[int] = []
        self._rows: List = []

    def open(self, path: str) -> bool:
        import pyarrow.parquet as pq
        try:
            self._file = pq.ParquetFile(path)
        except Exception:                            # noqa: BLE001 - a missing or malformed shard is reported, not raised
            self._file = None
            return False
        if self.column not in self._file.schema_arrow.names:
            self._file = None
            return False
        self.shard = ParquetShard(path, self._file.metadata.num_rows, 0)
        self.reset_counters()
        return True

    def _more_rows(self) -> bool:
        if self._file is None or self._group >= self._file.num_row_groups:
            return False
        self._rows = self._file.read_row_group(self._group, columns=[self.column]).column(0).to_pylist()
        self._group += 1
        return True

    def next_batch(self, max_tokens: int) -> torch.Tensor:
        out = self._carry
        self._carry = []
        while len(out) < max_tokens:
            if not self._rows and not self._more_rows():
                break
            row = self._rows.pop(0)
            self.rows_read += 1
            if row is None:
                continue
            ids = list(self.tokenizer.encode(row)) if isinstance(row, str) else [int(t) for t in row]
            if self.eos_id is not None:
                ids.append(self.eos_id)
            out.extend(ids)
        out, self._carry = out[:max_tokens], out[max_tokens:]
        self.total_tokens += len(out)
        if self.shard is not None:
            self.shard.num_tokens = self.total_tokens
        return torch.tensor(out, dtype=torch.long)

    def reset(self):
        if self._file is not None:
            self.reset_counters()

    def close(self):
        self._file = None
        self._rows, self._carry = [], []

    def batches(self, batch_size: int, seq_len: int):
        """(ids, labels) pairs of shape [batch_size, seq_len] until the shard runs out."""
        need = batch_size * seq_len + 1
        tail = torch.empty(0, dtype=torch.long)
        while True:
            chunk = torch.cat([tail, self.next_batch(need - tail.numel())])
            if chunk.numel() < need:
                return
            yield chunk[:-1].view(batch_size, seq_len), chunk[1:].view(batch_size, seq_len)
            tail = chunk[-1:]
