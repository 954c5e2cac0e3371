"""Datasets of (input ids, target ids) pairs and the combinators around them.

Reference behaviour covered (include/oil/dataset.h:18-202): ``Dataset`` (size / get), ``InMemoryDataset`` (from a text
file through a tokenizer with a stride, from a file of token ids, from a directory), ``StreamingDataset`` (files matched
by a pattern, read shard by shard through a shuffle buffer), ``ChunkedDataset`` (a token file cut into overlapping chunks
read on demand), ``FilterDataset`` / ``MapDataset`` / ``ConcatDataset`` / ``ShuffleDataset`` and ``split_dataset``.
Targets are the inputs shifted by one token. Token files are little-endian int32.
"""
from __future__ import annotations

import glob
import os
import random
from typing import Callable, Iterator, List, Optional, Sequence, Tuple

import numpy as np
import torch

Pair = Tuple[torch.Tensor, torch.Tensor]


class Dataset:
    def __len__(self) -> int:
        raise NotImplementedError

    def get(self, index: int) -> Pair:
        raise NotImplementedError

    def __getitem__(self, index: int) -> Pair:
        return self.get(index)

    def batches(self, batch_size: int, drop_last: bool = True) -> Iterator[Pair]:
        n = len(self)
        for i in range(0, n - (batch_size - 1 if drop_last else 0), batch_size):
            xs, ys = zip(*(self.get(j) for j in range(i, min(n, i + batch_size))))
            yield torch.stack(xs), torch.stack(ys)


def _windows(ids: Sequence[int], seq_len: int, stride: int, max_samples: int):
    ids = torch.as_tensor(np.asarray(ids, dtype=np.int64))
    out = []
    for s in range(0, max(0, ids.numel() - seq_len), stride):
        out.append((ids[s:s + seq_len].clone(), ids[s + 1:s + seq_len + 1].clone()))
        if 0 < max_samples <= len(out):
            break
    return out


class InMemoryDataset(Dataset):
    def __init__(self):
        self.inputs: List[torch.Tensor] = []
        self.targets: List[torch.Tensor] = []

    def __len__(self):
        return len(self.inputs)

    def get(self, index):
        return self.inputs[index], self.targets[index]

    def add_sample(self, inp: torch.Tensor, target: torch.Tensor):
        self.inputs.append(inp)
        self.targets.append(target)

    def clear(self):
        self.inputs.clear()
        self.targets.clear()

    def _extend(self, pairs):
        for x, y in pairs:
            self.add_sample(x, y)
        return self

    @classmethod
    def from_text_file(cls, path: str, tok, seq_len: int, stride: int = -1, max_samples: int = -1) -> "InMemoryDataset":
        ids = tok.encode(open(path, encoding="utf-8", errors="replace").read())
        return cls()._extend(_windows(ids, seq_len, seq_len if stride <= 0 else stride, max_samples))

    @classmethod
    def from_tokenized_file(cls, path: str, seq_len: int, max_samples: int = -1) -> "InMemoryDataset":
        return cls()._extend(_windows(np.fromfile(path, dtype="<i4"), seq_len, seq_len, max_samples))

    @classmethod
    def from_directory(cls, directory: str, ext: str, tok, seq_len: int) -> "InMemoryDataset":
        ds = cls()
        for p in sorted(glob.glob(os.path.join(directory, "*" + ext))):
            ds._extend(_windows(tok.encode(open(p, encoding="utf-8", errors="replace").read()), seq_len, seq_len, -1))
        return ds


class StreamingDataset(Dataset):
    """Token files matched by ``pattern`` are the shards; samples come out of a shuffle buffer that is refilled shard by
    shard, so memory stays at ``buffer_size`` samples whatever the corpus size. ``get(i)`` ignores ``i`` beyond bounds
    checking: the order is the stream's."""

    def __init__(self, pattern: str, seq_len: int, buffer_size: int = 10000, seed: int = 42):
        self.shards = sorted(glob.glob(pattern))
        self.seq_len, self.buffer_size = seq_len, buffer_size
        self.rng = random.Random(seed)
        self.sizes = [max(0, (os.path.getsize(p) // 4 - 1) // seq_len) for p in self.shards]
        self._buffer: List[Pair] = []
        self._shard = 0
        self._offset = 0

    def __len__(self):
        return sum(self.sizes)

    def _refill(self):
        while len(self._buffer) < self.buffer_size and self.shards:
            if self._offset >= self.sizes[self._shard]:
                last = self._shard + 1 == len(self.shards)
                self._shard, self._offset = (self._shard + 1) % len(self.shards), 0
                if sum(self.sizes) == 0 or (last and self._buffer):
                    return              # the next epoch starts only once this one has been handed out
                continue
            take = min(self.buffer_size - len(self._buffer), self.sizes[self._shard] - self._offset)
            ids = np.fromfile(self.shards[self._shard], dtype="<i4", count=take * self.seq_len + 1, offset=4 * self._offset * self.seq_len)
            self._buffer.extend(_windows(ids, self.seq_len, self.seq_len, -1))
            self._offset += take

    def get(self, index):
        if not 0 <= index < len(self):
            raise IndexError(index)
        if not self._buffer:
            self._refill()
        j = self.rng.randrange(len(self._buffer))
        self._buffer[j], self._buffer[-1] = self._buffer[-1], self._buffer[j]
        return self._buffer.pop()


class ChunkedDataset(Dataset):
    """A token file seen as chunks of ``chunk_size`` tokens that overlap by ``overlap``; a chunk is read from disk when one
    of its samples is asked for (one chunk cached)."""

    def __init__(self, path: str, chunk_size: int, overlap: int = 0, seq_len: int = 2048):
        assert chunk_size > overlap and chunk_size > seq_len
        self.path, self.chunk_size, self.overlap, self.seq_len = path, chunk_size, overlap, seq_len
        self.n_tokens = os.path.getsize(path) // 4
        step = chunk_size - overlap
        self.chunk_offsets = list(range(0, max(1, self.n_tokens - seq_len), step))
        self.per_chunk = [max(0, (min(chunk_size, self.n_tokens - o) - 1) // seq_len) for o in self.chunk_offsets]
        self._cum = np.cumsum([0] + self.per_chunk)
        self._cached = (-1, None)

    @property
    def num_chunks(self):
        return len(self.chunk_offsets)

    def __len__(self):
        return int(self._cum[-1])

    def read_chunk(self, c: int) -> np.ndarray:
        if self._cached[0] != c:
            self._cached = (c, np.fromfile(self.path, dtype="<i4", count=self.chunk_size, offset=4 * self.chunk_offsets[c]))
        return self._cached[1]

    def get(self, index):
        c = int(np.searchsorted(self._cum, index, side="right") - 1)
        ids = self.read_chunk(c)
        s = (index - int(self._cum[c])) * self.seq_len
        t = torch.as_tensor(ids[s:s + self.seq_len + 1].astype(np.int64))
        return t[:-1], t[1:]


class FilterDataset(Dataset):
    def __init__(self, base: Dataset, predicate: Callable[[torch.Tensor, torch.Tensor], bool]):
        self.base = base
        self.indices = [i for i in range(len(base)) if predicate(*base.get(i))]

    def __len__(self):
        return len(self.indices)

    def get(self, index):
        return self.base.get(self.indices[index])


class MapDataset(Dataset):
    def __init__(self, base: Dataset, fn: Callable[[torch.Tensor, torch.Tensor], Pair]):
        self.base, self.fn = base, fn

    def __len__(self):
        return len(self.base)

    def get(self, index):
        return self.fn(*self.base.get(index))


class ConcatDataset(Dataset):
    def __init__(self, parts: Sequence[Dataset]):
        self.parts = list(parts)
        self._cum = np.cumsum([0] + [len(p) for p in self.parts])

    def __len__(self):
        return int(self._cum[-1])

    def get(self, index):
        k = int(np.searchsorted(self._cum, index, side="right") - 1)
        return self.parts[k].get(index - int(self._cum[k]))


class ShuffleDataset(Dataset):
    """A fixed permutation of the base (``reshuffle`` draws the next epoch's)."""

    def __init__(self, base: Dataset, seed: int = 42):
        self.base = base
        self.rng = random.Random(seed)
        self.perm = list(range(len(base)))
        self.reshuffle()

    def reshuffle(self):
        self.rng.shuffle(self.perm)

    def __len__(self):
        return len(self.perm)

    def get(self, index):
        return self.base.get(self.perm[index])


class _Subset(Dataset):
    def __init__(self, base, indices):
        self.base, self.indices = base, indices

    def __len__(self):
        return len(self.indices)

    def get(self, index):
        return self.base.get(self.indices[index])


def split_dataset(base: Dataset, train_ratio: float, val_ratio: float, seed: int = 42):
    """-> (train, val, test): a seeded permutation cut at the two ratios, the remainder is the test set."""
    idx = list(range(len(base)))
    random.Random(seed).shuffle(idx)
    a = int(len(idx) * train_ratio)
    b = a + int(len(idx) * val_ratio)
    return _Subset(base, idx[:a]), _Subset(base, idx[a:b]), _Subset(base, idx[b:])
