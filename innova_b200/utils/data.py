"""Synthetic token streams and the token DataLoader.

``zipf_tokens`` draws ids i.i.d. from a truncated Zipf(s) law over the vocabulary (rank k has
probability proportional to k^-s), reproducibly from a seed. ``TokenLoader`` serves a flat token
array the way the reference's DataLoader does (src/trainer_data.cpp:238-280): batch i is tokens
[i*B*S, (i+1)*B*S) and the labels are the next tokens; it can shuffle per epoch and keeps batches in
pinned memory so that the host-to-device copy overlaps compute.
"""
from __future__ import annotations

import numpy as np
import torch


def zipf_probs(vocab: int, s: float = 1.1) -> np.ndarray:
    w = 1.0 / np.power(np.arange(1, vocab + 1, dtype=np.float64), s)
    return w / w.sum()


def zipf_tokens(n: int, vocab: int, s: float = 1.1, seed: int = 0) -> torch.Tensor:
    """n token ids in [0, vocab) with P(id = k-1) ~ k^-s."""
    rng = np.random.default_rng(seed)
    cdf = np.cumsum(zipf_probs(vocab, s))
    u = rng.random(n)
    ids = np.searchsorted(cdf, u, side="right")
    np.clip(ids, 0, vocab - 1, out=ids)
    return torch.from_numpy(ids.astype(np.int64))


class TokenLoader:
    """Batches of (ids [B,S], labels [B,S]) from a flat token tensor."""

    def __init__(self, tokens: torch.Tensor, batch_size: int, seq_len: int, shuffle: bool = False, seed: int = 0, pin: bool = False,
                 drop_last: bool = True):
        self.tokens = tokens.reshape(-1).long()
        self.B, self.S = batch_size, seq_len
        self.shuffle, self.seed, self.epoch = shuffle, seed, 0
        self.pin = pin and torch.cuda.is_available()
        per = batch_size * seq_len
        self.num_batches = (self.tokens.numel() - 1) // per
        if self.num_batches <= 0:
            raise ValueError("not enough tokens for one batch")

    def set_epoch(self, epoch: int):
        self.epoch = epoch

    def __len__(self):
        return self.num_batches

    def __iter__(self):
        order = np.arange(self.num_batches)
        if self.shuffle:
            np.random.default_rng(self.seed + self.epoch).shuffle(order)
        per = self.B * self.S
        for i in order:
            lo = int(i) * per
            ids = self.tokens[lo:lo + per].view(self.B, self.S)
            labels = self.tokens[lo + 1:lo + per + 1].view(self.B, self.S)
            if self.pin:
                ids, labels = ids.contiguous().pin_memory(), labels.contiguous().pin_memory()
            yield ids, labels


# ---------------------------------------------------------------------------------------------- file-backed, prefetching, curriculum
class MMapTokenLoader(TokenLoader):
    """Token ids in a flat binary file (uint16 / int32 / int64), memory-mapped: a corpus larger than host memory is paged in
    batch by batch (the reference's mmap / streaming loader, src/trainer_data.cpp:238-280)."""

    def __init__(self, path: str, batch_size: int, seq_len: int, dtype=np.uint16, **kw):
        self.mm = np.memmap(path, dtype=dtype, mode="r")
        self.B, self.S = batch_size, seq_len
        self.shuffle, self.seed, self.epoch = kw.get("shuffle", False), kw.get("seed", 0), 0
        self.pin = kw.get("pin", False) and torch.cuda.is_available()
        self.num_batches = (self.mm.shape[0] - 1) // (batch_size * seq_len)
        if self.num_batches <= 0:
            raise ValueError("not enough tokens for one batch")

    @staticmethod
    def write(path: str, tokens, dtype=np.uint16):
        np.asarray(tokens, dtype=dtype).tofile(path)

    def __iter__(self):
        order = np.arange(self.num_batches)
        if self.shuffle:
            np.random.default_rng(self.seed + self.epoch).shuffle(order)
        per = self.B * self.S
        for i in order:
            lo = int(i) * per
            chunk = torch.from_numpy(self.mm[lo:lo + per + 1].astype(np.int64))
            ids, labels = chunk[:-1].view(self.B, self.S), chunk[1:].view(self.B, self.S)
            if self.pin:
                ids, labels = ids.pin_memory(), labels.pin_memory()
            yield ids, labels


class PrefetchLoader:
    """Wraps a loader: a worker thread reads ``depth`` batches ahead; with a CUDA ``device`` the batches are staged in
    pinned memory and copied on a side stream, so the host-to-device transfer of step i + 1 overlaps the compute of
    step i (the consumer's stream waits on the copy's event only)."""

    def __init__(self, loader, depth: int = 2, device=None):
        self.loader, self.depth = loader, max(1, depth)
        self.device = torch.device(device) if device is not None else None
        self.cuda = self.device is not None and self.device.type == "cuda"
        self.stream = torch.cuda.Stream(self.device) if self.cuda else None

    def __len__(self):
        return len(self.loader)

    def _stage(self, batch):
        if not self.cuda:
            return batch, None
        with torch.cuda.stream(self.stream):
            out = tuple((t if t.is_pinned() else t.pin_memory()).to(self.device, non_blocking=True) for t in batch)
            ev = torch.cuda.Event()
            ev.record(self.stream)
        return out, ev

    def __iter__(self):
        import queue
        import threading
        q: "queue.Queue" = queue.Queue(maxsize=self.depth)
        end, failure = object(), []

        def work():
            try:
                for batch in self.loader:
                    q.put(self._stage(batch))
            except Exception as e:                    # noqa: BLE001 - handed to the consumer
                failure.append(e)
            q.put(end)
        t = threading.Thread(target=work, daemon=True)
        t.start()
        while True:
            item = q.get()
            if item is end:
                break
            batch, ev = item
            if ev is not None:
                torch.cuda.current_stream(self.device).wait_event(ev)
                for x in batch:
                    x.record_stream(torch.cuda.current_stream(self.device))
            yield batch
        t.join()
        if failure:
            raise failure[0]


class TokenAugmenter:
    """Input-side noise (labels untouched): each token is replaced by a random id with probability ``replace_p`` or by
    ``mask_id`` with probability ``mask_p`` (the reference's augmentation hook, src/trainer_data.cpp:282-306)."""

    def __init__(self, vocab: int, replace_p: float = 0.0, mask_p: float = 0.0, mask_id: int = 0, seed: int = 0):
        self.vocab, self.replace_p, self.mask_p, self.mask_id = vocab, replace_p, mask_p, mask_id
        self.gen = torch.Generator().manual_seed(seed)

    def __call__(self, ids: torch.Tensor) -> torch.Tensor:
        u = torch.rand(ids.shape, generator=self.gen)
        out = ids.clone()
        rep = u < self.replace_p
        out[rep] = torch.randint(0, self.vocab, (int(rep.sum()),), generator=self.gen)
        out[(u >= self.replace_p) & (u < self.replace_p + self.mask_p)] = self.mask_id
        return out


class CurriculumLoader:
    """Sequence length grows from ``start_len`` to the loader's full length over ``ramp_epochs`` epochs (rounded to
    ``multiple``): short contexts first. Batches are cut from the full-length batches, so no token is read twice."""

    def __init__(self, loader: TokenLoader, start_len: int, ramp_epochs: int, multiple: int = 16, augment=None):
        self.loader, self.start, self.ramp, self.multiple, self.augment = loader, start_len, max(1, ramp_epochs), multiple, augment
        self.epoch = 0

    def set_epoch(self, epoch: int):
        self.epoch = epoch
        self.loader.set_epoch(epoch)

    def current_len(self) -> int:
        full = self.loader.S
        frac = min(1.0, self.epoch / self.ramp)
        n = int(self.start + (full - self.start) * frac)
        return max(self.multiple, min(full, n // self.multiple * self.multiple))

    def __len__(self):
        return len(self.loader)

    def __iter__(self):
        n = self.current_len()
        for ids, labels in self.loader:
            ids, labels = ids[:, :n], labels[:, :n]
            yield (self.augment(ids) if self.augment is not None else ids), labels
