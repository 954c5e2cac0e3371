"""Streaming evaluation metrics on tensors.

Reference behaviour covered (include/oil/metrics.h:15-127): ``Accuracy`` (top-k), ``Perplexity``, ``F1Score`` (per class
and macro), ``BLEUScore`` (modified n-gram precision, brevity penalty), ``ROUGELScore`` (longest common subsequence F1),
``MeanAveragePrecision`` and ``ConfusionMatrix``. Counting is done with tensor operations on the device of the inputs
(``bincount`` for the confusion matrix, ``topk`` for accuracy, a log-softmax gather for perplexity); only the running
totals live on the host.
"""
from __future__ import annotations

import math
from collections import Counter
from typing import List, Sequence

import torch


def _ids(x) -> List[int]:
    return [int(v) for v in (x.flatten().tolist() if torch.is_tensor(x) else x)]


class Accuracy:
    def __init__(self, top_k: int = 1):
        self.top_k = top_k
        self.reset()

    def reset(self):
        self.correct, self.total = 0, 0

    def update(self, predictions: torch.Tensor, targets: torch.Tensor) -> float:
        """predictions [N, C] scores (or [N] class ids when top_k = 1); returns the accuracy of this batch."""
        t = targets.flatten().long()
        if predictions.dim() == 1 or predictions.shape[-1] == 1 and self.top_k == 1 and predictions.dtype in (torch.long, torch.int):
            hit = predictions.flatten().long() == t
        else:
            p = predictions.reshape(t.numel(), -1)
            hit = (p.topk(min(self.top_k, p.shape[1]), -1).indices == t[:, None]).any(-1)
        c = int(hit.sum())
        self.correct += c
        self.total += t.numel()
        return c / max(1, t.numel())

    def compute(self) -> float:
        return self.correct / max(1, self.total)


class Perplexity:
    def __init__(self, ignore_index: int = -100):
        self.ignore_index = ignore_index
        self.reset()

    def reset(self):
        self.nll, self.count = 0.0, 0

    def update(self, logits: torch.Tensor, targets: torch.Tensor) -> float:
        """logits [..., V], targets [...]; returns the perplexity of this batch."""
        t = targets.flatten().long()
        keep = t != self.ignore_index
        lp = torch.log_softmax(logits.reshape(t.numel(), -1).float(), -1)
        nll = -lp.gather(1, t.clamp_min(0)[:, None])[:, 0][keep]
        self.nll += float(nll.sum())
        self.count += int(keep.sum())
        return math.exp(float(nll.mean())) if nll.numel() else float("nan")

    def compute(self) -> float:
        return math.exp(self.nll / self.count) if self.count else float("nan")


class ConfusionMatrix:
    """``at(pred, true)`` counts; rows are predicted classes."""

    def __init__(self, num_classes: int):
        self.num_classes = num_classes
        self.reset()

    def reset(self):
        self.m = torch.zeros(self.num_classes, self.num_classes, dtype=torch.long)

    def update(self, predictions: torch.Tensor, targets: torch.Tensor, from_logits: bool = False):
        if from_logits or (predictions.dim() > 1 and predictions.shape[-1] == self.num_classes and predictions.is_floating_point()):
            predictions = predictions.reshape(-1, self.num_classes).argmax(-1)
        p, t = predictions.flatten().long(), targets.flatten().long()
        ok = (p >= 0) & (p < self.num_classes) & (t >= 0) & (t < self.num_classes)
        flat = torch.bincount(p[ok] * self.num_classes + t[ok], minlength=self.num_classes ** 2)
        self.m += flat.view(self.num_classes, self.num_classes).cpu()

    def at(self, pred_class: int, true_class: int) -> int:
        return int(self.m[pred_class, true_class])

    def true_positive(self, c: int) -> int:
        return int(self.m[c, c])

    def false_positive(self, c: int) -> int:
        return int(self.m[c].sum() - self.m[c, c])

    def false_negative(self, c: int) -> int:
        return int(self.m[:, c].sum() - self.m[c, c])

    def true_negative(self, c: int) -> int:
        return int(self.m.sum()) - self.true_positive(c) - self.false_positive(c) - self.false_negative(c)

    @property
    def total_samples(self) -> int:
        return int(self.m.sum())


class F1Score:
    """``class_idx = -1`` gives the macro average over classes that occur (as prediction or target)."""

    def __init__(self, num_classes: int = 2):
        self.num_classes = num_classes
        self.cm = ConfusionMatrix(num_classes)

    def reset(self):
        self.cm.reset()

    def update(self, predictions, targets):
        self.cm.update(predictions, targets)

    def _avg(self, fn, c):
        if c >= 0:
            return fn(c)
        seen = [k for k in range(self.num_classes) if self.cm.m[k].sum() + self.cm.m[:, k].sum() > 0]
        return sum(fn(k) for k in seen) / max(1, len(seen))

    def precision(self, class_idx: int = -1) -> float:
        return self._avg(lambda c: self.cm.true_positive(c) / max(1, self.cm.true_positive(c) + self.cm.false_positive(c)), class_idx)

    def recall(self, class_idx: int = -1) -> float:
        return self._avg(lambda c: self.cm.true_positive(c) / max(1, self.cm.true_positive(c) + self.cm.false_negative(c)), class_idx)

    def f1(self, class_idx: int = -1) -> float:
        def one(c):
            tp, fp, fn = self.cm.true_positive(c), self.cm.false_positive(c), self.cm.false_negative(c)
            return 2 * tp / max(1, 2 * tp + fp + fn)
        return self._avg(one, class_idx)


class BLEUScore:
    def __init__(self, max_n: int = 4):
        self.max_n = max_n

    @staticmethod
    def get_ngrams(seq: Sequence[int], n: int) -> Counter:
        return Counter(tuple(seq[i:i + n]) for i in range(len(seq) - n + 1))

    def compute(self, candidate, reference) -> float:
        c, r = _ids(candidate), _ids(reference)
        if not c or not r:
            return 0.0
        logp = 0.0
        for n in range(1, self.max_n + 1):
            cn, rn = self.get_ngrams(c, n), self.get_ngrams(r, n)
            total = sum(cn.values())
            if total == 0:
                return 0.0
            match = sum(min(v, rn[g]) for g, v in cn.items())
            if match == 0:
                return 0.0
            logp += math.log(match / total) / self.max_n
        bp = 1.0 if len(c) > len(r) else math.exp(1.0 - len(r) / len(c))
        return bp * math.exp(logp)


class ROUGELScore:
    def compute(self, candidate, reference) -> float:
        c, r = _ids(candidate), _ids(reference)
        if not c or not r:
            return 0.0
        prev = [0] * (len(r) + 1)
        for a in c:
            cur = [0]
            for j, b in enumerate(r):
                cur.append(prev[j] + 1 if a == b else max(prev[j + 1], cur[j]))
            prev = cur
        lcs = prev[-1]
        if lcs == 0:
            return 0.0
        p, q = lcs / len(c), lcs / len(r)
        return 2 * p * q / (p + q)


class MeanAveragePrecision:
    """Mean over queries of the average precision of a ranking (scores descending) against binary labels."""

    def __init__(self):
        self.reset()

    def reset(self):
        self.sum_ap, self.n = 0.0, 0

    @staticmethod
    def average_precision(scores: torch.Tensor, labels: torch.Tensor) -> float:
        order = scores.flatten().argsort(descending=True)
        rel = labels.flatten()[order].float()
        if rel.sum() == 0:
            return 0.0
        prec = rel.cumsum(0) / torch.arange(1, rel.numel() + 1, device=rel.device)
        return float((prec * rel).sum() / rel.sum())

    def compute(self, scores: torch.Tensor, labels: torch.Tensor) -> float:
        """scores, labels [Q, N] (or [N]); adds the queries to the running mean and returns it."""
        s, l = scores.reshape(-1, scores.shape[-1]), labels.reshape(-1, labels.shape[-1])
        for q in range(s.shape[0]):
            self.sum_ap += self.average_precision(s[q], l[q])
            self.n += 1
        return self.sum_ap / max(1, self.n)
