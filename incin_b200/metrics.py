"""Streaming evaluation metrics (crates/incin-core/src/metrics/mod.rs:10-272): Accuracy, Precision,
Recall, F1Score, MSE, ConfusionMatrix.  ``update`` accumulates on the host from device tensors; ``compute``
returns the value so far; ``reset`` starts over."""
from __future__ import annotations

import torch


class ConfusionMatrix:
    def __init__(self, num_classes: int):
        self.n = num_classes
        self.m = torch.zeros(num_classes, num_classes, dtype=torch.int64)

    def update(self, pred: torch.Tensor, target: torch.Tensor) -> None:
        p = pred.argmax(-1) if pred.dim() > target.dim() else pred
        idx = (target.reshape(-1).cpu().long() * self.n + p.reshape(-1).cpu().long())
        self.m += torch.bincount(idx, minlength=self.n * self.n).reshape(self.n, self.n)

    def compute(self) -> torch.Tensor:
        return self.m.clone()    # rows = truth, columns = prediction

    def reset(self) -> None:
        self.m.zero_()


class Accuracy:
    def __init__(self):
        self.correct = self.total = 0

    def update(self, pred, target) -> None:
        p = pred.argmax(-1) if pred.dim() > target.dim() else pred
        self.correct += int((p.reshape(-1).cpu() == target.reshape(-1).cpu()).sum())
        self.total += target.numel()

    def compute(self) -> float:
        return self.correct / self.total if self.total else 0.0

    def reset(self) -> None:
        self.correct = self.total = 0


class _PerClass:
    def __init__(self, num_classes: int, average: str = "macro"):
        self.cm, self.average = ConfusionMatrix(num_classes), average

    def update(self, pred, target) -> None:
        self.cm.update(pred, target)

    def reset(self) -> None:
        self.cm.reset()

    def _tp_fp_fn(self):
        m = self.cm.m.double()
        tp = m.diag()
        return tp, m.sum(0) - tp, m.sum(1) - tp

    def _avg(self, per_class, weight):
        if self.average == "micro":
            raise NotImplementedError
        return float((per_class * weight).sum() / weight.sum()) if self.average == "weighted" else float(per_class.mean())


class Precision(_PerClass):
    def compute(self) -> float:
        tp, fp, fn = self._tp_fp_fn()
        if self.average == "micro":
            return float(tp.sum() / (tp.sum() + fp.sum()).clamp(min=1))
        return self._avg(tp / (tp + fp).clamp(min=1), tp + fn)


class Recall(_PerClass):
    def compute(self) -> float:
        tp, fp, fn = self._tp_fp_fn()
        if self.average == "micro":
            return float(tp.sum() / (tp.sum() + fn.sum()).clamp(min=1))
        return self._avg(tp / (tp + fn).clamp(min=1), tp + fn)


class F1Score(_PerClass):
    def compute(self) -> float:
        tp, fp, fn = self._tp_fp_fn()
        if self.average == "micro":
            return float(2 * tp.sum() / (2 * tp.sum() + fp.sum() + fn.sum()).clamp(min=1))
        return self._avg(2 * tp / (2 * tp + fp + fn).clamp(min=1), tp + fn)


class MSE:
    def __init__(self):
        self.s, self.n = 0.0, 0

    def update(self, pred, target) -> None:
        self.s += float(((pred.float() - target.float()) ** 2).sum())
        self.n += target.numel()

    def compute(self) -> float:
        return self.s / self.n if self.n else 0.0

    def reset(self) -> None:
        self.s, self.n = 0.0, 0
