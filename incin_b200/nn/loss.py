"""Losses (crates/incin-core/src/nn/loss.rs:7-289, tensor/ops/loss.rs:35-146)."""
from __future__ import annotations

import torch
import torch.nn.functional as TF

from ..ops import functional as F


def cross_entropy_loss(logits, targets, num_classes: int | None = None):
    """Mean softmax cross-entropy; the bf16 CUDA path is the fused online-log-sum-exp kernel pair."""
    return F.cross_entropy(logits, targets, num_classes)


def mse_loss(pred, target):
    return ((pred.float() - target.float()) ** 2).mean()


def l1_loss(pred, target):
    return (pred.float() - target.float()).abs().mean()


def nll_loss(log_probs, targets):
    return TF.nll_loss(log_probs.float(), targets)


def bce_loss(prob, target, eps: float = 1e-7):
    p = prob.float().clamp(eps, 1 - eps)
    return -(target * p.log() + (1 - target) * (1 - p).log()).mean()


def bce_with_logits_loss(logits, target):
    return TF.binary_cross_entropy_with_logits(logits.float(), target.float())


def huber_loss(pred, target, delta: float = 1.0):
    return TF.huber_loss(pred.float(), target.float(), delta=delta)


def kl_div_loss(log_p, q):
    return TF.kl_div(log_p.float(), q.float(), reduction="batchmean")


class CrossEntropyLoss(torch.nn.Module):
    def forward(self, logits, targets):
        return cross_entropy_loss(logits, targets)


class MSELoss(torch.nn.Module):
    def forward(self, pred, target):
        return mse_loss(pred, target)
