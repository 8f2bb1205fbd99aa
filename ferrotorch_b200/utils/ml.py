"""scikit-learn-style metrics on tensors (ferrotorch-ml/src/metrics.rs)."""
from __future__ import annotations

import torch


def confusion_matrix(y_true: torch.Tensor, y_pred: torch.Tensor, num_classes: int | None = None) -> torch.Tensor:
    k = num_classes or int(max(y_true.max(), y_pred.max())) + 1
    return torch.bincount(y_true.long() * k + y_pred.long(), minlength=k * k).view(k, k)


def accuracy_score(y_true, y_pred) -> float:
    return float((y_true == y_pred).float().mean())


def precision_recall_f1(y_true, y_pred, average: str = "macro", num_classes: int | None = None):
    cm = confusion_matrix(y_true, y_pred, num_classes).double()
    tp, fp, fn = cm.diag(), cm.sum(0) - cm.diag(), cm.sum(1) - cm.diag()
    if average == "micro":
        p = tp.sum() / (tp.sum() + fp.sum()).clamp_min(1)
        r = tp.sum() / (tp.sum() + fn.sum()).clamp_min(1)
    else:
        p = (tp / (tp + fp).clamp_min(1)).mean()
        r = (tp / (tp + fn).clamp_min(1)).mean()
    f1 = 2 * p * r / (p + r).clamp_min(1e-12) if average == "micro" else \
        (2 * tp / (2 * tp + fp + fn).clamp_min(1)).mean()
    return float(p), float(r), float(f1)


def mean_squared_error(y_true, y_pred) -> float:
    return float(((y_true - y_pred) ** 2).mean())


def mean_absolute_error(y_true, y_pred) -> float:
    return float((y_true - y_pred).abs().mean())


def r2_score(y_true, y_pred) -> float:
    ss_res = ((y_true - y_pred) ** 2).sum()
    ss_tot = ((y_true - y_true.mean()) ** 2).sum()
    return float(1 - ss_res / ss_tot)


def roc_auc_score(y_true, scores) -> float:
    """Binary AUC by the rank statistic (ties get average ranks)."""
    order = scores.argsort()
    ranks = torch.empty_like(scores, dtype=torch.float64)
    sorted_scores = scores[order]
    i, n = 0, scores.numel()
    while i < n:
        j = i
        while j + 1 < n and sorted_scores[j + 1] == sorted_scores[i]:
            j += 1
        ranks[order[i:j + 1]] = (i + j) / 2.0 + 1.0
        i = j + 1
    pos = y_true.bool()
    n_pos, n_neg = int(pos.sum()), int((~pos).sum())
    return float((ranks[pos].sum() - n_pos * (n_pos + 1) / 2.0) / (n_pos * n_neg))


def train_test_split(*arrays, test_size: float = 0.25, seed: int = 0):
    n = arrays[0].shape[0]
    perm = torch.randperm(n, generator=torch.Generator().manual_seed(seed))
    k = int(round(n * (1 - test_size)))
    out = []
    for a in arrays:
        out += [a[perm[:k]], a[perm[k:]]]
    return out
