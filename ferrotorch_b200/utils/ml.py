"""scikit-learn-style metrics, toy datasets and array adapters on tensors
(ferrotorch-ml/src/{metrics,datasets,adapter}.rs): a few metrics in plain torch, the rest bridged to
scikit-learn the way the reference bridges to its classical-ML library."""
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


# --------------------------------------------------------------------------- bridge to scikit-learn
# The reference's ferrotorch-ml is a bridge too: tensors are converted to arrays, a classical-ML
# library (ferrolearn there, scikit-learn here) does the work, and results come back as floats or
# tensors (ferrotorch-ml/src/adapter.rs:52-218, metrics.rs, datasets.rs).  Names and argument
# order follow the reference / scikit-learn.
def tensor_to_array1(t: torch.Tensor):
    if t.dim() != 1:
        raise ValueError("tensor_to_array1: expected a 1-D tensor, got shape %s" % (tuple(t.shape),))
    return t.detach().cpu().numpy()


def tensor_to_array2(t: torch.Tensor):
    if t.dim() != 2:
        raise ValueError("tensor_to_array2: expected a 2-D tensor, got shape %s" % (tuple(t.shape),))
    return t.detach().cpu().numpy()


def tensor_to_array1_usize(t: torch.Tensor):
    """Class labels: finite, non-negative, integral values only (adapter.rs:218)."""
    a = tensor_to_array1(t)
    f = t.detach().cpu().double()
    if not bool(torch.isfinite(f).all()) or bool((f < 0).any()) or bool((f != f.round()).any()):
        raise ValueError("labels must be finite, non-negative integers")
    return a.astype("int64")


def array1_to_tensor(a, dtype=torch.float32) -> torch.Tensor:
    import numpy as np

    return torch.from_numpy(np.ascontiguousarray(a)).to(dtype)


array2_to_tensor = array1_to_tensor


def array1_usize_to_tensor(a, dtype=torch.float32) -> torch.Tensor:
    return array1_to_tensor(a, dtype)


def _np(x):
    return x.detach().cpu().numpy() if isinstance(x, torch.Tensor) else x


def _bridge(name: str, labels: tuple = ()):
    """A function ``name(*tensors, **kw)`` that calls ``sklearn.metrics.<name>`` on arrays;
    positional arguments listed in ``labels`` are checked as class labels first."""
    def fn(*args, **kw):
        import sklearn.metrics as M

        conv = [tensor_to_array1_usize(a) if i in labels and isinstance(a, torch.Tensor) else _np(a)
                for i, a in enumerate(args)]
        out = getattr(M, name)(*conv, **{k: _np(v) for k, v in kw.items()})
        return float(out) if getattr(out, "ndim", 0) == 0 else torch.from_numpy(out)

    fn.__name__ = fn.__qualname__ = name
    fn.__module__ = __name__
    fn.__doc__ = "``sklearn.metrics.%s`` on tensors (ferrotorch-ml/src/metrics.rs)." % name
    return fn


# regression
explained_variance_score = _bridge("explained_variance_score")
max_error = _bridge("max_error")
mean_absolute_percentage_error = _bridge("mean_absolute_percentage_error")
median_absolute_error = _bridge("median_absolute_error")
root_mean_squared_error = _bridge("root_mean_squared_error")
# classification
precision_score = _bridge("precision_score", (0, 1))
recall_score = _bridge("recall_score", (0, 1))
f1_score = _bridge("f1_score", (0, 1))
hamming_loss = _bridge("hamming_loss", (0, 1))
balanced_accuracy_score = _bridge("balanced_accuracy_score", (0, 1))
matthews_corrcoef = _bridge("matthews_corrcoef", (0, 1))
cohen_kappa_score = _bridge("cohen_kappa_score", (0, 1))
zero_one_loss = _bridge("zero_one_loss", (0, 1))
top_k_accuracy_score = _bridge("top_k_accuracy_score", (0,))
log_loss = _bridge("log_loss", (0,))
brier_score_loss = _bridge("brier_score_loss", (0,))
average_precision_score = _bridge("average_precision_score", (0,))
# ranking
dcg_score = _bridge("dcg_score")
ndcg_score = _bridge("ndcg_score")
coverage_error = _bridge("coverage_error")
label_ranking_average_precision_score = _bridge("label_ranking_average_precision_score")
label_ranking_loss = _bridge("label_ranking_loss")
# clustering
adjusted_rand_score = _bridge("adjusted_rand_score", (0, 1))
adjusted_mutual_info_score = _bridge("adjusted_mutual_info_score", (0, 1))
normalized_mutual_info_score = _bridge("normalized_mutual_info_score", (0, 1))
homogeneity_score = _bridge("homogeneity_score", (0, 1))
completeness_score = _bridge("completeness_score", (0, 1))
v_measure_score = _bridge("v_measure_score", (0, 1))
fowlkes_mallows_score = _bridge("fowlkes_mallows_score", (0, 1))
silhouette_score = _bridge("silhouette_score", (1,))
davies_bouldin_score = _bridge("davies_bouldin_score", (1,))
calinski_harabasz_score = _bridge("calinski_harabasz_score", (1,))


def d2_brier_score(y_true: torch.Tensor, y_prob: torch.Tensor) -> float:
    """Fraction of the Brier score explained: ``1 - BS(model) / BS(base rate)`` (binary)."""
    y = y_true.double()
    bs = float(((y_prob.double() - y) ** 2).mean())
    ref = float(((y.mean() - y) ** 2).mean())
    return 1.0 - bs / ref if ref > 0 else 0.0


# --------------------------------------------------------------------------- datasets (datasets.rs)
def _xy(x, y, y_dtype=torch.float32):
    return array2_to_tensor(x), array1_to_tensor(y, y_dtype)


def make_classification(n_samples: int = 100, n_features: int = 20, n_classes: int = 2, seed: int | None = None, **kw):
    from sklearn import datasets as D

    return _xy(*D.make_classification(n_samples=n_samples, n_features=n_features, n_classes=n_classes,
                                      random_state=seed, **kw))


def make_regression(n_samples: int = 100, n_features: int = 100, n_informative: int = 10, noise: float = 0.0,
                    seed: int | None = None, **kw):
    from sklearn import datasets as D

    return _xy(*D.make_regression(n_samples=n_samples, n_features=n_features, n_informative=n_informative,
                                  noise=noise, random_state=seed, **kw))


def make_blobs(n_samples: int = 100, n_features: int = 2, centers: int = 3, cluster_std: float = 1.0,
               seed: int | None = None, **kw):
    from sklearn import datasets as D

    return _xy(*D.make_blobs(n_samples=n_samples, n_features=n_features, centers=centers, cluster_std=cluster_std,
                             random_state=seed, **kw))


def make_moons(n_samples: int = 100, noise: float | None = None, seed: int | None = None):
    from sklearn import datasets as D

    return _xy(*D.make_moons(n_samples=n_samples, noise=noise, random_state=seed))


def make_circles(n_samples: int = 100, noise: float | None = None, factor: float = 0.8, seed: int | None = None):
    from sklearn import datasets as D

    return _xy(*D.make_circles(n_samples=n_samples, noise=noise, factor=factor, random_state=seed))


def load_iris():
    from sklearn import datasets as D

    return _xy(*D.load_iris(return_X_y=True))


def load_wine():
    from sklearn import datasets as D

    return _xy(*D.load_wine(return_X_y=True))


def load_breast_cancer():
    from sklearn import datasets as D

    return _xy(*D.load_breast_cancer(return_X_y=True))
