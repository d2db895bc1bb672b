"""Shared helpers of the classical-ML package: array coercion and the estimator interfaces
(ml/types.go:5-27).  Estimators are configured by keyword fields with the reference's names;
a zero / missing value means "use the default"."""
from __future__ import annotations

import numpy as np
import torch


def A(X, dtype=np.float64) -> np.ndarray:
    if isinstance(X, torch.Tensor):
        X = X.detach().cpu().numpy()
    return np.asarray(X, dtype=dtype)


def T(X, device=None) -> torch.Tensor:
    return torch.as_tensor(A(X), dtype=torch.float64, device=device)


class Estimator:
    _defaults: dict = {}

    def __init__(self, **kw):
        for k, v in self._defaults.items():
            setattr(self, k, v)
        for k, v in kw.items():
            if k not in self._defaults:
                raise TypeError(f"{type(self).__name__}: unknown field {k!r}")
            if v not in (0, None, "") or isinstance(v, bool):
                setattr(self, k, v)


class Regressor(Estimator):
    def Fit(self, X, y): raise NotImplementedError
    def Predict(self, X): raise NotImplementedError


class Classifier(Estimator):
    def Fit(self, X, y): raise NotImplementedError
    def Predict(self, X): raise NotImplementedError


class Clusterer(Estimator):
    def Fit(self, X): raise NotImplementedError


class Transformer(Estimator):
    def Fit(self, X): raise NotImplementedError
    def Transform(self, X): raise NotImplementedError

    def FitTransform(self, X):
        self.Fit(X)
        return self.Transform(X)


class LabelArray(np.ndarray):
    """Cluster labels that read both ways: as the array itself (``m.Labels[i]``) and through
    the reference's accessor call ``m.Labels()`` (ml/cluster_extras.go:89, 219)."""

    def __call__(self) -> np.ndarray:
        return np.asarray(self)


def as_labels(lab) -> LabelArray:
    return np.asarray(lab, dtype=np.int64).view(LabelArray)
