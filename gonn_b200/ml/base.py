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


def _np(v):
    return v.numpy() if isinstance(v, torch.Tensor) else v


# result fields under the reference's names, derived from what the estimators store
# (ml/linreg.go, logreg.go, svm.go, kmeans.go, knn.go, gmm.go, pca.go, lda.go ...): name -> getter
_FIELD_ALIASES = {
    # linear models keep (Coef, Intercept); classifiers a (d + 1, K) matrix W with the bias row last
    "Weights": lambda o: o.Coef if "Coef" in o.__dict__ else _np(o.W)[:-1].T,
    "Bias": lambda o: o.Intercept if "Intercept" in o.__dict__ else _np(o.W)[-1],
    "Centroids": lambda o: o.Centers,
    "Xtrain": lambda o: _np(o.__dict__["X"]),
    "XTrain": lambda o: _np(o.__dict__["X"]),
    "Ytrain": lambda o: _np(o.__dict__["y"]),
    "Covariances": lambda o: o.Variances,            # diagonal covariances
    "AlphaPrec": lambda o: o.AlphaEst,
    "LambdaPrec": lambda o: o.LambdaEst,
    "Components": lambda o: np.asarray(o.Scalings).T,                        # LDA: (NComponents, d)
    "Classes": lambda o: o.Categories[0],                                    # OneHotEncoder on one column
}


def _estimator_getattr(self, name):
    get = _FIELD_ALIASES.get(name)
    if get is not None:
        try:
            return get(self)
        except (KeyError, AttributeError):
            pass
    raise AttributeError(f"{type(self).__name__!r} object has no attribute {name!r}")


Estimator.__getattr__ = _estimator_getattr


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
