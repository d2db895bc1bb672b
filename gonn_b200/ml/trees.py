"""Decision trees and tree ensembles (ml/tree.go, forest.go, extratrees.go, adaboost.go,
gboost.go, iforest.go): CART with Gini / variance splits, bagging, extra-random splits,
SAMME AdaBoost, gradient boosting on squared error / log-loss, isolation forest."""
from __future__ import annotations

import math

import numpy as np

from .base import A, Classifier, Estimator, Regressor


class _Node:
    __slots__ = ("feat", "thr", "left", "right", "value")

    def __init__(self, value=None):
        self.feat, self.thr, self.left, self.right, self.value = -1, 0.0, None, None, value


def _impurity(y, classify, K):
    if classify:
        p = np.bincount(y, minlength=K) / len(y)
        return 1.0 - (p * p).sum()
    return y.var()


def _leaf(y, w, classify, K):
    if classify:
        return np.bincount(y, weights=w, minlength=K) / (w.sum() if w is not None else len(y))
    return float(np.average(y, weights=w))


def _build(X, y, w, depth, cfg, rng, classify, K):
    n, d = X.shape
    node = _Node(_leaf(y, w, classify, K))
    if (cfg["max_depth"] and depth >= cfg["max_depth"]) or n < max(cfg["min_split"], 2) or _impurity(y, classify, K) == 0:
        return node
    feats = np.arange(d)
    if cfg["max_features"] and cfg["max_features"] < d:
        feats = rng.choice(d, cfg["max_features"], replace=False)
    best = (0.0, -1, 0.0)
    parent = _impurity(y, classify, K)
    for f in feats:
        col = X[:, f]
        if cfg["extra"]:
            lo, hi = col.min(), col.max()
            if lo == hi:
                continue
            cands = [rng.uniform(lo, hi)]
        else:
            u = np.unique(col)
            if len(u) < 2:
                continue
            cands = (u[:-1] + u[1:]) / 2
            if len(cands) > 32:
                cands = np.quantile(col, np.linspace(0.03, 0.97, 32))
        for t in cands:
            m = col <= t
            nl = m.sum()
            if nl == 0 or nl == n:
                continue
            gain = parent - (nl * _impurity(y[m], classify, K) + (n - nl) * _impurity(y[~m], classify, K)) / n
            if gain > best[0] + 1e-12:
                best = (gain, f, t)
    if best[1] < 0:
        return node
    _, f, t = best
    m = X[:, f] <= t
    node.feat, node.thr = int(f), float(t)
    node.left = _build(X[m], y[m], None if w is None else w[m], depth + 1, cfg, rng, classify, K)
    node.right = _build(X[~m], y[~m], None if w is None else w[~m], depth + 1, cfg, rng, classify, K)
    return node


def _predict(node, X):
    out = [None] * len(X)
    stack = [(node, np.arange(len(X)))]
    while stack:
        nd, idx = stack.pop()
        if nd.left is None or len(idx) == 0:
            for i in idx:
                out[i] = nd.value
            continue
        m = X[idx, nd.feat] <= nd.thr
        stack.append((nd.left, idx[m]))
        stack.append((nd.right, idx[~m]))
    return np.asarray(out)


class _Tree(Estimator):
    _defaults = {"MaxDepth": 0, "MinSamplesSplit": 2, "MaxFeatures": 0, "Seed": 0}
    classify, extra = True, False

    def _cfg(self):
        return {"max_depth": int(self.MaxDepth), "min_split": int(self.MinSamplesSplit),
                "max_features": int(self.MaxFeatures), "extra": self.extra}

    def Fit(self, X, y, sample_weight=None):
        X = A(X)
        if self.classify:
            y = A(y, np.int64)
            self.Classes = np.unique(y)
            yi = np.searchsorted(self.Classes, y)
            self.root = _build(X, yi, sample_weight, 0, self._cfg(), np.random.default_rng(self.Seed), True, len(self.Classes))
        else:
            self.root = _build(X, A(y), sample_weight, 0, self._cfg(), np.random.default_rng(self.Seed), False, 0)
        return self

    def PredictProba(self, X):
        return _predict(self.root, A(X))

    def Predict(self, X):
        v = _predict(self.root, A(X))
        return self.Classes[v.argmax(1)] if self.classify else v.astype(float)


class DecisionTreeClassifier(_Tree, Classifier):
    classify = True


class DecisionTreeRegressor(_Tree, Regressor):
    classify = False


class _Forest(Estimator):
    _defaults = {"NEstimators": 100, "MaxDepth": 0, "MinSamplesSplit": 2, "MaxFeatures": 0, "Seed": 0, "Bootstrap": True}
    classify, extra = True, False

    def Fit(self, X, y):
        X = A(X)
        y = A(y, np.int64) if self.classify else A(y)
        n, d = X.shape
        rng = np.random.default_rng(self.Seed)
        mf = int(self.MaxFeatures) or (max(int(math.sqrt(d)), 1) if self.classify else max(d // 3, 1))
        if self.classify:
            self.Classes = np.unique(y)
        self.trees = []
        base = (DecisionTreeClassifier if self.classify else DecisionTreeRegressor)
        for i in range(int(self.NEstimators)):
            idx = rng.integers(0, n, n) if self.Bootstrap else np.arange(n)
            t = base(MaxDepth=self.MaxDepth, MinSamplesSplit=self.MinSamplesSplit, MaxFeatures=mf, Seed=int(rng.integers(1 << 31)))
            t.extra = self.extra
            t.Fit(X[idx], y[idx])
            self.trees.append(t)
        return self

    def PredictProba(self, X):
        X = A(X)
        P = np.zeros((len(X), len(self.Classes)))
        for t in self.trees:
            p = t.PredictProba(X)
            P[:, np.searchsorted(self.Classes, t.Classes)] += p
        return P / len(self.trees)

    def Predict(self, X):
        if self.classify:
            return self.Classes[self.PredictProba(X).argmax(1)]
        return np.mean([t.Predict(X) for t in self.trees], 0)


class RandomForestClassifier(_Forest, Classifier):
    classify, extra = True, False


class RandomForestRegressor(_Forest, Regressor):
    classify, extra = False, False


class ExtraTreesClassifier(_Forest, Classifier):
    _defaults = dict(_Forest._defaults, Bootstrap=False)
    classify, extra = True, True


class ExtraTreesRegressor(_Forest, Regressor):
    _defaults = dict(_Forest._defaults, Bootstrap=False)
    classify, extra = False, True


class AdaBoostClassifier(Classifier):
    """SAMME with depth-limited trees."""
    _defaults = {"NEstimators": 50, "LearningRate": 1.0, "MaxDepth": 1, "Seed": 0}

    def Fit(self, X, y):
        X, y = A(X), A(y, np.int64)
        self.Classes = np.unique(y)
        K, n = len(self.Classes), len(X)
        w = np.full(n, 1.0 / n)
        self.stumps, self.alphas = [], []
        rng = np.random.default_rng(self.Seed)
        for _ in range(int(self.NEstimators)):
            idx = rng.choice(n, n, p=w)
            t = DecisionTreeClassifier(MaxDepth=self.MaxDepth, Seed=int(rng.integers(1 << 31))).Fit(X[idx], y[idx])
            miss = t.Predict(X) != y
            err = float((w * miss).sum())
            if err >= 1 - 1.0 / K:
                continue
            alpha = self.LearningRate * (math.log((1 - err) / max(err, 1e-12)) + math.log(K - 1))
            self.stumps.append(t)
            self.alphas.append(alpha)
            if err == 0:
                break
            w = w * np.exp(alpha * miss)
            w /= w.sum()
        return self

    def _votes(self, X):
        X = A(X)
        votes = np.zeros((len(X), len(self.Classes)))
        for t, a in zip(self.stumps, self.alphas):
            votes[np.arange(len(X)), np.searchsorted(self.Classes, t.Predict(X))] += a
        return votes

    def Predict(self, X):
        return self.Classes[self._votes(X).argmax(1)]

    def PredictProba(self, X):
        """Softmax over the weighted votes (ml/adaboost.go:136-161)."""
        v = self._votes(X)
        e = np.exp(v - v.max(1, keepdims=True))
        return e / e.sum(1, keepdims=True)


class GradientBoostingRegressor(Regressor):
    _defaults = {"NEstimators": 100, "LR": 0.1, "MaxDepth": 3, "Seed": 0}

    def Fit(self, X, y):
        X, y = A(X), A(y)
        self.init = float(y.mean())
        pred = np.full(len(y), self.init)
        self.trees = []
        for i in range(int(self.NEstimators)):
            t = DecisionTreeRegressor(MaxDepth=self.MaxDepth, Seed=self.Seed + i).Fit(X, y - pred)
            pred += self.LR * t.Predict(X)
            self.trees.append(t)
        return self

    def Predict(self, X):
        X = A(X)
        return self.init + self.LR * sum(t.Predict(X) for t in self.trees)


class GradientBoostingClassifier(Classifier):
    """Binary log-loss boosting (one-vs-rest for more classes)."""
    _defaults = {"NEstimators": 100, "LR": 0.1, "MaxDepth": 3, "Seed": 0}

    def Fit(self, X, y):
        X, y = A(X), A(y, np.int64)
        self.Classes = np.unique(y)
        self.models = []
        for c in self.Classes:
            t = (y == c).astype(float)
            p0 = np.clip(t.mean(), 1e-6, 1 - 1e-6)
            f0 = math.log(p0 / (1 - p0))
            F = np.full(len(y), f0)
            trees = []
            for i in range(int(self.NEstimators)):
                p = 1 / (1 + np.exp(-F))
                tr = DecisionTreeRegressor(MaxDepth=self.MaxDepth, Seed=self.Seed + i).Fit(X, t - p)
                F += self.LR * tr.Predict(X)
                trees.append(tr)
            self.models.append((f0, trees))
            if len(self.Classes) == 2:
                break
        return self

    def _raw(self, X):
        X = A(X)
        return np.stack([f0 + self.LR * sum(t.Predict(X) for t in trees) for f0, trees in self.models], 1)

    def PredictProba(self, X):
        r = 1 / (1 + np.exp(-self._raw(X)))
        if len(self.Classes) == 2:
            return np.stack([r[:, 0], 1 - r[:, 0]], 1)
        return r / r.sum(1, keepdims=True)

    def Predict(self, X):
        return self.Classes[self.PredictProba(X).argmax(1)]


def _c(n):
    return 2 * (math.log(n - 1) + 0.5772156649) - 2 * (n - 1) / n if n > 2 else (1.0 if n == 2 else 0.0)


class IsolationForest(Estimator):
    _defaults = {"NEstimators": 100, "MaxSamples": 256, "ContaminationRate": 0.1, "Seed": 0}

    def Fit(self, X):
        X = A(X)
        rng = np.random.default_rng(self.Seed)
        self.psi = min(int(self.MaxSamples), len(X))
        limit = math.ceil(math.log2(max(self.psi, 2)))
        self.trees = []

        def build(S, depth):
            if depth >= limit or len(S) <= 1:
                return ("leaf", len(S))
            f = int(rng.integers(S.shape[1]))
            lo, hi = S[:, f].min(), S[:, f].max()
            if lo == hi:
                return ("leaf", len(S))
            t = rng.uniform(lo, hi)
            m = S[:, f] < t
            return ("node", f, t, build(S[m], depth + 1), build(S[~m], depth + 1))

        for _ in range(int(self.NEstimators)):
            self.trees.append(build(X[rng.choice(len(X), self.psi, replace=False)], 0))
        s = self.AnomalyScore(X)
        self.Threshold = float(np.quantile(s, 1 - self.ContaminationRate))
        return self

    def _path(self, tree, x, depth=0):
        while tree[0] == "node":
            tree = tree[3] if x[tree[1]] < tree[2] else tree[4]
            depth += 1
        return depth + _c(tree[1])

    def AnomalyScore(self, X):
        X = A(X)
        h = np.array([np.mean([self._path(t, x) for t in self.trees]) for x in X])
        return 2.0 ** (-h / _c(self.psi))

    def Predict(self, X):
        """-1 for anomalies, 1 for inliers."""
        return np.where(self.AnomalyScore(X) > self.Threshold, -1, 1)
