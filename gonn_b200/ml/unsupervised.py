"""Clustering, decomposition, manifold learning, preprocessing, metrics, model selection
(ml/kmeans.go, dbscan.go, agglomerative.go, meanshift.go, gmm.go, pca.go, kernel_pca.go, ica.go,
tsne.go, preprocess.go, metrics.go, model_selection.go)."""
from __future__ import annotations

import itertools
import math

import numpy as np
import torch

from .base import A, Clusterer, Estimator, T, Transformer, as_labels


class KMeans(Clusterer):
    _defaults = {"K": 8, "MaxIter": 300, "Tol": 1e-4, "Seed": 0}

    def Fit(self, X):
        X = T(X)
        g = torch.Generator().manual_seed(int(self.Seed))
        n = X.shape[0]
        # k-means++ seeding
        C = [X[int(torch.randint(n, (1,), generator=g))]]
        for _ in range(1, int(self.K)):
            d2 = torch.cdist(X, torch.stack(C)).min(1).values ** 2
            C.append(X[int(torch.multinomial(d2 / d2.sum(), 1, generator=g))])
        C = torch.stack(C)
        for _ in range(int(self.MaxIter)):
            lab = torch.cdist(X, C).argmin(1)
            newC = torch.stack([X[lab == k].mean(0) if bool((lab == k).any()) else C[k] for k in range(int(self.K))])
            shift = float((newC - C).norm())
            C = newC
            if shift < self.Tol:
                break
        self.Centers, self.Labels = C.numpy(), as_labels(torch.cdist(X, C).argmin(1).numpy())
        self.Inertia = float((torch.cdist(X, C).min(1).values ** 2).sum())
        return self

    def Predict(self, X):
        return torch.cdist(T(X), torch.as_tensor(self.Centers)).argmin(1).numpy()


class DBSCAN(Clusterer):
    _defaults = {"Eps": 0.5, "MinSamples": 5}

    def Fit(self, X):
        X = T(X)
        D = torch.cdist(X, X).numpy()
        n = len(D)
        nb = [np.nonzero(D[i] <= self.Eps)[0] for i in range(n)]
        lab = np.full(n, -2)
        c = 0
        for i in range(n):
            if lab[i] != -2:
                continue
            if len(nb[i]) < self.MinSamples:
                lab[i] = -1
                continue
            lab[i] = c
            queue = list(nb[i])
            while queue:
                j = queue.pop()
                if lab[j] == -1:
                    lab[j] = c
                if lab[j] != -2:
                    continue
                lab[j] = c
                if len(nb[j]) >= self.MinSamples:
                    queue.extend(nb[j])
            c += 1
        self.Labels = as_labels(lab)
        self.Xtrain = X.numpy().copy()
        return self

    def Predict(self, X):
        """The label of the nearest training point if it lies within ``Eps``, else -1
        (ml/cluster_extras.go:65-86)."""
        d, j = torch.cdist(T(X), T(self.Xtrain)).min(1)
        lab = np.asarray(self.Labels)[j.numpy()]
        return np.where(d.numpy() > self.Eps, -1, lab)


class AgglomerativeClustering(Clusterer):
    _defaults = {"NClusters": 2, "Linkage": "average"}

    def Fit(self, X):
        D = torch.cdist(T(X), T(X)).numpy()
        clusters = {i: [i] for i in range(len(D))}
        agg = {"single": np.min, "complete": np.max, "average": np.mean}[self.Linkage]
        while len(clusters) > int(self.NClusters):
            best = (math.inf, None)
            keys = list(clusters)
            for a, b in itertools.combinations(keys, 2):
                d = agg(D[np.ix_(clusters[a], clusters[b])])
                if d < best[0]:
                    best = (d, (a, b))
            a, b = best[1]
            clusters[a] += clusters.pop(b)
        lab = np.zeros(len(D), dtype=np.int64)
        for k, (_, members) in enumerate(sorted(clusters.items())):
            lab[members] = k
        self.Labels = as_labels(lab)
        self.Xtrain = A(X).copy()
        return self

    def Predict(self, X):
        """The cluster of the nearest training point (ml/cluster_extras.go:200-216)."""
        j = torch.cdist(T(X), T(self.Xtrain)).argmin(1).numpy()
        return np.asarray(self.Labels)[j]


class MeanShift(Clusterer):
    _defaults = {"Bandwidth": 1.0, "MaxIter": 300, "Tol": 1e-3}

    def Fit(self, X):
        X = T(X)
        P = X.clone()
        for _ in range(int(self.MaxIter)):
            W = (torch.cdist(P, X) <= self.Bandwidth).to(X.dtype)
            newP = (W @ X) / W.sum(1, keepdim=True).clamp_min(1)
            moved = float((newP - P).norm(dim=1).max())
            P = newP
            if moved < self.Tol:
                break
        centers = []
        lab = np.zeros(len(X), dtype=np.int64)
        for i, p in enumerate(P):
            for k, c in enumerate(centers):
                if float((p - c).norm()) < self.Bandwidth / 2:
                    lab[i] = k
                    break
            else:
                centers.append(p)
                lab[i] = len(centers) - 1
        self.Centers, self.Labels = torch.stack(centers).numpy(), as_labels(lab)
        return self

    def Predict(self, X):
        """Index of the nearest centre (ml/meanshift.go:117-132)."""
        return torch.cdist(T(X), T(self.Centers)).argmin(1).numpy()


class GaussianMixture(Clusterer):
    """EM with diagonal covariances."""
    _defaults = {"NComponents": 2, "MaxIter": 100, "Tol": 1e-4, "Seed": 0}

    def Fit(self, X):
        X = A(X)
        n, d = X.shape
        K = int(self.NComponents)
        km = KMeans(K=K, Seed=self.Seed).Fit(X)
        mu = km.Centers.copy()
        var = np.stack([X[km.Labels == k].var(0) + 1e-6 if (km.Labels == k).sum() > 1 else X.var(0) for k in range(K)])
        pi = np.bincount(km.Labels, minlength=K) / n
        prev = -np.inf
        for _ in range(int(self.MaxIter)):
            logp = -0.5 * (((X[:, None] - mu[None]) ** 2 / var[None]) + np.log(2 * np.pi * var)[None]).sum(2) + np.log(pi + 1e-300)
            m = logp.max(1, keepdims=True)
            ll = float((m[:, 0] + np.log(np.exp(logp - m).sum(1))).sum())
            R = np.exp(logp - m)
            R /= R.sum(1, keepdims=True)
            Nk = R.sum(0) + 1e-12
            mu = (R.T @ X) / Nk[:, None]
            var = (R.T @ (X ** 2)) / Nk[:, None] - mu ** 2 + 1e-6
            pi = Nk / n
            if abs(ll - prev) < self.Tol:
                break
            prev = ll
        self.Means, self.Variances, self.Weights, self.Resp = mu, var, pi, R
        self.LogLikelihood = ll
        self.Labels = as_labels(R.argmax(1))
        return self

    def PredictProba(self, X):
        """Posterior probabilities over the components: softmax of log weight + log density
        (ml/gmm.go:181-193)."""
        X = A(X)
        logp = -0.5 * (((X[:, None] - self.Means[None]) ** 2 / self.Variances[None])
                       + np.log(2 * np.pi * self.Variances)[None]).sum(2) + np.log(self.Weights + 1e-300)
        logp -= logp.max(1, keepdims=True)
        p = np.exp(logp)
        return p / p.sum(1, keepdims=True)

    def Predict(self, X):
        return self.PredictProba(X).argmax(1)


class PCA(Transformer):
    _defaults = {"NComponents": 2}

    def Fit(self, X):
        X = T(X)
        self.Mean = X.mean(0)
        U, S, Vt = torch.linalg.svd(X - self.Mean, full_matrices=False)
        k = int(self.NComponents)
        # deterministic sign: the largest-magnitude entry of each component is positive
        sign = torch.sign(Vt[torch.arange(Vt.shape[0]), Vt.abs().argmax(1)])
        Vt = Vt * sign[:, None]
        self.Components = Vt[:k]
        self.ExplainedVariance = (S[:k] ** 2 / (X.shape[0] - 1)).numpy()
        self.ExplainedVarianceRatio = (S[:k] ** 2 / (S ** 2).sum()).numpy()
        return self

    def Transform(self, X):
        return ((T(X) - self.Mean) @ self.Components.T).numpy()

    def InverseTransform(self, Z):
        return (T(Z) @ self.Components + self.Mean).numpy()


class KernelPCA(Transformer):
    _defaults = {"NComponents": 2, "Kernel": "rbf", "Gamma": 0.0, "Degree": 3, "Coef0": 1.0}

    def _k(self, Xa, Xb):
        g = self.Gamma or 1.0 / Xa.shape[1]
        if self.Kernel == "linear":
            return Xa @ Xb.T
        if self.Kernel == "poly":
            return (g * Xa @ Xb.T + self.Coef0) ** int(self.Degree)
        if self.Kernel == "sigmoid":
            return torch.tanh(g * Xa @ Xb.T + self.Coef0)
        return torch.exp(-g * torch.cdist(Xa, Xb) ** 2)

    def Fit(self, X):
        X = T(X)
        self.X = X
        K = self._k(X, X)
        n = K.shape[0]
        one = torch.full((n, n), 1.0 / n, dtype=K.dtype)
        self._Krow, self._Kall = K.mean(0), K.mean()
        Kc = K - one @ K - K @ one + one @ K @ one
        ev, evec = torch.linalg.eigh(Kc)
        idx = torch.argsort(ev, descending=True)[:int(self.NComponents)]
        self.Lambdas, self.Alphas = ev[idx].clamp_min(1e-12), evec[:, idx]
        return self

    def Transform(self, X):
        K = self._k(T(X), self.X)
        Kc = K - K.mean(1, keepdim=True) - self._Krow[None] + self._Kall
        return (Kc @ (self.Alphas / self.Lambdas.sqrt())).numpy()


class FastICA(Transformer):
    _defaults = {"NComponents": 2, "MaxIter": 200, "Tol": 1e-4, "Seed": 0}

    def Fit(self, X):
        X = T(X)
        self.Mean = X.mean(0)
        Xc = (X - self.Mean).T
        k = int(self.NComponents)
        ev, E = torch.linalg.eigh(Xc @ Xc.T / Xc.shape[1])
        idx = torch.argsort(ev, descending=True)[:k]
        self.Whitening = (E[:, idx] / ev[idx].sqrt()).T
        Z = self.Whitening @ Xc
        g = torch.Generator().manual_seed(int(self.Seed))
        W = torch.randn(k, k, generator=g, dtype=torch.float64)

        def sym(W):
            s, u = torch.linalg.eigh(W @ W.T)
            return u @ torch.diag(1 / s.sqrt()) @ u.T @ W
        W = sym(W)
        for _ in range(int(self.MaxIter)):
            WX = W @ Z
            gx = torch.tanh(WX)
            Wn = sym((gx @ Z.T) / Z.shape[1] - torch.diag((1 - gx ** 2).mean(1)) @ W)
            lim = float((torch.diag(Wn @ W.T).abs() - 1).abs().max())
            W = Wn
            if lim < self.Tol:
                break
        self.Components = W.numpy()          # the unmixing rotation in whitened space (ml/ica.go:23)
        self.Unmixing = W @ self.Whitening
        return self

    def Transform(self, X):
        return ((T(X) - self.Mean) @ self.Unmixing.T).numpy()


class TSNE(Estimator):
    _defaults = {"NComponents": 2, "Perplexity": 30.0, "LearningRate": 200.0, "NIter": 500, "Seed": 0,
                 "EarlyExaggeration": 12.0}

    def Fit(self, X):
        """Computes the embedding and keeps it in ``Embedding`` (ml/tsne.go:18-21); t-SNE has no
        out-of-sample transform."""
        self.Embedding = self.FitTransform(X)
        return self

    def FitTransform(self, X):
        X = T(X)
        n = X.shape[0]
        D = torch.cdist(X, X) ** 2
        P = torch.zeros(n, n, dtype=torch.float64)
        target = math.log(min(self.Perplexity, max(n - 1, 2) / 1.0))
        for i in range(n):
            lo, hi, beta = 0.0, math.inf, 1.0
            di = torch.cat([D[i, :i], D[i, i + 1:]])
            for _ in range(50):
                p = torch.exp(-di * beta)
                s = float(p.sum()) + 1e-300
                H = math.log(s) + beta * float((di * p).sum()) / s
                if abs(H - target) < 1e-5:
                    break
                if H > target:
                    lo, beta = beta, beta * 2 if hi == math.inf else (beta + hi) / 2
                else:
                    hi, beta = beta, (beta + lo) / 2
            p = p / s
            P[i, :i], P[i, i + 1:] = p[:i], p[i:]
        P = (P + P.T) / (2 * n)
        P = P.clamp_min(1e-12)
        g = torch.Generator().manual_seed(int(self.Seed))
        Y = torch.randn(n, int(self.NComponents), generator=g, dtype=torch.float64) * 1e-4
        V = torch.zeros_like(Y)
        for it in range(int(self.NIter)):
            ex = self.EarlyExaggeration if it < 100 else 1.0
            num = 1 / (1 + torch.cdist(Y, Y) ** 2)
            num.fill_diagonal_(0)
            Q = (num / num.sum()).clamp_min(1e-12)
            PQ = (ex * P - Q) * num
            grad = 4 * ((torch.diag(PQ.sum(1)) - PQ) @ Y)
            V = (0.5 if it < 250 else 0.8) * V - self.LearningRate * grad
            Y = Y + V
            Y = Y - Y.mean(0)
        self.Embedding = Y.numpy()
        return self.Embedding


class StandardScaler(Transformer):
    def Fit(self, X):
        X = A(X)
        self.Mean, self.Std = X.mean(0), X.std(0)
        self.Std[self.Std == 0] = 1.0
        return self

    def Transform(self, X):
        return (A(X) - self.Mean) / self.Std

    def InverseTransform(self, Z):
        return A(Z) * self.Std + self.Mean


class MinMaxScaler(Transformer):
    def Fit(self, X):
        X = A(X)
        self.Min, self.Max = X.min(0), X.max(0)
        return self

    def Transform(self, X):
        rng = np.where(self.Max - self.Min == 0, 1.0, self.Max - self.Min)
        return (A(X) - self.Min) / rng


class OneHotEncoder(Transformer):
    def Fit(self, X):
        X = A(X)
        X = X[:, None] if X.ndim == 1 else X
        self.Categories = [np.unique(X[:, j]) for j in range(X.shape[1])]
        return self

    def Transform(self, X):
        X = A(X)
        X = X[:, None] if X.ndim == 1 else X
        return np.concatenate([(X[:, j][:, None] == c[None]).astype(float) for j, c in enumerate(self.Categories)], 1)


class LabelEncoder(Estimator):
    def Fit(self, y):
        self.Classes = sorted(set(list(y)))
        self._map = {c: i for i, c in enumerate(self.Classes)}
        return self

    def Transform(self, y):
        return np.array([self._map[v] for v in y], dtype=np.int64)

    def FitTransform(self, y):
        return self.Fit(y).Transform(y)

    def InverseTransform(self, idx):
        return [self.Classes[int(i)] for i in idx]


class PolynomialFeatures(Transformer):
    _defaults = {"Degree": 2, "IncludeBias": True}

    def Fit(self, X):
        d = A(X).shape[1]
        self.Powers = [c for deg in range(0 if self.IncludeBias else 1, int(self.Degree) + 1)
                       for c in itertools.combinations_with_replacement(range(d), deg)]
        return self

    def Transform(self, X):
        X = A(X)
        return np.stack([np.prod(X[:, list(c)], 1) if c else np.ones(len(X)) for c in self.Powers], 1)


# ---- metrics --------------------------------------------------------------------------------
def Accuracy(y_true, y_pred):
    return float((A(y_true) == A(y_pred)).mean())


def ConfusionMatrix(y_true, y_pred, n_classes=None):
    """``M[t, p]`` counts.  With ``n_classes`` the labels are indices ``0..n_classes-1`` and pairs
    outside the range are dropped (ml/metrics.go:23-34); without it the sorted distinct labels of
    both arrays index the matrix."""
    yt, yp = A(y_true, np.int64), A(y_pred, np.int64)
    if n_classes is not None:
        M = np.zeros((n_classes, n_classes), dtype=np.int64)
        ok = (yt >= 0) & (yt < n_classes) & (yp >= 0) & (yp < n_classes)
        np.add.at(M, (yt[ok], yp[ok]), 1)
        return M
    cls = np.unique(np.concatenate([yt, yp]))
    M = np.zeros((len(cls), len(cls)), dtype=np.int64)
    np.add.at(M, (np.searchsorted(cls, yt), np.searchsorted(cls, yp)), 1)
    return M


def _per_class(y_true, y_pred):
    """Per-class tp / fp / fn / support over the sorted union of labels (ml/metrics.go:52-76)."""
    M = ConfusionMatrix(y_true, y_pred)
    tp = np.diag(M).astype(np.float64)
    return tp, M.sum(0) - tp, M.sum(1) - tp, M.sum(1).astype(np.float64)


def _ratio(num, den):
    return np.divide(num, den, out=np.zeros_like(num, dtype=np.float64), where=den > 0)


def _average(vals, support, average):
    """``"macro"`` (the default: plain mean over classes) or ``"weighted"`` (by support), as in
    ml/metrics.go:127-147; an integer label selects that class alone (binary use)."""
    if len(vals) == 0:
        return 0.0
    if average == "weighted":
        w = support.sum()
        return float((vals * support).sum() / w) if w else 0.0
    return float(vals.mean())


def _prf(y_true, y_pred, average, positive):
    tp, fp, fn, support = _per_class(y_true, y_pred)
    prec, rec = _ratio(tp, tp + fp), _ratio(tp, tp + fn)
    f1 = _ratio(2 * prec * rec, prec + rec)
    if positive is not None or not isinstance(average, str):
        cls = np.unique(np.concatenate([A(y_true, np.int64), A(y_pred, np.int64)]))
        want = positive if positive is not None else average
        i = np.searchsorted(cls, want)
        if i >= len(cls) or cls[i] != want:
            return 0.0, 0.0, 0.0
        return float(prec[i]), float(rec[i]), float(f1[i])
    return _average(prec, support, average), _average(rec, support, average), _average(f1, support, average)


def Precision(y_true, y_pred, average="macro", positive=None): return _prf(y_true, y_pred, average, positive)[0]
def Recall(y_true, y_pred, average="macro", positive=None): return _prf(y_true, y_pred, average, positive)[1]
def F1(y_true, y_pred, average="macro", positive=None): return _prf(y_true, y_pred, average, positive)[2]


def MeanSquaredError(y_true, y_pred):
    yt = A(y_true)
    return float(((yt - A(y_pred)) ** 2).mean()) if len(yt) else 0.0


def MeanAbsoluteError(y_true, y_pred):
    yt = A(y_true)
    return float(np.abs(yt - A(y_pred)).mean()) if len(yt) else 0.0


def R2Score(y_true, y_pred):
    """Coefficient of determination; 0 for an empty or constant target (ml/metrics.go:175-195)."""
    yt, yp = A(y_true), A(y_pred)
    if len(yt) == 0:
        return 0.0
    ss = ((yt - yt.mean()) ** 2).sum()
    return float(1 - ((yt - yp) ** 2).sum() / ss) if ss else 0.0


MSE, MAE, R2 = MeanSquaredError, MeanAbsoluteError, R2Score


def SilhouetteScore(X, labels):
    """Mean silhouette coefficient with Euclidean distances; points alone in their cluster add
    0, fewer than two clusters give 0 (ml/metrics.go:198-245)."""
    lab = A(labels, np.int64)
    if len(lab) == 0 or len(np.unique(lab)) < 2:
        return 0.0
    D = torch.cdist(T(X), T(X)).numpy()
    s = []
    for i in range(len(D)):
        same = lab == lab[i]
        if same.sum() <= 1:
            s.append(0.0)
            continue
        a = D[i, same].sum() / (same.sum() - 1)
        b = min(D[i, lab == c].mean() for c in np.unique(lab) if c != lab[i])
        s.append((b - a) / max(a, b) if max(a, b) > 0 else 0.0)
    return float(np.mean(s))


Silhouette = SilhouetteScore


def ROCAUC(y_true, scores):
    yt, sc = A(y_true), A(scores)
    order = np.argsort(sc, kind="stable")
    ranks = np.empty(len(sc))
    ranks[order] = np.arange(1, len(sc) + 1)
    for v in np.unique(sc):            # average ranks over ties
        m = sc == v
        ranks[m] = ranks[m].mean()
    pos = yt == 1
    n1, n0 = pos.sum(), (~pos).sum()
    return float((ranks[pos].sum() - n1 * (n1 + 1) / 2) / (n1 * n0)) if n1 and n0 else 0.5


# ---- model selection ---------------------------------------------------------------------------
def TrainTestSplit(X, y, test_size: float = 0.25, seed: int = 0):
    X, y = A(X), A(y)
    perm = np.random.default_rng(seed).permutation(len(X))
    k = int(round(len(X) * test_size))
    return X[perm[k:]], X[perm[:k]], y[perm[k:]], y[perm[:k]]


class KFold(Estimator):
    _defaults = {"NSplits": 5, "Shuffle": False, "Seed": 0}

    def Split(self, n: int):
        idx = np.random.default_rng(self.Seed).permutation(n) if self.Shuffle else np.arange(n)
        for f in np.array_split(idx, int(self.NSplits)):
            yield np.setdiff1d(idx, f, assume_unique=True), f


def CrossValScore(model_factory, X, y, k: int = 5):
    """``model_factory()`` returns a fresh estimator; the score is accuracy for classifiers
    (integer targets) and R^2 otherwise."""
    X, y = A(X), A(y)
    scores = []
    for tr, te in KFold(NSplits=k).Split(len(X)):
        m = model_factory().Fit(X[tr], y[tr])
        p = m.Predict(X[te])
        scores.append(Accuracy(y[te], p) if np.issubdtype(np.asarray(p).dtype, np.integer) else R2(y[te], p))
    return scores
