"""Linear models, discriminant analysis, naive Bayes, nearest neighbours, SVM
(ml/linreg.go, ridge/lasso/elasticnet, bayesian_ridge.go, logreg.go, lda.go, qda.go, nb.go,
knn.go, svc.go).  Dense linear algebra runs through torch (float64)."""
from __future__ import annotations

import numpy as np
import torch

from .base import A, Classifier, Regressor, T


def _add_bias(X):
    return torch.cat([X, torch.ones(X.shape[0], 1, dtype=X.dtype)], 1)


class LinearRegression(Regressor):
    def Fit(self, X, y):
        Xb, y = _add_bias(T(X)), T(y)
        w = torch.linalg.lstsq(Xb, y[:, None]).solution[:, 0]
        self.Coef, self.Intercept = w[:-1].numpy(), float(w[-1])
        return self

    def Predict(self, X):
        return A(X) @ self.Coef + self.Intercept


class Ridge(Regressor):
    _defaults = {"Alpha": 1.0}

    def Fit(self, X, y):
        X, y = T(X), T(y)
        mu, ym = X.mean(0), y.mean()
        Xc = X - mu
        w = torch.linalg.solve(Xc.T @ Xc + self.Alpha * torch.eye(X.shape[1], dtype=X.dtype), Xc.T @ (y - ym))
        self.Coef, self.Intercept = w.numpy(), float(ym - mu @ w)
        return self

    def Predict(self, X):
        return A(X) @ self.Coef + self.Intercept


class ElasticNet(Regressor):
    """Coordinate descent on (1/2n)||y - Xw||^2 + alpha*l1_ratio*|w|_1 + alpha*(1-l1_ratio)/2*|w|^2."""
    _defaults = {"Alpha": 1.0, "L1Ratio": 0.5, "MaxIter": 1000, "Tol": 1e-6}

    def Fit(self, X, y):
        X, y = A(X), A(y)
        n, d = X.shape
        mu, ym = X.mean(0), y.mean()
        Xc, yc = X - mu, y - ym
        w = np.zeros(d)
        l1, l2 = self.Alpha * self.L1Ratio, self.Alpha * (1 - self.L1Ratio)
        col_sq = (Xc ** 2).sum(0) / n
        r = yc.copy()
        for _ in range(int(self.MaxIter)):
            wmax = 0.0
            for j in range(d):
                if col_sq[j] == 0:
                    continue
                rho = Xc[:, j] @ (r + Xc[:, j] * w[j]) / n
                nw = np.sign(rho) * max(abs(rho) - l1, 0.0) / (col_sq[j] + l2)
                if nw != w[j]:
                    r -= Xc[:, j] * (nw - w[j])
                    wmax = max(wmax, abs(nw - w[j]))
                    w[j] = nw
            if wmax < self.Tol:
                break
        self.Coef, self.Intercept = w, float(ym - mu @ w)
        return self

    def Predict(self, X):
        return A(X) @ self.Coef + self.Intercept


class Lasso(ElasticNet):
    _defaults = {"Alpha": 1.0, "L1Ratio": 1.0, "MaxIter": 1000, "Tol": 1e-6}


class BayesianRidge(Regressor):
    _defaults = {"Alpha1": 1e-6, "Alpha2": 1e-6, "Lambda1": 1e-6, "Lambda2": 1e-6, "MaxIter": 300, "Tol": 1e-3}

    def Fit(self, X, y):
        X, y = A(X), A(y)
        n, d = X.shape
        mu, ym = X.mean(0), y.mean()
        Xc, yc = X - mu, y - ym
        alpha, lam = 1.0 / (yc.var() + 1e-12), 1.0
        XtX, Xty = Xc.T @ Xc, Xc.T @ yc
        w = np.zeros(d)
        for _ in range(int(self.MaxIter)):
            S = np.linalg.inv(lam * np.eye(d) + alpha * XtX)
            w_new = alpha * S @ Xty
            gamma = d - lam * np.trace(S)
            lam = (gamma + 2 * self.Lambda1) / (w_new @ w_new + 2 * self.Lambda2)
            alpha = (n - gamma + 2 * self.Alpha1) / (((yc - Xc @ w_new) ** 2).sum() + 2 * self.Alpha2)
            done = np.abs(w_new - w).sum() < self.Tol
            w = w_new
            if done:
                break
        self.Coef, self.Intercept, self.Sigma, self.AlphaEst, self._mu = w, float(ym - mu @ w), S, alpha, mu
        self.LambdaEst = lam
        return self

    def Predict(self, X):
        return A(X) @ self.Coef + self.Intercept

    def PredictWithStd(self, X):
        Xc = A(X) - self._mu
        var = 1.0 / self.AlphaEst + np.einsum("ij,jk,ik->i", Xc, self.Sigma, Xc)
        return self.Predict(X), np.sqrt(var)


class LogisticRegression(Classifier):
    """Multinomial softmax regression by full-batch gradient descent."""
    _defaults = {"LR": 0.1, "MaxIter": 1000, "Tol": 1e-6, "Seed": 0}

    def Fit(self, X, y):
        X, yi = T(X), torch.as_tensor(A(y, np.int64))
        self.Classes = torch.unique(yi).numpy()
        idx = torch.searchsorted(torch.as_tensor(self.Classes), yi)
        K = len(self.Classes)
        W = torch.zeros(X.shape[1] + 1, K, dtype=torch.float64, requires_grad=True)
        Xb = _add_bias(X)
        prev = float("inf")
        for _ in range(int(self.MaxIter)):
            loss = torch.nn.functional.cross_entropy(Xb @ W, idx)
            (g,) = torch.autograd.grad(loss, W)
            with torch.no_grad():
                W -= self.LR * g
            if abs(prev - float(loss.detach())) < self.Tol:
                break
            prev = float(loss.detach())
        self.W = W.detach()
        return self

    def PredictProba(self, X):
        return torch.softmax(_add_bias(T(X)) @ self.W, 1).numpy()

    def Predict(self, X):
        return self.Classes[self.PredictProba(X).argmax(1)]


class LinearSVC(Classifier):
    """One-vs-rest linear SVM, hinge loss + L2, sub-gradient descent."""
    _defaults = {"C": 1.0, "MaxIter": 1000, "LR": 0.01, "Seed": 0}

    def Fit(self, X, y):
        X, y = T(X), A(y, np.int64)
        self.Classes = np.unique(y)
        Xb = _add_bias(X)
        Ws = []
        for c in self.Classes:
            t = torch.as_tensor(np.where(y == c, 1.0, -1.0))
            w = torch.zeros(Xb.shape[1], dtype=torch.float64)
            for _ in range(int(self.MaxIter)):
                m = t * (Xb @ w)
                act = (m < 1).to(torch.float64)
                g = w.clone()
                g[-1] = 0
                g -= self.C * (Xb * (act * t)[:, None]).mean(0) * Xb.shape[0] / Xb.shape[0]
                w -= self.LR * g
            Ws.append(w)
        self.W = torch.stack(Ws, 1)
        return self

    def DecisionFunction(self, X):
        return (_add_bias(T(X)) @ self.W).numpy()

    def Predict(self, X):
        s = self.DecisionFunction(X)
        if len(self.Classes) == 2:
            return self.Classes[(s[:, 1] > s[:, 0]).astype(int)]
        return self.Classes[s.argmax(1)]


class LDA(Classifier):
    _defaults = {"NComponents": 0}

    def Fit(self, X, y):
        X, y = A(X), A(y, np.int64)
        self.Classes = np.unique(y)
        n, d = X.shape
        self.Means = np.stack([X[y == c].mean(0) for c in self.Classes])
        self.Priors = np.array([(y == c).mean() for c in self.Classes])
        Sw = sum(((X[y == c] - m).T @ (X[y == c] - m)) for c, m in zip(self.Classes, self.Means)) / (n - len(self.Classes))
        self.Cov = Sw + 1e-9 * np.eye(d)
        self.CovInv = np.linalg.inv(self.Cov)
        mu = X.mean(0)
        Sb = sum((y == c).sum() * np.outer(m - mu, m - mu) for c, m in zip(self.Classes, self.Means)) / n
        ev, evec = np.linalg.eig(self.CovInv @ Sb)
        order = np.argsort(-ev.real)
        k = self.NComponents or min(len(self.Classes) - 1, d)
        self.Scalings = evec.real[:, order[:k]]
        self._mu = mu
        return self

    def _scores(self, X):
        X = A(X)
        return X @ self.CovInv @ self.Means.T - 0.5 * np.einsum("kd,de,ke->k", self.Means, self.CovInv, self.Means) + np.log(self.Priors)

    def PredictProba(self, X):
        s = self._scores(X)
        s = np.exp(s - s.max(1, keepdims=True))
        return s / s.sum(1, keepdims=True)

    def Predict(self, X):
        return self.Classes[self._scores(X).argmax(1)]

    def Transform(self, X):
        return (A(X) - self._mu) @ self.Scalings


class QDA(Classifier):
    def Fit(self, X, y):
        X, y = A(X), A(y, np.int64)
        self.Classes = np.unique(y)
        d = X.shape[1]
        self.Means, self.Covs, self.Priors = [], [], []
        for c in self.Classes:
            Xc = X[y == c]
            self.Means.append(Xc.mean(0))
            self.Covs.append(np.cov(Xc.T).reshape(d, d) + 1e-6 * np.eye(d))
            self.Priors.append(len(Xc) / len(X))
        return self

    def _discriminant(self, X):
        X = A(X)
        s = []
        for m, C, p in zip(self.Means, self.Covs, self.Priors):
            Ci = np.linalg.inv(C)
            dlt = X - m
            s.append(-0.5 * np.einsum("ij,jk,ik->i", dlt, Ci, dlt) - 0.5 * np.linalg.slogdet(C)[1] + np.log(p))
        return np.stack(s, 1)

    def Predict(self, X):
        return self.Classes[self._discriminant(X).argmax(1)]

    def PredictProba(self, X):
        """Softmax of the quadratic discriminants (ml/lda.go:365-371)."""
        s = self._discriminant(X)
        e = np.exp(s - s.max(1, keepdims=True))
        return e / e.sum(1, keepdims=True)


class GaussianNB(Classifier):
    def Fit(self, X, y):
        X, y = A(X), A(y, np.int64)
        self.Classes = np.unique(y)
        self.Theta = np.stack([X[y == c].mean(0) for c in self.Classes])
        self.Var = np.stack([X[y == c].var(0) for c in self.Classes]) + 1e-9 * X.var(0).max()
        self.Priors = np.array([(y == c).mean() for c in self.Classes])
        return self

    def Predict(self, X):
        X = A(X)[:, None, :]
        ll = -0.5 * (np.log(2 * np.pi * self.Var)[None] + (X - self.Theta[None]) ** 2 / self.Var[None]).sum(2)
        return self.Classes[(ll + np.log(self.Priors)[None]).argmax(1)]


class MultinomialNB(Classifier):
    _defaults = {"Alpha": 1.0}

    def Fit(self, X, y):
        X, y = A(X), A(y, np.int64)
        self.Classes = np.unique(y)
        cnt = np.stack([X[y == c].sum(0) for c in self.Classes]) + self.Alpha
        self.LogProb = np.log(cnt / cnt.sum(1, keepdims=True))
        self.LogPrior = np.log(np.array([(y == c).mean() for c in self.Classes]))
        return self

    def Predict(self, X):
        return self.Classes[(A(X) @ self.LogProb.T + self.LogPrior).argmax(1)]


class BernoulliNB(Classifier):
    _defaults = {"Alpha": 1.0, "Binarize": 0.0}

    def Fit(self, X, y):
        X, y = (A(X) > self.Binarize).astype(float), A(y, np.int64)
        self.Classes = np.unique(y)
        self.P = np.stack([(X[y == c].sum(0) + self.Alpha) / ((y == c).sum() + 2 * self.Alpha) for c in self.Classes])
        self.LogPrior = np.log(np.array([(y == c).mean() for c in self.Classes]))
        return self

    def Predict(self, X):
        X = (A(X) > self.Binarize).astype(float)
        ll = X @ np.log(self.P).T + (1 - X) @ np.log(1 - self.P).T
        return self.Classes[(ll + self.LogPrior).argmax(1)]


class _KNN:
    _defaults = {"K": 5, "Weights": "uniform"}

    def Fit(self, X, y):
        self.X, self.y = T(X), A(y)
        return self

    def _neighbours(self, X):
        d = torch.cdist(T(X), self.X)
        k = min(int(self.K), self.X.shape[0])
        dist, idx = torch.topk(d, k, dim=1, largest=False)
        w = torch.ones_like(dist) if self.Weights != "distance" else 1.0 / (dist + 1e-12)
        return idx.numpy(), w.numpy()


class KNNClassifier(_KNN, Classifier):
    def Predict(self, X):
        idx, w = self._neighbours(X)
        labs = self.y[idx].astype(np.int64)
        classes = np.unique(self.y).astype(np.int64)
        votes = np.stack([(w * (labs == c)).sum(1) for c in classes], 1)
        return classes[votes.argmax(1)]


class KNNRegressor(_KNN, Regressor):
    def Predict(self, X):
        idx, w = self._neighbours(X)
        return (self.y[idx] * w).sum(1) / w.sum(1)
