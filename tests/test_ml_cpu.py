"""Classical ML: shape and "recovers known structure" checks (ml/*_test.go of the reference)."""
import numpy as np
import pytest

from gonn_b200 import data as D
from gonn_b200 import ml


def _blobs():
    X, y = D.MakeBlobs(240, 4, 3, 3, std=1.0)
    return X.numpy(), y.numpy()


def test_regressors_recover_linear_model():
    xy = D.MakeRegression(300, 5, 0.01, 1)
    (X, y), w = xy, xy.Weights
    X, y, w = X.numpy(), y.numpy(), w.numpy()
    for m in (ml.LinearRegression(), ml.Ridge(Alpha=1e-3), ml.Lasso(Alpha=1e-4), ml.ElasticNet(Alpha=1e-4),
              ml.BayesianRidge()):
        m.Fit(X, y)
        assert np.abs(m.Coef - w).max() < 0.05, type(m).__name__
        assert ml.R2(y, m.Predict(X)) > 0.99
    p, s = ml.BayesianRidge().Fit(X, y).PredictWithStd(X[:3])
    assert p.shape == s.shape == (3,) and (s > 0).all()


@pytest.mark.parametrize("make", [
    lambda: ml.LogisticRegression(LR=0.5, MaxIter=500), lambda: ml.LDA(), lambda: ml.QDA(), lambda: ml.GaussianNB(),
    lambda: ml.KNNClassifier(K=5), lambda: ml.KNNClassifier(K=5, Weights="distance"), lambda: ml.LinearSVC(MaxIter=300),
    lambda: ml.DecisionTreeClassifier(MaxDepth=6), lambda: ml.RandomForestClassifier(NEstimators=15, MaxDepth=6),
    lambda: ml.ExtraTreesClassifier(NEstimators=15, MaxDepth=8), lambda: ml.AdaBoostClassifier(NEstimators=20, MaxDepth=2),
    lambda: ml.GradientBoostingClassifier(NEstimators=20, MaxDepth=2)])
def test_classifiers_separate_blobs(make):
    X, y = _blobs()
    Xtr, Xte, ytr, yte = ml.TrainTestSplit(X, y, 0.25, 0)
    m = make().Fit(Xtr, ytr.astype(np.int64))
    assert ml.Accuracy(yte.astype(np.int64), m.Predict(Xte)) > 0.9


def test_tree_regressors_and_boosting():
    r = np.random.default_rng(0)
    X = r.uniform(-2, 2, (300, 2))
    y = np.sin(X[:, 0]) + 0.5 * X[:, 1] ** 2
    for m in (ml.DecisionTreeRegressor(MaxDepth=8), ml.RandomForestRegressor(NEstimators=20, MaxDepth=8),
              ml.ExtraTreesRegressor(NEstimators=20, MaxDepth=10), ml.GradientBoostingRegressor(NEstimators=60),
              ml.KNNRegressor(K=3)):
        assert ml.R2(y, m.Fit(X, y).Predict(X)) > 0.85, type(m).__name__


def test_count_naive_bayes():
    r = np.random.default_rng(0)
    y = r.integers(0, 2, 200)
    X = r.poisson(np.where(y[:, None] == 0, [5, 1, 1], [1, 1, 5]), (200, 3)).astype(float)
    assert ml.Accuracy(y, ml.MultinomialNB().Fit(X, y).Predict(X)) > 0.9
    assert ml.Accuracy(y, ml.BernoulliNB(Binarize=2.0).Fit(X, y).Predict(X)) > 0.8


def test_clusterers_find_blobs():
    X, y = _blobs()
    km = ml.KMeans(K=3, Seed=0).Fit(X)
    assert ml.Silhouette(X, km.Labels) > 0.5 and km.Predict(X[:5]).shape == (5,)
    assert len(set(ml.AgglomerativeClustering(NClusters=3).Fit(X[:80]).Labels)) == 3
    db = ml.DBSCAN(Eps=2.5, MinSamples=4).Fit(X)
    assert len(set(db.Labels) - {-1}) >= 2
    assert len(ml.MeanShift(Bandwidth=4.0).Fit(X).Centers) >= 2
    gm = ml.GaussianMixture(NComponents=3, Seed=0).Fit(X)
    assert ml.Silhouette(X, gm.Labels) > 0.5


def test_decompositions():
    r = np.random.default_rng(0)
    Z = r.standard_normal((200, 2))
    X = Z @ np.array([[3.0, 1.0, 0.0], [0.0, 0.5, 2.0]]) + 0.01 * r.standard_normal((200, 3))
    p = ml.PCA(NComponents=2).Fit(X)
    assert p.ExplainedVarianceRatio.sum() > 0.99
    assert np.abs(p.InverseTransform(p.Transform(X)) - X).max() < 0.1
    assert ml.KernelPCA(NComponents=2, Kernel="rbf").FitTransform(X).shape == (200, 2)
    S = np.stack([np.sign(np.sin(np.linspace(0, 20, 300))), np.sin(np.linspace(0, 33, 300))], 1)
    rec = ml.FastICA(NComponents=2, Seed=0).FitTransform(S @ np.array([[1.0, 0.5], [0.3, 1.0]]))
    c = np.abs(np.corrcoef(rec.T, S.T)[:2, 2:])
    assert c.max(1).min() > 0.9
    emb = ml.TSNE(NIter=120, Perplexity=10).FitTransform(_blobs()[0][:60])
    assert emb.shape == (60, 2) and np.isfinite(emb).all()


def test_preprocessing_metrics_selection():
    X = np.array([[1.0, 10.0], [2.0, 20.0], [3.0, 30.0]])
    assert np.allclose(ml.StandardScaler().FitTransform(X).mean(0), 0)
    assert np.allclose(ml.MinMaxScaler().FitTransform(X).max(0), 1)
    assert ml.OneHotEncoder().FitTransform(np.array([0, 2, 1, 2])).shape == (4, 3)
    le = ml.LabelEncoder()
    assert le.InverseTransform(le.FitTransform(["b", "a", "b"])) == ["b", "a", "b"]
    assert ml.PolynomialFeatures(Degree=2).FitTransform(X).shape == (3, 6)
    yt, yp = [1, 0, 1, 1, 0], [1, 0, 0, 1, 1]
    assert ml.ConfusionMatrix(yt, yp).tolist() == [[1, 1], [1, 2]]
    assert abs(ml.Precision(yt, yp, positive=1) - 2 / 3) < 1e-12 and abs(ml.Recall(yt, yp, positive=1) - 2 / 3) < 1e-12
    # macro (default) and support-weighted averages over classes {0: p=r=1/2, 1: p=r=2/3}
    for f in (ml.Precision, ml.Recall, ml.F1):
        assert abs(f(yt, yp) - 7 / 12) < 1e-12 and abs(f(yt, yp, "weighted") - 0.6) < 1e-12
    assert ml.ConfusionMatrix([0, 2, 5], [0, 1, 5], 3).tolist() == [[1, 0, 0], [0, 0, 0], [0, 1, 0]]
    assert ml.MeanSquaredError([1.0, 3.0], [2.0, 5.0]) == 2.5 and ml.MeanAbsoluteError([1.0, 3.0], [2.0, 5.0]) == 1.5
    assert ml.MeanSquaredError([], []) == 0.0 and ml.R2Score([2.0, 2.0], [1.0, 3.0]) == 0.0
    assert abs(ml.R2Score([1.0, 2.0, 3.0], [1.0, 2.0, 4.0]) - 0.5) < 1e-12
    assert ml.SilhouetteScore([[0.0], [1.0]], [0, 0]) == 0.0
    assert abs(ml.SilhouetteScore([[0.0], [1.0], [10.0], [11.0]], [0, 0, 1, 1]) - (9.5 / 10.5 + 8.5 / 9.5) / 2) < 1e-12
    assert abs(ml.ROCAUC([0, 0, 1, 1], [0.1, 0.4, 0.35, 0.8]) - 0.75) < 1e-12
    folds = list(ml.KFold(NSplits=4).Split(10))
    assert len(folds) == 4 and sorted(np.concatenate([f for _, f in folds])) == list(range(10))
    Xb, yb = _blobs()
    assert min(ml.CrossValScore(lambda: ml.GaussianNB(), Xb, yb.astype(np.int64), 4)) > 0.9
    iso = ml.IsolationForest(NEstimators=30, Seed=0).Fit(np.vstack([Xb[yb == 0], [[60.0, 60.0, 60.0, 60.0]]]))
    s = iso.AnomalyScore(np.vstack([Xb[yb == 0][:5], [[60.0, 60.0, 60.0, 60.0]]]))
    assert s[-1] > s[:5].max()
