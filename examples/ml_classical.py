"""Classical estimators on synthetic data (the reference's examples/ml_classical/main.go):
train/test split, scaling, a few classifiers, k-means and PCA."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from gonn_b200 import ml  # noqa: E402
from gonn_b200.data import MakeBlobs  # noqa: E402


def main():
    X, y = MakeBlobs(300, 4, centers=3, std=1.0, seed=3)
    X, y = X.tolist(), y.tolist()
    Xtr, Xte, ytr, yte = ml.TrainTestSplit(X, y, test_size=0.25, seed=0)
    scaler = ml.StandardScaler()
    Xtr, Xte = scaler.FitTransform(Xtr), None if Xte is None else scaler.Transform(Xte)
    scores = {}
    for name, est in (("logistic", ml.LogisticRegression()), ("tree", ml.DecisionTreeClassifier()),
                      ("forest", ml.RandomForestClassifier()), ("knn", ml.KNNClassifier()),
                      ("nb", ml.GaussianNB())):
        est.Fit(Xtr, ytr)
        scores[name] = ml.Accuracy(yte, est.Predict(Xte))
        print(f"{name:10s} accuracy {scores[name]:.3f}")
    km = ml.KMeans(K=3, Seed=0)
    km.Fit(Xtr)
    print("k-means inertia", round(km.Inertia, 2))
    pca = ml.PCA(NComponents=2)
    Z = pca.FitTransform(Xtr)
    print("PCA explained variance ratio", [round(float(v), 3) for v in pca.ExplainedVarianceRatio])
    return scores


if __name__ == "__main__":
    main()
