"""Classical machine learning on plain arrays (ml/*.go): linear models, trees and ensembles,
neighbours, naive Bayes, clustering, decomposition, manifold learning, preprocessing, metrics
and model selection.  Independent of the nn / tensor packages; torch is used for the dense
linear algebra."""
from .base import Regressor, Classifier, Clusterer, Transformer  # noqa
from .linear import *  # noqa
from .trees import (DecisionTreeClassifier, DecisionTreeRegressor, RandomForestClassifier, RandomForestRegressor,  # noqa
                    ExtraTreesClassifier, ExtraTreesRegressor, AdaBoostClassifier, GradientBoostingRegressor,
                    GradientBoostingClassifier, IsolationForest)
from .unsupervised import *  # noqa

# the long names the reference's documentation uses for the discriminant models
LinearDiscriminantAnalysis, QuadraticDiscriminantAnalysis = LDA, QDA  # noqa: F405
