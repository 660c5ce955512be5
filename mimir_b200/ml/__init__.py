"""Classical machine learning on tables (reference: tabular/, tree/, linear/, svm/, neighbors/, bayes/,
cluster/, decompose/, forecast/, recommend/, rules/, automl/).

One module per family, named as the reference's packages: ``tabular`` (tables, splits, cross-validation),
``tree`` (boosted trees, forests, isolation forests; histograms and tree growth in native code),
``linear`` (least squares with lasso / ridge penalties, logistic and softmax regression), ``svm`` (kernel
machines by SMO, linear classifiers by native dual coordinate descent, regression), ``neighbors``,
``bayes``, ``cluster`` (k-means, mixtures, DBSCAN, Ward's hierarchy, silhouette), ``decompose`` (PCA),
``forecast``, ``recommend``, ``rules``, ``automl``; ``modules`` serves fitted models as ``nn.Module``s.
Fits standardize the features, count a missing value (NaN) as the feature's mean, and return models of
plain fields with ``to_json`` / ``from_json``.  The short function names below are the array-level
entry points (``ridge(X, y)``, ``kmeans(X, k)``, ...)."""
from . import automl, base, bayes, cluster, decompose, forecast, linear, modules, neighbors, recommend, rules, svm, tabular, tree  # noqa: F401
from .base import CLASSIFICATION, REGRESSION, Task  # noqa: F401
from .linear import KernelSVM, elastic_net, fista_lasso, lasso, linear_svm, logistic, ridge  # noqa: F401
from .neighbors import KNN, GaussianNB, MultinomialNB, dbscan, gmm, kmeans, pca, ward  # noqa: F401
from .tabular import Data, cross_validate, fit_scaler, split  # noqa: F401
from .tree import decision_tree, gradient_boosting, isolation_forest, random_forest  # noqa: F401
