"""Classical machine learning (reference: tabular/, tree/, linear/, logistic/, svm/, neighbors/,
bayes/, cluster/, decomp/, forecast/, recommend/, rules/, automl/)."""
from . import linear, misc, neighbors, tabular, tree
from .linear import KernelSVM, elastic_net, fista_lasso, lasso, linear_svm, logistic, ridge
from .misc import ALS, HoltWinters, apriori, automl, autoregressive
from .neighbors import KNN, GaussianNB, MultinomialNB, dbscan, gmm, kmeans, pca, ward
from .tabular import Data, cross_validate, fit_scaler, split
from .tree import decision_tree, gradient_boosting, isolation_forest, random_forest
