"""catboost_b200: a Blackwell-native gradient-boosted decision tree framework with CatBoost's capabilities.

Public API mirrors ``catboost``: :class:`CatBoost`, :class:`CatBoostClassifier`, :class:`CatBoostRegressor`,
:class:`CatBoostRanker`, :class:`Pool`, :func:`train`, :func:`cv`, :func:`sum_models`.
"""
from .core import (CatBoost, CatBoostClassifier, CatBoostRanker, CatBoostRegressor, EFstrType, sum_models,  # noqa: F401
                   to_classifier, to_ranker, to_regressor, train)
from .data.pool import CatBoostError, Pool  # noqa: F401
from .cv import cv  # noqa: F401
from .eval_features import eval_features  # noqa: F401

from .gp import sample_gaussian_process  # noqa: F401
from .compat import (EFeaturesSelectionAlgorithm, EFeaturesSelectionGrouping, EShapCalcType, FeaturesData,  # noqa: F401
                     MultiRegressionCustomMetric, MultiRegressionCustomObjective, MultiTargetCustomMetric,
                     MultiTargetCustomObjective)

from .widget import MetricVisualizer  # noqa: E402,F401

CatboostError = CatBoostError          # spelling kept by the reference for old code
__version__ = "0.1.0"
__all__ = ["CatBoost", "CatBoostClassifier", "CatBoostRegressor", "CatBoostRanker", "Pool", "CatBoostError", "train",
           "cv", "sum_models", "to_classifier", "to_regressor", "to_ranker", "EFstrType", "EShapCalcType",
           "EFeaturesSelectionAlgorithm", "EFeaturesSelectionGrouping", "FeaturesData", "CatboostError",
           "sample_gaussian_process", "eval_features", "MultiRegressionCustomMetric", "MultiRegressionCustomObjective",
           "MultiTargetCustomMetric", "MultiTargetCustomObjective", "MetricVisualizer"]
