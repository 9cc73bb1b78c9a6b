"""Small public types of the reference package that carry no algorithm: enumerations, the FeaturesData container and the
base classes users derive multi-target custom metrics / objectives from (catboost/python-package/catboost/core.py)."""
from __future__ import annotations

import numpy as np

from .data.pool import CatBoostError


class EShapCalcType:
    Regular = "Regular"
    Approximate = "Approximate"
    Exact = "Exact"


class EFeaturesSelectionAlgorithm:
    RecursiveByPredictionValuesChange = "RecursiveByPredictionValuesChange"
    RecursiveByLossFunctionChange = "RecursiveByLossFunctionChange"
    RecursiveByShapValues = "RecursiveByShapValues"


class EFeaturesSelectionGrouping:
    Individual = "Individual"
    ByTags = "ByTags"


class FeaturesData:
    """Numerical features as a float32 matrix and categorical features as a matrix of strings / bytes, with optional
    names.  In a Pool the numerical columns come first."""

    def __init__(self, num_feature_data=None, cat_feature_data=None, num_feature_names=None, cat_feature_names=None):
        if num_feature_data is None and cat_feature_data is None:
            raise CatBoostError("FeaturesData needs num_feature_data or cat_feature_data")
        self.num_feature_data = None if num_feature_data is None else np.asarray(num_feature_data)
        self.cat_feature_data = None if cat_feature_data is None else np.asarray(cat_feature_data, dtype=object)
        if self.num_feature_data is not None and self.num_feature_data.dtype != np.float32:
            raise CatBoostError("num_feature_data must have dtype float32")
        for a in (self.num_feature_data, self.cat_feature_data):
            if a is not None and a.ndim != 2:
                raise CatBoostError("feature data must be two-dimensional")
        if self.num_feature_data is not None and self.cat_feature_data is not None \
                and len(self.num_feature_data) != len(self.cat_feature_data):
            raise CatBoostError("num_feature_data and cat_feature_data have different numbers of objects")
        self.num_feature_names = list(num_feature_names) if num_feature_names is not None else None
        self.cat_feature_names = list(cat_feature_names) if cat_feature_names is not None else None

    def get_object_count(self):
        a = self.num_feature_data if self.num_feature_data is not None else self.cat_feature_data
        return int(a.shape[0])

    def get_num_feature_count(self):
        return 0 if self.num_feature_data is None else int(self.num_feature_data.shape[1])

    def get_cat_feature_count(self):
        return 0 if self.cat_feature_data is None else int(self.cat_feature_data.shape[1])

    def get_feature_count(self):
        return self.get_num_feature_count() + self.get_cat_feature_count()

    def get_feature_names(self):
        nn, nc = self.get_num_feature_count(), self.get_cat_feature_count()
        names = list(self.num_feature_names) if self.num_feature_names is not None else [""] * nn
        names += list(self.cat_feature_names) if self.cat_feature_names is not None else [""] * nc
        return [nm if nm else str(i) for i, nm in enumerate(names)]

    def columns(self):
        """(list of column arrays, categorical column indices) in Pool order."""
        cols = [self.num_feature_data[:, j] for j in range(self.get_num_feature_count())]
        nn = len(cols)
        for j in range(self.get_cat_feature_count()):
            col = self.cat_feature_data[:, j]
            cols.append(np.array([v.decode("utf-8") if isinstance(v, bytes) else str(v) for v in col], dtype=object))
        return cols, list(range(nn, len(cols)))


class MultiTargetCustomMetric:
    """Base class of custom metrics for multi-target models: implement ``evaluate(approxes, targets, weight)`` (lists of
    per-dimension sequences) -> (error sum, weight sum), ``is_max_optimal()`` and ``get_final_error(error, weight)``."""

    def evaluate(self, approxes, targets, weight):
        raise NotImplementedError

    def is_max_optimal(self):
        return False

    def get_final_error(self, error, weight):
        return error / (weight + 1e-38)


class MultiTargetCustomObjective:
    """Base class of custom objectives for multi-target models: implement ``calc_ders_multi(approxes, targets, weight)``
    -> (first derivatives [dims], second derivatives [dims][dims]) for one object."""

    def calc_ders_multi(self, approxes, targets, weight):
        raise NotImplementedError


MultiRegressionCustomMetric = MultiTargetCustomMetric
MultiRegressionCustomObjective = MultiTargetCustomObjective
