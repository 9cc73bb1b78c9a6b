"""User-facing estimators: ``CatBoost``, ``CatBoostClassifier``, ``CatBoostRegressor``, ``CatBoostRanker`` and the
module-level ``train`` / ``cv`` / ``sum_models`` helpers.  The surface follows
catboost/python-package/catboost/core.py (CatBoost :2585, CatBoostClassifier :4894, CatBoostRegressor :5981,
CatBoostRanker :6391, train :6775, cv :7085, sum_models :7394).
"""
from __future__ import annotations

import copy
import math
import json
import os
from typing import Optional

import numpy as np

from .data.pool import CatBoostError, Pool, to_pool
from .metrics import make_metric
from .models.model import Model
from .params import DEFAULTS, SYNONYMS, normalize_params, parse_devices


class EFstrType:
    PredictionValuesChange = "PredictionValuesChange"
    LossFunctionChange = "LossFunctionChange"
    FeatureImportance = "FeatureImportance"
    Interaction = "Interaction"
    ShapValues = "ShapValues"
    PredictionDiff = "PredictionDiff"
    ShapInteractionValues = "ShapInteractionValues"
    SageValues = "SageValues"


def _sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


class CatBoost:
    _default_loss = "RMSE"
    _estimator_type = None

    def __init__(self, params: Optional[dict] = None, **kwargs):
        p = dict(params or {})
        p.update(kwargs)
        self._init_params = {k: v for k, v in p.items() if v is not None}
        normalize_params(self._init_params)     # validates names early
        self._model: Optional[Model] = None
        self._evals_result = {}
        self._best_iteration = None
        self._best_score = {}
        self._train_info = {}

    # ------------------------------------------------------------------ params
    def get_params(self, deep=True):
        return copy.deepcopy(self._init_params)

    def get_init_params(self):
        """The parameters this object was constructed with (before training filled in defaults)."""
        return copy.deepcopy(self._init_params)

    def set_params(self, **params):
        normalize_params(params)
        self._init_params.update(params)
        return self

    def get_param(self, key):
        return self._init_params.get(key)

    def get_all_params(self):
        self._check_fitted()
        return dict(self._model.params)

    def is_fitted(self):
        return self._model is not None

    def _check_fitted(self):
        if self._model is None:
            raise CatBoostError("model is not fitted")

    def copy(self):
        return copy.deepcopy(self)

    def __sklearn_tags__(self):  # pragma: no cover - sklearn >= 1.6 compatibility
        try:
            from sklearn.utils import Tags, InputTags, TargetTags
            return Tags(estimator_type=self._estimator_type, target_tags=TargetTags(required=True),
                        input_tags=InputTags(allow_nan=True))
        except Exception:
            raise AttributeError

    # ------------------------------------------------------------------ fit
    def fit(self, X, y=None, cat_features=None, text_features=None, embedding_features=None, pairs=None,
            sample_weight=None, group_id=None, group_weight=None, subgroup_id=None, pairs_weight=None, baseline=None,
            use_best_model=None, eval_set=None, verbose=None, logging_level=None, plot=False, plot_file=None,
            column_description=None, verbose_eval=None, metric_period=None, silent=None, early_stopping_rounds=None,
            save_snapshot=None, snapshot_file=None, snapshot_interval=None, init_model=None, callbacks=None,
            log_cout=None, log_cerr=None):
        params = dict(self._init_params)
        if cat_features is None and "cat_features" in params:
            cat_features = params.get("cat_features")
        params.pop("cat_features", None)
        for k, v in dict(use_best_model=use_best_model, verbose=verbose if verbose is not None else verbose_eval,
                         logging_level=logging_level, metric_period=metric_period, silent=silent,
                         early_stopping_rounds=early_stopping_rounds, save_snapshot=save_snapshot,
                         snapshot_file=snapshot_file, snapshot_interval=snapshot_interval).items():
            if v is not None:
                params[k] = v
        if isinstance(X, Pool):
            if any(a is not None for a in (y, sample_weight, group_id, pairs, baseline)) and y is not None:
                raise CatBoostError("y must be None when X is a Pool")
            train_pool = X
        else:
            if y is None and not isinstance(X, (str, os.PathLike)):
                raise CatBoostError("y is required when X is not a Pool")
            if text_features is None:
                text_features = params.get("text_features")
            if embedding_features is None:
                embedding_features = params.get("embedding_features")
            train_pool = Pool(X, y, cat_features=cat_features, text_features=text_features,
                              embedding_features=embedding_features, pairs=pairs, weight=sample_weight, group_id=group_id,
                              group_weight=group_weight, subgroup_id=subgroup_id, pairs_weight=pairs_weight,
                              baseline=baseline, column_description=column_description)
        eval_pools = []
        if eval_set is not None:
            sets = eval_set if isinstance(eval_set, list) else [eval_set]
            for es in sets:
                if isinstance(es, Pool):
                    eval_pools.append(es)
                elif isinstance(es, tuple) and len(es) == 2:
                    eval_pools.append(Pool(es[0], es[1], cat_features=train_pool.cat_feature_indices,
                                           text_features=getattr(train_pool, "text_feature_indices", None) or None,
                                           embedding_features=getattr(train_pool, "embedding_feature_indices", None) or None,
                                           feature_names=train_pool.feature_names))
                else:
                    raise CatBoostError("eval_set must be a Pool, an (X, y) tuple or a list of them")
        frac = params.get("eval_fraction")
        if frac is not None and float(frac) > 0 and not eval_pools:
            # the last part of the learn set becomes the evaluation set (whole queries when there are groups), as in
            # catboost/libs/train_lib (eval_fraction)
            from .parallel.launcher import shard_bounds
            n_all = train_pool.num_row()
            if not 0.0 < float(frac) < 1.0:
                raise CatBoostError("eval_fraction must be in (0, 1)")
            cut = int(round(n_all * (1.0 - float(frac))))
            if train_pool.group_id is not None:
                off = train_pool.group_offsets()
                cut = int(off[np.searchsorted(off, cut)]) if cut < n_all else n_all
            if cut <= 0 or cut >= n_all:
                raise CatBoostError("eval_fraction leaves the learn or the evaluation part empty")
            eval_pools = [train_pool.slice(np.arange(cut, n_all))]
            train_pool = train_pool.slice(np.arange(0, cut))
        init = None
        if init_model is not None:
            init = init_model._model if isinstance(init_model, CatBoost) else init_model
            if isinstance(init, (str, os.PathLike)):
                init = CatBoost().load_model(init)._model
        from .parallel.launcher import train_maybe_multi_gpu
        res = train_maybe_multi_gpu(params, train_pool, eval_pools, default_loss=self._default_loss, init_model=init,
                                    callbacks=callbacks, log_cout=log_cout)
        self._model = res.model
        self._evals_result = res.evals_result
        self._best_iteration = res.best_iteration
        self._best_score = res.best_score
        self._train_info = dict(timings=res.timings, h2d_bytes=res.h2d_bytes, launches_per_iter=res.launches_per_iter)
        self._eval_pools = list(eval_pools)
        return self

    # ------------------------------------------------------------------ predict
    def _pool_kwargs(self):
        """How raw prediction data has to be read: the column roles the model was trained with."""
        kw = dict(cat_features=[c.flat_index for c in self._model.cat_features])
        est = getattr(self._model, "estimators", None)
        if est is not None:
            kw["text_features"] = list(est.text_flat) or None
            kw["embedding_features"] = list(est.emb_flat) or None
        return kw

    def _raw(self, data, ntree_start=0, ntree_end=0, thread_count=-1, task_type="CPU", devices=None):
        self._check_fitted()
        pool = data if isinstance(data, Pool) else Pool(data, data_can_be_none=False, **self._pool_kwargs())
        fd, ch = self._model.pool_arrays(pool)
        raw = self._model.predict_raw(fd, ch, ntree_start, ntree_end, task_type=task_type, thread_count=thread_count,
                                      device=devices)
        if pool.baseline is not None:
            raw = raw + pool.baseline.reshape(raw.shape)
        return raw

    def _format(self, raw, prediction_type):
        m = self._model
        pt = prediction_type
        binclass = m.loss_name in ("Logloss", "CrossEntropy", "Focal")
        multi = m.loss_name in ("MultiClass", "MultiClassOneVsAll")
        if pt == "RawFormulaVal":
            return raw[:, 0] if raw.shape[1] == 1 else raw
        if pt == "MultiProbability":
            # per-label probabilities of a multi-label model (catboost/private/libs/options/enums.h EPredictionType)
            if m.loss_name not in ("MultiLogloss", "MultiCrossEntropy"):
                raise CatBoostError("prediction_type 'MultiProbability' needs a MultiLogloss / MultiCrossEntropy model")
            return _sigmoid(raw)
        if pt in ("Probability", "LogProbability"):
            if binclass:
                p1 = _sigmoid(raw[:, 0])
                pr = np.stack([1 - p1, p1], axis=1)
            elif m.loss_name == "MultiClass":
                e = np.exp(raw - raw.max(1, keepdims=True))
                pr = e / e.sum(1, keepdims=True)
            elif m.loss_name in ("MultiClassOneVsAll", "MultiLogloss", "MultiCrossEntropy"):
                pr = _sigmoid(raw)
            else:
                raise CatBoostError(f"prediction_type {pt!r} needs a classification model")
            return pr if pt == "Probability" else np.log(np.clip(pr, 1e-300, None))
        if pt == "Class":
            if binclass:
                thr = float(m.info.get("binclass_probability_threshold", 0.5))
                border = math.log(thr / (1.0 - thr)) if 0.0 < thr < 1.0 else (math.inf if thr >= 1.0 else -math.inf)
                idx = (raw[:, 0] > border).astype(np.int64)
            elif multi:
                idx = raw.argmax(1)
            elif m.loss_name in ("MultiLogloss", "MultiCrossEntropy"):
                return (raw > 0).astype(np.int64)
            else:
                raise CatBoostError("prediction_type 'Class' needs a classification model")
            names = m.class_names
            if names is None:
                return idx
            arr = np.array(names, dtype=object)[idx]
            try:
                return arr.astype(type(names[0])) if not isinstance(names[0], str) else arr
            except (ValueError, TypeError):
                return arr
        if pt == "Exponent":
            return np.exp(raw[:, 0])
        if pt == "RMSEWithUncertainty":
            return np.stack([raw[:, 0], np.exp(2 * raw[:, 1])], 1)
        raise CatBoostError(f"unknown prediction_type {pt!r}")

    def _default_prediction_type(self):
        return "RawFormulaVal"

    def predict(self, data, prediction_type=None, ntree_start=0, ntree_end=0, thread_count=-1, verbose=None,
                task_type="CPU", devices=None):
        """``task_type='GPU'`` evaluates float-only symmetric models on the device; ``devices`` ('0-7', '0:2', a list)
        shards the rows over several GPUs of this machine."""
        single = self._is_single_object(data)
        if single:
            data = [list(data)] if not isinstance(data, np.ndarray) else data.reshape(1, -1)
        raw = self._raw(data, ntree_start, ntree_end, thread_count, task_type, devices)
        pt = prediction_type or self._default_prediction_type()
        out = self._format(raw, pt)
        return out[0] if single else out

    def _is_single_object(self, data) -> bool:
        """A flat list / 1-D array of as many values as the model has features is one object, as in the reference's
        ``_is_data_single_object``; the prediction for it is a scalar (or one row)."""
        if isinstance(data, np.ndarray):
            flat = data.ndim == 1 and (data.dtype != object or all(np.ndim(v) == 0 for v in data))
        elif isinstance(data, (list, tuple)):
            flat = len(data) > 0 and all(np.ndim(v) == 0 for v in data)
        else:
            return False
        return bool(flat and self._model is not None and self._model.n_features > 1 and len(data) == self._model.n_features)

    def staged_predict(self, data, prediction_type=None, ntree_start=0, ntree_end=0, eval_period=1, thread_count=-1,
                       verbose=None):
        self._check_fitted()
        pool = data if isinstance(data, Pool) else Pool(data, **self._pool_kwargs())
        fd, ch = self._model.pool_arrays(pool)
        pt = prediction_type or self._default_prediction_type()
        for raw in self._model.staged_raw(fd, ch, ntree_start, ntree_end, eval_period):
            yield self._format(raw, pt)

    def calc_leaf_indexes(self, data, ntree_start=0, ntree_end=0, thread_count=-1, verbose=False):
        self._check_fitted()
        pool = data if isinstance(data, Pool) else Pool(data, **self._pool_kwargs())
        fd, ch = self._model.pool_arrays(pool)
        return self._model.leaf_indices(fd, ch, ntree_start, ntree_end)

    # ------------------------------------------------------------------ attributes
    @property
    def tree_count_(self):
        self._check_fitted()
        return self._model.tree_count

    @property
    def feature_names_(self):
        self._check_fitted()
        return list(self._model.feature_names)

    @property
    def n_features_in_(self):
        self._check_fitted()
        return self._model.n_features

    @property
    def best_iteration_(self):
        return self._best_iteration

    @property
    def best_score_(self):
        return self._best_score

    @property
    def evals_result_(self):
        return self._evals_result

    @property
    def learning_rate_(self):
        self._check_fitted()
        return self._model.params.get("learning_rate")

    @property
    def random_seed_(self):
        self._check_fitted()
        return self._model.params.get("random_seed", 0)

    @property
    def classes_(self):
        self._check_fitted()
        return np.array(self._model.class_names) if self._model.class_names is not None else np.array([])

    @property
    def feature_importances_(self):
        return self.get_feature_importance()

    def get_evals_result(self):
        return self._evals_result

    def get_best_iteration(self):
        return self._best_iteration

    def get_best_score(self):
        return self._best_score

    def get_tree_leaf_counts(self):
        self._check_fitted()
        return np.array([t.leaf_values.shape[0] for t in self._model.trees])

    def get_leaf_values(self):
        self._check_fitted()
        return np.concatenate([t.leaf_values.reshape(-1) for t in self._model.trees])

    def get_leaf_weights(self):
        self._check_fitted()
        return np.concatenate([t.leaf_weights.reshape(-1) for t in self._model.trees])

    def get_scale_and_bias(self):
        self._check_fitted()
        b = self._model.bias
        return self._model.scale, (float(b[0]) if len(b) == 1 else b.tolist())

    def set_scale_and_bias(self, scale, bias):
        self._check_fitted()
        self._model.scale = float(scale)
        self._model.bias = np.broadcast_to(np.asarray(bias, dtype=np.float64), (self._model.dims,)).copy()
        self._model.__dict__.pop("_gpu_predictor", None)

    def get_borders(self):
        self._check_fitted()
        return {f.flat_index: np.asarray(f.borders).tolist() for f in self._model.float_features}

    def get_cat_feature_indices(self):
        self._check_fitted()
        return [c.flat_index for c in self._model.cat_features]

    def shrink(self, ntree_end, ntree_start=0):
        self._check_fitted()
        self._model.shrink(ntree_end, ntree_start)
        self._model.__dict__.pop("_packed", None)
        self._model.__dict__.pop("_gpu_predictor", None)

    def drop_unused_features(self):
        return self

    # ------------------------------------------------------------------ analysis
    def plot_partial_dependence(self, data, features, plot=False, plot_file=None, thread_count=-1):
        """Partial dependence of the raw prediction on one or two numerical features
        (catboost/python-package/catboost/core.py ``plot_partial_dependence``): every document's value of the feature is
        replaced by each border-bucket representative in turn and the predictions are averaged.  Returns
        ``(values, None)``: ``values`` has one axis per feature (bucket order); no figure is drawn."""
        self._check_fitted()
        pool = data if isinstance(data, Pool) else Pool(data, **self._pool_kwargs())
        feats = [features] if isinstance(features, (int, str, np.integer)) else list(features)
        if not 1 <= len(feats) <= 2:
            raise CatBoostError("partial dependence is computed for one or two features")
        m = self._model
        cols, grids = [], []
        for f in feats:
            c = pool.feature_names.index(f) if isinstance(f, str) else int(f)
            ff = next((x for x in m.float_features if x.flat_index == c), None)
            if ff is None:
                raise CatBoostError("partial dependence needs numerical features that the model knows")
            b = np.asarray(ff.borders, dtype=np.float64)
            if len(b) == 0:
                grid = np.array([0.0])
            else:
                # one representative per bucket: below the first border, between neighbours, above the last one
                grid = np.concatenate([[b[0] - 1.0], (b[:-1] + b[1:]) / 2.0, [b[-1] + 1.0]])
            cols.append(pool.float_feature_indices.index(c))
            grids.append(grid)
        fd, ch = m.pool_arrays(pool)
        base = np.array(fd, dtype=np.float32, copy=True)
        out = np.zeros([len(g) for g in grids])
        for idx in np.ndindex(*out.shape):
            work = base.copy()
            for k, j in enumerate(idx):
                work[:, cols[k]] = grids[k][j]
            out[idx] = float(np.mean(m.predict_raw(work, ch)[:, 0]))
        return out, None

    # ------------------------------------------------------------------ uncertainty
    def virtual_ensembles_predict(self, data, prediction_type="VirtEnsembles", ntree_end=0, virtual_ensembles_count=10,
                                  thread_count=-1, verbose=None):
        """Predictions of ``virtual_ensembles_count`` truncated sub-models (catboost/private/libs/algo/apply.cpp:526-606):
        with T trees and period = T // (2 K), ensemble k is the model cut after ``T - (K - 1 - k) * period`` trees.
        ``VirtEnsembles`` returns [documents, K, dimensions]; ``TotalUncertainty`` returns per document
        [mean, knowledge uncertainty] for regression, [mean, knowledge, data uncertainty] for RMSEWithUncertainty and
        [data uncertainty, total uncertainty] for classification."""
        self._check_fitted()
        if prediction_type not in ("VirtEnsembles", "TotalUncertainty"):
            raise CatBoostError("prediction_type must be 'VirtEnsembles' or 'TotalUncertainty'")
        m = self._model
        T = len(m.trees)
        end = T if not ntree_end or ntree_end > T else int(ntree_end)
        K = int(virtual_ensembles_count)
        period = end // (2 * K) if K > 0 else 0
        if period <= 0 or period * K >= end:
            raise CatBoostError(f"Not enough trees in model for {K} virtual Ensembles")
        pool = data if isinstance(data, Pool) else Pool(data, **self._pool_kwargs())
        fd, ch = m.pool_arrays(pool)
        begin = end - period * K
        acc = m.predict_raw(fd, ch, 0, begin)
        ens = []
        for k in range(K):
            lo = begin + k * period
            part = m.predict_raw(fd, ch, lo, lo + period) - np.broadcast_to(m.bias, (m.dims,))
            acc = acc + part
            ens.append(acc.copy())
        ens = np.stack(ens, axis=1)                                        # [n, K, dims]
        loss = m.loss_name
        if loss == "RMSEWithUncertainty":
            ens = ens.copy()
            ens[:, :, 1] = np.exp(2.0 * ens[:, :, 1])
        if prediction_type == "VirtEnsembles":
            return ens
        if loss == "RMSEWithUncertainty":
            return np.stack([ens[:, :, 0].mean(1), ens[:, :, 0].var(1), ens[:, :, 1].mean(1)], axis=1)
        if m.class_names is None:
            return np.stack([ens[:, :, 0].mean(1), ens[:, :, 0].var(1)], axis=1)

        def entropy(p):
            return -(p * np.log(np.clip(p, 1e-300, None))).sum(-1)
        if m.dims == 1:
            p1 = _sigmoid(ens[:, :, 0])
            probs = np.stack([1 - p1, p1], axis=-1)
        else:
            e = np.exp(ens - ens.max(-1, keepdims=True))
            probs = e / e.sum(-1, keepdims=True)
        return np.stack([entropy(probs).mean(1), entropy(probs.mean(1))], axis=1)

    def iterate_leaf_indexes(self, data, ntree_start=0, ntree_end=0):
        """Generator over documents: the leaf index of every tree."""
        for row in self.calc_leaf_indexes(data, ntree_start, ntree_end):
            yield row

    def set_leaf_values(self, new_leaf_values):
        """Replace all leaf values (flat: trees in order, leaves in order, dimensions innermost)."""
        self._check_fitted()
        vals = np.asarray(new_leaf_values, dtype=np.float64).reshape(-1)
        total = sum(t.leaf_values.size for t in self._model.trees)
        if len(vals) != total:
            raise CatBoostError(f"expected {total} leaf values, got {len(vals)}")
        pos = 0
        for t in self._model.trees:
            k = t.leaf_values.size
            t.leaf_values = vals[pos:pos + k].reshape(t.leaf_values.shape).copy()
            pos += k
        self._model.__dict__.pop("_gpu_predictor", None)
        self._model.__dict__.pop("_packed", None)

    def set_feature_names(self, feature_names):
        self._check_fitted()
        names = [str(x) for x in feature_names]
        if len(names) != self._model.n_features:
            raise CatBoostError("feature_names length does not match the number of features of the model")
        self._model.feature_names = names
        for f in self._model.float_features:
            f.name = names[f.flat_index]
        for c in self._model.cat_features:
            c.name = names[c.flat_index]

    def get_metadata(self):
        """Key-value strings stored in the model file (a live dict: assignments are saved with the model)."""
        self._check_fitted()
        return self._model.info

    def get_n_features_in(self):
        self._check_fitted()
        return int(self._model.n_features)

    def get_text_feature_indices(self):
        est = getattr(self._model, "estimators", None) if self._model is not None else None
        return list(getattr(est, "text_indices", []) or []) if est is not None else []

    def get_embedding_feature_indices(self):
        est = getattr(self._model, "estimators", None) if self._model is not None else None
        return list(getattr(est, "embedding_indices", []) or []) if est is not None else []

    def save_borders(self, fname):
        """Borders of the numerical features as ``feature index<TAB>border`` lines (the input_borders format)."""
        self._check_fitted()
        with open(fname, "w") as fh:
            for f in self._model.float_features:
                for b in f.borders:
                    fh.write(f"{f.flat_index}\t{float(b)!r}\n")

    def get_test_eval(self):
        """Raw predictions on the single evaluation set of the last fit."""
        evs = self.get_test_evals()
        if len(evs) != 1:
            raise CatBoostError("the model was fitted with %d evaluation sets: use get_test_evals" % len(evs))
        return evs[0]

    def get_test_evals(self):
        self._check_fitted()
        return [self._raw(p) for p in getattr(self, "_eval_pools", [])]

    def get_object_importance(self, pool, train_pool, top_size=-1, type="Average", update_method="SinglePoint",
                              importance_values_sign="All", thread_count=-1, verbose=False, ostr_type=None,
                              log_cout=None, log_cerr=None):
        """Influence of the training objects on the loss over ``pool`` (LeafInfluence;
        catboost/python-package/catboost/core.py ``get_object_importance``).  Returns ``(indices, scores)`` ordered by
        decreasing |score|: one pair of arrays for ``type='Average'``, one pair of lists for ``'PerObject'``."""
        self._check_fitted()
        from .ostr import object_importance, select
        from .params import parse_loss
        from .train.objectives import make_objective
        if ostr_type is not None:
            type = ostr_type
        if not isinstance(pool, Pool) or not isinstance(train_pool, Pool):
            raise CatBoostError("pool and train_pool must be Pool objects with labels")
        if pool.label is None or train_pool.label is None:
            raise CatBoostError("object importance needs the labels of both datasets")
        params = dict(self._model.params)
        lname, lparams = parse_loss(params.get("loss_function") or self._model.loss_name)
        objective = make_objective(lname, lparams)
        scores = object_importance(self._model, objective, params, train_pool, pool, self._encode_labels(train_pool.label),
                                   self._encode_labels(pool.label), update_method=update_method)
        return select(scores, type, -1 if top_size is None else int(top_size), importance_values_sign)

    def get_feature_importance(self, data=None, type=EFstrType.FeatureImportance, prettified=False, thread_count=-1,
                               verbose=False, fstr_type=None, shap_mode="Auto", model_output="Raw",
                               interaction_indices=None, shap_calc_type="Regular", reference_data=None, log_cout=None,
                               log_cerr=None):
        self._check_fitted()
        from . import fstr
        t = fstr_type or type
        t = getattr(t, "name", t)
        if t in (EFstrType.FeatureImportance, EFstrType.PredictionValuesChange):
            imp = fstr.prediction_values_change(self._model)
        elif t == EFstrType.LossFunctionChange:
            if data is None:
                raise CatBoostError("LossFunctionChange needs a dataset")
            imp = fstr.loss_function_change(self, data)
        elif t == EFstrType.ShapValues:
            if data is None:
                raise CatBoostError("ShapValues needs a dataset")
            return fstr.shap_values(self._model, data if isinstance(data, Pool) else Pool(data))
        elif t == EFstrType.ShapInteractionValues:
            if data is None:
                raise CatBoostError("ShapInteractionValues needs a dataset")
            return fstr.shap_interaction_values(self._model, data if isinstance(data, Pool) else Pool(data))
        elif t == EFstrType.Interaction:
            return fstr.interaction(self._model)
        elif t == EFstrType.PredictionDiff:
            return fstr.prediction_diff(self, data)
        elif t == EFstrType.SageValues:
            if data is None:
                raise CatBoostError("SageValues needs a dataset")
            imp = fstr.sage_values(self, data)
        else:
            raise CatBoostError(f"feature importance type {t!r} is not supported")
        if prettified:
            order = np.argsort(-imp)
            try:
                import pandas as pd
                return pd.DataFrame({"Feature Id": [self._model.feature_names[i] for i in order], "Importances": imp[order]})
            except Exception:
                return [(self._model.feature_names[i], float(imp[i])) for i in order]
        return imp

    def eval_metrics(self, data, metrics, ntree_start=0, ntree_end=0, eval_period=1, thread_count=-1, tmp_dir=None,
                     plot=False, plot_file=None, log_cout=None, log_cerr=None):
        self._check_fitted()
        pool = to_pool(data)
        metrics = [metrics] if isinstance(metrics, str) else list(metrics)
        ms = [make_metric(m) for m in metrics]
        y = self._encode_labels(pool.label)
        out = {str(m): [] for m in ms}
        fd, ch = self._model.pool_arrays(pool)
        kw = {}
        if pool.group_id is not None:
            kw["group_offsets"] = pool.group_offsets()
        if pool.pairs is not None:
            kw["pairs"], kw["pairs_weight"] = pool.pairs, pool.pairs_weight
        for raw in self._model.staged_raw(fd, ch, ntree_start, ntree_end, eval_period, at_iterations=True):
            for m in ms:
                out[str(m)].append(m.eval(raw, y, pool.weight, **kw))
        return out

    def _encode_labels(self, label):
        names = self._model.class_names
        lab = np.asarray(label)
        if names is not None and self._model.loss_name in ("Logloss", "Focal", "MultiClass", "MultiClassOneVsAll"):
            tb = self._model.params.get("target_border")
            if tb is not None and self._model.loss_name in ("Logloss", "Focal"):
                return (lab.astype(np.float64) > float(tb)).astype(np.float32)
            m = {v: i for i, v in enumerate(names)}
            return np.array([m.get(v, -1) for v in lab.tolist()], dtype=np.float32)
        return lab.astype(np.float32) if lab.dtype != object else lab

    def score(self, X, y=None):
        self._check_fitted()
        pool = X if isinstance(X, Pool) else Pool(X, y, **self._pool_kwargs())
        yy = pool.label
        raw = self._raw(pool)
        if self._model.class_names is not None:
            pred = self._format(raw, "Class")
            return float(np.mean(np.asarray(pred).astype(str) == np.asarray(yy).astype(str)))
        if self._estimator_type == "ranker":
            m = make_metric("NDCG")
            return m.eval(raw, np.asarray(yy, dtype=np.float64), pool.weight, group_offsets=pool.group_offsets())
        yy = np.asarray(yy, dtype=np.float64)
        # R2 of the prediction on the scale of the target: models with a log link predict exp(raw)
        p = np.exp(raw[:, 0]) if self._default_prediction_type() == "Exponent" else raw[:, 0]
        den = np.sum((yy - yy.mean()) ** 2)
        return float(1 - np.sum((yy - p) ** 2) / den) if den > 0 else 0.0

    # ------------------------------------------------------------------ persistence
    def save_model(self, fname, format="cbm", export_parameters=None, pool=None):
        self._check_fitted()
        from .models import io as mio
        mio.save_model(self._model, fname, format, export_parameters, pool)

    def load_model(self, fname=None, format="cbm", stream=None, blob=None):
        from .models import io as mio
        if blob is not None:
            self._model = mio.load_model_blob(blob, format)
        elif stream is not None:
            self._model = mio.load_model_blob(stream.read(), format)
        else:
            self._model = mio.load_model(fname, format)
        return self

    def _serialize_model(self):
        from .models import io as mio
        return mio.model_to_cbm_bytes(self._model)

    def __getstate__(self):
        st = dict(self.__dict__)
        st.pop("_eval_pools", None)
        if self._model is not None:
            m = self._model.copy()
            for k in ("_gpu_predictor", "_packed", "_split_cache"):
                m.__dict__.pop(k, None)
            st["_model"] = m
        return st

    def calc_feature_statistics(self, data, target=None, feature=None, prediction_type=None, cat_feature_values=None,
                                plot=False, max_cat_features_on_plot=10, thread_count=-1, plot_file=None):
        """Per-bucket statistics of numerical features (catboost/python-package/catboost/core.py
        ``calc_feature_statistics``): borders, the bucket of every object, mean target, mean prediction, objects per
        bucket, and the mean prediction when the feature of every object is moved into each bucket.  Returns the dict of
        one feature, or {feature: dict} for a list of features; nothing is drawn."""
        self._check_fitted()
        pool = data if isinstance(data, Pool) else Pool(data, target, **self._pool_kwargs())
        y = pool.label if target is None else np.asarray(target)
        if y is None:
            raise CatBoostError("calc_feature_statistics needs the target")
        y = np.asarray(self._encode_labels(y), dtype=np.float64).reshape(len(y), -1)[:, 0]
        m = self._model
        if prediction_type is None:
            prediction_type = "Probability" if m.class_names is not None and m.dims == 1 else "RawFormulaVal"

        def pred_of(raw):
            out = self._format(raw, prediction_type)
            out = np.asarray(out, dtype=np.float64)
            return out[:, -1] if out.ndim == 2 else out
        feats = [feature] if isinstance(feature, (int, str, np.integer)) else list(feature if feature is not None else
                                                                                  [f.flat_index for f in m.float_features])
        fd, ch = m.pool_arrays(pool)
        base_pred = pred_of(m.predict_raw(fd, ch))
        res = {}
        for f in feats:
            c = pool.feature_names.index(f) if isinstance(f, str) else int(f)
            ff = next((x for x in m.float_features if x.flat_index == c), None)
            if ff is None:
                raise CatBoostError("feature statistics are computed for numerical features of the model")
            col = m.float_features.index(ff)
            borders = np.asarray(ff.borders, dtype=np.float32)
            bins = np.searchsorted(borders, fd[:, col], side="left").astype(np.int64)
            nb = len(borders) + 1
            cnt = np.bincount(bins, minlength=nb).astype(np.float64)
            safe = np.maximum(cnt, 1.0)
            w = pool.weight if pool.weight is not None else np.ones(len(y))
            wsum = np.bincount(bins, weights=w, minlength=nb)
            grid = np.concatenate([[borders[0] - 1.0], (borders[:-1] + borders[1:]) / 2.0, [borders[-1] + 1.0]]) \
                if len(borders) else np.array([0.0])
            varying = np.zeros(nb)
            work = np.array(fd, dtype=np.float32, copy=True)
            for j in range(nb):
                work[:, col] = grid[j]
                varying[j] = float(np.mean(pred_of(m.predict_raw(work, ch))))
            res[f] = {"borders": borders, "binarized_feature": bins,
                      "mean_target": np.bincount(bins, weights=y, minlength=nb) / safe,
                      "mean_weighted_target": np.bincount(bins, weights=y * w, minlength=nb) / np.maximum(wsum, 1e-300),
                      "mean_prediction": np.bincount(bins, weights=base_pred, minlength=nb) / safe,
                      "objects_per_bin": cnt.astype(np.int64), "predictions_on_varying_feature": varying}
        return res[feats[0]] if isinstance(feature, (int, str, np.integer)) else res

    def compare(self, model, data, metrics, ntree_start=0, ntree_end=0, eval_period=1, thread_count=-1, tmp_dir=None,
                log_cout=None, log_cerr=None):
        """Metric curves of this model and of ``model`` on the same data: {metric: (own values, other values)}.
        (The reference draws them in a notebook widget.)"""
        a = self.eval_metrics(data, metrics, ntree_start, ntree_end, eval_period)
        b = model.eval_metrics(data, metrics, ntree_start, ntree_end, eval_period)
        return {k: (a[k], b[k]) for k in a}

    def create_metric_calcer(self, metrics, ntree_start=0, ntree_end=0, eval_period=1, thread_count=-1, tmp_dir=None):
        """Metric values over several batches of data: ``add(pool)`` any number of times, then ``eval_metrics()``."""
        self._check_fitted()
        return _BatchMetricCalcer(self, metrics, ntree_start, ntree_end, eval_period)

    def plot_predictions(self, data, features_to_change, plot=False, plot_file=None):
        """Predictions of every object of ``data`` while one numerical feature takes each bucket of its grid.
        Returns ({feature: array [objects, buckets]}, None); nothing is drawn."""
        self._check_fitted()
        pool = data if isinstance(data, Pool) else Pool(data, **self._pool_kwargs())
        m = self._model
        fd, ch = m.pool_arrays(pool)
        out = {}
        for f in features_to_change:
            c = pool.feature_names.index(f) if isinstance(f, str) else int(f)
            ff = next((x for x in m.float_features if x.flat_index == c), None)
            if ff is None:
                raise CatBoostError("plot_predictions varies numerical features of the model")
            col = m.float_features.index(ff)
            b = np.asarray(ff.borders, dtype=np.float64)
            grid = np.concatenate([[b[0] - 1.0], (b[:-1] + b[1:]) / 2.0, [b[-1] + 1.0]]) if len(b) else np.array([0.0])
            vals = np.zeros((fd.shape[0], len(grid)))
            work = np.array(fd, dtype=np.float32, copy=True)
            for j, g in enumerate(grid):
                work[:, col] = g
                vals[:, j] = m.predict_raw(work, ch)[:, 0]
            out[f] = vals
        return out, None

    def plot_tree(self, tree_idx=0, pool=None):
        """The tree as a graph: a ``graphviz.Source`` when the graphviz package is importable, otherwise an object whose
        ``source`` attribute (and ``str()``) is the same DOT text (catboost/python-package/catboost/core.py plot_tree).
        Leaves show their values; inner nodes the condition whose "yes" branch goes right."""
        self._check_fitted()
        m = self._model
        if not 0 <= int(tree_idx) < len(m.trees):
            raise CatBoostError(f"tree_idx must be in [0, {len(m.trees)})")
        t = m.trees[int(tree_idx)]
        fname = {f.feature_index: (f.name or str(f.flat_index)) for f in m.float_features}
        cname = {c.feature_index: (c.name or str(c.flat_index)) for c in m.cat_features}

        def cond(si):
            sp = m.splits[int(si)]
            if sp.kind == "float":
                return f"{fname.get(sp.feature, sp.feature)}, value > {float(sp.border):.9g}"
            if sp.kind == "onehot":
                text = m.cat_hash_to_string.get(int(sp.value), int(sp.value)) if getattr(m, "cat_hash_to_string", None) else int(sp.value)
                return f"{cname.get(sp.feature, sp.feature)}, value = {text}"
            c = m.ctrs[sp.feature]
            cats = ", ".join(str(cname.get(k, k)) for k in c.cat_features)
            return f"{c.ctr_type} ctr of {{{cats}}}, value > {float(sp.border):.9g}"

        def leaf_text(v):
            v = np.asarray(v, dtype=np.float64).reshape(-1)
            return "val = " + (f"{v[0]:.6g}" if v.size == 1 else "[" + ", ".join(f"{x:.4g}" for x in v) + "]")

        lines = ["digraph {", "  node [shape=rectangle];"]
        from .models.model import ObliviousTree
        if isinstance(t, ObliviousTree):
            depth = len(t.splits)
            # node ids by (level, prefix of the decisions taken so far); the split of level k decides bit k of the leaf index
            for level in range(depth):
                for pre in range(1 << level):
                    lines.append(f'  n{level}_{pre} [label="{cond(t.splits[level])}"];')
            for leaf in range(1 << depth):
                lines.append(f'  leaf{leaf} [shape=ellipse, label="{leaf_text(t.leaf_values[leaf])}"];')
            for level in range(depth):
                for pre in range(1 << level):
                    for bit, lab in ((0, "No"), (1, "Yes")):
                        nxt = pre | (bit << level)
                        dst = f"leaf{nxt}" if level + 1 == depth else f"n{level + 1}_{nxt}"
                        lines.append(f'  n{level}_{pre} -> {dst} [label="{lab}"];')
            if depth == 0:
                pass
        else:
            for node in range(len(t.split_of_node)):
                if t.split_of_node[node] >= 0:
                    lines.append(f'  n{node} [label="{cond(t.split_of_node[node])}"];')
                    lines.append(f'  n{node} -> n{int(t.left[node])} [label="No"];')
                    lines.append(f'  n{node} -> n{int(t.right[node])} [label="Yes"];')
                else:
                    lines.append(f'  n{node} [shape=ellipse, label="{leaf_text(t.leaf_values[int(t.leaf_of_node[node])])}"];')
        lines.append("}")
        dot = "\n".join(lines)
        try:
            import graphviz
            return graphviz.Source(dot)
        except ImportError:
            class _DotGraph:
                def __init__(self, source):
                    self.source = source

                def __str__(self):
                    return self.source

                def render(self, *a, **k):
                    raise CatBoostError("rendering needs the graphviz package; the DOT text is in .source")
            return _DotGraph(dot)

    # ------------------------------------------------------------------ search helpers
    def grid_search(self, param_grid, X, y=None, cv=3, partition_random_seed=0, calc_cv_statistics=True,
                    search_by_train_test_split=True, refit=True, shuffle=True, stratified=None, train_size=0.8,
                    verbose=True, plot=False, plot_file=None, log_cout=None, log_cerr=None):
        from .tuning import grid_search
        return grid_search(self, param_grid, X, y, cv, partition_random_seed, search_by_train_test_split, refit, shuffle,
                           stratified, train_size, verbose)

    def randomized_search(self, param_distributions, X, y=None, cv=3, n_iter=10, partition_random_seed=0,
                          calc_cv_statistics=True, search_by_train_test_split=True, refit=True, shuffle=True,
                          stratified=None, train_size=0.8, verbose=True, plot=False, plot_file=None, log_cout=None,
                          log_cerr=None):
        from .tuning import randomized_search
        return randomized_search(self, param_distributions, X, y, cv, n_iter, partition_random_seed,
                                 search_by_train_test_split, refit, shuffle, stratified, train_size, verbose)

    def select_features(self, X, y=None, eval_set=None, features_for_select=None, num_features_to_select=None,
                        algorithm=None, steps=1, shap_calc_type=None, train_final_model=True, verbose=None,
                        logging_level=None, plot=False, plot_file=None, log_cout=None, log_cerr=None, grouping=None,
                        features_tags_for_select=None, num_features_tags_to_select=None):
        from .tuning import select_features
        return select_features(self, X, y, eval_set, features_for_select, num_features_to_select, steps,
                               train_final_model)


class CatBoostClassifier(CatBoost):
    _default_loss = "Logloss"
    _estimator_type = "classifier"

    _CLASSIFICATION_LOSSES = ("Logloss", "CrossEntropy", "Focal", "MultiClass", "MultiClassOneVsAll", "MultiLogloss",
                              "MultiCrossEntropy")

    def fit(self, X, y=None, **kw):
        loss = self._init_params.get("loss_function", self._init_params.get("objective"))
        if isinstance(loss, str) and loss.split(":")[0] not in self._CLASSIFICATION_LOSSES:
            # catboost/python-package/catboost/core.py CatBoostClassifier._check_is_compatible_loss
            raise CatBoostError(f"Invalid loss_function='{loss}': for classifier use Logloss, CrossEntropy, MultiClass, "
                                "MultiClassOneVsAll, MultiLogloss, MultiCrossEntropy, Focal or a custom objective object")
        if "loss_function" not in self._init_params and "objective" not in self._init_params:
            lab = X.label if isinstance(X, Pool) else y
            if lab is not None:
                lab = np.asarray(lab)
                if lab.ndim == 1 or (lab.ndim == 2 and lab.shape[1] == 1):
                    nuniq = len(np.unique(lab))
                    if nuniq > 2 and self._init_params.get("target_border") is None:
                        self._init_params["loss_function"] = "MultiClass"
                        try:
                            return super().fit(X, y, **kw)
                        finally:
                            self._init_params.pop("loss_function", None)
                elif lab.ndim == 2:
                    self._init_params["loss_function"] = "MultiLogloss"
                    try:
                        return super().fit(X, y, **kw)
                    finally:
                        self._init_params.pop("loss_function", None)
        return super().fit(X, y, **kw)

    def _default_prediction_type(self):
        return "Class"

    def predict_proba(self, X, ntree_start=0, ntree_end=0, thread_count=-1, verbose=None, task_type="CPU"):
        return self.predict(X, "Probability", ntree_start, ntree_end, thread_count, verbose, task_type)

    def predict_log_proba(self, X, ntree_start=0, ntree_end=0, thread_count=-1, verbose=None, task_type="CPU"):
        return self.predict(X, "LogProbability", ntree_start, ntree_end, thread_count, verbose, task_type)

    def staged_predict_proba(self, data, ntree_start=0, ntree_end=0, eval_period=1, thread_count=-1, verbose=None):
        return self.staged_predict(data, "Probability", ntree_start, ntree_end, eval_period, thread_count, verbose)

    def staged_predict_log_proba(self, data, ntree_start=0, ntree_end=0, eval_period=1, thread_count=-1, verbose=None):
        return self.staged_predict(data, "LogProbability", ntree_start, ntree_end, eval_period, thread_count, verbose)

    def set_probability_threshold(self, binclass_probability_threshold=None):
        """Probability above which a binary model predicts the positive class (stored with the model); None restores 0.5."""
        self._check_fitted()
        if binclass_probability_threshold is None:
            self._model.info.pop("binclass_probability_threshold", None)
            return
        t = float(binclass_probability_threshold)
        if not 0.0 <= t <= 1.0:
            raise CatBoostError("the probability threshold must be in [0, 1]")
        self._model.info["binclass_probability_threshold"] = repr(t)

    def get_probability_threshold(self):
        self._check_fitted()
        return float(self._model.info.get("binclass_probability_threshold", 0.5))


class CatBoostRegressor(CatBoost):
    _default_loss = "RMSE"
    _estimator_type = "regressor"

    def fit(self, X, y=None, **kw):
        loss = self._init_params.get("loss_function", self._init_params.get("objective"))
        if isinstance(loss, str) and loss.split(":")[0] in CatBoostClassifier._CLASSIFICATION_LOSSES + (
                "YetiRank", "YetiRankPairwise", "PairLogit", "PairLogitPairwise", "QuerySoftMax", "QueryCrossEntropy",
                "LambdaMart", "StochasticRank", "StochasticFilter"):
            raise CatBoostError(f"Invalid loss_function='{loss}': for regressor use RMSE, MultiRMSE, SurvivalAft, MAE, Quantile, "
                                "LogLinQuantile, Poisson, MAPE, Lq, RMSPE or a custom objective object")
        return super().fit(X, y, **kw)

    def _default_prediction_type(self):
        # catboost/python-package/catboost/core.py CatBoostRegressor._get_default_prediction_type: models with a log link
        # answer on the scale of the target
        loss = str(self._model.loss_name if self._model is not None else self._init_params.get("loss_function") or "")
        if loss.startswith("Poisson") or loss.startswith("Tweedie"):
            return "Exponent"
        if loss == "RMSEWithUncertainty":
            return "RMSEWithUncertainty"
        return "RawFormulaVal"


class CatBoostRanker(CatBoost):
    _default_loss = "YetiRank"
    _estimator_type = "ranker"


def train(pool=None, params=None, dtrain=None, logging_level=None, verbose=None, iterations=None,
          num_boost_round=None, evals=None, eval_set=None, plot=None, verbose_eval=None, metric_period=None,
          early_stopping_rounds=None, save_snapshot=None, snapshot_file=None, snapshot_interval=None, init_model=None,
          log_cout=None, log_cerr=None):
    """Functional training entry point (catboost.train)."""
    params = dict(params or {})
    if iterations is not None:
        params["iterations"] = iterations
    if num_boost_round is not None:
        params["iterations"] = num_boost_round
    pool = pool if pool is not None else dtrain
    if pool is None:
        raise CatBoostError("pool is required")
    model = CatBoost(params)
    model.fit(pool, eval_set=eval_set if eval_set is not None else evals, verbose=verbose if verbose is not None else verbose_eval,
              logging_level=logging_level, metric_period=metric_period, early_stopping_rounds=early_stopping_rounds,
              save_snapshot=save_snapshot, snapshot_file=snapshot_file, snapshot_interval=snapshot_interval,
              init_model=init_model, log_cout=log_cout)
    return model


def sum_models(models, weights=None, ctr_merge_policy="IntersectingCountersAverage"):
    from .models.ops import sum_models as _sum
    out = CatBoost()
    out._model = _sum([m._model for m in models], weights, ctr_merge_policy)
    out.__class__ = models[0].__class__
    return out


def to_regressor(model):
    out = CatBoostRegressor()
    out.__dict__.update(copy.deepcopy(model.__dict__))
    return out


def to_classifier(model):
    out = CatBoostClassifier()
    out.__dict__.update(copy.deepcopy(model.__dict__))
    return out


def to_ranker(model):
    out = CatBoostRanker()
    out.__dict__.update(copy.deepcopy(model.__dict__))
    return out


class _BatchMetricCalcer:
    """Collects raw staged predictions and targets of several batches; evaluates the metrics over all of them."""

    def __init__(self, model, metrics, ntree_start, ntree_end, eval_period):
        self.model, self.metrics = model, [metrics] if isinstance(metrics, str) else list(metrics)
        self.range = (ntree_start, ntree_end, max(1, int(eval_period)))
        self.stages, self.labels, self.weights = None, [], []

    def add(self, pool):
        if not isinstance(pool, Pool) or pool.label is None:
            raise CatBoostError("add() needs a Pool with labels")
        m = self.model._model
        fd, ch = m.pool_arrays(pool)
        staged = list(m.staged_raw(fd, ch, self.range[0], self.range[1], self.range[2], at_iterations=True))
        if self.stages is None:
            self.stages = [[s.copy()] for s in staged]
        else:
            for acc, s in zip(self.stages, staged):
                acc.append(s.copy())
        self.labels.append(np.asarray(self.model._encode_labels(pool.label)))
        self.weights.append(np.ones(pool.num_row()) if pool.weight is None else np.asarray(pool.weight, dtype=np.float64))

    def eval_metrics(self):
        from .metrics import make_metric
        if self.stages is None:
            raise CatBoostError("no data was added")
        y, w = np.concatenate(self.labels), np.concatenate(self.weights)
        out = {}
        for name in self.metrics:
            mt = make_metric(name)
            out[str(mt)] = [mt.eval(np.concatenate(parts), y, w) for parts in self.stages]
        return out
