"""Model algebra: weighted sum of models (``sum_models``, catboost/libs/model/model.cpp SumModels)."""
from __future__ import annotations

import numpy as np

from ..data.pool import CatBoostError
from .model import Model, NonSymmetricTree, ObliviousTree


def sum_models(models, weights=None, ctr_merge_policy="IntersectingCountersAverage") -> Model:
    if not models:
        raise CatBoostError("sum_models needs at least one model")
    weights = [1.0] * len(models) if weights is None else list(weights)
    if len(weights) != len(models):
        raise CatBoostError("weights and models differ in length")
    base = models[0]
    out = base.copy()
    out.trees, out.splits = [], []
    out.__dict__.pop("_split_cache", None)
    out.__dict__.pop("_packed", None)
    out.__dict__.pop("_gpu_predictor", None)
    out.bias = np.zeros(base.dims)
    out.scale = 1.0
    # union of borders per float feature
    for m in models:
        if m.dims != base.dims:
            raise CatBoostError("models have different prediction dimensions")
        if len(m.float_features) != len(base.float_features):
            raise CatBoostError("models were trained on different feature sets")
    for j, ff in enumerate(out.float_features):
        allb = np.unique(np.concatenate([np.asarray(m.float_features[j].borders, dtype=np.float32) for m in models]))
        out.float_features[j] = type(ff)(ff.flat_index, ff.feature_index, allb, ff.nan_mode, ff.has_nans, ff.name)
    out.ctrs = []
    for m, w in zip(models, weights):
        ctr_shift = len(out.ctrs)
        out.ctrs += list(m.ctrs)
        for k, v in m.one_hot.items():
            out.one_hot.setdefault(k, v)
        out.bias = out.bias + w * np.broadcast_to(m.bias, (base.dims,))
        remap = {}
        for i, sp in enumerate(m.splits):
            sp2 = type(sp)(sp.kind, sp.feature + (ctr_shift if sp.kind == "ctr" else 0), sp.border, sp.value)
            remap[i] = out.split_index(sp2)
        for t in m.trees:
            if isinstance(t, ObliviousTree):
                out.trees.append(ObliviousTree([remap[s] for s in t.splits], t.leaf_values * (w * m.scale), t.leaf_weights))
            else:
                so = np.array([remap[s] if s >= 0 else -1 for s in t.split_of_node], dtype=np.int32)
                out.trees.append(NonSymmetricTree(so, t.left, t.right, t.leaf_of_node, t.leaf_values * (w * m.scale),
                                                  t.leaf_weights))
    return out


def carry_model(model: Model, float_values: dict) -> Model:
    """A copy of ``model`` with some float features fixed to given values (the reference's ``CarryModel``,
    catboost/libs/carry_model/carry.h): every split on a carried feature has a known outcome, so symmetric trees lose
    those levels (their leaves are the matching half of the old ones) and the model no longer reads the feature --
    whatever value the data holds for it.  ``float_values``: {float feature index: value}.  Oblivious trees only."""
    out = model.copy()
    for key in ("_split_cache", "_packed", "_gpu_predictor", "_gpu_predictor_multi"):
        out.__dict__.pop(key, None)
    carried = {int(k): float(v) for k, v in float_values.items()}
    new_trees = []
    for t in model.trees:
        if not isinstance(t, ObliviousTree):
            raise CatBoostError("carry_model supports symmetric (oblivious) trees")
        keep_levels, fixed_bits = [], 0
        for level, s in enumerate(t.splits):
            sp = model.splits[s]
            if sp.kind == "float" and sp.feature in carried:
                v = carried[sp.feature]
                goes_right = (not np.isnan(v)) and v > sp.border
                if np.isnan(v):
                    ff = model.float_features[sp.feature]
                    goes_right = str(getattr(ff, "nan_mode", "Min")) == "Max"
                fixed_bits |= (1 if goes_right else 0) << level
            else:
                keep_levels.append(level)
        n_new = 1 << len(keep_levels)
        idx = np.zeros(n_new, dtype=np.int64)
        for j in range(n_new):
            old = fixed_bits
            for k, level in enumerate(keep_levels):
                old |= ((j >> k) & 1) << level
            idx[j] = old
        vals = np.asarray(t.leaf_values)[idx]
        wts = np.asarray(t.leaf_weights)[idx] if len(t.leaf_weights) else np.zeros(n_new)
        new_trees.append(ObliviousTree([t.splits[level] for level in keep_levels], vals, wts))
    out.trees = new_trees
    return out
