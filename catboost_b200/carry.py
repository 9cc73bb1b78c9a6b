"""``carry`` and ``uplift`` (catboost/python-package/catboost/carry.py, catboost/libs/carry_model/carry.h): models with some
float features fixed.

``carry(model, {feature: value})`` returns a model that no longer reads the given features: every split on them has a
known outcome.  With lists of values (all of one length k) the result has k output dimensions, one per set of values.
``uplift(model, {feature: (base, next)})`` returns the model of the difference f(x | features = next) - f(x | features =
base) in raw-formula units.  Features are named by flat index (the column in the data) or by name.  Symmetric trees only.
"""
from __future__ import annotations

import numpy as np

from .data.pool import CatBoostError
from .models.model import ObliviousTree
from .models.ops import carry_model


def _float_index(core, key):
    for ff in core.float_features:
        if (isinstance(key, str) and ff.name == key) or (not isinstance(key, str) and ff.flat_index == int(key)):
            return ff.feature_index
    if isinstance(key, str) and key in list(core.feature_names):
        return _float_index(core, list(core.feature_names).index(key))
    raise CatBoostError(f"carry: {key!r} is not a float feature of the model")


def _wrap(model, core):
    out = model.copy() if hasattr(model, "copy") else model
    if hasattr(out, "_model"):
        out._model = core
        return out
    return core


def _checked(features):
    if not isinstance(features, dict):
        raise CatBoostError("features must be a dict")
    kinds = {type(k) is str for k in features}
    if len(kinds) > 1:
        raise CatBoostError("feature keys must be all names or all flat indices")


def carry(model, features):
    _checked(features)
    core = model._model if hasattr(model, "_model") else model
    lists = {k: (list(v) if isinstance(v, (list, tuple)) else [v]) for k, v in features.items()}
    if not lists:
        return _wrap(model, core.copy())
    k = {len(v) for v in lists.values()}
    if len(k) != 1:
        raise CatBoostError("carry: value lists must all have the same length")
    k = k.pop()
    variants = [carry_model(core, {_float_index(core, f): float(v[j]) for f, v in lists.items()}) for j in range(k)]
    if k == 1:
        return _wrap(model, variants[0])
    if core.dims != 1:
        raise CatBoostError("carry with several values needs a one-dimensional model")
    out = variants[0].copy()
    out.trees = [ObliviousTree(list(t0.splits), np.stack([np.asarray(v.trees[i].leaf_values).reshape(-1) for v in variants], 1),
                               np.asarray(t0.leaf_weights)) for i, t0 in enumerate(variants[0].trees)]
    out.dims = k
    out.bias = np.repeat(np.asarray(core.bias, dtype=np.float64).reshape(-1)[:1], k)
    return _wrap(model, out)


def uplift(model, features):
    _checked(features)
    core = model._model if hasattr(model, "_model") else model
    if core.dims != 1:
        raise CatBoostError("uplift needs a one-dimensional model")
    base = carry_model(core, {_float_index(core, f): float(v[0]) for f, v in features.items()})
    nxt = carry_model(core, {_float_index(core, f): float(v[1]) for f, v in features.items()})
    out = base.copy()
    out.trees = [ObliviousTree(list(tb.splits), np.asarray(tn.leaf_values, dtype=np.float64) - np.asarray(tb.leaf_values, dtype=np.float64),
                               np.asarray(tb.leaf_weights)) for tb, tn in zip(base.trees, nxt.trees)]
    out.bias = np.zeros_like(np.asarray(core.bias, dtype=np.float64))
    return _wrap(model, out)
