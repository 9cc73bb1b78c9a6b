"""Polynomial view of a model of oblivious trees (catboost/python-package/catboost/monoforest.py,
catboost/libs/monoforest): every tree is a function of its binary split indicators, so it expands into a multilinear
polynomial; equal monomials of different trees are merged.

For a tree with splits s_0..s_{d-1} and leaf values v[mask] (bit k of ``mask`` = outcome of split k) the coefficient of
the monomial prod_{k in S} s_k is the Moebius transform  c[S] = sum_{T subset of S} (-1)^{|S| - |T|} v[T].  Inside a
monomial two conditions on the same numerical feature collapse into the stronger one (x > a and x > b = x > max(a, b)).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import numpy as np

from .data.pool import CatBoostError
from .models.model import ObliviousTree


class Split:
    def __init__(self, feature_idx, split_type, border):
        self.feature_idx, self.split_type, self.border = feature_idx, split_type, border

    def __str__(self):
        return f"[F{self.feature_idx} {'>' if self.split_type == 'TakeGreater' else '='} {self.border}]"

    __repr__ = __str__


class Monom:
    def __init__(self, splits, value, weight):
        self.splits, self.value, self.weight = splits, value, weight

    def __str__(self):
        head = "(" + ", ".join(f"{v:.9g}" for v in self.value) + ")"
        return head + ("" if not self.splits else " * " + " * ".join(str(s) for s in self.splits))

    __repr__ = __str__


class BorderExplanation:
    def __init__(self, border, probability, expected_value_change):
        self.border, self.probability, self.expected_value_change = border, probability, expected_value_change

    def __repr__(self):
        return f"(border={self.border}, probability={self.probability:.4g}, expected_value_change={self.expected_value_change})"


class FeatureExplanation:
    def __init__(self, feature, type, expected_bias, borders_explanations):
        self.feature, self.type = feature, type
        self.expected_bias, self.borders_explanations = expected_bias, borders_explanations

    def __repr__(self):
        return f"FeatureExplanation(feature={self.feature}, type={self.type}, borders={self.borders_explanations})"

    def dimension(self):
        return len(self.expected_bias)

    def calc_strength(self, dim=None):
        """Standard deviation of the feature's contribution if its border indicators were independent."""
        dims = range(self.dimension()) if dim is None else [dim]
        tot = 0.0
        for b in self.borders_explanations:
            p = b.probability
            tot += sum(b.expected_value_change[d] ** 2 for d in dims) * p * (1.0 - p)
        return float(np.sqrt(tot))

    def calc_pdp(self, dim=None):
        """(borders, values): the expected contribution of the feature below the first border and after each border."""
        d = 0 if dim is None else dim
        xs = [b.border for b in self.borders_explanations]
        ys = [self.expected_bias[d]]
        for b in self.borders_explanations:
            ys.append(ys[-1] + b.expected_value_change[d])
        return xs, ys


def _check_model(model):
    m = getattr(model, "_model", model)
    if m is None:
        raise CatBoostError("model is not fitted")
    if not all(isinstance(t, ObliviousTree) for t in m.trees):
        raise CatBoostError("the polynomial view needs a model of symmetric trees")
    if m.ctrs:
        raise CatBoostError("models with CTR features have no polynomial over raw features")
    return m


def _split_key(m, si) -> Tuple:
    sp = m.splits[si]
    if sp.kind == "float":
        return (m.float_features[sp.feature].flat_index, "TakeGreater", float(sp.border))
    return (m.cat_features[sp.feature].flat_index if sp.feature < len(m.cat_features) else sp.feature, "TakeEqual",
            int(sp.value))


def to_polynom(model) -> List[Monom]:
    m = _check_model(model)
    dims = m.dims
    acc: Dict[Tuple, np.ndarray] = {}
    wacc: Dict[Tuple, float] = {}
    for t in m.trees:
        d = len(t.splits)
        coef = np.array(t.leaf_values, dtype=np.float64).reshape(1 << d, dims) * m.scale
        for k in range(d):                                    # in-place Moebius transform over the subset lattice
            bit = 1 << k
            idx = np.arange(1 << d)
            hi = idx[(idx & bit) != 0]
            coef[hi] -= coef[hi ^ bit]
        keys = [_split_key(m, si) for si in t.splits]
        wts = np.asarray(t.leaf_weights, dtype=np.float64).reshape(-1) if t.leaf_weights is not None else np.zeros(1 << d)
        for mask in range(1 << d):
            if not np.any(coef[mask]):
                continue
            chosen = [keys[k] for k in range(d) if mask >> k & 1]
            merged: Dict[Tuple, float] = {}
            contradiction = False
            for f, kind, b in chosen:
                if kind == "TakeGreater":
                    merged[(f, kind)] = max(merged.get((f, kind), -np.inf), b)
                else:
                    if (f, kind) in merged and merged[(f, kind)] != b:
                        contradiction = True               # a category cannot equal two values: the monomial is zero
                    merged[(f, kind)] = b
            if contradiction:
                continue
            key = tuple(sorted((f, kind, b) for (f, kind), b in merged.items()))
            acc[key] = acc.get(key, 0.0) + coef[mask]
            # weight of a monomial: training weight of the leaves where all of its conditions hold
            sel = [l for l in range(1 << d) if (l & mask) == mask]
            wacc[key] = wacc.get(key, 0.0) + float(wts[sel].sum()) if len(wts) == (1 << d) else 0.0
    bias = np.broadcast_to(np.asarray(m.bias, dtype=np.float64), (dims,))
    acc[()] = acc.get((), 0.0) + bias
    out = []
    for key in sorted(acc, key=lambda k: (len(k), k)):
        if np.any(acc[key]) or key == ():
            out.append(Monom([Split(f, kind, b) for f, kind, b in key], [float(v) for v in np.ravel(acc[key])],
                             wacc.get(key, 0.0)))
    return out


def to_polynom_string(model) -> str:
    return " + ".join(str(mn) for mn in to_polynom(model))


def eval_polynom(monoms: List[Monom], X: np.ndarray, cat_hashes: Optional[Dict[int, np.ndarray]] = None) -> np.ndarray:
    """Value of the polynomial on rows of ``X`` (flat feature order; ``cat_hashes`` maps a categorical flat index to the
    hashes of its column)."""
    X = np.asarray(X, dtype=np.float32)
    dims = len(monoms[0].value)
    out = np.zeros((X.shape[0], dims))
    for mn in monoms:
        ind = np.ones(X.shape[0], dtype=bool)
        for s in mn.splits:
            if s.split_type == "TakeGreater":
                ind &= X[:, s.feature_idx] > np.float32(s.border)
            else:
                ind &= (cat_hashes or {})[s.feature_idx] == s.border
        out[ind] += np.asarray(mn.value)
    return out


def explain_features(model) -> List[FeatureExplanation]:
    """Per feature: for every border the weighted probability of passing it and the change of the expected model value
    when it is passed, both estimated from the leaf weights stored in the model."""
    m = _check_model(model)
    dims = m.dims
    change: Dict[Tuple, np.ndarray] = {}
    prob_num: Dict[Tuple, float] = {}
    prob_den: Dict[Tuple, float] = {}
    for t in m.trees:
        d = len(t.splits)
        vals = np.array(t.leaf_values, dtype=np.float64).reshape(1 << d, dims) * m.scale
        w = np.asarray(t.leaf_weights, dtype=np.float64).reshape(-1)
        if len(w) != (1 << d) or w.sum() <= 0:
            w = np.ones(1 << d)
        leaves = np.arange(1 << d)
        for k, si in enumerate(t.splits):
            on = (leaves >> k & 1) == 1
            w1, w0 = w[on].sum(), w[~on].sum()
            if w1 <= 0 or w0 <= 0:
                continue
            key = _split_key(m, si)
            delta = (vals[on] * w[on, None]).sum(0) / w1 - (vals[~on] * w[~on, None]).sum(0) / w0
            change[key] = change.get(key, 0.0) + delta
            prob_num[key] = prob_num.get(key, 0.0) + w1
            prob_den[key] = prob_den.get(key, 0.0) + w1 + w0
    by_feature: Dict[Tuple, list] = {}
    for key in change:
        by_feature.setdefault((key[0], key[1]), []).append(key)
    out = []
    for (f, kind), keys in sorted(by_feature.items()):
        keys.sort(key=lambda k: k[2])
        borders = [BorderExplanation(k[2], prob_num[k] / prob_den[k], [float(v) for v in change[k]]) for k in keys]
        bias = -np.sum([np.asarray(b.expected_value_change) * b.probability for b in borders], axis=0)
        out.append(FeatureExplanation(f, "Float" if kind == "TakeGreater" else "OneHot", [float(v) for v in bias], borders))
    return out


def calc_features_strength(model) -> List[float]:
    m = _check_model(model)
    res = [0.0] * m.n_features
    for fe in explain_features(model):
        res[fe.feature] = fe.calc_strength()
    return res
