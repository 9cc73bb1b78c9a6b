"""Feature importances and SHAP values.

* PredictionValuesChange: for every split, the weighted squared deviation of the two children's values from their
  weighted mean, summed over the trees and normalised to 100 (catboost/libs/fstr/calc_fstr.cpp).
* ShapValues: exact TreeSHAP (path-dependent, covers = leaf weights), the algorithm the reference implements in
  catboost/libs/fstr/shap_values.cpp; output ``[n, n_features + 1]`` (last column = expected value), or
  ``[n, dims, n_features + 1]`` for multi-dimensional models.
* LossFunctionChange: change of the loss when a feature's SHAP contribution is replaced by its mean.
* SageValues: Shapley additive global importance by sampling (marginal imputation of features in random order).
* Interaction: pairwise strength of features that meet in the same tree.
"""
from __future__ import annotations

import math

import numpy as np

from .data.pool import CatBoostError, Pool
from .metrics import make_metric
from .models.model import Model, NonSymmetricTree, ObliviousTree


def _split_flat_features(m: Model, sp):
    """Flat (user column) indices a split depends on."""
    if sp.kind == "float":
        return [m.float_features[sp.feature].flat_index]
    if sp.kind == "onehot":
        return [m.cat_features[sp.feature].flat_index]
    ctr = m.ctrs[sp.feature]
    return [m.cat_features[c].flat_index for c in ctr.cat_features]


def _as_nonsymmetric(t):
    if isinstance(t, NonSymmetricTree):
        return t
    from .models.io import oblivious_to_nonsymmetric
    return oblivious_to_nonsymmetric(t)


def _node_stats(t: NonSymmetricTree, dims):
    """cover and weighted mean value of every node (children before parents by reverse order)."""
    n = len(t.split_of_node)
    cover = np.zeros(n)
    mean = np.zeros((n, dims))
    order = _topo(t)
    for node in reversed(order):
        if t.split_of_node[node] < 0:
            lf = t.leaf_of_node[node]
            cover[node] = max(float(t.leaf_weights[lf]), 0.0) if lf < len(t.leaf_weights) else 0.0
            mean[node] = t.leaf_values[lf]
        else:
            l, r = t.left[node], t.right[node]
            cover[node] = cover[l] + cover[r]
            if cover[node] > 0:
                mean[node] = (mean[l] * cover[l] + mean[r] * cover[r]) / cover[node]
            else:
                mean[node] = 0.5 * (mean[l] + mean[r])
    return cover, mean


def _topo(t: NonSymmetricTree):
    order, stack = [], [0]
    while stack:
        node = stack.pop()
        order.append(node)
        if t.split_of_node[node] >= 0:
            stack += [int(t.right[node]), int(t.left[node])]
    return order


def prediction_values_change(m: Model) -> np.ndarray:
    imp = np.zeros(m.n_features)
    for t in m.trees:
        ns = _as_nonsymmetric(t)
        cover, mean = _node_stats(ns, m.dims)
        for node in range(len(ns.split_of_node)):
            si = ns.split_of_node[node]
            if si < 0:
                continue
            l, r = ns.left[node], ns.right[node]
            w0, w1 = cover[l], cover[r]
            if w0 + w1 <= 0:
                continue
            avg = (mean[l] * w0 + mean[r] * w1) / (w0 + w1)
            val = float((((mean[l] - avg) ** 2) * w0 + ((mean[r] - avg) ** 2) * w1).sum())
            feats = _split_flat_features(m, m.splits[si])
            for f in feats:
                imp[f] += val / len(feats)
    tot = imp.sum()
    return imp / tot * 100.0 if tot > 0 else imp


def interaction(m: Model):
    pair = {}
    for t in m.trees:
        ns = _as_nonsymmetric(t)
        cover, mean = _node_stats(ns, m.dims)
        feats_in_tree = {}
        for node in range(len(ns.split_of_node)):
            si = ns.split_of_node[node]
            if si < 0:
                continue
            l, r = ns.left[node], ns.right[node]
            w0, w1 = cover[l], cover[r]
            if w0 + w1 <= 0:
                continue
            avg = (mean[l] * w0 + mean[r] * w1) / (w0 + w1)
            val = float((((mean[l] - avg) ** 2) * w0 + ((mean[r] - avg) ** 2) * w1).sum())
            for f in _split_flat_features(m, m.splits[si]):
                feats_in_tree[f] = feats_in_tree.get(f, 0.0) + val
        fl = sorted(feats_in_tree)
        for i in range(len(fl)):
            for j in range(i + 1, len(fl)):
                pair[(fl[i], fl[j])] = pair.get((fl[i], fl[j]), 0.0) + min(feats_in_tree[fl[i]], feats_in_tree[fl[j]])
    tot = sum(pair.values())
    out = [[a, b, v / tot * 100.0 if tot > 0 else 0.0] for (a, b), v in pair.items()]
    return sorted(out, key=lambda x: -x[2])


# ---- TreeSHAP ---------------------------------------------------------------------------------------------
class _Path:
    __slots__ = ("d", "z", "o", "w")

    def __init__(self, d, z, o, w):
        self.d, self.z, self.o, self.w = d, z, o, w


def _extend(path, pz, po, pi):
    l = len(path)
    path = [_Path(p.d, p.z, p.o, p.w) for p in path]
    path.append(_Path(pi, pz, po, 1.0 if l == 0 else 0.0))
    for i in range(l - 1, -1, -1):
        path[i + 1].w += po * path[i].w * (i + 1) / (l + 1)
        path[i].w = pz * path[i].w * (l - i) / (l + 1)
    return path


def _unwind(path, i):
    l = len(path) - 1
    path = [_Path(p.d, p.z, p.o, p.w) for p in path]
    n = path[l].w
    o, z = path[i].o, path[i].z
    for j in range(l - 1, -1, -1):
        if o != 0:
            t = path[j].w
            path[j].w = n * (l + 1) / ((j + 1) * o)
            n = t - path[j].w * z * (l - j) / (l + 1)
        else:
            path[j].w = path[j].w * (l + 1) / (z * (l - j))
    for j in range(i, l):
        path[j].d, path[j].z, path[j].o = path[j + 1].d, path[j + 1].z, path[j + 1].o
    return path[:l]


def _unwound_sum(path, i):
    l = len(path) - 1
    o, z = path[i].o, path[i].z
    n = path[l].w
    tot = 0.0
    for j in range(l - 1, -1, -1):
        if o != 0:
            t = n * (l + 1) / ((j + 1) * o)
            tot += t
            n = path[j].w - t * z * (l - j) / (l + 1)
        else:
            tot += path[j].w / (z * (l - j) / (l + 1))
    return tot


def _tree_shap_row(m, ns, cover, outcomes_col, phi, split_feat, condition=0, condition_feature=-1):
    """Accumulate SHAP values of one tree for one row.  outcomes_col: bool per model split.
    condition = +1 / -1 fixes ``condition_feature`` as present / absent (used for the interaction values)."""

    def recurse(node, path, pz, po, pi, cfrac):
        if cfrac == 0.0:
            return
        if condition == 0 or condition_feature != pi:
            path = _extend(path, pz, po, pi)
        si = ns.split_of_node[node]
        if si < 0:
            v = ns.leaf_values[ns.leaf_of_node[node]]
            for i in range(1, len(path)):
                w = _unwound_sum(path, i)
                phi[path[i].d] += w * (path[i].o - path[i].z) * v * cfrac
            return
        hot, cold = (ns.right[node], ns.left[node]) if outcomes_col[si] else (ns.left[node], ns.right[node])
        f = split_feat[si]
        iz, io = 1.0, 1.0
        k = next((i for i in range(1, len(path)) if path[i].d == f), None)
        if k is not None:
            iz, io = path[k].z, path[k].o
            path = _unwind(path, k)
        c = cover[node]
        if c <= 0:
            return
        # a branch no training row reached carries no weight: skip it when it is the cold one, and give the hot one a
        # vanishing (but non-zero) fraction so that the path algebra stays finite
        hot_z = max(cover[hot] / c, 1e-9)
        cold_z = cover[cold] / c
        hot_c, cold_c = cfrac, cfrac
        if condition > 0 and f == condition_feature:
            cold_c = 0.0
        elif condition < 0 and f == condition_feature:
            hot_c *= hot_z
            cold_c *= cold_z
        recurse(hot, path, iz * hot_z, io, f, hot_c)
        if cover[cold] > 0:
            recurse(cold, path, iz * cold_z, 0.0, f, cold_c)

    recurse(0, [], 1.0, 1.0, -1, 1.0)


def shap_values(m: Model, pool: Pool) -> np.ndarray:
    fd, ch = m.pool_arrays(pool)
    n = pool.num_row()
    F = m.n_features
    out = np.zeros((n, F + 1, m.dims))
    oc = m._split_outcomes_block(fd, ch, m._ctr_values(ch))
    split_feat = [(_split_flat_features(m, sp)[0]) for sp in m.splits]
    bias = np.broadcast_to(m.bias, (m.dims,)).astype(np.float64)
    expected = bias.copy()
    prepared = []
    for t in m.trees:
        ns = _as_nonsymmetric(t)
        cover, mean = _node_stats(ns, m.dims)
        prepared.append((ns, cover))
        expected = expected + mean[0] * m.scale
    import sys
    sys.setrecursionlimit(max(sys.getrecursionlimit(), 10000))
    for r in range(n):
        phi = np.zeros((F + 1, m.dims))
        col = oc[:, r]
        for ns, cover in prepared:
            if cover[0] <= 0:
                continue
            _tree_shap_row(m, ns, cover, col, phi, split_feat)
        out[r, :F] = phi[:F] * m.scale
        out[r, F] = expected
    if m.dims == 1:
        return out[:, :, 0]
    return np.transpose(out, (0, 2, 1))


def shap_interaction_values(m: Model, pool: Pool) -> np.ndarray:
    """Exact TreeSHAP interaction values ``[n, F + 1, F + 1]`` (one-dimensional models): entry (i, j), i != j, is half
    the difference of feature i's SHAP value with feature j fixed present and fixed absent; the diagonal holds the
    rest of feature i's SHAP value; the last row / column carry the expected value in their corner
    (catboost/libs/fstr/shap_interaction_values.cpp)."""
    if m.dims != 1:
        raise CatBoostError("ShapInteractionValues are implemented for one-dimensional models")
    fd, ch = m.pool_arrays(pool)
    n, F = pool.num_row(), m.n_features
    oc = m._split_outcomes_block(fd, ch, m._ctr_values(ch))
    split_feat = [(_split_flat_features(m, sp)[0]) for sp in m.splits]
    prepared = []
    for t in m.trees:
        ns = _as_nonsymmetric(t)
        cover, _ = _node_stats(ns, 1)
        if cover[0] > 0:
            prepared.append((ns, cover, {split_feat[si] for si in ns.split_of_node if si >= 0}))
    base = shap_values(m, pool)                                   # [n, F + 1]
    out = np.zeros((n, F + 1, F + 1))
    import sys
    sys.setrecursionlimit(max(sys.getrecursionlimit(), 10000))
    for r in range(n):
        col = oc[:, r]
        for j in range(F):
            on = np.zeros((F + 1, 1))
            off = np.zeros((F + 1, 1))
            for ns, cover, used in prepared:
                if j not in used:
                    continue                                      # fixing an unused feature changes nothing
                _tree_shap_row(m, ns, cover, col, on, split_feat, 1, j)
                _tree_shap_row(m, ns, cover, col, off, split_feat, -1, j)
            half = (on[:F, 0] - off[:F, 0]) * 0.5 * m.scale
            half[j] = 0.0
            out[r, :F, j] = half
        for i in range(F):
            out[r, i, i] = base[r, i] - out[r, i, :F].sum()
        out[r, F, F] = base[r, F]
    return out


def loss_function_change(estimator, data) -> np.ndarray:
    m = estimator._model
    pool = data if isinstance(data, Pool) else Pool(data)
    if pool.label is None:
        raise CatBoostError("LossFunctionChange needs labels")
    sv = shap_values(m, pool)
    raw = estimator._raw(pool)
    y = estimator._encode_labels(pool.label)
    loss = m.params.get("loss_function", m.loss_name) if isinstance(m.params.get("loss_function", None), str) else m.loss_name
    metric = make_metric(loss)
    kw = {}
    if pool.group_id is not None:
        kw["group_offsets"] = pool.group_offsets()
    base = metric.eval(raw, y, pool.weight, **kw)
    imp = np.zeros(m.n_features)
    for f in range(m.n_features):
        contrib = sv[:, f] if m.dims == 1 else sv[:, :, f]
        if not np.any(contrib):
            continue
        alt = raw - contrib.reshape(raw.shape) + contrib.reshape(raw.shape).mean(axis=0, keepdims=True)
        v = metric.eval(alt, y, pool.weight, **kw)
        imp[f] = (base - v) if metric.is_max_optimal else (v - base)
    return imp


def prediction_diff(estimator, data) -> np.ndarray:
    pool = data if isinstance(data, Pool) else Pool(data)
    if pool.num_row() != 2:
        raise CatBoostError("PredictionDiff needs exactly two rows")
    sv = shap_values(estimator._model, pool)
    d = sv[0, :-1] - sv[1, :-1] if sv.ndim == 2 else (sv[0, :, :-1] - sv[1, :, :-1]).sum(0)
    return np.abs(d)


def sage_values(estimator, data, n_samples: int = 128, batch_size: int = 512, detect_convergence: bool = True,
                seed: int = 228) -> np.ndarray:
    """SAGE (Shapley additive global importance) of every feature: the mean rise of the model's loss when the feature's
    column is replaced by draws from its marginal distribution, averaged over random feature orders and random batches
    (catboost/libs/fstr/sage_values.cpp:334-426: a batch of rows, a random order of the features, the features are
    imputed one after another and every step's loss change is credited to the feature just imputed; sampling stops
    early when the widest 95 % confidence interval is below a tenth of the largest value)."""
    m = estimator._model
    if m.dims != 1:
        raise CatBoostError("SageValues: the model must have one dimension")
    pool = data if isinstance(data, Pool) else Pool(data)
    if pool.label is None:
        raise CatBoostError("SageValues needs labels")
    loss = m.params.get("loss_function", m.loss_name) if isinstance(m.params.get("loss_function", None), str) else m.loss_name
    metric = make_metric(loss)
    rng = np.random.default_rng(seed)
    n = pool.num_row()
    batch_size = min(int(batch_size), n)
    columns = [("float", j, c) for j, c in enumerate(pool.float_feature_indices)] + \
              [("cat", j, c) for j, c in enumerate(pool.cat_feature_indices)] + \
              [("text", j, c) for j, c in enumerate(getattr(pool, "text_feature_indices", []) or [])] + \
              [("emb", j, c) for j, c in enumerate(getattr(pool, "embedding_feature_indices", []) or [])]
    n_ext = max([c for _, _, c in columns] + [m.n_features - 1]) + 1
    samples = [[0.0] for _ in range(n_ext)]
    groups = pool.group_offsets() if pool.group_id is not None else None

    def batch_loss(b):
        raw = estimator._raw(b)
        kw = {"group_offsets": b.group_offsets()} if b.group_id is not None else {}
        v = metric.eval(raw, estimator._encode_labels(b.label), b.weight, **kw)
        return -v if metric.is_max_optimal else v

    for _ in range(int(n_samples)):
        if groups is None:
            rows = rng.choice(n, batch_size, replace=False)
        else:
            order, rows, got = rng.permutation(len(groups) - 1), [], 0
            for g in order:
                rows.append(np.arange(groups[g], groups[g + 1]))
                got += groups[g + 1] - groups[g]
                if got >= batch_size:
                    break
            rows = np.concatenate(rows)
        b = pool.slice(rows)
        prev = batch_loss(b)
        for k in rng.permutation(len(columns)):
            kind, j, ext = columns[k]
            draw = rng.integers(0, n, size=b.num_row())
            if kind == "float":
                b.float_data[:, j] = pool.float_data[draw, j]
            elif kind == "cat":
                b.cat_hashes[j] = pool.cat_hashes[j, draw]
                b.__dict__.pop("_cat_hash_tensors", None)
            elif kind == "text":
                b.text_data[j] = pool.text_data[j][draw]
            else:
                b.embedding_data[j] = pool.embedding_data[j][draw]
            cur = batch_loss(b)
            samples[ext].append(cur - prev)
            prev = cur
        if detect_convergence:
            means = np.array([np.mean(s) for s in samples])
            half = np.array([1.96 * np.std(s) / math.sqrt(len(s)) for s in samples])
            if half.max() / (np.abs(means).max() + 1e-12) <= 0.1:
                break
    return np.array([float(np.mean(s)) for s in samples])
