"""Hyper-parameter search and feature selection helpers
(catboost/private/libs/hyperparameter_tuning, catboost/libs/features_selection)."""
from __future__ import annotations

import itertools

import numpy as np

from .cv import _fold_indices
from .data.pool import CatBoostError, Pool, to_pool
from .metrics import make_metric


def _candidates(grid):
    grids = grid if isinstance(grid, list) else [grid]
    for g in grids:
        keys = list(g)
        for combo in itertools.product(*[g[k] if isinstance(g[k], (list, tuple, np.ndarray)) else [g[k]] for k in keys]):
            yield dict(zip(keys, combo))


def _evaluate(est, params, pool, cv, seed, by_split, shuffle, stratified, train_size):
    from .core import CatBoost
    base = est.get_params()
    base.update(params)
    base.setdefault("verbose", False)
    base["allow_writing_files"] = False
    n = pool.num_row()
    if by_split:
        rng = np.random.RandomState(seed)
        idx = rng.permutation(n) if shuffle else np.arange(n)
        k = int(n * train_size)
        splits = [(np.sort(idx[:k]), np.sort(idx[k:]))]
    else:
        splits = _fold_indices(pool, cv if isinstance(cv, int) else 3, shuffle, seed, bool(stratified))
    scores = []
    metric_name = None
    maximize = False
    for tr, te in splits:
        m = est.__class__(**base)
        m.fit(pool.slice(tr), eval_set=pool.slice(te), use_best_model=False)
        ev = m.get_evals_result()["validation"]
        metric_name = list(ev)[0]
        maximize = make_metric(metric_name).is_max_optimal
        scores.append(max(ev[metric_name]) if maximize else min(ev[metric_name]))
    return float(np.mean(scores)), metric_name, maximize


def _search(est, cands, X, y, cv, seed, by_split, refit, shuffle, stratified, train_size, verbose):
    pool = to_pool(X, y) if not isinstance(X, Pool) else X
    best, best_score, results = None, None, []
    for i, cand in enumerate(cands):
        score, name, maximize = _evaluate(est, cand, pool, cv, seed, by_split, shuffle, stratified, train_size)
        results.append({"params": cand, "score": score})
        if best is None or (score > best_score if maximize else score < best_score):
            best, best_score = cand, score
        if verbose:
            print(f"{i}: {name}={score:.6f} best={best_score:.6f} params={cand}")
    if best is None:
        raise CatBoostError("empty parameter grid")
    if refit:
        est.set_params(**best)
        est.fit(pool)
    return {"params": best, "cv_results": {"scores": [r["score"] for r in results], "params": [r["params"] for r in results]}}


def grid_search(est, param_grid, X, y=None, cv=3, partition_random_seed=0, search_by_train_test_split=True, refit=True,
                shuffle=True, stratified=None, train_size=0.8, verbose=True):
    return _search(est, list(_candidates(param_grid)), X, y, cv, partition_random_seed, search_by_train_test_split, refit,
                   shuffle, stratified, train_size, verbose)


def randomized_search(est, param_distributions, X, y=None, cv=3, n_iter=10, partition_random_seed=0,
                      search_by_train_test_split=True, refit=True, shuffle=True, stratified=None, train_size=0.8,
                      verbose=True):
    rng = np.random.RandomState(partition_random_seed)
    cands = []
    for _ in range(n_iter):
        c = {}
        for k, v in param_distributions.items():
            if hasattr(v, "rvs"):
                c[k] = v.rvs(random_state=rng)
            else:
                vals = list(v)
                c[k] = vals[rng.randint(len(vals))]
        cands.append(c)
    return _search(est, cands, X, y, cv, partition_random_seed, search_by_train_test_split, refit, shuffle, stratified,
                   train_size, verbose)


def select_features(est, X, y=None, eval_set=None, features_for_select=None, num_features_to_select=None, steps=1,
                    train_final_model=True):
    """Recursive feature elimination by PredictionValuesChange."""
    pool = to_pool(X, y) if not isinstance(X, Pool) else X
    feats = list(range(pool.n_features)) if features_for_select is None else \
        [pool.feature_names.index(f) if isinstance(f, str) else int(f) for f in features_for_select]
    target = num_features_to_select or max(1, len(feats) // 2)
    if target > len(feats):
        raise CatBoostError("num_features_to_select exceeds the number of candidate features")
    eliminated, active = [], list(feats)
    per_step = max(1, int(np.ceil((len(active) - target) / max(1, steps))))
    params = est.get_params()
    params.setdefault("verbose", False)
    params["allow_writing_files"] = False
    loss_curve = []
    while len(active) > target:
        ignored = [f for f in range(pool.n_features) if f not in active and f in feats]
        m = est.__class__(**{**params, "ignored_features": ignored})
        m.fit(pool, eval_set=eval_set)
        imp = m.get_feature_importance()
        order = sorted(active, key=lambda f: imp[f])
        drop = order[: min(per_step, len(active) - target)]
        eliminated += drop
        active = [f for f in active if f not in drop]
        ev = m.get_evals_result()
        key = "validation" if "validation" in ev else "learn"
        loss_curve.append(ev[key][list(ev[key])[0]][-1])
    if train_final_model:
        est.set_params(ignored_features=[f for f in feats if f not in active])
        est.fit(pool, eval_set=eval_set)
    return {"selected_features": active, "eliminated_features": eliminated,
            "selected_features_names": [pool.feature_names[f] for f in active],
            "eliminated_features_names": [pool.feature_names[f] for f in eliminated],
            "loss_graph": {"loss_values": loss_curve}}
