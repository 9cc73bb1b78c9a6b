"""Cross-validation (catboost.cv, catboost/libs/train_lib/cross_validation.cpp): k folds, optional
stratification, group-aware splitting, per-iteration mean/std of every metric."""
from __future__ import annotations

import numpy as np

from .data.pool import CatBoostError, Pool


def _fold_indices(pool: Pool, fold_count, shuffle, seed, stratified, inverted=False):
    n = pool.num_row()
    rng = np.random.RandomState(seed)
    if pool.group_id is not None:
        off = pool.group_offsets()
        g = np.arange(len(off) - 1)
        if shuffle:
            rng.shuffle(g)
        parts = np.array_split(g, fold_count)
        folds = [np.concatenate([np.arange(off[k], off[k + 1]) for k in np.sort(p)]) if len(p) else np.zeros(0, int) for p in parts]
    elif stratified and pool.label is not None:
        lab = np.asarray(pool.label)
        folds = [[] for _ in range(fold_count)]
        for c in np.unique(lab):
            idx = np.nonzero(lab == c)[0]
            if shuffle:
                rng.shuffle(idx)
            for k, part in enumerate(np.array_split(idx, fold_count)):
                folds[k].append(part)
        folds = [np.sort(np.concatenate(f)) for f in folds]
    else:
        idx = np.arange(n)
        if shuffle:
            rng.shuffle(idx)
        folds = [np.sort(p) for p in np.array_split(idx, fold_count)]
    out = []
    for k in range(fold_count):
        test = folds[k]
        train = np.sort(np.concatenate([folds[j] for j in range(fold_count) if j != k]))
        out.append((test, train) if inverted else (train, test))
    return out


def cv(pool=None, params=None, dtrain=None, iterations=None, num_boost_round=None, fold_count=None, nfold=None,
       inverted=False, partition_random_seed=0, seed=None, shuffle=True, logging_level=None, stratified=None,
       as_pandas=True, metric_period=None, verbose=None, verbose_eval=None, plot=False, plot_file=None,
       early_stopping_rounds=None, save_snapshot=None, snapshot_file=None, snapshot_interval=None,
       metric_update_interval=0.5, folds=None, type="Classical", return_models=False, log_cout=None, log_cerr=None):
    from .core import CatBoost
    pool = pool if pool is not None else dtrain
    if pool is None or params is None:
        raise CatBoostError("cv needs a pool and params")
    params = dict(params)
    if iterations is not None or num_boost_round is not None:
        params["iterations"] = iterations if iterations is not None else num_boost_round
    if "loss_function" not in params and "objective" not in params:
        raise CatBoostError("cv needs loss_function in params")
    k = fold_count or nfold or 3
    loss = params.get("loss_function", params.get("objective"))
    if stratified is None:
        stratified = isinstance(loss, str) and loss.split(":")[0] in ("Logloss", "Focal", "MultiClass", "MultiClassOneVsAll")
    seed = partition_random_seed if seed is None else seed
    splits = folds if folds is not None else _fold_indices(pool, k, shuffle, seed, stratified, inverted)
    params.setdefault("verbose", bool(verbose or verbose_eval) if (verbose or verbose_eval) is not None else False)
    params["allow_writing_files"] = False
    if early_stopping_rounds is not None:
        params["early_stopping_rounds"] = early_stopping_rounds
    results, models = [], []
    for tr, te in splits:
        m = CatBoost(params)
        m.fit(pool.slice(tr), eval_set=pool.slice(te), use_best_model=False)
        results.append(m.get_evals_result())
        models.append(m)
    names = list(results[0]["learn"].keys())
    length = min(len(r["validation"][names[0]]) for r in results)
    table = {"iterations": list(range(length))}
    for nm in names:
        te = np.array([r["validation"][nm][:length] for r in results])
        trn = np.array([r["learn"][nm][:length] for r in results])
        table[f"test-{nm}-mean"] = te.mean(0)
        table[f"test-{nm}-std"] = te.std(0, ddof=1) if len(results) > 1 else np.zeros(length)
        table[f"train-{nm}-mean"] = trn.mean(0)
        table[f"train-{nm}-std"] = trn.std(0, ddof=1) if len(results) > 1 else np.zeros(length)
    if as_pandas:
        try:
            import pandas as pd
            table = pd.DataFrame(table)
        except Exception:
            pass
    return (table, models) if return_models else table
