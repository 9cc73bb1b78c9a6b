"""Feature evaluation: does a set of features improve the model?  (catboost/python-package/catboost/eval/
catboost_evaluation.py, catboost/libs/train_lib/eval_feature.cpp.)

Folds of the dataset are trained twice or more: a baseline that ignores every feature under evaluation, and test cases
that bring features back (``All``: all of them at once; ``SeqAdd``: one at a time; ``SeqRem``: all but one;
``SeqAddAndAll``: both).  Every case is scored on the held-out part of its fold; a case is compared with the baseline
by the paired per-fold differences (Wilcoxon signed-rank test, like the reference's EvaluationResult).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np

from .cv import _fold_indices
from .data.pool import CatBoostError, Pool

EVAL_TYPES = ("All", "SeqAdd", "SeqRem", "SeqAddAndAll")


def _cases(features: List[int], eval_type: str):
    """(label, ignored features) of the baseline and of every test case."""
    if not features:
        raise CatBoostError("provide at least one feature to evaluate")
    if eval_type not in EVAL_TYPES:
        raise CatBoostError(f"eval_type must be one of {EVAL_TYPES}")
    baseline = ("baseline", list(features))
    tests = []
    if eval_type in ("All", "SeqAddAndAll") or len(features) == 1:
        tests.append(("all features", []))
    if len(features) > 1:
        if eval_type == "SeqRem":
            tests += [(f"without {f}", [f]) for f in features]
        elif eval_type in ("SeqAdd", "SeqAddAndAll"):
            tests += [(f"with {f}", [g for g in features if g != f]) for f in features]
    return baseline, tests


def _wilcoxon_p(diffs: np.ndarray) -> float:
    d = diffs[diffs != 0]
    if len(d) < 2:
        return float("nan")
    try:
        from scipy.stats import wilcoxon
        return float(wilcoxon(d).pvalue)
    except Exception:  # pragma: no cover - scipy missing or degenerate input
        return float("nan")


def eval_features(pool: Pool, params: dict, features_to_eval: Sequence, eval_type: str = "SeqAdd", fold_count: int = 5,
                  eval_metrics: Optional[Sequence[str]] = None, partition_random_seed: int = 0,
                  significance: float = 0.05) -> Dict[str, dict]:
    """Returns {metric: {"baseline": [per fold], "cases": {label: {"values", "delta_mean", "pvalue", "decision"}}}}.
    ``delta_mean`` is oriented so that positive means better than the baseline."""
    from .core import CatBoost
    from .metrics import make_metric
    params = dict(params)
    if "loss_function" not in params:
        raise CatBoostError("provide loss_function in params")
    names = pool.feature_names
    feats = sorted({names.index(f) if isinstance(f, str) else int(f) for f in features_to_eval})
    metrics = list(dict.fromkeys(list(eval_metrics or []) + [params["loss_function"]]))
    baseline, tests = _cases(feats, eval_type)
    user_ignored = list(params.pop("ignored_features", None) or [])
    params.setdefault("verbose", False)
    params.setdefault("allow_writing_files", False)
    stratified = str(params["loss_function"]).split(":")[0] in ("Logloss", "Focal", "MultiClass", "MultiClassOneVsAll")
    folds = _fold_indices(pool, fold_count, True, partition_random_seed, stratified)
    values = {m: {lab: [] for lab, _ in [baseline] + tests} for m in metrics}
    for train_idx, test_idx in folds:
        tr, te = pool.slice(train_idx), pool.slice(test_idx)
        for label, ignored in [baseline] + tests:
            model = CatBoost(dict(params, ignored_features=sorted(set(user_ignored) | set(ignored))))
            model.fit(tr)
            res = model.eval_metrics(te, metrics, eval_period=max(1, model.tree_count_))
            for m in metrics:
                values[m][label].append(float(res[m][-1]))
    out = {}
    for m in metrics:
        higher = bool(make_metric(m).is_max_optimal)
        base = np.array(values[m]["baseline"])
        cases = {}
        for label, _ in tests:
            v = np.array(values[m][label])
            diff = (v - base) if higher else (base - v)
            p = _wilcoxon_p(diff)
            if not np.isfinite(p) or p > significance:
                decision = "UNKNOWN"
            else:
                decision = "GOOD" if diff.mean() > 0 else "BAD"
            cases[label] = {"values": v.tolist(), "delta_mean": float(diff.mean()), "pvalue": p, "decision": decision}
        out[m] = {"baseline": base.tolist(), "cases": cases}
    return out
