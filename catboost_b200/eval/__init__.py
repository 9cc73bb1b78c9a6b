"""Evaluation of features and of training configurations on small learn folds (the ``catboost.eval`` interface:
catboost/python-package/catboost/eval/catboost_evaluation.py, evaluation_result.py, execution_case.py).

The dataset is permuted (whole groups when a group column exists) and cut into folds of ``fold_size`` documents.  Each
of the first ``fold_count`` folds is a learn set of its own; the model of a fold is scored on all the other folds, at
every ``eval_step`` trees, and the best value along that curve is the fold's score.  Cases (parameter sets) are compared
with the baseline case by the paired per-fold differences: Wilcoxon signed-rank p-value, mean difference with a bootstrap
confidence interval, and a GOOD / BAD / UNKNOWN decision.

Unlike the reference, which streams the file into fold files on disk, the folds are index sets over one in-memory pool;
``CatboostEvaluation`` also accepts a ready ``Pool`` in place of the dataset path.
"""
from __future__ import annotations

import json
import os
from enum import Enum
from typing import Dict, Iterable, List, Optional, Sequence

import numpy as np

from ..data.pool import CatBoostError, Pool

__all__ = ["EvalType", "CatboostEvaluation", "ScoreType", "ScoreConfig", "CaseEvaluationResult", "MetricEvaluationResult",
           "EvaluationResults", "calc_wilcoxon_test", "calc_bootstrap_ci_for_mean", "ExecutionCase", "LabelMode",
           "make_dirs_if_not_exists", "series_to_line", "save_plot"]


# ---- small helpers ---------------------------------------------------------------------------------------------
def make_dirs_if_not_exists(name):
    os.makedirs(name, exist_ok=True)


def series_to_line(row, sep):
    return sep.join(str(x) for x in row)


def save_plot(fig, file_name=None):
    """Writes a plotly figure to an html file; needs plotly, which is optional."""
    try:
        from plotly.offline import plot
    except ImportError as e:
        raise CatBoostError("save_plot needs the plotly package") from e
    plot(fig, filename=file_name or "plot.html", auto_open=False)


def calc_wilcoxon_test(baseline, test) -> float:
    d = np.asarray(baseline, dtype=np.float64) - np.asarray(test, dtype=np.float64)
    if len(d) < 2 or not np.any(d != 0):
        return 1.0
    from scipy.stats import wilcoxon
    return float(wilcoxon(d[d != 0]).pvalue) if np.count_nonzero(d) > 1 else 1.0


def calc_bootstrap_ci_for_mean(samples, level=0.05, tries=999, seed: int = 0):
    s = np.asarray(samples, dtype=np.float64)
    if s.size == 0 or not np.any(s != 0):
        return 0.0, 0.0
    rng = np.random.default_rng(seed)
    means = np.sort(rng.choice(s, size=(tries, s.size)).mean(1))
    return float(means[int(tries * (level / 2))]), float(means[min(tries - 1, int(tries * (1.0 - level / 2)))])


def _ranges(features: Optional[Iterable[int]]) -> str:
    """{1, 2, 3, 7} -> '1-3;7'."""
    f = sorted(set(int(x) for x in (features or [])))
    if not f:
        return "None"
    out, start, prev = [], f[0], f[0]
    for x in f[1:] + [None]:
        if x is None or x != prev + 1:
            out.append(str(start) if start == prev else f"{start}-{prev}")
            start = x
        prev = x if x is not None else prev
    return ";".join(out)


# ---- enums and configuration -------------------------------------------------------------------------------------
class EvalType(Enum):
    All = "All"                  # all evaluated features at once
    SeqRem = "SeqRem"            # each feature removed while the others stay
    SeqAdd = "SeqAdd"            # each feature added while the others stay out
    SeqAddAndAll = "SeqAddAndAll"


class LabelMode(Enum):
    AddFeature = "AddFeature"
    IgnoreFeature = "IgnoreFeature"


class ScoreType(Enum):
    Abs = "AbsoluteDiff"
    Rel = "RelativeDiff"


class ScoreConfig:
    """How differences are reported: absolute or relative (in percent), test level, confidence interval level."""

    def __init__(self, score_type=ScoreType.Rel, multiplier=100, score_level=0.01, interval_level=0.01,
                 overfit_iterations_info=True):
        self.type = score_type
        self.multiplier = multiplier
        self.score_level = score_level
        self.interval_level = interval_level
        self.overfit_overfit_iterations_info = overfit_iterations_info

    @staticmethod
    def abs_score(level=0.01):
        return ScoreConfig(ScoreType.Abs, multiplier=1, score_level=level)

    @staticmethod
    def rel_score(level=0.01):
        return ScoreConfig(ScoreType.Rel, multiplier=100, score_level=level)


class ExecutionCase:
    """One training configuration of a comparison: parameters, a label, extra features to ignore."""

    def __init__(self, params, label=None, ignored_features=None, learning_rate=None):
        p = dict(params)
        if learning_rate is not None:
            p["learning_rate"] = learning_rate
        ign = set(p.get("ignored_features") or [])
        if ignored_features is not None:
            ign |= set(ignored_features)
        p["ignored_features"] = sorted(int(x) for x in ign)
        self._label = label if label is not None else ""
        self._ignored_features = ignored_features
        self._params = p

    def _key(self):
        return json.dumps(self._params, sort_keys=True, default=lambda o: o.tolist() if hasattr(o, "tolist") else str(o))

    def _set_thread_count(self, thread_count):
        if thread_count is not None and thread_count != -1:
            self._params["thread_count"] = thread_count

    def get_params(self):
        return dict(self._params)

    def get_label(self):
        return self._label

    def __str__(self):
        return self._label if self._label else f"Ignore: {_ranges(self._ignored_features)}"

    __repr__ = __str__

    def __eq__(self, other):
        return isinstance(other, ExecutionCase) and self._key() == other._key() and self._label == other._label

    def __hash__(self):
        return hash((self._key(), self._label))


# ---- results ---------------------------------------------------------------------------------------------------
class _MetricDescription(str):
    """A metric description string that also knows its direction."""

    def is_max_optimal(self) -> bool:
        from ..metrics import make_metric
        return bool(make_metric(str(self)).is_max_optimal)


class CaseEvaluationResult:
    """Learning curves of one case and one metric, one curve per learn fold."""

    def __init__(self, case, metric_description, eval_step):
        self._case = case
        self._metric_description = _MetricDescription(metric_description)
        self._eval_step = int(eval_step)
        self._fold_ids: List[int] = []
        self._curves: Dict[int, np.ndarray] = {}

    def _add(self, fold_id, learning_curve):
        if fold_id in self._curves:
            raise CatBoostError(f"fold {fold_id} was added twice")
        self._fold_ids.append(int(fold_id))
        self._curves[int(fold_id)] = np.asarray(learning_curve, dtype=np.float64)

    def __eq__(self, other):
        return (isinstance(other, CaseEvaluationResult) and self._case == other._case
                and self._metric_description == other._metric_description and self._fold_ids == other._fold_ids
                and all(np.array_equal(self._curves[f], other._curves[f]) for f in self._fold_ids))

    def get_case(self):
        return self._case

    def get_fold_ids(self):
        return list(self._fold_ids)

    def _best_index(self, fold):
        c = self._curves[fold]
        return int(np.argmax(c) if self._metric_description.is_max_optimal() else np.argmin(c))

    def get_best_metric_for_fold(self, fold):
        return float(self._curves[fold][self._best_index(fold)])

    def get_best_iterations(self):
        import pandas as pd
        return pd.Series({f: self._best_index(f) * self._eval_step for f in self._fold_ids})

    def get_best_metrics(self):
        import pandas as pd
        return pd.Series({f: self.get_best_metric_for_fold(f) for f in self._fold_ids})

    def get_fold_curve(self, fold):
        return self._curves[fold]

    def get_metric_description(self):
        return self._metric_description

    def get_eval_step(self):
        return self._eval_step

    def count_under_and_over_fits(self, overfit_border=0.15, underfit_border=0.95):
        """Folds whose best iteration lies in the first ``overfit_border`` or after ``underfit_border`` of the curve."""
        over = under = 0
        for f in self._fold_ids:
            frac = self._best_index(f) / max(len(self._curves[f]) - 1, 1)
            over += frac < overfit_border
            under += frac > underfit_border
        return int(under), int(over)

    def estimate_fit_quality(self):
        under, over = self.count_under_and_over_fits()
        if under > over:
            return "Underfitting"
        return "Overfitting" if over > under else "Good"


class MetricEvaluationResult:
    """All cases of one metric, compared against a baseline case."""

    def __init__(self, case_results: Sequence[CaseEvaluationResult]):
        if not case_results:
            raise CatBoostError("need at least one case result")
        self._case_results = {r.get_case(): r for r in case_results}
        self._metric_description = case_results[0].get_metric_description()
        self._baseline_case = case_results[0].get_case()
        self._score_config = ScoreConfig()
        folds = case_results[0].get_fold_ids()
        for r in case_results:
            if r.get_metric_description() != self._metric_description or r.get_fold_ids() != folds:
                raise CatBoostError("case results must share the metric and the folds")
        self._tables = {}

    def _table(self, baseline_case):
        import pandas as pd
        cfg = self._score_config
        base = self._case_results[baseline_case].get_best_metrics()
        base_it = self._case_results[baseline_case].get_best_iterations()
        rows = {}
        for case, res in self._case_results.items():
            if case == baseline_case:
                continue
            test = res.get_best_metrics()
            diff = base - test
            if cfg.type == ScoreType.Rel:
                diff = diff / base.abs()
            if self._metric_description.is_max_optimal():
                diff = -diff
            lo, hi = calc_bootstrap_ci_for_mean(diff.values, cfg.interval_level)
            p = calc_wilcoxon_test(base.values, test.values)
            mean = float(diff.mean())
            row = {"PValue": p, "Score": mean * cfg.multiplier,
                   f"Quantile {cfg.score_level / 2}": lo * cfg.multiplier,
                   f"Quantile {1.0 - cfg.score_level / 2}": hi * cfg.multiplier,
                   "Decision": ("GOOD" if mean > 0 else "BAD" if mean < 0 else "UNKNOWN") if p < cfg.score_level else "UNKNOWN"}
            if cfg.overfit_overfit_iterations_info:
                it = res.get_best_iterations()
                row["Overfit iter diff"] = float((it - base_it).mean())
                row["Overfit iter pValue"] = calc_wilcoxon_test(base_it.values, it.values)
            rows[str(case)] = row
        t = pd.DataFrame.from_dict(rows, orient="index")
        return t.sort_values(by=["Score"], ascending=False) if len(t) else t

    def _change_score_config(self, config):
        if config is not None:
            self._score_config = ScoreConfig.abs_score() if config == ScoreType.Abs else \
                ScoreConfig.rel_score() if config == ScoreType.Rel else config
            self._tables = {}

    def get_baseline_case(self):
        return self._baseline_case

    def get_cases(self):
        return list(self._case_results.keys())

    def get_metric_description(self):
        return self._metric_description

    def get_baseline_comparison(self, score_config=None):
        return self.get_case_comparison(self._baseline_case, score_config)

    def get_case_comparison(self, case, score_config=None):
        self._change_score_config(score_config)
        if case not in self._tables:
            self._tables[case] = self._table(case)
        return self._tables[case]

    def change_baseline_case(self, case):
        if case not in self._case_results:
            raise CatBoostError(f"case {case} is not among the results")
        self._baseline_case = case

    def get_case_result(self, case):
        return self._case_results[case]

    def get_fold_ids(self):
        return self._case_results[self._baseline_case].get_fold_ids()

    def get_eval_step(self):
        return self._case_results[self._baseline_case].get_eval_step()

    def __eq__(self, other):
        return isinstance(other, MetricEvaluationResult) and self._case_results == other._case_results


class EvaluationResults:
    def __init__(self, metric_results: Sequence[MetricEvaluationResult]):
        if not metric_results:
            raise CatBoostError("need at least one metric result")
        self._results = {str(r.get_metric_description()): r for r in metric_results}
        self._metrics = {str(r.get_metric_description()): r.get_metric_description() for r in metric_results}
        self._cases = metric_results[0].get_cases()

    def get_metric_results(self, metric):
        return self._results[str(metric)]

    def get_metrics(self):
        return dict(self._metrics)

    def get_results(self):
        return dict(self._results)

    def set_baseline_case(self, case):
        for r in self._results.values():
            r.change_baseline_case(case)


# ---- the evaluator -----------------------------------------------------------------------------------------------
class CatboostEvaluation:
    """Compares training configurations on learn folds of ``fold_size`` documents.

    ``path_to_dataset`` is a delimited file read with ``column_description`` (as ``Pool`` reads it) or a ``Pool``.
    ``group_column`` is accepted for interface compatibility: grouping comes from the column description."""

    def __init__(self, path_to_dataset, fold_size, fold_count, column_description=None, fold_offset=0, group_column=None,
                 working_dir=None, remove_models=True, delimiter="\t", has_header=False, partition_random_seed=0,
                 min_fold_count=1):
        self._source = path_to_dataset
        self._column_description = column_description
        self._fold_size, self._fold_count, self._fold_offset = int(fold_size), int(fold_count), int(fold_offset)
        self._delimiter, self._has_header = delimiter, bool(has_header)
        self._seed, self._min_fold_count = int(partition_random_seed), int(min_fold_count)
        self._remove_models = bool(remove_models)
        self._group_column = group_column
        if working_dir is None:
            import tempfile
            working_dir = tempfile.mkdtemp()
        self._working_dir = working_dir
        self._pool: Optional[Pool] = None
        if self._fold_size < 1:
            raise CatBoostError("fold_size must be positive")

    def get_working_dir(self):
        return self._working_dir

    def _load(self) -> Pool:
        if self._pool is None:
            src = self._source
            self._pool = src if isinstance(src, Pool) else Pool(src, column_description=self._column_description,
                                                                delimiter=self._delimiter, has_header=self._has_header)
        return self._pool

    def _folds(self, pool: Pool) -> List[np.ndarray]:
        """Index sets of the folds: a random order of documents (of whole groups when there are groups), cut every
        ``fold_size`` documents; a last short piece joins the fold before it."""
        rng = np.random.default_rng(self._seed)
        n = pool.num_row()
        if pool.group_id is not None:
            off = np.asarray(pool.group_offsets())
            order = rng.permutation(len(off) - 1)
            folds, cur, size = [], [], 0
            for g in order:
                cur.append(np.arange(off[g], off[g + 1]))
                size += off[g + 1] - off[g]
                if size >= self._fold_size:
                    folds.append(np.concatenate(cur))
                    cur, size = [], 0
            if cur:
                tail = np.concatenate(cur)
                if folds:
                    folds[-1] = np.concatenate([folds[-1], tail])
                else:
                    folds.append(tail)
        else:
            perm = rng.permutation(n)
            k = max(n // self._fold_size, 1)
            folds = [perm[i * self._fold_size: (i + 1) * self._fold_size if i < k - 1 else n] for i in range(k)]
        if len(folds) < max(self._min_fold_count, 2):
            raise CatBoostError(f"the dataset gives {len(folds)} folds of {self._fold_size} documents; at least "
                                f"{max(self._min_fold_count, 2)} are needed")
        return [np.sort(f) for f in folds]

    @staticmethod
    def _create_eval_feature_cases(params, features_to_eval, eval_type, label_mode=LabelMode.AddFeature):
        feats = sorted(set(int(f) for f in features_to_eval))
        if not feats:
            raise CatBoostError("provide at least one feature to evaluate")
        et = EvalType(eval_type) if not isinstance(eval_type, EvalType) else eval_type
        ignored = set(params.get("ignored_features") or [])
        for f in feats:
            if f in ignored:
                raise CatBoostError(f"Feature {f} is in ignored set and in tmp-features set at the same time")
        baseline = ExecutionCase(params, ignored_features=feats, label="Features: None")
        cases = []
        if et in (EvalType.All, EvalType.SeqAddAndAll) or len(feats) == 1:
            cases.append(ExecutionCase(params, ignored_features=[], label=f"Features: {_ranges(feats)}"))
        if len(feats) > 1:
            if et == EvalType.SeqRem:
                for f in feats:
                    cases.append(ExecutionCase(params, ignored_features=[f], label=(
                        f"Features: {_ranges([g for g in feats if g != f])}" if label_mode == LabelMode.AddFeature
                        else f"Ignore: {f}")))
            elif et in (EvalType.SeqAdd, EvalType.SeqAddAndAll):
                for f in feats:
                    cases.append(ExecutionCase(params, ignored_features=[g for g in feats if g != f],
                                               label=f"Features: {f}"))
        return baseline, cases

    def _calculate_result_metrics(self, cases, metrics, thread_count=-1, evaluation_step=1):
        from ..core import CatBoost
        if len(set(cases)) != len(cases):
            raise CatBoostError(f"Found duplicate cases in {cases}")
        if self._fold_count <= self._fold_offset:
            raise AttributeError(f"Count of folds(folds_count - offset) need to be at least one: offset "
                                 f"{self._fold_offset}, folds_count {self._fold_count}.")
        pool = self._load()
        folds = self._folds(pool)
        learn_ids = list(range(self._fold_offset, min(self._fold_count, len(folds))))
        if not learn_ids:
            raise CatBoostError("fold_offset leaves no fold to learn on")
        metrics = [str(m) for m in metrics]
        step = max(1, int(evaluation_step))
        results = {m: {c: CaseEvaluationResult(c, m, step) for c in cases} for m in metrics}
        n = pool.num_row()
        for fid in learn_ids:
            learn = pool.slice(folds[fid])
            rest_mask = np.ones(n, dtype=bool)
            rest_mask[folds[fid]] = False
            rest = pool.slice(np.nonzero(rest_mask)[0])
            for case in cases:
                p = case.get_params()
                p.setdefault("verbose", False)
                p.setdefault("allow_writing_files", False)
                if thread_count is not None and thread_count != -1:
                    p["thread_count"] = thread_count
                model = CatBoost(p).fit(learn)
                curves = model.eval_metrics(rest, metrics, eval_period=step)
                for m in metrics:
                    results[m][case]._add(fid, curves[m])
        return EvaluationResults([MetricEvaluationResult([results[m][c] for c in cases]) for m in metrics])

    def eval_features(self, learn_config, features_to_eval, loss_function=None, eval_type=EvalType.SeqAdd, eval_metrics=None,
                      thread_count=-1, eval_step=None, label_mode=LabelMode.AddFeature):
        """Baseline = all evaluated features ignored; test cases bring them back according to ``eval_type``."""
        params = dict(learn_config.get_params() if hasattr(learn_config, "get_params") else learn_config)
        if loss_function is not None:
            if "loss_function" in params and params["loss_function"] != loss_function:
                raise CatBoostError(f"Loss function in params {params['loss_function']} should be equal to feature "
                                    f"evaluation objective function {loss_function}")
            params["loss_function"] = loss_function
        elif "loss_function" not in params:
            raise CatBoostError("Provide loss function in params or as option to eval_features method")
        if params["loss_function"] == "PairLogit":
            raise CatBoostError("Pair classification is not supported")
        metrics = list(eval_metrics) if isinstance(eval_metrics, (list, tuple)) else ([] if eval_metrics is None else [eval_metrics])
        if params["loss_function"] not in metrics:
            metrics.append(params["loss_function"])
        baseline, cases = self._create_eval_feature_cases(params, features_to_eval, eval_type, label_mode)
        return self.eval_cases(baseline, cases, metrics, thread_count=thread_count, eval_step=eval_step or 1)

    def eval_cases(self, baseline_case, compare_cases, eval_metrics, thread_count=-1, eval_step=1):
        compare = list(compare_cases) if isinstance(compare_cases, (list, tuple)) else [compare_cases]
        metrics = list(eval_metrics) if isinstance(eval_metrics, (list, tuple)) else [eval_metrics]
        res = self._calculate_result_metrics([baseline_case] + compare, metrics, thread_count=thread_count,
                                             evaluation_step=eval_step)
        res.set_baseline_case(baseline_case)
        return res
