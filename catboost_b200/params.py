"""Training options: CatBoost-named flat parameters -> validated, defaulted option set.

Reproduces the parts of the reference's option system that the trainers consume
(catboost/private/libs/options/: plain_options_helper.cpp for the flat names, catboost_options.cpp:31-271
for the per-loss leaf-estimation defaults, :774-990 for cross defaults, defaults_helper.h:33-42 for the
boosting-type rule, data_processing_options.cpp:16 for border_count 128 on GPU / 254 on CPU,
catboost/python-package/catboost/core.py:1601-1700 for the synonyms).
"""
from __future__ import annotations

import copy
import json
import re
from typing import Any, Dict, Optional

from .data.pool import CatBoostError

SYNONYMS = {
    "objective": "loss_function", "eta": "learning_rate", "n_estimators": "iterations", "num_boost_round": "iterations",
    "num_trees": "iterations", "max_depth": "depth", "reg_lambda": "l2_leaf_reg", "random_state": "random_seed",
    "max_bin": "border_count", "colsample_bylevel": "rsm", "min_child_samples": "min_data_in_leaf",
    "num_leaves": "max_leaves", "verbose_eval": "verbose", "early_stopping_rounds": "od_wait_alias",
    "scale_pos_weight": "scale_pos_weight",
}

DEFAULTS: Dict[str, Any] = dict(
    iterations=1000, learning_rate=None, depth=6, l2_leaf_reg=None, model_size_reg=0.5, rsm=1.0,
    loss_function=None, border_count=None, feature_border_type="GreedyLogSum", per_float_feature_quantization=None,
    input_borders=None, output_borders=None, fold_permutation_block=None, od_pval=0.0, od_wait=20, od_type="IncToDec",
    nan_mode="Min", counter_calc_method="SkipTest", leaf_estimation_iterations=None, leaf_estimation_method=None,
    thread_count=-1, random_seed=0, use_best_model=None, best_model_min_trees=1, verbose=None, silent=None,
    logging_level=None, metric_period=1, ctr_leaf_count_limit=None, store_all_simple_ctr=False, max_ctr_complexity=None,
    has_time=False, allow_const_label=False, target_border=None, classes_count=None, class_weights=None,
    auto_class_weights=None, class_names=None, one_hot_max_size=None, random_strength=1.0, random_score_type="NormalWithModelSizeDecrease",
    name="experiment", ignored_features=None, train_dir="catboost_info", custom_loss=None, custom_metric=None,
    eval_metric=None, bagging_temperature=None, save_snapshot=None, snapshot_file=None, snapshot_interval=600,
    fold_len_multiplier=2.0, used_ram_limit=None, gpu_ram_part=0.95, pinned_memory_size=1 << 30,
    allow_writing_files=True, final_ctr_computation_mode="Default", approx_on_full_history=False,
    boosting_type=None, simple_ctr=None, combinations_ctr=None, per_feature_ctr=None, ctr_description=None,
    ctr_target_border_count=None, ctr_border_count=15, task_type="CPU", device_config=None, devices=None,
    bootstrap_type=None, subsample=None, mvs_reg=None, sampling_frequency="PerTree", sampling_unit="Object",
    dev_score_calc_obj_block_size=None, dev_efb_max_buckets=None, sparse_features_conflict_fraction=0.0,
    grow_policy="SymmetricTree", min_data_in_leaf=1, max_leaves=31, score_function=None, leaf_estimation_backtracking=None,
    ctr_history_unit="Sample", monotone_constraints=None, feature_weights=None, penalties_coefficient=1.0,
    first_feature_use_penalties=None, per_object_feature_penalties=None, model_shrink_rate=None,
    model_shrink_mode=None, langevin=False, diffusion_temperature=10000.0, posterior_sampling=False,
    boost_from_average=None, text_features=None, tokenizers=None, dictionaries=None, feature_calcers=None,
    text_processing=None, embedding_features=None, eval_fraction=None, fixed_binary_splits=None,
    data_partition=None, permutation_count=None, min_fold_size=100, cat_features=None, scale_pos_weight=None,
    gpu_cat_features_storage="GpuRam", observations_to_bootstrap="TestOnly", fused_levels=True,
    histogram_reduce="fused", histogram_cells="narrow", bayesian_matrix_reg=0.1, node_type="SingleHost", callback=None,
)

GPU_ONLY = {"gpu_ram_part", "pinned_memory_size", "gpu_cat_features_storage", "data_partition", "fold_len_multiplier",
            "min_fold_size", "observations_to_bootstrap", "devices", "fused_levels", "histogram_reduce", "histogram_cells"}
CPU_ONLY = {"rsm", "sampling_frequency", "approx_on_full_history", "model_shrink_rate", "model_shrink_mode",
            "langevin", "diffusion_temperature", "posterior_sampling", "monotone_constraints", "dev_efb_max_buckets",
            "sparse_features_conflict_fraction", "random_score_type"}

# Options that only steer how much memory or which internal block sizes the reference uses: accepted for script
# compatibility, they have no counterpart here and change no result.
RESOURCE_HINTS = {"used_ram_limit", "gpu_ram_part", "pinned_memory_size", "device_config", "gpu_cat_features_storage",
                  "data_partition", "node_type", "dev_score_calc_obj_block_size", "dev_efb_max_buckets",
                  "observations_to_bootstrap", "fused_levels", "model_size_reg"}
# Options of the reference whose behaviour is not implemented: a value that differs from the default is refused with an
# error instead of being silently dropped.
NOT_IMPLEMENTED = {"counter_calc_method", "ctr_leaf_count_limit", "store_all_simple_ctr", "final_ctr_computation_mode",
                   "ctr_history_unit", "approx_on_full_history", "fixed_binary_splits",
                   "sparse_features_conflict_fraction"}

POINTWISE_LOSSES = {"RMSE", "Logloss", "CrossEntropy", "Poisson", "MAE", "Quantile", "LogLinQuantile", "MAPE", "Huber",
                    "Lq", "Expectile", "Tweedie", "LogCosh", "Focal"}
MULTI_LOSSES = {"MultiClass", "MultiClassOneVsAll", "MultiLogloss", "MultiCrossEntropy", "MultiRMSE", "RMSEWithUncertainty",
                "MultiQuantile", "PythonUserDefinedMultiTarget"}
SURVIVAL_LOSSES = {"Cox", "SurvivalAft"}
COMBINED_LOSSES = {"Combination"}
RANKING_LOSSES = {"YetiRank", "YetiRankPairwise", "PairLogit", "PairLogitPairwise", "QueryRMSE", "QuerySoftMax",
                  "QueryCrossEntropy", "LambdaMart", "StochasticRank", "StochasticFilter", "GroupQuantile"}
PAIRWISE_HIST_LOSSES = {"YetiRankPairwise", "PairLogitPairwise", "QueryCrossEntropy"}
ALL_LOSSES = (POINTWISE_LOSSES | MULTI_LOSSES | RANKING_LOSSES | SURVIVAL_LOSSES | COMBINED_LOSSES
              | {"PythonUserDefinedPerObject", "PythonUserDefinedMultiTarget"})

# (newton iterations, gradient iterations, method, l2)  -- catboost_options.cpp:31-271
_LEAF_DEFAULTS = {
    "RMSE": (1, 1, "Newton", 3.0), "MultiRMSE": (1, 1, "Newton", 3.0), "RMSEWithUncertainty": (1, 1, "Newton", 3.0),
    "Huber": (1, 1, "Newton", 3.0), "LogCosh": (1, 1, "Exact", 3.0), "QueryRMSE": (1, 1, "Newton", 3.0),
    "QuerySoftMax": (10, 100, "Gradient", 3.0), "MultiClass": (1, 10, "Newton", 3.0),
    "MultiClassOneVsAll": (1, 10, "Newton", 3.0), "MAE": (1, 1, "Gradient", 3.0), "MAPE": (1, 1, "Gradient", 3.0),
    "Quantile": (1, 1, "Gradient", 3.0), "LogLinQuantile": (1, 1, "Gradient", 3.0), "Expectile": (5, 10, "Newton", 3.0),
    "PairLogit": (10, 40, "Newton", 3.0), "PairLogitPairwise": (1, 5, "Newton", 5.0), "Poisson": (10, 1, "Newton", 3.0),
    "Logloss": (10, 40, "Newton", 3.0), "CrossEntropy": (10, 40, "Newton", 3.0), "MultiLogloss": (10, 40, "Newton", 3.0),
    "MultiCrossEntropy": (10, 40, "Newton", 3.0), "YetiRank": (1, 1, "Newton", 0.0),
    "YetiRankPairwise": (1, 1, "Simple", 0.0), "QueryCrossEntropy": (10, 1, "Newton", 1.0),
    "LambdaMart": (1, 1, "Newton", 0.0), "StochasticRank": (1, 1, "Gradient", 3.0),
    "StochasticFilter": (1, 100, "Gradient", 3.0), "Tweedie": (1, 1, "Newton", 3.0), "Lq": (1, 1, "Newton", 3.0),
    "PythonUserDefinedPerObject": (1, 1, "Gradient", 3.0), "PythonUserDefinedMultiTarget": (1, 1, "Newton", 3.0),
    "MultiQuantile": (1, 1, "Gradient", 3.0),
    "GroupQuantile": (1, 1, "Gradient", 3.0), "Focal": (1, 1, "Newton", 3.0), "Cox": (1, 1, "Newton", 3.0),
    "SurvivalAft": (1, 1, "Gradient", 3.0),
}


def parse_loss(desc: str):
    """``'Quantile:alpha=0.3;delta=0.01'`` -> ('Quantile', {'alpha': 0.3, 'delta': 0.01})."""
    if not isinstance(desc, str):
        return "PythonUserDefinedPerObject", {}
    name, _, rest = desc.partition(":")
    params = {}
    if rest:
        for tok in re.split(r"[;,]", rest):
            if not tok:
                continue
            if "=" not in tok and params:
                # 'alpha=0.2,0.8': a bare token continues the list value of the key before it
                last = next(reversed(params))
                params[last] = f"{params[last]:g},{tok.strip()}" if isinstance(params[last], float) else f"{params[last]},{tok.strip()}"
                continue
            k, _, v = tok.partition("=")
            try:
                params[k.strip()] = float(v)
            except ValueError:
                params[k.strip()] = v.strip()
    return name.strip(), params


def parse_devices(spec, available: Optional[int] = None):
    """``'0'``, ``'0:1:3'``, ``'0-7'``, ``'-1'`` (all) -> sorted list of ordinals
    (catboost/cuda/cuda_lib/devices_provider.h:33-44, helpers.h ParseRangeString)."""
    if spec is None or spec == "" or spec == "-1" or spec == -1:
        return list(range(available)) if available is not None else [0]
    if isinstance(spec, int):
        return [spec]
    if isinstance(spec, (list, tuple)):
        return sorted({int(x) for x in spec})
    out = set()
    for part in str(spec).split(":"):
        part = part.strip()
        if "-" in part:
            a, b = part.split("-")
            if int(b) < int(a):
                raise CatBoostError(f"bad device range {part!r}")
            out.update(range(int(a), int(b) + 1))
        elif part:
            out.add(int(part))
    out = sorted(out)
    if available is not None and any(d >= available or d < 0 for d in out):
        raise CatBoostError(f"device ordinal out of range in {spec!r} (available: {available})")
    return out


class Options(dict):
    """Resolved options; attribute access for convenience."""

    def __getattr__(self, k):
        try:
            return self[k]
        except KeyError as e:
            raise AttributeError(k) from e

    def __setattr__(self, k, v):
        self[k] = v

    def to_json(self) -> str:
        def enc(o):
            if callable(o) or hasattr(o, "calc_ders_range") or hasattr(o, "evaluate"):
                return f"<python object {type(o).__name__}>"
            if hasattr(o, "tolist"):
                return o.tolist()
            return str(o)
        return json.dumps({k: v for k, v in self.items() if k not in ("callback",)}, default=enc, sort_keys=True)


def normalize_params(params: Optional[dict]) -> dict:
    """Resolve synonyms; reject unknown names and duplicates given through different synonyms."""
    out = {}
    for k, v in (params or {}).items():
        if v is None:
            continue
        name = SYNONYMS.get(k, k)
        if name == "od_wait_alias":
            out["od_type"] = "Iter"
            out["od_wait"] = int(v)
            out["od_pval"] = 0.0
            continue
        if name not in DEFAULTS:
            raise CatBoostError(f"unknown parameter {k!r}")
        if name in out and out[name] != v:
            raise CatBoostError(f"parameter {name!r} is given twice through synonyms")
        if name in ("loss_function", "eval_metric", "custom_metric", "custom_loss"):
            v = _metric_objects_to_text(v)
        out[name] = v
    return out


def _metric_objects_to_text(v):
    """Metric objects of ``catboost_b200.metrics`` (``metrics.AUC(type='Ranking')``) stand for their description."""
    def one(x):
        return str(x) if type(x).__mro__[1:2] and any(c.__name__ == "BuiltinMetric" for c in type(x).__mro__) else x
    if isinstance(v, (list, tuple)):
        return [one(x) for x in v]
    return one(v)


def resolve_options(params: Optional[dict], default_loss: str = "RMSE", n_rows: Optional[int] = None,
                    has_cat: bool = False, n_classes: Optional[int] = None, has_eval: bool = False) -> Options:
    user = normalize_params(params)
    o = Options(copy.copy(DEFAULTS))
    o.update(user)
    o["_user_keys"] = sorted(user.keys())
    task = str(o.task_type).upper()
    if task not in ("CPU", "GPU"):
        raise CatBoostError(f"task_type must be 'CPU' or 'GPU', got {o.task_type!r}")
    o.task_type = task
    for k in user:
        if k in NOT_IMPLEMENTED and user[k] is not None and user[k] != DEFAULTS.get(k):
            raise CatBoostError(f"option {k}={user[k]!r} is not implemented in this framework (only its default "
                                f"{DEFAULTS.get(k)!r} is accepted)")
        # GPU-only knobs on CPU and the resource hints are accepted and change nothing (the reference's TGpuOnlyOption
        # warns and continues)
    # loss
    loss = o.loss_function if o.loss_function is not None else default_loss
    lname, lparams = parse_loss(loss)
    if lname not in ALL_LOSSES:
        raise CatBoostError(f"unknown loss_function {lname!r}")
    o.loss_function = loss
    o["loss_name"], o["loss_params"] = lname, lparams
    # tree
    if not (1 <= int(o.depth) <= 16):
        raise CatBoostError("depth must be in [1, 16]")
    if lname in PAIRWISE_HIST_LOSSES and int(o.depth) > 8:
        raise CatBoostError("pairwise losses support depth <= 8")
    if o.grow_policy not in ("SymmetricTree", "Depthwise", "Lossguide", "Region"):
        raise CatBoostError(f"unknown grow_policy {o.grow_policy!r}")
    if int(o.iterations) < 0:
        raise CatBoostError("iterations must be non-negative")
    if o.border_count is None:
        o.border_count = 128 if task == "GPU" else 254
        if lname in PAIRWISE_HIST_LOSSES and task == "GPU":
            o.border_count = 32
    if not (1 <= int(o.border_count) <= 255):
        raise CatBoostError("border_count must be in [1, 255]")
    nnewton, ngrad, method, l2 = _LEAF_DEFAULTS.get(lname, (1, 1, "Newton", 3.0))
    if lname == "PairLogitPairwise" and task == "CPU":
        method, ngrad = "Gradient", 50
    if lname == "YetiRankPairwise" and task == "CPU":
        method = "Gradient"
    if lname == "Tweedie" and False:
        pass
    if o.leaf_estimation_method is None:
        o.leaf_estimation_method = method
    if o.leaf_estimation_method not in ("Newton", "Gradient", "Exact", "Simple"):
        raise CatBoostError(f"unknown leaf_estimation_method {o.leaf_estimation_method!r}")
    if o.leaf_estimation_iterations is None:
        o.leaf_estimation_iterations = {"Newton": nnewton, "Gradient": ngrad}.get(o.leaf_estimation_method, 1)
    if o.l2_leaf_reg is None:
        o.l2_leaf_reg = l2
    if float(o.l2_leaf_reg) < 0:
        raise CatBoostError("l2_leaf_reg must be non-negative")
    if float(o.l2_leaf_reg) == 0.0:
        o.l2_leaf_reg = 1e-20
    if o.leaf_estimation_backtracking is None:
        o.leaf_estimation_backtracking = "AnyImprovement"
    # score function: Cosine is the default on both devices; non-symmetric trees on GPU need an L2 family
    if o.score_function is None:
        o.score_function = "Cosine"
    if o.score_function not in ("Cosine", "L2", "NewtonCosine", "NewtonL2", "SolarL2", "LOOL2", "SatL2"):
        raise CatBoostError(f"unknown score_function {o.score_function!r}")
    # bootstrap (catboost_options.cpp: GPU default Bayesian; CPU default MVS for non-multiclass with subsample 0.8)
    if o.bootstrap_type is None:
        if o.subsample is not None and o.bagging_temperature is None:
            o.bootstrap_type = "Bernoulli"
        elif task == "GPU" or lname in MULTI_LOSSES or o.bagging_temperature is not None:
            o.bootstrap_type = "Bayesian"
        else:
            o.bootstrap_type = "MVS"
    if o.bootstrap_type not in ("Bayesian", "Bernoulli", "Poisson", "MVS", "No"):
        raise CatBoostError(f"unknown bootstrap_type {o.bootstrap_type!r}")
    if o.bootstrap_type == "Poisson" and task != "GPU":
        raise CatBoostError("Poisson bootstrap is supported on GPU only")
    if o.bootstrap_type == "Bayesian":
        if o.subsample is not None:
            raise CatBoostError("subsample is not used with the Bayesian bootstrap")
        if o.bagging_temperature is None:
            o.bagging_temperature = 1.0
    else:
        if o.bagging_temperature is not None and o.bootstrap_type != "No":
            raise CatBoostError("bagging_temperature requires bootstrap_type='Bayesian'")
        if o.subsample is None:
            o.subsample = {"Bernoulli": 0.66, "Poisson": 0.66, "MVS": 0.8, "No": 1.0}[o.bootstrap_type]
    if o.sampling_unit not in (None, "Object", "Group"):
        raise CatBoostError(f"unknown sampling_unit {o.sampling_unit!r}")
    if o.sampling_unit == "Group" and o.bootstrap_type == "MVS":
        raise CatBoostError("sampling_unit='Group' is not used with the MVS bootstrap")
    if o.posterior_sampling:
        # catboost/libs/train_lib/options_helper.cpp:376-392 and catboost_options.cpp:744-751: Langevin boosting whose
        # diffusion temperature is the number of objects and whose shrink rate is 1 / (2 n)
        if "langevin" in o["_user_keys"] and not o.langevin:
            raise CatBoostError("posterior_sampling requires Langevin boosting")
        if "diffusion_temperature" in o["_user_keys"]:
            raise CatBoostError("diffusion_temperature is set by posterior_sampling")
        if o.model_shrink_mode not in (None, "Constant"):
            raise CatBoostError("posterior_sampling requires the Constant model shrink mode")
        o.langevin = True
        if n_rows:
            o.diffusion_temperature = float(n_rows)
            o.model_shrink_rate = 1.0 / (2.0 * float(n_rows))
    # learning rate (options_helper.cpp:269 auto-tunes from the dataset size; this is the same functional form)
    if o.learning_rate is None:
        o.learning_rate = auto_learning_rate(lname, int(o.iterations), n_rows, has_eval) if n_rows else 0.03
    if float(o.learning_rate) <= 0:
        raise CatBoostError("learning_rate must be positive")
    # boosting type (defaults_helper.h:33-42): Ordered only for small data on GPU-like defaults
    if o.boosting_type is None:
        small = n_rows is not None and n_rows < 50000 and int(o.iterations) >= 500
        nonsym = o.grow_policy != "SymmetricTree"
        o.boosting_type = "Ordered" if (task == "GPU" and small and not nonsym and lname not in MULTI_LOSSES
                                        and lname not in PAIRWISE_HIST_LOSSES and has_cat) else "Plain"
    if o.boosting_type not in ("Plain", "Ordered"):
        raise CatBoostError(f"unknown boosting_type {o.boosting_type!r}")
    if o.boosting_type == "Ordered" and o.grow_policy != "SymmetricTree":
        raise CatBoostError("Ordered boosting supports only SymmetricTree grow policy")
    if o.one_hot_max_size is None:
        o.one_hot_max_size = 2
    if int(o.one_hot_max_size) > 255:
        raise CatBoostError("one_hot_max_size must be <= 255")
    if o.max_ctr_complexity is None:
        o.max_ctr_complexity = 4
    if o.permutation_count is None:
        o.permutation_count = 4 if has_cat else 1
    if o.boost_from_average is None:
        o.boost_from_average = lname in ("RMSE", "Logloss", "CrossEntropy", "Quantile", "MAE", "MAPE", "MultiRMSE")
    if o.use_best_model is None:
        o.use_best_model = bool(has_eval)
    if o.od_type not in ("IncToDec", "Iter", "Wilcoxon"):
        raise CatBoostError(f"unknown od_type {o.od_type!r}")
    if o.eval_metric is None:
        o.eval_metric = default_eval_metric(loss)
    if o.verbose is None and o.silent is None and o.logging_level is None:
        o.verbose = True
    if o.silent:
        o.verbose = False
    if o.logging_level is not None:
        o.verbose = o.logging_level not in ("Silent",)
    if float(o.rsm) <= 0 or float(o.rsm) > 1:
        raise CatBoostError("rsm must be in (0, 1]")
    return o


def auto_learning_rate(loss_name: str, iterations: int, n_rows: int, has_eval: bool) -> float:
    """Data-dependent default learning rate (same functional form as options_helper.cpp:269: an exponential of a
    linear function of log(rows), corrected for the iteration count), rounded to 6 digits."""
    import math
    if loss_name not in ("Logloss", "CrossEntropy", "RMSE", "MultiClass", "MultiClassOneVsAll"):
        return 0.03
    n = max(int(n_rows), 10)
    if has_eval:
        a, b, c, d = 0.105, -3.276, -0.428, 0.911
    else:
        a, b, c, d = 0.283, -6.044, -0.891, 2.620
    custom_iter_const = math.exp(c * math.log(max(iterations, 1)) + d)
    default_iter_const = math.exp(c * math.log(1000) + d)
    default_lr = math.exp(a * math.log(n) + b)
    return round(min(default_lr * custom_iter_const / default_iter_const, 0.5), 6)


def default_eval_metric(loss: str) -> str:
    name, _ = parse_loss(loss)
    return {"YetiRank": "PFound", "YetiRankPairwise": "PFound", "PairLogitPairwise": "PairLogit",
            "LambdaMart": "NDCG", "StochasticRank": "NDCG", "StochasticFilter": "FilteredDCG",
            "PythonUserDefinedPerObject": "RMSE", "PythonUserDefinedMultiTarget": "MultiRMSE"}.get(name, loss)
