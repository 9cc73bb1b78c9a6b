"""Boosting driver: data preparation, trainer selection, the iteration loop with metrics / overfitting detector /
snapshots / callbacks, and assembly of the final model.

Corresponds to the reference's ``TrainModel`` -> ``TBoosting::Run`` / ``Train`` path
(catboost/libs/train_lib/train_model.cpp:950-1179, catboost/cuda/methods/doc_parallel_boosting.h:302-529,
catboost/private/libs/algo/train.cpp:170-402) with one structural difference: on the GPU the symmetric-tree /
pointwise case never returns to the host inside an iteration (see ``gpu_engine``).
"""
from __future__ import annotations

import math
import os
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import numpy as np
import torch

from ..data.pool import CatBoostError, Pool
from ..data.quantization import (BinnedStore, FeatureQuantization, FlatFeature, build_quantization, make_store,
                                 pack_columns_into, quantize_floats_into)
from ..metrics import make_metric
from ..models.model import (CatFeatureInfo, FloatFeatureInfo, Model, NonSymmetricTree, ObliviousTree, OneHotFeatureInfo,
                            Split)
from ..params import MULTI_LOSSES, Options, RANKING_LOSSES, resolve_options
from ..parallel.runtime import DistContext
from ..utils.logging import TrainLogger
from ..utils.overfit import OverfittingDetector
from ..utils.profiler import Profiler
from .objectives import make_objective


@dataclass
class TrainResult:
    model: Model
    evals_result: Dict[str, Dict[str, List[float]]]
    best_iteration: Optional[int]
    best_score: Dict[str, Dict[str, float]]
    options: Options
    timings: Dict[str, float] = field(default_factory=dict)
    h2d_bytes: int = 0
    launches_per_iter: int = 0


# ---------------------------------------------------------------------------------------------------------
def _unique_labels(lab: np.ndarray) -> np.ndarray:
    """Distinct label values.  Numeric labels with at most two values (the usual binary target) are recognised by three
    passes instead of a sort (np.unique takes 26 ms on 10.5M floats)."""
    lab = np.asarray(lab)
    if lab.dtype.kind in "fiub" and lab.size:
        mn, mx = lab.min(), lab.max()
        if mn == mn and mx == mx and bool(((lab == mn) | (lab == mx)).all()):
            return np.array([mn] if mn == mx else [mn, mx], dtype=lab.dtype)
    return np.unique(lab)


class LabelCodec:
    """Target preparation: class-name mapping, target border, class weights
    (catboost/private/libs/labels/label_converter.cpp, target/data_providers.cpp)."""

    def __init__(self, o: Options, label: np.ndarray, ctx: DistContext):
        self.loss = o.loss_name
        self.class_names = None
        self.n_classes = None
        self.is_binclass = self.loss in ("Logloss", "CrossEntropy", "Focal")
        self.is_multiclass = self.loss in ("MultiClass", "MultiClassOneVsAll")
        lab = np.asarray(label)
        if self.loss in ("Logloss", "Focal"):
            if o.target_border is not None:
                self.border = float(o.target_border)
                self.class_names = [0, 1]
            else:
                self.border = None
                uniq = sorted(set().union(*ctx.all_gather_object(set(_unique_labels(lab).tolist()))))
                if o.class_names is not None:
                    uniq = list(o.class_names)
                if len(uniq) > 2:
                    raise CatBoostError(f"{self.loss} needs a binary target; got {len(uniq)} distinct values "
                                        "(set target_border or use MultiClass)")
                if len(uniq) < 2 and not o.allow_const_label:
                    raise CatBoostError("target contains only one unique value")
                self.class_names = uniq if len(uniq) == 2 else (uniq + [uniq[0] if not uniq else uniq[0]])[:2]
        elif self.is_multiclass:
            uniq = sorted(set().union(*ctx.all_gather_object(set(_unique_labels(lab).tolist()))))
            if o.class_names is not None:
                uniq = list(o.class_names)
            if o.classes_count:
                uniq = list(range(int(o.classes_count)))
            self.class_names = uniq
            self.n_classes = len(uniq)
            if self.n_classes < 2 and not o.allow_const_label:
                raise CatBoostError("target contains only one unique value")

    def _map(self, lab: np.ndarray) -> np.ndarray:
        names = self.class_names
        # few numeric classes: one vectorised comparison per class (a search per label costs a second per 10M rows)
        if lab.dtype.kind in "fiub" and lab.size and len(names) <= 32 and \
                all(isinstance(v, (int, float, np.integer, np.floating)) for v in names):
            out = np.zeros(lab.shape, dtype=np.float32)
            hits = 0
            for i, v in enumerate(names):
                m = lab == v
                hits += int(np.count_nonzero(m))
                if i == 1:
                    out += m
                elif i:
                    out += m.astype(np.float32) * np.float32(i)
            if hits != lab.size:
                bad = lab[~np.isin(lab, np.asarray(names, dtype=lab.dtype))]
                raise CatBoostError(f"label {bad[0]!r} was not seen in the training data")
            return out
        try:
            arr = np.asarray(names, dtype=lab.dtype if lab.dtype.kind in "fiub" else None)
            order = np.argsort(arr, kind="stable")
            srt = arr[order]
            pos = np.clip(np.searchsorted(srt, lab), 0, len(srt) - 1)
            ok = srt[pos] == lab
            if not bool(np.all(ok)):
                bad = lab[~ok][0]
                raise CatBoostError(f"label {bad!r} was not seen in the training data")
            return order[pos].astype(np.float32)
        except TypeError:
            m = {v: i for i, v in enumerate(names)}
            try:
                return np.array([m[v] for v in lab.tolist()], dtype=np.float32)
            except KeyError as e:
                raise CatBoostError(f"label {e.args[0]!r} was not seen in the training data")

    def encode(self, label) -> np.ndarray:
        lab = np.asarray(label)
        if self.loss in ("Logloss", "Focal"):
            if self.border is not None:
                return (lab.astype(np.float64) > self.border).astype(np.float32)
            return self._map(lab)
        if self.is_multiclass:
            return self._map(lab)
        if lab.dtype == object or lab.dtype.kind in "US":
            raise CatBoostError("string labels need a classification loss")
        return lab.astype(np.float32)


def class_weight_vector(o: Options, codec: LabelCodec, y: np.ndarray) -> Optional[np.ndarray]:
    cw = o.class_weights
    if o.scale_pos_weight is not None:
        cw = [1.0, float(o.scale_pos_weight)]
    if cw is None and o.auto_class_weights not in (None, "None"):
        k = 2 if codec.is_binclass else (codec.n_classes or 2)
        counts = np.bincount(y.astype(np.int64), minlength=k).astype(np.float64)
        if o.auto_class_weights == "Balanced":
            cw = counts.max() / np.maximum(counts, 1)
        elif o.auto_class_weights == "SqrtBalanced":
            cw = np.sqrt(counts.max() / np.maximum(counts, 1))
        else:
            raise CatBoostError(f"unknown auto_class_weights {o.auto_class_weights!r}")
    if cw is None:
        return None
    if isinstance(cw, dict):
        cw = [float(cw.get(c, 1.0)) for c in (codec.class_names or sorted(cw))]
    cw = np.asarray(cw, dtype=np.float32)
    return cw[y.astype(np.int64)]


# ---------------------------------------------------------------------------------------------------------
class FeaturePlan:
    """Which flat (binned) features exist and how they map to model splits."""

    def __init__(self):
        self.features: List[FlatFeature] = []
        self.quant: Optional[FeatureQuantization] = None
        self.float_subset: List[int] = []
        self.onehot: Dict[int, np.ndarray] = {}       # cat feature index -> sorted uint32 values
        self.ctr_plan = None


def plan_features(o: Options, pool: Pool, ctx: DistContext, quant: Optional[FeatureQuantization]) -> FeaturePlan:
    plan = FeaturePlan()
    ignored = set()
    for x in (o.ignored_features or []):
        ignored.add(pool.feature_names.index(x) if isinstance(x, str) and x in pool.feature_names else int(x))
    if quant is None:
        quant = build_quantization(pool, int(o.border_count), o.feature_border_type, o.nan_mode,
                                   o.per_float_feature_quantization, o.input_borders, seed=int(o.random_seed),
                                   ctx=ctx if ctx.is_distributed else None)
    plan.quant = quant
    for j, c in enumerate(pool.float_feature_indices):
        if c in ignored or len(quant.borders[j]) == 0:
            continue
        plan.float_subset.append(j)
        plan.features.append(FlatFeature("float", j, borders=quant.borders[j], n_bins=len(quant.borders[j]) + 1))
    # float features occupy whole groups so that the quantise kernel writes them without read-modify-write
    while len(plan.features) % 4 != 0 and len(pool.cat_feature_indices) > 0:
        plan.features.append(FlatFeature("float", -1, borders=np.zeros(0, np.float32), n_bins=1))
    ctr_cats = []
    for j, c in enumerate(pool.cat_feature_indices):
        if c in ignored:
            continue
        uniq = pool.cat_distinct_values(j)
        if ctx.is_distributed:
            uniq = np.unique(np.concatenate(ctx.all_gather_object(uniq)))
        if len(uniq) <= 1:
            continue
        if len(uniq) <= int(o.one_hot_max_size):
            plan.onehot[j] = uniq
            plan.features.append(FlatFeature("onehot", j, values=uniq, n_bins=len(uniq)))
        else:
            ctr_cats.append(j)
    if ctr_cats:
        from .ctr import plan_ctrs
        plan.ctr_plan = plan_ctrs(o, pool, ctr_cats, ctx)
    return plan


def onehot_bins(values: np.ndarray, hashes: np.ndarray) -> np.ndarray:
    """bin k = position of the hash among the training values; unseen values get bin 255 (matches nothing)."""
    pos = np.searchsorted(values, hashes)
    pos = np.clip(pos, 0, len(values) - 1)
    ok = values[pos] == hashes
    return np.where(ok, pos, 255).astype(np.uint8)


def build_store(plan: FeaturePlan, pool: Pool, device, feature_weights=None, extra_features=None,
                extra_cols: Optional[torch.Tensor] = None):
    feats = list(plan.features) + list(extra_features or [])
    fw = np.ones(len(feats), dtype=np.float32)
    for i, f in enumerate(feats):
        if f.kind == "float" and f.source < 0:
            fw[i] = 0.0
    if feature_weights is not None:
        for i, f in enumerate(feats):
            if f.kind == "float" and f.source >= 0:
                fw[i] *= float(feature_weights.get(pool.float_feature_indices[f.source], 1.0))
    store = make_store(feats, pool.num_row(), device, fw)
    h2d = 0
    if plan.float_subset:
        h2d += quantize_floats_into(store, pool.float_data, plan.quant, 0, plan.float_subset)
    k = len([f for f in plan.features if f.kind == "float"])
    oh = [f for f in plan.features if f.kind == "onehot"]
    if oh:
        cols = np.stack([onehot_bins(f.values, pool.cat_hashes[f.source]) for f in oh])
        h2d += cols.nbytes
        pack_columns_into(store, torch.from_numpy(cols).to(store.bins.device), k)
    if extra_cols is not None and extra_cols.shape[0] > 0:
        pack_columns_into(store, extra_cols, len(plan.features))
    return store, h2d


# ---------------------------------------------------------------------------------------------------------
def pick_device(o: Options, ctx: DistContext):
    if o.task_type != "GPU":
        return torch.device("cpu")
    if not torch.cuda.is_available():
        raise CatBoostError("task_type='GPU' was requested but no CUDA device is available")
    from ..params import parse_devices
    devs = parse_devices(o.devices, torch.cuda.device_count())
    if ctx.is_distributed:
        local = int(os.environ.get("LOCAL_RANK", ctx.rank % max(1, torch.cuda.device_count())))
        idx = devs[local % len(devs)] if len(devs) >= ctx.world else local
    else:
        idx = devs[0]
    torch.cuda.set_device(idx)
    return torch.device("cuda", idx)


def _metric_list(o: Options):
    descs = [o.eval_metric] if isinstance(o.eval_metric, str) else [o.eval_metric]
    for extra in (o.custom_metric, o.custom_loss):
        if extra is None:
            continue
        descs += [extra] if isinstance(extra, str) else list(extra)
    if isinstance(o.loss_function, str) and o.loss_function not in descs and not o.loss_function.startswith("PythonUserDefined"):
        descs.append(o.loss_function)
    out, seen = [], set()
    from ..metrics import BuiltinMetric
    descs = [str(d) if isinstance(d, BuiltinMetric) else d for d in descs]        # metric objects: their description
    for d in descs:
        if not isinstance(d, str):
            out.append(d)
            continue
        if d not in seen:
            seen.add(d)
            try:
                out.append(make_metric(d))
            except ValueError as e:
                raise CatBoostError(str(e))
    return out


class _UserMetric:
    """Python custom metric object with evaluate / get_final_error / is_max_optimal."""

    def __init__(self, obj):
        self.obj, self.desc, self.name = obj, type(obj).__name__, type(obj).__name__
        self.is_max_optimal = bool(obj.is_max_optimal())

    def __str__(self):
        return self.desc

    def eval(self, approx, target, weight=None, **kw):
        a = np.asarray(approx, dtype=np.float64)
        cols = [a[:, k] for k in range(a.shape[1])] if a.ndim == 2 else [a]
        err, wsum = self.obj.evaluate(cols, np.asarray(target), None if weight is None else np.asarray(weight))
        return float(self.obj.get_final_error(err, wsum))


# ---------------------------------------------------------------------------------------------------------
def train_model(params: dict, train_pool: Pool, eval_pools: Optional[List[Pool]] = None, *, default_loss="RMSE",
                init_model: Optional[Model] = None, ctx: Optional[DistContext] = None, callbacks=None,
                log_cout=None, record_timings: bool = True) -> TrainResult:
    t_start = time.time()
    eval_pools = list(eval_pools or [])
    ctx = ctx or DistContext.current()
    if train_pool.label is None:
        raise CatBoostError("the training pool has no label")
    user_obj = params.get("loss_function") if params and not isinstance(params.get("loss_function"), (str, type(None))) else None
    p = dict(params or {})
    if user_obj is not None:
        # objects with calc_ders_multi drive a multi-dimensional model (one dimension per target column or per class)
        p["loss_function"] = "PythonUserDefinedMultiTarget" if hasattr(user_obj, "calc_ders_multi") else "PythonUserDefinedPerObject"
    n_rows = train_pool.num_row()
    if ctx.is_distributed:
        n_rows = int(sum(ctx.all_gather_object(n_rows)))
    o = resolve_options(p, default_loss=default_loss, n_rows=n_rows, has_cat=bool(train_pool.cat_feature_indices),
                        has_eval=bool(eval_pools))
    prof = Profiler(enabled=record_timings)
    device = pick_device(o, ctx)
    ctx.device = device
    if o.task_type == "CPU" and int(o.thread_count) > 0:
        from ..ops import native
        native.cpu_lib().cbc_set_num_threads(int(o.thread_count))
        torch.set_num_threads(int(o.thread_count))

    # ---- targets ---------------------------------------------------------------------------------------
    codec = LabelCodec(o, train_pool.label, ctx)
    multi_target = o.loss_name in ("MultiRMSE", "MultiLogloss", "MultiCrossEntropy", "SurvivalAft")
    user_dims = None
    if o.loss_name == "PythonUserDefinedMultiTarget":
        lab2 = np.asarray(train_pool.label)
        multi_target = lab2.ndim == 2 and lab2.shape[1] > 1
        if not multi_target:
            # class labels 0 .. K-1: one dimension per class
            user_dims = int(o.classes_count) if o.classes_count else int(np.asarray(lab2, dtype=np.float64).max()) + 1
            if o.eval_metric == "MultiRMSE":
                o.eval_metric = "MultiClass"
    if multi_target:
        y_train = np.asarray(train_pool.label, dtype=np.float32).reshape(train_pool.num_row(), -1)
        n_targets = y_train.shape[1]
    else:
        y_train = codec.encode(train_pool.label)
        n_targets = 1
    objective = make_objective(user_obj if user_obj is not None else o.loss_name, o.loss_params,
                               n_classes=codec.n_classes if user_dims is None else user_dims, n_targets=n_targets)
    dims = objective.dims
    w_train = train_pool.weight
    cw = class_weight_vector(o, codec, y_train) if objective.is_classification and not multi_target else None
    if cw is not None:
        w_train = cw if w_train is None else w_train * cw
    if objective.needs_groups and train_pool.group_id is None:
        raise CatBoostError(f"{o.loss_name} needs group_id")
    if o.loss_name == "Cox" and ctx.is_distributed:
        raise CatBoostError("Cox couples all documents through one sorted pass: train it on one rank")
    if o.loss_name == "SurvivalAft" and n_targets != 2:
        raise CatBoostError("SurvivalAft needs two label columns: lower and upper bound (-1 = open end)")

    # ---- text / embedding columns -> estimated numeric features ----------------------------------------
    estimators = None
    if getattr(train_pool, "text_data", None) or getattr(train_pool, "embedding_data", None):
        if ctx.is_distributed:
            raise CatBoostError("text and embedding features are supported on one rank only")
        if multi_target:
            raise CatBoostError("text and embedding features need a single target")
        from ..data.estimated import EstimatedFeatures
        with prof.span("estimated_features"):
            estimators = EstimatedFeatures(o.text_processing if isinstance(o.text_processing, dict) else None,
                                           seed=int(o.random_seed), tokenizers=o.tokenizers, dictionaries=o.dictionaries,
                                           feature_calcers=o.feature_calcers)
            n_cls = (codec.n_classes or 2) if objective.is_classification else 0
            estimators.set_device(device if device.type == "cuda" else None)
            learn = estimators.fit(train_pool, np.asarray(y_train), int(n_cls))
            train_pool = train_pool.with_estimated(learn, estimators.names)
            eval_pools = [ep.with_estimated(estimators.transform(ep), estimators.names) for ep in eval_pools]
            estimators.set_device(None)                   # the stored model searches on the host

    # ---- features --------------------------------------------------------------------------------------
    with prof.span("quantization"):
        with prof.span("quantization.borders"):
            plan = plan_features(o, train_pool, ctx, getattr(train_pool, "_quantized", None))
        if o.output_borders and (ctx is None or ctx.rank == 0):
            # the border grid that training uses, one "float_feature_index<TAB>border" line each (output_borders option)
            with open(o.output_borders, "w") as fh:
                for f, b in enumerate(plan.quant.borders):
                    for v in b:
                        fh.write(f"{f}\t{float(v):.9g}\n")
        fweights = None
        if o.feature_weights is not None:
            fw = o.feature_weights
            fweights = ({i: float(v) for i, v in enumerate(fw)} if not isinstance(fw, dict) else
                        {(train_pool.feature_names.index(k) if isinstance(k, str) else int(k)): float(v) for k, v in fw.items()})
        ctr_state = None
        extra_feats, extra_cols, eval_extra_cols = [], None, [None] * len(eval_pools)
        if plan.ctr_plan is not None:
            from .ctr import compute_ctr_features
            with prof.span("quantization.ctrs"):
                ctr_state = compute_ctr_features(plan.ctr_plan, o, train_pool, y_train, w_train, eval_pools, device, ctx,
                                                 codec)
            extra_feats, extra_cols, eval_extra_cols = ctr_state.flat_features, ctr_state.train_bins, ctr_state.eval_bins
        store, h2d_bytes = build_store(plan, train_pool, device, fweights, extra_feats, extra_cols)
        if store.F == 0 or all(f.n_bins <= 1 for f in store.features):
            raise CatBoostError("all features are constant or ignored: nothing to train on")
        eval_stores = []
        for ep, ec in zip(eval_pools, eval_extra_cols):
            es, b = build_store(plan, _align_pool(ep, train_pool), device, None, extra_feats, ec)
            h2d_bytes += b
            eval_stores.append(es)

    # ---- starting approx -------------------------------------------------------------------------------
    n = train_pool.num_row()
    bias = np.zeros(dims)
    if init_model is not None:
        fd, ch = init_model.pool_arrays(train_pool)
        base_train = init_model.predict_raw(fd, ch).T
        base_evals = []
        for ep in eval_pools:
            fd, ch = init_model.pool_arrays(ep)
            base_evals.append(init_model.predict_raw(fd, ch).T)
    else:
        if train_pool.baseline is None and o.boost_from_average:
            bias = np.asarray(_global_start_constant(objective, y_train, w_train, ctx), dtype=np.float64).reshape(dims)
        base_train = np.repeat(bias.reshape(dims, 1), n, axis=1)
        if train_pool.baseline is not None:
            base_train = base_train + np.asarray(train_pool.baseline).T.reshape(dims, n)
        base_evals = []
        for ep in eval_pools:
            b = np.repeat(bias.reshape(dims, 1), ep.num_row(), axis=1)
            if ep.baseline is not None:
                b = b + np.asarray(ep.baseline).T.reshape(dims, -1)
            base_evals.append(b)

    # ---- eval targets ----------------------------------------------------------------------------------
    eval_y, eval_w = [], []
    for ep in eval_pools:
        if ep.label is None:
            raise CatBoostError("evaluation pool has no label")
        eval_y.append(np.asarray(ep.label, dtype=np.float32).reshape(ep.num_row(), -1) if multi_target
                      else codec.encode(ep.label))
        eval_w.append(ep.weight)

    metrics = [m if not (hasattr(m, "evaluate") and not hasattr(m, "eval")) else _UserMetric(m) for m in _metric_list(o)]
    eval_metric = metrics[0]
    logger = TrainLogger(o, [str(m) for m in metrics], len(eval_pools), log_cout, enabled=(ctx.rank == 0))
    od = OverfittingDetector(o.od_type, int(o.od_wait), float(o.od_pval), eval_metric.is_max_optimal) \
        if eval_pools and (o.od_type == "Iter" or float(o.od_pval) > 0 or "od_wait" in o["_user_keys"]) else None

    from .loop import run_boosting
    res = run_boosting(o, objective, store, eval_stores, y_train, w_train, base_train, eval_y, eval_w, base_evals,
                       train_pool, eval_pools, metrics, logger, od, ctx, prof, callbacks, plan, ctr_state)

    # ---- model ----------------------------------------------------------------------------------------
    with prof.span("model"):
        model = assemble_model(o, plan, train_pool, store, res.trees, dims, bias if init_model is None else np.zeros(dims),
                               codec, ctr_state)
        if init_model is not None:
            from ..models.ops import sum_models
            model = sum_models([init_model, model], [1.0, 1.0])
        best_it = res.best_iteration
        if o.use_best_model and best_it is not None and eval_pools:
            keep = max(best_it + 1, int(o.best_model_min_trees))
            base_trees = init_model.tree_count if init_model is not None else 0
            model.shrink(base_trees + keep)
        model.estimators = estimators
        model.params = {k: v for k, v in o.items() if not k.startswith("_") and k != "callback"}
        model.info["params"] = o.to_json()
        model.info["catboost_b200_version"] = "0.1"
        model.info["train_finish_time"] = time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime())
    timings = prof.report()
    timings["total"] = time.time() - t_start
    logger.close()
    return TrainResult(model, res.evals_result, res.best_iteration, res.best_score, o, timings, h2d_bytes,
                       res.launches_per_iter)


def _align_pool(ep: Pool, train_pool: Pool) -> Pool:
    if ep.n_features != train_pool.n_features:
        raise CatBoostError(f"evaluation pool has {ep.n_features} features, training pool has {train_pool.n_features}")
    if list(ep.cat_feature_indices) != list(train_pool.cat_feature_indices):
        raise CatBoostError("categorical feature indices differ between the training and evaluation pools")
    return ep


def _global_start_constant(objective, y, w, ctx: DistContext):
    c = np.asarray(objective.start_constant(y, w), dtype=np.float64)
    if not ctx.is_distributed:
        return c
    parts = ctx.all_gather_object((c, float(len(y)) if w is None else float(np.sum(w))))
    tot = sum(p[1] for p in parts)
    if objective.name in ("Logloss", "CrossEntropy"):
        pm = sum(1.0 / (1.0 + np.exp(-p[0])) * p[1] for p in parts) / tot
        return np.log(pm / (1 - pm))
    return sum(p[0] * p[1] for p in parts) / tot


# ---------------------------------------------------------------------------------------------------------
def assemble_model(o: Options, plan: FeaturePlan, pool: Pool, store: BinnedStore, trees, dims: int, bias, codec,
                   ctr_state=None) -> Model:
    m = Model()
    m.dims = dims
    m.bias = np.asarray(bias, dtype=np.float64).reshape(dims)
    m.loss_name = o.loss_name
    m.class_names = codec.class_names
    m.feature_names = list(pool.feature_names)
    m.n_features = pool.n_features
    q = plan.quant
    for j, c in enumerate(pool.float_feature_indices):
        m.float_features.append(FloatFeatureInfo(c, j, np.asarray(q.borders[j], dtype=np.float32),
                                                 "Max" if q.nan_is_max[j] else "Min", bool(q.has_nan[j]),
                                                 pool.feature_names[c]))
    for j, c in enumerate(pool.cat_feature_indices):
        m.cat_features.append(CatFeatureInfo(c, j, pool.feature_names[c]))
        for s, h in pool.cat_strings[j].items():
            m.cat_hash_to_string[int(h)] = s
    for j, vals in plan.onehot.items():
        m.one_hot[j] = OneHotFeatureInfo(j, vals)
    if ctr_state is not None:
        m.ctrs = ctr_state.model_ctrs
    feats = store.features

    def to_split(f: int, b: int) -> int:
        ff = feats[f]
        if ff.kind == "float":
            return m.split_index(Split("float", ff.source, border=float(ff.borders[b])))
        if ff.kind == "onehot":
            return m.split_index(Split("onehot", ff.source, value=int(ff.values[b])))
        return m.split_index(Split("ctr", ff.source, border=float(ff.borders[b])))

    for t in trees:
        if t["kind"] == "oblivious":
            sp = t["splits"]
            vals = np.asarray(t["values"], dtype=np.float64).reshape(-1, dims)
            wts = np.asarray(t["weights"], dtype=np.float64).reshape(-1)
            depth = sp.shape[0]
            keep_levels = [k for k in range(depth) if sp[k, 0] >= 0]
            if len(keep_levels) != depth:
                # drop empty levels: keep the leaves whose bit for a dropped level is 0
                idx = np.arange(1 << len(keep_levels))
                full = np.zeros_like(idx)
                for newk, k in enumerate(keep_levels):
                    full |= ((idx >> newk) & 1) << k
                vals, wts = vals[full], wts[full]
            m.trees.append(ObliviousTree([to_split(int(sp[k, 0]), int(sp[k, 1])) for k in keep_levels], vals, wts))
        else:
            ns = t["node_split"]
            split_of_node = np.full(len(ns), -1, dtype=np.int32)
            left = np.zeros(len(ns), dtype=np.int32)
            right = np.zeros(len(ns), dtype=np.int32)
            for k in range(len(ns)):
                if ns[k, 0] >= 0:
                    split_of_node[k] = to_split(int(ns[k, 0]), int(ns[k, 1]))
                    left[k], right[k] = ns[k, 3], ns[k, 3] + 1
            m.trees.append(NonSymmetricTree(split_of_node, left, right, t["leaf_of_node"].astype(np.int32),
                                            np.asarray(t["values"], dtype=np.float64).reshape(-1, dims),
                                            np.asarray(t["weights"], dtype=np.float64).reshape(-1)))
    return m
