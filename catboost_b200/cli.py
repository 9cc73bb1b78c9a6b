"""Command-line interface: ``python -m catboost_b200 <mode> ...`` with the reference's mode names
(catboost/app/main.cpp:21-35): fit, calc, fstr, eval-metrics, metadata, model-sum, normalize-model, select-features,
dataset-statistics, dump-options, roc.  Option names follow catboost/private/libs/app_helpers/bind_options.cpp."""
from __future__ import annotations

import argparse
import json
import sys

import numpy as np


def _add_pool_args(ap, prefix=""):
    ap.add_argument("-f", "--learn-set", dest="learn_set")
    ap.add_argument("-t", "--test-set", dest="test_set", action="append", default=[])
    ap.add_argument("--column-description", "--cd", dest="cd")
    ap.add_argument("--delimiter", default="\t")
    ap.add_argument("--has-header", action="store_true")
    ap.add_argument("--learn-pairs")
    ap.add_argument("--test-pairs")


def _pool(path, args, pairs=None):
    from .data.pool import Pool
    return Pool(path, column_description=args.cd, delimiter=args.delimiter, has_header=args.has_header, pairs=pairs)


_FIT_PARAMS = [("--loss-function", str, "loss_function"), ("-i", int, "iterations"), ("--iterations", int, "iterations"),
               ("-w", float, "learning_rate"), ("--learning-rate", float, "learning_rate"), ("-n", int, "depth"),
               ("--depth", int, "depth"), ("--l2-leaf-reg", float, "l2_leaf_reg"), ("-x", int, "border_count"),
               ("--border-count", int, "border_count"), ("--feature-border-type", str, "feature_border_type"),
               ("-r", int, "random_seed"), ("--random-seed", int, "random_seed"), ("--task-type", str, "task_type"),
               ("--devices", str, "devices"), ("--grow-policy", str, "grow_policy"), ("--max-leaves", int, "max_leaves"),
               ("--min-data-in-leaf", int, "min_data_in_leaf"), ("--bootstrap-type", str, "bootstrap_type"),
               ("--bagging-temperature", float, "bagging_temperature"), ("--subsample", float, "subsample"),
               ("--random-strength", float, "random_strength"), ("--rsm", float, "rsm"),
               ("--leaf-estimation-method", str, "leaf_estimation_method"),
               ("--leaf-estimation-iterations", int, "leaf_estimation_iterations"), ("--score-function", str, "score_function"),
               ("--eval-metric", str, "eval_metric"), ("--custom-metric", str, "custom_metric"),
               ("--one-hot-max-size", int, "one_hot_max_size"), ("--max-ctr-complexity", int, "max_ctr_complexity"),
               ("--od-type", str, "od_type"), ("--od-wait", int, "od_wait"), ("--od-pval", float, "od_pval"),
               ("--metric-period", int, "metric_period"), ("--train-dir", str, "train_dir"),
               ("--snapshot-file", str, "snapshot_file"), ("--snapshot-interval", float, "snapshot_interval"),
               ("-T", int, "thread_count"), ("--thread-count", int, "thread_count"), ("--nan-mode", str, "nan_mode"),
               ("--boosting-type", str, "boosting_type"), ("--boost-from-average", str, "boost_from_average"),
               ("--class-weights", str, "class_weights"), ("--auto-class-weights", str, "auto_class_weights"),
               ("--target-border", float, "target_border"), ("--simple-ctr", str, "simple_ctr"),
               ("--combinations-ctr", str, "combinations_ctr"), ("--ignore-features", str, "ignored_features"),
               ("--permutations", int, "permutation_count"), ("--logging-level", str, "logging_level")]


def _fit_params(args):
    params = {}
    if args.params_file:
        with open(args.params_file) as fh:
            params.update(json.load(fh))
    for _, _, dest in _FIT_PARAMS:
        v = getattr(args, dest, None)
        if v is not None:
            params[dest] = v
    if "class_weights" in params and isinstance(params["class_weights"], str):
        params["class_weights"] = [float(x) for x in params["class_weights"].split(",")]
    if "ignored_features" in params and isinstance(params["ignored_features"], str):
        out = []
        for tok in params["ignored_features"].replace(":", ",").split(","):
            if "-" in tok:
                a, b = tok.split("-")
                out += list(range(int(a), int(b) + 1))
            elif tok:
                out.append(int(tok))
        params["ignored_features"] = out
    if "boost_from_average" in params:
        params["boost_from_average"] = str(params["boost_from_average"]).lower() in ("1", "true", "yes")
    if args.use_best_model is not None:
        params["use_best_model"] = args.use_best_model.lower() in ("1", "true", "yes")
    if args.save_snapshot:
        params["save_snapshot"] = True
    return params


def mode_fit(argv):
    ap = argparse.ArgumentParser(prog="catboost_b200 fit")
    _add_pool_args(ap)
    ap.add_argument("-m", "--model-file", default="model.bin")
    ap.add_argument("--model-format", default="CatboostBinary")
    ap.add_argument("--params-file")
    ap.add_argument("--eval-file")
    ap.add_argument("--use-best-model")
    ap.add_argument("--save-snapshot", action="store_true")
    ap.add_argument("--fstr-file")
    ap.add_argument("--verbose", type=int, default=1)
    for flag, typ, dest in _FIT_PARAMS:
        ap.add_argument(flag, type=typ, dest=dest, default=None)
    args = ap.parse_args(argv)
    if not args.learn_set:
        ap.error("--learn-set is required")
    from .core import CatBoost
    params = _fit_params(args)
    params.setdefault("verbose", bool(args.verbose))
    learn = _pool(args.learn_set, args, args.learn_pairs)
    tests = [_pool(t, args, args.test_pairs) for t in args.test_set]
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        # a rank of a multi-process run (run-worker / torchrun): every rank read the whole file, keeps its row shard
        # (queries whole) and fit() is a collective call
        from .parallel.launcher import shard_bounds
        r, w = dist.get_rank(), dist.get_world_size()
        b = shard_bounds(learn, w)
        learn = learn.slice_range(b[r], b[r + 1])
        tests = [t.slice_range(*[shard_bounds(t, w)[k] for k in (r, r + 1)]) for t in tests]
    model = CatBoost(params)
    model.fit(learn, eval_set=tests or None)
    if dist.is_available() and dist.is_initialized() and dist.get_rank() != 0:
        return 0
    for fmt in args.model_format.split(","):
        fmt = {"CatboostBinary": "cbm", "Json": "json", "Cpp": "cpp", "Python": "python"}.get(fmt, fmt.lower())
        name = args.model_file if fmt == "cbm" else f"{args.model_file}.{fmt}"
        model.save_model(name, format=fmt)
    if args.eval_file and tests:
        raw = model.predict(tests[0], prediction_type="RawFormulaVal")
        _write_eval(args.eval_file, raw, tests[0], ["RawFormulaVal"])
    if args.fstr_file:
        imp = model.get_feature_importance()
        with open(args.fstr_file, "w") as fh:
            for i in np.argsort(-imp):
                fh.write(f"{imp[i]:.9g}\t{model.feature_names_[i]}\n")
    return 0


def _write_eval(path, preds, pool, types):
    preds = np.asarray(preds)
    if preds.ndim == 1:
        preds = preds.reshape(-1, 1)
    with open(path, "w") as fh:
        cols = ["SampleId"] + [f"{types[0]}" if preds.shape[1] == 1 else f"{types[0]}:Dim={k}" for k in range(preds.shape[1])]
        if pool.label is not None:
            cols.append("Label")
        fh.write("\t".join(cols) + "\n")
        for i in range(preds.shape[0]):
            row = [str(i)] + [f"{v:.9g}" for v in preds[i]]
            if pool.label is not None:
                row.append(str(pool.label[i]))
            fh.write("\t".join(row) + "\n")


def mode_calc(argv):
    ap = argparse.ArgumentParser(prog="catboost_b200 calc")
    ap.add_argument("-m", "--model-file", default="model.bin")
    ap.add_argument("--model-format", default="CatboostBinary")
    ap.add_argument("--input-path", required=True)
    ap.add_argument("--column-description", "--cd", dest="cd")
    ap.add_argument("--delimiter", default="\t")
    ap.add_argument("--has-header", action="store_true")
    ap.add_argument("-o", "--output-path", default="output.tsv")
    ap.add_argument("--prediction-type", default="RawFormulaVal")
    ap.add_argument("--tree-count-limit", type=int, default=0)
    ap.add_argument("--task-type", default="CPU")
    args = ap.parse_args(argv)
    from .core import CatBoost
    fmt = {"CatboostBinary": "cbm", "Json": "json"}.get(args.model_format, args.model_format.lower())
    model = CatBoost().load_model(args.model_file, format=fmt)
    pool = _pool(args.input_path, args)
    types = args.prediction_type.split(",")
    preds = model.predict(pool, prediction_type=types[0], ntree_end=args.tree_count_limit, task_type=args.task_type)
    _write_eval(args.output_path, preds, pool, types)
    return 0


def mode_fstr(argv):
    ap = argparse.ArgumentParser(prog="catboost_b200 fstr")
    ap.add_argument("-m", "--model-file", default="model.bin")
    ap.add_argument("--input-path")
    ap.add_argument("--column-description", "--cd", dest="cd")
    ap.add_argument("--delimiter", default="\t")
    ap.add_argument("--has-header", action="store_true")
    ap.add_argument("-o", "--output-path", default="feature_strength.tsv")
    ap.add_argument("--fstr-type", default="FeatureImportance")
    args = ap.parse_args(argv)
    from .core import CatBoost
    model = CatBoost().load_model(args.model_file)
    data = _pool(args.input_path, args) if args.input_path else None
    imp = model.get_feature_importance(data, type=args.fstr_type)
    with open(args.output_path, "w") as fh:
        if args.fstr_type in ("ShapValues",):
            for row in np.asarray(imp):
                fh.write("\t".join(f"{v:.9g}" for v in np.ravel(row)) + "\n")
        elif args.fstr_type == "Interaction":
            for a, b, v in imp:
                fh.write(f"{v:.9g}\t{a}\t{b}\n")
        else:
            for i in np.argsort(-np.asarray(imp)):
                fh.write(f"{imp[i]:.9g}\t{model.feature_names_[i]}\n")
    return 0


def mode_eval_metrics(argv):
    ap = argparse.ArgumentParser(prog="catboost_b200 eval-metrics")
    ap.add_argument("-m", "--model-file", default="model.bin")
    ap.add_argument("--input-path", required=True)
    ap.add_argument("--column-description", "--cd", dest="cd")
    ap.add_argument("--delimiter", default="\t")
    ap.add_argument("--has-header", action="store_true")
    ap.add_argument("-o", "--output-path", default="eval_metrics.tsv")
    ap.add_argument("--metrics", required=True)
    ap.add_argument("--eval-period", type=int, default=1)
    args = ap.parse_args(argv)
    from .core import CatBoost
    model = CatBoost().load_model(args.model_file)
    res = model.eval_metrics(_pool(args.input_path, args), args.metrics.split(","), eval_period=args.eval_period)
    names = list(res)
    with open(args.output_path, "w") as fh:
        fh.write("iter\t" + "\t".join(names) + "\n")
        for i in range(len(res[names[0]])):
            fh.write(f"{i}\t" + "\t".join(f"{res[n][i]:.9g}" for n in names) + "\n")
    return 0


def mode_metadata(argv):
    ap = argparse.ArgumentParser(prog="catboost_b200 metadata")
    ap.add_argument("action", choices=["get", "set", "dump"])
    ap.add_argument("-m", "--model-file", default="model.bin")
    ap.add_argument("--key")
    ap.add_argument("--value")
    args = ap.parse_args(argv)
    from .core import CatBoost
    model = CatBoost().load_model(args.model_file)
    if args.action == "dump":
        for k, v in model._model.info.items():
            print(f"{k}\t{v}")
    elif args.action == "get":
        print(model._model.info.get(args.key, ""))
    else:
        model._model.info[args.key] = args.value
        model.save_model(args.model_file)
    return 0


def mode_model_sum(argv):
    ap = argparse.ArgumentParser(prog="catboost_b200 model-sum")
    ap.add_argument("-m", "--model", action="append", default=[], help="path or path=weight")
    ap.add_argument("-o", "--output-path", default="model.bin")
    args = ap.parse_args(argv)
    from .core import CatBoost, sum_models
    models, weights = [], []
    for spec in args.model:
        path, _, w = spec.partition("=")
        models.append(CatBoost().load_model(path))
        weights.append(float(w) if w else 1.0)
    sum_models(models, weights).save_model(args.output_path)
    return 0


def mode_normalize_model(argv):
    ap = argparse.ArgumentParser(prog="catboost_b200 normalize-model")
    ap.add_argument("-m", "--model-file", "--model-path", dest="model_file", default="model.bin")
    ap.add_argument("--set-scale", type=float)
    ap.add_argument("--set-bias", type=float)
    ap.add_argument("-o", "--output-model")
    ap.add_argument("--output-model-format", default=None)
    ap.add_argument("--print-scale-and-bias", action="store_true")
    ap.add_argument("-i", "--input-path", action="append", default=[],
                    help="pool(s): scale and bias are chosen so that the model's values on them span [0, 1]")
    ap.add_argument("--column-description", "--cd", dest="cd")
    ap.add_argument("--delimiter", default="\t")
    ap.add_argument("--has-header", action="store_true")
    ap.add_argument("-T", "--thread-count", type=int, default=-1)
    ap.add_argument("--logging-level", default="Info")
    args = ap.parse_args(argv)
    from .core import CatBoost
    from .data.pool import CatBoostError
    model = CatBoost().load_model(args.model_file)
    scale, bias = model.get_scale_and_bias()
    before = (scale, bias)
    if args.print_scale_and_bias:
        print(f"Input model scale {scale} bias {bias}")
    if args.input_path:
        # catboost/app/mode_normalize_model.cpp: minimum and maximum of the unscaled model over all pools
        if args.set_scale is not None or args.set_bias is not None:
            raise CatBoostError("Conflicting options: -i and --set-scale/bias")
        model.set_scale_and_bias(1.0, 0.0)
        lo, hi = float("inf"), float("-inf")
        for path in args.input_path:
            raw = np.asarray(model.predict(_pool(path, args), prediction_type="RawFormulaVal"))
            if raw.ndim != 1:
                raise CatBoostError("No sense in normalizing a multiclass/multitarget model")
            lo, hi = min(lo, float(raw.min())), max(hi, float(raw.max()))
        if not lo < hi:
            raise CatBoostError("Model gives same result on all docs")
        model.set_scale_and_bias(1.0 / (hi - lo), -lo / (hi - lo))
    else:
        model.set_scale_and_bias(args.set_scale if args.set_scale is not None else scale,
                                 args.set_bias if args.set_bias is not None else bias)
    after = model.get_scale_and_bias()
    if after != before or args.output_model:
        if args.print_scale_and_bias:
            print(f"Output model scale {after[0]} bias {after[1]}")
        out = args.output_model or args.model_file
        if args.output_model_format:
            model.save_model(out, format=args.output_model_format.lower().replace("catboostbinary", "cbm"))
        else:
            model.save_model(out)
    return 0


def mode_select_features(argv):
    ap = argparse.ArgumentParser(prog="catboost_b200 select-features")
    _add_pool_args(ap)
    ap.add_argument("--params-file")
    ap.add_argument("--features-for-select", required=True)
    ap.add_argument("--num-features-to-select", type=int, required=True)
    ap.add_argument("--features-selection-steps", type=int, default=1)
    ap.add_argument("--features-selection-result-path", default="selection_result.json")
    ap.add_argument("--features-selection-algorithm", default="RecursiveByShapValues")
    ap.add_argument("--shap-calc-type", default="Regular")
    ap.add_argument("--train-final-model", action="store_true")
    ap.add_argument("-m", "--model-file", default=None, help="where the final model goes with --train-final-model")
    ap.add_argument("--verbose", type=int, default=0)
    ap.add_argument("--use-best-model")
    ap.add_argument("--save-snapshot", action="store_true")
    for flag, typ, dest in _FIT_PARAMS:
        ap.add_argument(flag, type=typ, dest=dest, default=None)
    args = ap.parse_args(argv)
    from .core import CatBoost
    feats = []
    for tok in args.features_for_select.split(","):
        if "-" in tok:
            a, b = tok.split("-")
            feats += list(range(int(a), int(b) + 1))
        else:
            feats.append(int(tok))
    fp = _fit_params(args)
    extra = {} if fp.get("train_dir") else {"allow_writing_files": False}
    est = CatBoost({**fp, "verbose": bool(args.verbose), **extra})
    evals = [_pool(t, args) for t in args.test_set]
    res = est.select_features(_pool(args.learn_set, args), eval_set=evals[0] if evals else None, features_for_select=feats,
                              num_features_to_select=args.num_features_to_select, steps=args.features_selection_steps,
                              algorithm=args.features_selection_algorithm, shap_calc_type=args.shap_calc_type,
                              train_final_model=args.train_final_model, logging_level="Verbose" if args.verbose else "Silent")
    if args.train_final_model and args.model_file:
        est.save_model(args.model_file)
    with open(args.features_selection_result_path, "w") as fh:
        json.dump(res, fh)
    return 0


def mode_dataset_statistics(argv):
    ap = argparse.ArgumentParser(prog="catboost_b200 dataset-statistics")
    ap.add_argument("--input-path", required=True)
    ap.add_argument("--column-description", "--cd", dest="cd")
    ap.add_argument("--delimiter", default="\t")
    ap.add_argument("--has-header", action="store_true")
    ap.add_argument("-o", "--output-path", default="statistics.json")
    args = ap.parse_args(argv)
    pool = _pool(args.input_path, args)
    fd = pool.float_data
    stats = {"object_count": pool.num_row(), "feature_count": pool.num_col(),
             "float_features": [{"min": float(np.nanmin(fd[:, j])), "max": float(np.nanmax(fd[:, j])),
                                 "mean": float(np.nanmean(fd[:, j])), "nan_count": int(np.isnan(fd[:, j]).sum())}
                                for j in range(fd.shape[1])],
             "cat_features": [{"unique_values": int(len(np.unique(pool.cat_hashes[j])))} for j in range(len(pool.cat_feature_indices))]}
    if pool.label is not None and np.asarray(pool.label).dtype.kind in "fiu":
        lab = np.asarray(pool.label, dtype=np.float64)
        stats["target"] = {"min": float(lab.min()), "max": float(lab.max()), "mean": float(lab.mean())}
    with open(args.output_path, "w") as fh:
        json.dump(stats, fh, indent=1)
    return 0


def mode_dump_options(argv):
    ap = argparse.ArgumentParser(prog="catboost_b200 dump-options")
    ap.add_argument("--params-file")
    ap.add_argument("-o", "--output-path")
    ap.add_argument("--use-best-model")
    ap.add_argument("--save-snapshot", action="store_true")
    for flag, typ, dest in _FIT_PARAMS:
        ap.add_argument(flag, type=typ, dest=dest, default=None)
    args = ap.parse_args(argv)
    from .params import resolve_options
    o = resolve_options(_fit_params(args))
    text = o.to_json()
    if args.output_path:
        with open(args.output_path, "w") as fh:
            fh.write(text)
    else:
        print(text)
    return 0


def mode_roc(argv):
    ap = argparse.ArgumentParser(prog="catboost_b200 roc")
    ap.add_argument("-m", "--model-file", default="model.bin")
    ap.add_argument("--input-path", required=True)
    ap.add_argument("--column-description", "--cd", dest="cd")
    ap.add_argument("--delimiter", default="\t")
    ap.add_argument("--has-header", action="store_true")
    ap.add_argument("-o", "--output-path", default="roc.tsv")
    args = ap.parse_args(argv)
    from .core import CatBoost
    from .utils.roc import roc_curve
    model = CatBoost().load_model(args.model_file)
    pool = _pool(args.input_path, args)
    fpr, tpr, thr = roc_curve(model, pool)
    with open(args.output_path, "w") as fh:
        fh.write("FPR\tTPR\tThreshold\n")
        for a, b, c in zip(fpr, tpr, thr):
            fh.write(f"{a:.9g}\t{b:.9g}\t{c:.9g}\n")
    return 0


def mode_ostr(argv):
    """Object importance (catboost/app/mode_ostr.cpp): one line per scored training object."""
    ap = argparse.ArgumentParser(prog="catboost_b200 ostr")
    ap.add_argument("-m", "--model-file", default="model.bin")
    ap.add_argument("-f", "--learn-set", required=True)
    ap.add_argument("-t", "--test-set", required=True)
    ap.add_argument("--column-description", "--cd", dest="cd")
    ap.add_argument("--delimiter", default="\t")
    ap.add_argument("--has-header", action="store_true")
    ap.add_argument("-o", "--output-path", default="object_importances.tsv")
    ap.add_argument("--ostr-type", default="Average", choices=["Average", "PerObject"])
    ap.add_argument("--top-size", type=int, default=-1)
    ap.add_argument("--update-method", default="SinglePoint")
    ap.add_argument("--importance-values-sign", default="All", choices=["All", "Positive", "Negative"])
    args = ap.parse_args(argv)
    from .core import CatBoost
    model = CatBoost().load_model(args.model_file)
    idx, val = model.get_object_importance(_pool(args.test_set, args), _pool(args.learn_set, args), top_size=args.top_size,
                                           type=args.ostr_type, update_method=args.update_method,
                                           importance_values_sign=args.importance_values_sign)
    with open(args.output_path, "w") as fh:
        if args.ostr_type == "Average":
            for i, v in zip(idx, val):
                fh.write(f"{int(i)}\t{v:.9g}\n")
        else:
            for ii, vv in zip(idx, val):
                fh.write("\t".join(f"{int(i)}:{v:.9g}" for i, v in zip(ii, vv)) + "\n")
    return 0


def mode_eval_feature(argv):
    """Feature evaluation on folds of one dataset (catboost/app/mode_eval_feature.cpp)."""
    ap = argparse.ArgumentParser(prog="catboost_b200 eval-feature")
    ap.add_argument("-f", "--learn-set", required=True)
    ap.add_argument("--column-description", "--cd", dest="cd")
    ap.add_argument("--delimiter", default="\t")
    ap.add_argument("--has-header", action="store_true")
    ap.add_argument("--features-to-evaluate", required=True, help="comma separated feature indices or names")
    ap.add_argument("--feature-eval-mode", default="SeqAdd", choices=["All", "SeqAdd", "SeqRem", "SeqAddAndAll"])
    ap.add_argument("--fold-count", type=int, default=5)
    ap.add_argument("--loss-function", default="RMSE")
    ap.add_argument("-i", "--iterations", type=int, default=100)
    ap.add_argument("--params-file")
    ap.add_argument("--task-type", default="CPU")
    ap.add_argument("-o", "--output-path", default="feature_eval.json")
    args = ap.parse_args(argv)
    import json
    from .eval_features import eval_features
    params = {}
    if args.params_file:
        with open(args.params_file) as fh:
            params = json.load(fh)
    params.setdefault("loss_function", args.loss_function)
    params.setdefault("iterations", args.iterations)
    params.setdefault("task_type", args.task_type)
    feats = [int(x) if x.strip().lstrip("-").isdigit() else x.strip() for x in args.features_to_evaluate.split(",")]
    res = eval_features(_pool(args.learn_set, args), params, feats, eval_type=args.feature_eval_mode,
                        fold_count=args.fold_count)
    with open(args.output_path, "w") as fh:
        json.dump(res, fh, indent=1)
    return 0


def mode_run_worker(argv):
    """One rank of a training run over several processes / hosts (the counterpart of the reference's
    ``catboost run-worker`` + master, catboost/app/main.cpp:21-35, catboost/private/libs/distributed): every participant
    runs ``run-worker --rank R --world-size W --master-addr A --master-port P -- <fit options>``; the ranks join one
    process group (gloo for CPU training, NCCL for task_type GPU), each trains on its row shard of the learn set and rank
    0 writes the model."""
    import os
    if "--" in argv:
        k = argv.index("--")
        own, fit_args = argv[:k], argv[k + 1:]
    else:
        own, fit_args = argv, []
    ap = argparse.ArgumentParser(prog="catboost_b200 run-worker")
    ap.add_argument("--rank", type=int, default=int(os.environ.get("RANK", 0)))
    ap.add_argument("--world-size", type=int, default=int(os.environ.get("WORLD_SIZE", 1)))
    ap.add_argument("--master-addr", default=os.environ.get("MASTER_ADDR", "127.0.0.1"))
    ap.add_argument("--master-port", type=int, default=int(os.environ.get("MASTER_PORT", 29500)))
    ap.add_argument("--backend", default=None, help="gloo (CPU) or nccl (GPU); default: by --task-type of the fit options")
    args = ap.parse_args(own)
    import torch
    import torch.distributed as dist
    gpu = any(a.upper() == "GPU" for a in fit_args)
    backend = args.backend or ("nccl" if gpu and torch.cuda.is_available() else "gloo")
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = args.master_addr, str(args.master_port)
    kw = {}
    if backend == "nccl":
        local = int(os.environ.get("LOCAL_RANK", args.rank % max(1, torch.cuda.device_count())))
        torch.cuda.set_device(local)
        kw["device_id"] = torch.device("cuda", local)
    dist.init_process_group(backend, rank=args.rank, world_size=args.world_size, **kw)
    try:
        return mode_fit(fit_args)
    finally:
        try:
            dist.barrier()
        except Exception:
            pass
        dist.destroy_process_group()


def mode_model_based_eval(argv):
    """Feature evaluation that starts from a trained baseline (catboost/app/mode_model_based_eval.cpp, catboost/libs/
    train_lib/model_based_eval.cpp): for every feature set the baseline's first trees are kept and training continues
    once without the set (ignored) and once with it; the report gives the final metric of both continuations."""
    ap = argparse.ArgumentParser(prog="catboost_b200 model-based-eval")
    _add_pool_args(ap)
    ap.add_argument("--features-to-evaluate", required=True, help="feature sets separated by ';', indices by ','")
    ap.add_argument("--baseline-model-snapshot", "--baseline-model", dest="baseline", required=True)
    ap.add_argument("--offset", type=int, default=0, help="trees of the baseline that are kept")
    ap.add_argument("--experiment-size", type=int, default=100, help="iterations of every continuation")
    ap.add_argument("--loss-function", default=None)
    ap.add_argument("--task-type", default="CPU")
    ap.add_argument("-o", "--output-path", default="model_based_eval.json")
    args = ap.parse_args(argv)
    import json
    from .core import CatBoost
    learn = _pool(args.learn_set, args, args.learn_pairs)
    tests = [_pool(t, args, args.test_pairs) for t in args.test_set]
    base = CatBoost().load_model(args.baseline)
    loss = args.loss_function or base._model.loss_name
    if args.offset > 0:
        base.shrink(args.offset)
    sets = [[int(x) for x in part.split(",") if x.strip()] for part in args.features_to_evaluate.split(";") if part.strip()]
    report = []
    for fs in sets:
        row = {"features": fs}
        for name, ignored in (("without", fs), ("with", [])):
            m = CatBoost(dict(loss_function=loss, iterations=args.experiment_size, task_type=args.task_type,
                              ignored_features=ignored, verbose=False, allow_writing_files=False))
            m.fit(learn, eval_set=tests or None, init_model=base)
            ev = m.get_evals_result()
            key = "validation" if tests else "learn"
            metric = next(iter(ev[key]))
            row[name] = {"metric": metric, "value": float(ev[key][metric][-1])}
        row["delta"] = row["with"]["value"] - row["without"]["value"]
        report.append(row)
    with open(args.output_path, "w") as fh:
        json.dump(report, fh, indent=1)
    return 0


def mode_dsv_diff(argv):
    ap = argparse.ArgumentParser(prog="catboost_b200 dsv-diff")
    ap.add_argument("file_a")
    ap.add_argument("file_b")
    ap.add_argument("-d", "--delimiter", default="\t")
    ap.add_argument("--have-header", action="store_true")
    ap.add_argument("--diff-limit", type=float, default=0.0)
    a = ap.parse_args(argv)
    from .difftools import dsv_diff
    diffs = dsv_diff(a.file_a, a.file_b, a.diff_limit, a.delimiter, a.have_header)
    for d in diffs:
        print(d)
    return 1 if diffs else 0


def mode_json_diff(argv):
    ap = argparse.ArgumentParser(prog="catboost_b200 json-diff")
    ap.add_argument("file_a")
    ap.add_argument("file_b")
    ap.add_argument("--diff-limit", type=float, default=0.0)
    ap.add_argument("--ignore-keys", default="")
    a = ap.parse_args(argv)
    import json
    from .difftools import json_diff
    with open(a.file_a) as fa, open(a.file_b) as fb:
        diffs = json_diff(json.load(fa), json.load(fb), a.diff_limit,
                          ignore_keys=tuple(k for k in a.ignore_keys.split(",") if k))
    for d in diffs:
        print(d)
    return 1 if diffs else 0


def mode_numpy_diff(argv):
    ap = argparse.ArgumentParser(prog="catboost_b200 numpy-diff")
    ap.add_argument("file_a")
    ap.add_argument("file_b")
    ap.add_argument("--diff-limit", type=float, default=0.0)
    a = ap.parse_args(argv)
    from .difftools import numpy_diff
    diffs = numpy_diff(a.file_a, a.file_b, a.diff_limit)
    for d in diffs:
        print(d)
    return 1 if diffs else 0


def mode_compare_models(argv):
    ap = argparse.ArgumentParser(prog="catboost_b200 compare-models")
    ap.add_argument("model_a")
    ap.add_argument("model_b")
    ap.add_argument("--diff-limit", type=float, default=0.0)
    ap.add_argument("--format-a", default=None)
    ap.add_argument("--format-b", default=None)
    a = ap.parse_args(argv)
    from .difftools import compare_models
    from .models.io import load_model
    fmt = lambda path, f: f or ("json" if path.endswith(".json") else "cbm")
    diffs = compare_models(load_model(a.model_a, fmt(a.model_a, a.format_a)), load_model(a.model_b, fmt(a.model_b, a.format_b)),
                           a.diff_limit)
    for d in diffs:
        print(d)
    print("MODELS ARE EQUAL" if not diffs else "MODELS DIFFER")
    return 1 if diffs else 0


def mode_model_perftest(argv):
    ap = argparse.ArgumentParser(prog="catboost_b200 model-perftest")
    ap.add_argument("-m", "--model-file", required=True)
    ap.add_argument("--rows", type=int, default=100_000)
    ap.add_argument("--repeats", type=int, default=5)
    ap.add_argument("--task-type", default="CPU")
    ap.add_argument("--devices", default=None)
    a = ap.parse_args(argv)
    import json
    from .difftools import model_perftest
    from .models.io import load_model
    print(json.dumps(model_perftest(load_model(a.model_file, "json" if a.model_file.endswith(".json") else "cbm"), a.rows,
                                    a.repeats, task_type=a.task_type, devices=a.devices)))
    return 0


MODES = {"dsv-diff": mode_dsv_diff, "json-diff": mode_json_diff, "numpy-diff": mode_numpy_diff,
         "compare-models": mode_compare_models, "model-perftest": mode_model_perftest, "run-worker": mode_run_worker, "model-based-eval": mode_model_based_eval, "ostr": mode_ostr, "eval-feature": mode_eval_feature, "fit": mode_fit, "calc": mode_calc, "fstr": mode_fstr, "eval-metrics": mode_eval_metrics,
         "metadata": mode_metadata, "model-sum": mode_model_sum, "normalize-model": mode_normalize_model,
         "select-features": mode_select_features, "dataset-statistics": mode_dataset_statistics,
         "dump-options": mode_dump_options, "roc": mode_roc}


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help"):
        print("usage: python -m catboost_b200 <mode> [options]\nmodes: " + ", ".join(MODES))
        return 0
    mode = argv[0]
    if mode not in MODES:
        print(f"unknown mode {mode!r}; modes: " + ", ".join(MODES), file=sys.stderr)
        return 2
    return MODES[mode](argv[1:])
