"""Helper functions of the public package (catboost/python-package/catboost/utils.py): column-description files,
metric evaluation on raw arrays, ROC / FPR / FNR curves and threshold selection, confusion matrix, dataset
quantisation from a file, quantisation grids, ONNX export as an object."""
from __future__ import annotations

import os
from typing import Dict, Optional, Sequence

import numpy as np

from ..data.pool import CatBoostError, Pool

_CD_TYPES = {"label": "Label", "weight": "Weight", "baseline": "Baseline", "doc_id": "DocId", "group_id": "GroupId",
             "subgroup_id": "SubgroupId", "timestamp": "Timestamp"}
_FEATURE_COLUMN_TYPES = ("Num", "Categ", "Text", "NumVector")


def create_cd(label=None, cat_features=None, text_features=None, embedding_features=None, weight=None, baseline=None,
              doc_id=None, group_id=None, subgroup_id=None, timestamp=None, auxiliary_columns=None, feature_names=None,
              output_path="train.cd"):
    """Write a column-description file: ``index<TAB>type<TAB>name`` for every column that is not a plain number."""
    cols: Dict[int, list] = {}

    def put(index, kind):
        if not isinstance(index, (int, np.integer)):
            raise CatBoostError(f"Unsupported index type. Expected int, got {type(index)}")
        if int(index) in cols:
            raise CatBoostError(f"The index {index} occurs more than once")
        cols[int(index)] = [kind, ""]

    for value, kind in ((cat_features, "Categ"), (text_features, "Text"), (embedding_features, "NumVector"),
                        (auxiliary_columns, "Auxiliary")):
        if value is None:
            continue
        for index in ([value] if isinstance(value, (int, np.integer)) else value):
            put(index, kind)
    for key, value in (("label", label), ("weight", weight), ("baseline", baseline), ("doc_id", doc_id),
                       ("group_id", group_id), ("subgroup_id", subgroup_id), ("timestamp", timestamp)):
        if value is not None:
            put(value, _CD_TYPES[key])
    for index, name in (feature_names or {}).items():
        entry = cols.setdefault(int(index), ["Num", ""])
        if entry[0] not in _FEATURE_COLUMN_TYPES:
            raise CatBoostError(f"feature_names contains index {index} that does not correspond to feature column")
        entry[1] = str(name)
    with open(os.fspath(output_path), "w") as fh:
        for index in sorted(cols):
            fh.write(f"{index}\t{cols[index][0]}\t{cols[index][1]}\n")


def read_cd(cd_file, column_count: Optional[int] = None, data_file=None, canonize_column_types: bool = False):
    """Parse a column-description file.  Returns a dict with ``column_type_to_indices``, ``column_dtypes``,
    ``cat_feature_indices``, ``text_feature_indices``, ``embedding_feature_indices`` (feature numbering, i.e. counted
    over feature columns only), ``column_names`` and ``non_feature_column_indices``."""
    entries: Dict[int, tuple] = {}
    with open(os.fspath(cd_file)) as fh:
        for line in fh:
            parts = line.rstrip("\n").split("\t")
            if not parts or not parts[0].strip():
                continue
            kind = parts[1].strip() if len(parts) > 1 else "Num"
            if canonize_column_types:
                kind = {"Target": "Label", "DocId": "SampleId", "QueryId": "GroupId"}.get(kind, kind)
            entries[int(parts[0])] = (kind, parts[2].strip() if len(parts) > 2 else "")
    if column_count is None and data_file is not None:
        with open(os.fspath(data_file)) as fh:
            column_count = len(fh.readline().rstrip("\n").split("\t"))
    if column_count is None:
        column_count = (max(entries) + 1) if entries else 0
    by_type: Dict[str, list] = {}
    dtypes, names, non_feature = {}, [], []
    cat_idx, text_idx, emb_idx = [], [], []
    feature_no = 0
    for c in range(column_count):
        kind, name = entries.get(c, ("Num", ""))
        by_type.setdefault(kind, []).append(c)
        col_name = name or (f"feature_{feature_no}" if kind in _FEATURE_COLUMN_TYPES else kind)
        names.append(col_name)
        if kind in _FEATURE_COLUMN_TYPES:
            if kind == "Categ":
                cat_idx.append(feature_no)
            elif kind == "Text":
                text_idx.append(feature_no)
            elif kind == "NumVector":
                emb_idx.append(feature_no)
            dtypes[col_name] = np.float32 if kind == "Num" else object
            feature_no += 1
        else:
            non_feature.append(c)
            dtypes[col_name] = object if kind in ("DocId", "SampleId", "GroupId", "SubgroupId", "Auxiliary") else np.float64
    return {"column_type_to_indices": by_type, "column_dtypes": dtypes, "cat_feature_indices": cat_idx,
            "text_feature_indices": text_idx, "embedding_feature_indices": emb_idx, "column_names": names,
            "non_feature_column_indices": non_feature}


def eval_metric(label, approx, metric, weight=None, group_id=None, group_weight=None, subgroup_id=None, pairs=None,
                thread_count=-1):
    """Value(s) of ``metric`` for raw formula values ``approx`` ([n] or [n, dims] or a list of per-dimension arrays).
    Returns a list with one value, like the reference."""
    from ..metrics import make_metric
    a = np.asarray(approx, dtype=np.float64)
    y = np.asarray(label)
    if a.ndim == 2 and a.shape[0] != len(y) and a.shape[1] == len(y):
        a = a.T
    offsets = None
    if group_id is not None:
        g = np.asarray(group_id)
        change = np.nonzero(g[1:] != g[:-1])[0] + 1
        offsets = np.concatenate([[0], change, [len(g)]])
    w = weight if weight is not None else group_weight
    m = make_metric(metric)
    return [m.eval(a, y.astype(np.float64) if y.dtype != object else y, w, group_offsets=offsets,
                   pairs=None if pairs is None else np.asarray(pairs))]


def get_gpu_device_count() -> int:
    import torch
    return int(torch.cuda.device_count()) if torch.cuda.is_available() else 0


def _binary_scores(model, data):
    if not isinstance(data, Pool):
        raise CatBoostError("data must be a Pool with labels")
    if data.label is None:
        raise CatBoostError("data has no labels")
    raw = np.asarray(model.predict(data, prediction_type="RawFormulaVal"), dtype=np.float64)
    if raw.ndim != 1:
        raise CatBoostError("the curve is defined for binary classification models")
    return 1.0 / (1.0 + np.exp(-raw)), model._encode_labels(data.label) > 0.5


def get_roc_curve(model, data, thread_count=-1, plot=False):
    """(fpr, tpr, thresholds): thresholds decrease from 1 to the smallest predicted probability."""
    pools = data if isinstance(data, (list, tuple)) else [data]
    ps, ys = zip(*[_binary_scores(model, d) for d in pools])
    p, y = np.concatenate(ps), np.concatenate(ys)
    order = np.argsort(-p, kind="stable")
    p, y = p[order], y[order]
    tp, fp = np.cumsum(y), np.cumsum(~y)
    distinct = np.r_[np.nonzero(np.diff(p))[0], len(p) - 1]
    tpr = np.r_[0.0, tp[distinct] / max(tp[-1], 1)]
    fpr = np.r_[0.0, fp[distinct] / max(fp[-1], 1)]
    thr = np.r_[1.0, p[distinct]]
    return fpr, tpr, thr


def get_fpr_curve(model=None, data=None, curve=None, thread_count=-1, plot=False):
    """(thresholds, fpr) from a model and data, or from a ROC ``curve``."""
    if curve is None:
        curve = get_roc_curve(model, data)
    fpr, _, thr = curve
    return np.asarray(thr), np.asarray(fpr)


def get_fnr_curve(model=None, data=None, curve=None, thread_count=-1, plot=False):
    """(thresholds, fnr) from a model and data, or from a ROC ``curve``."""
    if curve is None:
        curve = get_roc_curve(model, data)
    _, tpr, thr = curve
    return np.asarray(thr), 1.0 - np.asarray(tpr)


def select_threshold(model=None, data=None, curve=None, FPR=None, FNR=None, thread_count=-1):
    """Probability boundary that reaches the wanted FPR or FNR; with neither given, the point where FPR = FNR."""
    if FPR is not None and FNR is not None:
        raise CatBoostError("only one of FPR and FNR can be given")
    if curve is None:
        curve = get_roc_curve(model, data)
    fpr, tpr, thr = (np.asarray(v) for v in curve)
    if FPR is not None:
        ok = np.nonzero(fpr <= FPR)[0]
        return float(thr[ok[-1]])
    if FNR is not None:
        ok = np.nonzero(1 - tpr <= FNR)[0]
        return float(thr[ok[0]])
    return float(thr[int(np.argmin(np.abs(fpr - (1 - tpr))))])


def get_confusion_matrix(model, data, thread_count=-1):
    """Counts [true class, predicted class] in the order of the model's classes."""
    if not isinstance(data, Pool) or data.label is None:
        raise CatBoostError("data must be a Pool with labels")
    names = list(model._model.class_names) if model._model.class_names is not None else None
    if names is None:
        raise CatBoostError("confusion matrix needs a classification model")
    pred = np.asarray(model.predict(data, prediction_type="Class")).reshape(-1)
    pos = {str(v): k for k, v in enumerate(names)}
    truth = model._encode_labels(data.label).astype(np.int64) if model._model.params.get("target_border") is not None \
        else np.array([pos.get(str(v), pos.get(str(_as_number(v)), -1)) for v in np.asarray(data.label).tolist()])
    pk = np.array([pos.get(str(v), pos.get(str(_as_number(v)), -1)) for v in pred.tolist()])
    cm = np.zeros((len(names), len(names)), dtype=np.float64)
    ok = (truth >= 0) & (pk >= 0)
    np.add.at(cm, (truth[ok], pk[ok]), 1.0 if data.weight is None else np.asarray(data.weight)[ok])
    return cm


def _as_number(v):
    try:
        f = float(v)
        return int(f) if f == int(f) else f
    except (TypeError, ValueError):
        return v


def quantize(data_path, column_description=None, pairs=None, graph=None, delimiter="\t", has_header=False,
             ignore_csv_quoting=False, feature_names=None, thread_count=-1, ignored_features=None,
             per_float_feature_quantization=None, border_count=None, max_bin=None, feature_border_type=None,
             nan_mode=None, input_borders=None, task_type=None, used_ram_limit=None, random_seed=None, **kwargs) -> Pool:
    """Load a dataset file and quantise it; the returned Pool trains without quantising again."""
    pool = Pool(os.fspath(data_path), column_description=column_description, pairs=pairs, delimiter=delimiter,
                has_header=has_header, ignore_csv_quoting=ignore_csv_quoting, feature_names=feature_names,
                thread_count=thread_count)
    pool.quantize(ignored_features=ignored_features, per_float_feature_quantization=per_float_feature_quantization,
                  border_count=border_count if border_count is not None else max_bin,
                  feature_border_type=feature_border_type, nan_mode=nan_mode, input_borders=input_borders,
                  task_type=task_type, random_seed=random_seed)
    return pool


def calculate_quantization_grid(values, border_count, border_type="Median"):
    """Borders for one column of values."""
    from ..data.quantization import select_borders
    v = np.asarray(values, dtype=np.float32).reshape(-1, 1)
    borders, _ = select_borders(v, int(border_count), border_type)
    return np.asarray(borders[0], dtype=np.float32)


def convert_to_onnx_object(model, export_parameters=None, **kwargs):
    """The ONNX model.  With the ``onnx`` package present this is an ``onnx.ModelProto``; otherwise the serialised
    protobuf bytes (the same content)."""
    from ..models.export import model_to_onnx_bytes
    blob = model_to_onnx_bytes(model._model)
    try:
        import onnx
        return onnx.load_model_from_string(blob)
    except ImportError:
        return blob
