"""Tolerant comparison tools for test and release work: delimiter-separated files, JSON documents, numpy files and
models.  They play the part of the reference's ``catboost/tools/limited_precision_dsv_diff``,
``limited_precision_json_diff``, ``limited_precision_numpy_diff``, ``model_comparator`` and ``model_perftest``:
two artefacts are "equal" when every pair of numbers differs by at most ``diff_limit`` in the relative-or-absolute sense
``|a - b| <= diff_limit * max(1, |a|, |b|)`` and everything else matches exactly.

CLI: ``python -m catboost_b200 dsv-diff | json-diff | numpy-diff | compare-models | model-perftest``; every comparison
exits 0 when the inputs agree and 1 with the first differences printed otherwise.
"""
from __future__ import annotations

import json
import math
import time
from typing import List, Optional

import numpy as np


def _as_float(tok: str) -> Optional[float]:
    try:
        return float(tok)
    except ValueError:
        return None


def numbers_close(a: float, b: float, diff_limit: float) -> bool:
    if a == b or (math.isnan(a) and math.isnan(b)):
        return True
    if math.isinf(a) or math.isinf(b) or math.isnan(a) or math.isnan(b):
        return False
    return abs(a - b) <= diff_limit * max(1.0, abs(a), abs(b))


def dsv_diff(path_a: str, path_b: str, diff_limit: float = 0.0, delimiter: str = "\t", have_header: bool = False,
             max_report: int = 10) -> List[str]:
    """Differences between two delimiter-separated files (empty list = equal)."""
    out: List[str] = []
    with open(path_a) as fa, open(path_b) as fb:
        la, lb = fa.read().splitlines(), fb.read().splitlines()
    if len(la) != len(lb):
        return [f"line counts differ: {len(la)} vs {len(lb)}"]
    for ln, (ra, rb) in enumerate(zip(la, lb)):
        if ra == rb:
            continue
        ca, cb = ra.split(delimiter), rb.split(delimiter)
        if len(ca) != len(cb):
            out.append(f"line {ln + 1}: {len(ca)} fields vs {len(cb)}")
        else:
            for k, (x, y) in enumerate(zip(ca, cb)):
                if x == y:
                    continue
                fx, fy = (None, None) if (have_header and ln == 0) else (_as_float(x), _as_float(y))
                if fx is None or fy is None or not numbers_close(fx, fy, diff_limit):
                    out.append(f"line {ln + 1}, field {k + 1}: {x!r} vs {y!r}")
                    break
        if len(out) >= max_report:
            break
    return out


def json_diff(a, b, diff_limit: float = 0.0, path: str = "$", out: Optional[List[str]] = None, max_report: int = 10,
              ignore_keys=()) -> List[str]:
    """Differences between two parsed JSON values."""
    out = [] if out is None else out
    if len(out) >= max_report:
        return out
    if isinstance(a, dict) and isinstance(b, dict):
        for k in sorted(set(a) | set(b)):
            if k in ignore_keys:
                continue
            if k not in a or k not in b:
                out.append(f"{path}.{k}: present in one document only")
            else:
                json_diff(a[k], b[k], diff_limit, f"{path}.{k}", out, max_report, ignore_keys)
    elif isinstance(a, list) and isinstance(b, list):
        if len(a) != len(b):
            out.append(f"{path}: lengths {len(a)} vs {len(b)}")
        else:
            for i, (x, y) in enumerate(zip(a, b)):
                json_diff(x, y, diff_limit, f"{path}[{i}]", out, max_report, ignore_keys)
    elif isinstance(a, (int, float)) and isinstance(b, (int, float)) and not isinstance(a, bool) and not isinstance(b, bool):
        if not numbers_close(float(a), float(b), diff_limit):
            out.append(f"{path}: {a!r} vs {b!r}")
    elif a != b:
        out.append(f"{path}: {a!r} vs {b!r}")
    return out


def numpy_diff(path_a: str, path_b: str, diff_limit: float = 0.0) -> List[str]:
    a, b = np.load(path_a, allow_pickle=False), np.load(path_b, allow_pickle=False)
    if a.shape != b.shape:
        return [f"shapes differ: {a.shape} vs {b.shape}"]
    if a.dtype.kind not in "fiub" or b.dtype.kind not in "fiub":
        return [] if np.array_equal(a, b) else ["non-numeric arrays differ"]
    x, y = a.astype(np.float64), b.astype(np.float64)
    bad = ~((np.abs(x - y) <= diff_limit * np.maximum(1.0, np.maximum(np.abs(x), np.abs(y)))) | (np.isnan(x) & np.isnan(y)))
    if not bad.any():
        return []
    idx = np.argwhere(bad)[:10]
    return [f"index {tuple(int(v) for v in i)}: {x[tuple(i)]!r} vs {y[tuple(i)]!r}" for i in idx]


def compare_models(model_a, model_b, diff_limit: float = 0.0, ignore_keys=("params", "model_guid", "train_finish_time",
                                                                           "catboost_version_info", "training")) -> List[str]:
    """Structural comparison of two models (trees, splits, borders, leaf values and weights, scale and bias, CTR tables'
    shapes): leaf values and borders within ``diff_limit``, everything else exact."""
    out: List[str] = []
    a, b = model_a, model_b
    if a.dims != b.dims:
        return [f"dimensions differ: {a.dims} vs {b.dims}"]
    if len(a.trees) != len(b.trees):
        out.append(f"tree counts differ: {len(a.trees)} vs {len(b.trees)}")
    if len(a.float_features) != len(b.float_features):
        out.append(f"float feature counts differ: {len(a.float_features)} vs {len(b.float_features)}")
    else:
        for j, (fa, fb) in enumerate(zip(a.float_features, b.float_features)):
            ba, bb = np.asarray(fa.borders, dtype=np.float64), np.asarray(fb.borders, dtype=np.float64)
            if ba.shape != bb.shape or not all(numbers_close(float(x), float(y), diff_limit) for x, y in zip(ba, bb)):
                out.append(f"borders of float feature {j} differ")
    if not all(numbers_close(float(x), float(y), diff_limit) for x, y in
               zip(np.broadcast_to(a.bias, (a.dims,)), np.broadcast_to(b.bias, (b.dims,)))) or \
            not numbers_close(float(a.scale), float(b.scale), diff_limit):
        out.append("scale / bias differ")

    def split_key(m, s):
        sp = m.splits[s]
        return (sp.kind, int(sp.feature), None if sp.border is None else float(sp.border),
                None if sp.value is None else int(sp.value))

    for t, (ta, tb) in enumerate(zip(a.trees, b.trees)):
        if type(ta) is not type(tb):
            out.append(f"tree {t}: different kinds")
            continue
        if hasattr(ta, "splits"):
            ka, kb = [split_key(a, s) for s in ta.splits], [split_key(b, s) for s in tb.splits]
            same = len(ka) == len(kb) and all(x[0] == y[0] and x[1] == y[1] and x[3] == y[3] and
                                              (x[2] is None) == (y[2] is None) and
                                              (x[2] is None or numbers_close(x[2], y[2], diff_limit)) for x, y in zip(ka, kb))
            if not same:
                out.append(f"tree {t}: splits differ")
        va, vb = np.asarray(ta.leaf_values, dtype=np.float64), np.asarray(tb.leaf_values, dtype=np.float64)
        if va.shape != vb.shape:
            out.append(f"tree {t}: leaf counts differ")
        elif not (np.abs(va - vb) <= diff_limit * np.maximum(1.0, np.maximum(np.abs(va), np.abs(vb)))).all():
            out.append(f"tree {t}: leaf values differ by up to {float(np.abs(va - vb).max()):.3g}")
        if len(out) >= 10:
            break
    if len(a.ctrs) != len(b.ctrs):
        out.append(f"CTR feature counts differ: {len(a.ctrs)} vs {len(b.ctrs)}")
    return out


def model_perftest(model, rows: int = 100_000, repeats: int = 5, seed: int = 0, task_type: str = "CPU", devices=None) -> dict:
    """Apply speed of a model on random rows (rows / second, best of ``repeats``), like the reference's
    ``model_perftest``: one block of standard-normal float features, hashed integers for the categorical ones."""
    from .core import CatBoost
    m = model if isinstance(model, CatBoost) else None
    core = model._model if m is not None else model
    rng = np.random.default_rng(seed)
    X = rng.standard_normal((rows, max(1, len(core.float_features)))).astype(np.float32)
    cats = rng.integers(0, 2 ** 31, size=(len(core.cat_features), rows), dtype=np.int64).astype(np.uint32) \
        if core.cat_features else None
    best = float("inf")
    for _ in range(repeats + 1):
        t0 = time.perf_counter()
        core.predict_raw(X, cats, task_type=task_type, device=devices)
        best = min(best, time.perf_counter() - t0)
    return {"rows": rows, "trees": len(core.trees), "seconds": best, "rows_per_second": rows / best,
            "tree_rows_per_second": rows * len(core.trees) / best, "task_type": task_type}
