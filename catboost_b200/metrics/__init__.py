"""Evaluation metrics (host side, numpy).

Names, parameters (``'Metric:param=value;...'``) and definitions follow catboost/libs/metrics/metric.cpp; the
``is_max_optimal`` flags drive best-iteration selection and the overfitting detector.  Loss-type metrics of the
training objective are additionally accumulated on the device by the trainers (``cb_metric_sum``), so the hot
loop does not need these functions.
"""
from __future__ import annotations

import math
from typing import Callable, Dict, Optional

import numpy as np

from ..params import parse_loss


def _w(weight, n):
    return np.ones(n) if weight is None else np.asarray(weight, dtype=np.float64)


def _sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def _softmax(a):
    a = a - a.max(axis=1, keepdims=True)
    e = np.exp(a)
    return e / e.sum(axis=1, keepdims=True)


class Metric:
    def __init__(self, desc: str):
        self.desc = desc
        self.name, self.params = parse_loss(desc)
        if self.name == "Combination":
            # a combination of losses is reported by the metric of its first loss with a non-zero weight
            # (catboost/private/libs/options/loss_description.cpp GetMetricFromCombination)
            first = next((str(self.params[f"loss{i}"]) for i in range(len(self.params) // 2)
                          if f"loss{i}" in self.params and float(self.params.get(f"weight{i}", 0.0)) != 0.0), None)
            if first is None:
                raise ValueError("Combination loss must have one or more non-zero weights")
            inner = Metric(first)
            self.params, self.fn, self.is_max_optimal, self.needs = inner.params, inner.fn, inner.is_max_optimal, inner.needs
            return
        if self.name not in _METRICS:
            raise ValueError(f"unknown metric {self.name!r}")
        self.fn, self.is_max_optimal, self.needs = _METRICS[self.name]

    def __str__(self):
        return self.desc

    def eval(self, approx: np.ndarray, target: np.ndarray, weight=None, group_offsets=None, pairs=None,
             pairs_weight=None) -> float:
        """approx: [n, dims] raw formula values."""
        approx = np.asarray(approx, dtype=np.float64)
        if approx.ndim == 1:
            approx = approx.reshape(-1, 1)
        return float(self.fn(approx, target, _w(weight, approx.shape[0]), self.params,
                             dict(group_offsets=group_offsets, pairs=pairs, pairs_weight=pairs_weight)))


# ---- regression -------------------------------------------------------------------------------------------
def _rmse(a, y, w, p, c):
    return math.sqrt(np.sum(w * (a[:, 0] - y) ** 2) / w.sum())


def _mae(a, y, w, p, c):
    return np.sum(w * np.abs(a[:, 0] - y)) / w.sum()


def _mape(a, y, w, p, c):
    return np.sum(w * np.abs(a[:, 0] - y) / np.maximum(1.0, np.abs(y))) / w.sum()


def _smape(a, y, w, p, c):
    d = np.abs(a[:, 0]) + np.abs(y)
    return 100.0 * np.sum(w * np.where(d > 0, 2 * np.abs(a[:, 0] - y) / np.where(d > 0, d, 1), 0)) / w.sum()


def _msle(a, y, w, p, c):
    return np.sum(w * (np.log1p(np.maximum(a[:, 0], -1 + 1e-12)) - np.log1p(y)) ** 2) / w.sum()


def _r2(a, y, w, p, c):
    m = np.sum(w * y) / w.sum()
    den = np.sum(w * (y - m) ** 2)
    return 1.0 - np.sum(w * (y - a[:, 0]) ** 2) / den if den > 0 else 0.0


def _median_abs(a, y, w, p, c):
    return float(np.median(np.abs(a[:, 0] - y)))


def _quantile(a, y, w, p, c):
    alpha, delta = float(p.get("alpha", 0.5)), float(p.get("delta", 1e-6))
    d = y - a[:, 0]
    v = np.where(d > delta, alpha * d, np.where(d < -delta, -(1 - alpha) * d, 0.0))
    return np.sum(w * v) / w.sum()


def _loglinquantile(a, y, w, p, c):
    alpha = float(p.get("alpha", 0.5))
    d = y - np.exp(a[:, 0])
    return np.sum(w * np.where(d > 0, alpha * d, -(1 - alpha) * d)) / w.sum()


def _poisson(a, y, w, p, c):
    return np.sum(w * (np.exp(a[:, 0]) - y * a[:, 0])) / w.sum()


def _huber(a, y, w, p, c):
    dl = float(p.get("delta", 1.0))
    d = np.abs(y - a[:, 0])
    return np.sum(w * np.where(d <= dl, 0.5 * d * d, dl * (d - 0.5 * dl))) / w.sum()


def _lq(a, y, w, p, c):
    return np.sum(w * np.abs(y - a[:, 0]) ** float(p.get("q", 2))) / w.sum()


def _expectile(a, y, w, p, c):
    alpha = float(p.get("alpha", 0.5))
    d = y - a[:, 0]
    return np.sum(w * np.where(d > 0, alpha, 1 - alpha) * d * d) / w.sum()


def _tweedie(a, y, w, p, c):
    vp = float(p.get("variance_power", 1.5))
    return np.sum(w * (-y * np.exp((1 - vp) * a[:, 0]) / (1 - vp) + np.exp((2 - vp) * a[:, 0]) / (2 - vp))) / w.sum()


def _logcosh(a, y, w, p, c):
    d = np.abs(y - a[:, 0])
    return np.sum(w * (d + np.log1p(np.exp(-2 * d)) - math.log(2))) / w.sum()


def _fair(a, y, w, p, c):
    s = float(p.get("smoothness", 1.0))
    d = np.abs(y - a[:, 0])
    return np.sum(w * s * s * (d / s - np.log1p(d / s))) / w.sum()


def _numerrors(a, y, w, p, c):
    return np.sum(w * (np.abs(a[:, 0] - y) > float(p.get("greater_than", 0.5)))) / w.sum()


def _multirmse(a, y, w, p, c):
    y = np.asarray(y, dtype=np.float64).reshape(a.shape)
    return math.sqrt(np.sum(w * ((a - y) ** 2).sum(1)) / w.sum())


# ---- binary classification ----------------------------------------------------------------------------------
def _logloss(a, y, w, p, c):
    x = np.ascontiguousarray(a[:, 0], dtype=np.float64)
    if x.size >= 20000:
        # large batches: the vectorised, threaded softplus (exact in float64 with the linear branch from 40 on)
        import torch
        tx = torch.from_numpy(x)
        v = torch.nn.functional.softplus(tx, threshold=40.0) - torch.from_numpy(np.ascontiguousarray(y, dtype=np.float64)) * tx
        return float((v * torch.from_numpy(np.ascontiguousarray(w, dtype=np.float64))).sum()) / float(w.sum())
    return np.sum(w * (np.logaddexp(0, x) - y * x)) / w.sum()


def _bin_counts(a, y, w, p):
    border = float(p.get("border", 0.5))
    pred = (_sigmoid(a[:, 0]) > border) if not p.get("_raw") else (a[:, 0] > 0)
    yb = y > 0.5
    tp = np.sum(w * (pred & yb)); fp = np.sum(w * (pred & ~yb)); fn = np.sum(w * (~pred & yb)); tn = np.sum(w * (~pred & ~yb))
    return tp, fp, fn, tn


def _classes(a):
    return (a[:, 0] > 0).astype(np.int64) if a.shape[1] == 1 else a.argmax(1)


def _accuracy(a, y, w, p, c):
    return np.sum(w * (_classes(a) == np.asarray(y).astype(np.int64))) / w.sum()


def _zero_one(a, y, w, p, c):
    return 1.0 - _accuracy(a, y, w, p, c)


def _precision(a, y, w, p, c):
    tp, fp, fn, tn = _bin_counts(a, y, w, p)
    return tp / (tp + fp) if tp + fp > 0 else 1.0


def _recall(a, y, w, p, c):
    tp, fp, fn, tn = _bin_counts(a, y, w, p)
    return tp / (tp + fn) if tp + fn > 0 else 1.0


def _f1(a, y, w, p, c):
    tp, fp, fn, tn = _bin_counts(a, y, w, p)
    return 2 * tp / (2 * tp + fp + fn) if 2 * tp + fp + fn > 0 else 0.0


def _balanced_accuracy(a, y, w, p, c):
    tp, fp, fn, tn = _bin_counts(a, y, w, p)
    return 0.5 * ((tp / (tp + fn) if tp + fn > 0 else 0) + (tn / (tn + fp) if tn + fp > 0 else 0))


def _balanced_error(a, y, w, p, c):
    return 1.0 - _balanced_accuracy(a, y, w, p, c)


def _mcc(a, y, w, p, c):
    if a.shape[1] > 1:
        return _multiclass_mcc(a, y, w)
    tp, fp, fn, tn = _bin_counts(a, y, w, p)
    den = math.sqrt((tp + fp) * (tp + fn) * (tn + fp) * (tn + fn))
    return (tp * tn - fp * fn) / den if den > 0 else 0.0


def _multiclass_mcc(a, y, w):
    k = a.shape[1]
    pred, yy = a.argmax(1), np.asarray(y).astype(np.int64)
    cm = np.zeros((k, k))
    np.add.at(cm, (yy, pred), w)
    t, pr, cdiag, s = cm.sum(1), cm.sum(0), np.trace(cm), cm.sum()
    den = math.sqrt((s * s - (pr ** 2).sum()) * (s * s - (t ** 2).sum()))
    return (cdiag * s - (t * pr).sum()) / den if den > 0 else 0.0


def _kappa(a, y, w, p, c):
    k = max(2, a.shape[1])
    pred, yy = _classes(a), np.asarray(y).astype(np.int64)
    cm = np.zeros((k, k))
    np.add.at(cm, (yy, pred), w)
    s = cm.sum()
    po = np.trace(cm) / s
    pe = (cm.sum(0) * cm.sum(1)).sum() / (s * s)
    return (po - pe) / (1 - pe) if pe < 1 else 0.0


def _brier(a, y, w, p, c):
    return np.sum(w * (_sigmoid(a[:, 0]) - y) ** 2) / w.sum()


def _hinge(a, y, w, p, c):
    return np.sum(w * np.maximum(0.0, 1.0 - (2 * y - 1) * a[:, 0])) / w.sum()


def _ctr_factor(a, y, w, p, c):
    s = np.sum(w * _sigmoid(a[:, 0]))
    return np.sum(w * y) / s if s > 0 else 0.0


def _norm_gini(a, y, w, p, c):
    return 2 * _auc(a, y, w, p, c) - 1


def auc_binary(score, y, w):
    order = np.argsort(score, kind="stable")
    s, yy, ww = score[order], y[order] > 0.5, w[order]
    # ties: average rank over equal scores via grouped sums
    pos_w, neg_w = ww * yy, ww * (~yy)
    tot_pos, tot_neg = pos_w.sum(), neg_w.sum()
    if tot_pos == 0 or tot_neg == 0:
        return 0.5
    change = np.ones(len(s), dtype=bool)
    change[1:] = s[1:] != s[:-1]
    gid = np.cumsum(change) - 1
    gp = np.bincount(gid, weights=pos_w)
    gn = np.bincount(gid, weights=neg_w)
    cn = np.cumsum(gn) - gn
    return float(np.sum(gp * (cn + 0.5 * gn)) / (tot_pos * tot_neg))


def _auc(a, y, w, p, c):
    y = np.asarray(y, dtype=np.float64)
    if a.shape[1] == 1:
        return auc_binary(a[:, 0], y, w)
    k = a.shape[1]       # Mu-like one-vs-rest average
    return float(np.mean([auc_binary(a[:, j], (y == j).astype(np.float64), w) for j in range(k)]))


# ---- multiclass ---------------------------------------------------------------------------------------------
def _multiclass(a, y, w, p, c):
    lp = np.log(np.clip(_softmax(a), 1e-300, None))
    return -np.sum(w * lp[np.arange(len(y)), np.asarray(y).astype(np.int64)]) / w.sum()


def _multiclass_ova(a, y, w, p, c):
    yy = np.zeros_like(a)
    yy[np.arange(len(y)), np.asarray(y).astype(np.int64)] = 1
    return np.sum(w * (np.logaddexp(0, a) - yy * a).mean(1)) / w.sum()


def _multilogloss(a, y, w, p, c):
    yy = np.asarray(y, dtype=np.float64).reshape(a.shape)
    return np.sum(w * (np.logaddexp(0, a) - yy * a).mean(1)) / w.sum()


def _total_f1(a, y, w, p, c):
    k = max(2, a.shape[1])
    pred, yy = _classes(a), np.asarray(y).astype(np.int64)
    f1s, ws = [], []
    for j in range(k):
        tp = np.sum(w * ((pred == j) & (yy == j))); fp = np.sum(w * ((pred == j) & (yy != j))); fn = np.sum(w * ((pred != j) & (yy == j)))
        f1s.append(2 * tp / (2 * tp + fp + fn) if 2 * tp + fp + fn > 0 else 0.0)
        ws.append(np.sum(w * (yy == j)))
    avg = p.get("average", "Weighted")
    if avg == "Macro":
        return float(np.mean(f1s))
    return float(np.sum(np.array(f1s) * np.array(ws)) / max(np.sum(ws), 1e-300))


def _hamming(a, y, w, p, c):
    if a.shape[1] > 1 and np.asarray(y).ndim == 2:
        return np.sum(w * ((a > 0) != (np.asarray(y) > 0.5)).mean(1)) / w.sum()
    return _zero_one(a, y, w, p, c)


# ---- ranking ------------------------------------------------------------------------------------------------
def _groups(c, n):
    off = c.get("group_offsets")
    return np.arange(n + 1) if off is None else np.asarray(off)


def _dcg_at(rel, top, exp_num, log_den=True):
    k = len(rel) if top <= 0 else min(top, len(rel))
    g = (2.0 ** rel[:k] - 1.0) if exp_num else rel[:k]
    d = np.log2(np.arange(2, k + 2)) if log_den else np.arange(1, k + 1)
    return float(np.sum(g / d))


def _ndcg_like(a, y, w, p, c, normalize):
    off = _groups(c, len(y))
    top = int(p.get("top", -1))
    exp_num = str(p.get("type", "Base")) == "Exp"
    log_den = str(p.get("denominator", "LogPosition")) == "LogPosition"
    tot, cnt = 0.0, 0.0
    for s, e in zip(off[:-1], off[1:]):
        rel = np.asarray(y[s:e], dtype=np.float64)
        order = np.argsort(-a[s:e, 0], kind="stable")
        dcg = _dcg_at(rel[order], top, exp_num, log_den)
        gw = w[s]
        if normalize:
            ideal = _dcg_at(np.sort(rel)[::-1], top, exp_num, log_den)
            tot += gw * (dcg / ideal if ideal > 0 else 1.0)
        else:
            tot += gw * dcg
        cnt += gw
    return tot / max(cnt, 1e-300)


def _ndcg(a, y, w, p, c):
    return _ndcg_like(a, y, w, p, c, True)


def _dcg(a, y, w, p, c):
    return _ndcg_like(a, y, w, p, c, False)


def _pfound(a, y, w, p, c):
    off = _groups(c, len(y))
    top, decay = int(p.get("top", -1)), float(p.get("decay", 0.85))
    tot, cnt = 0.0, 0.0
    for s, e in zip(off[:-1], off[1:]):
        rel = np.asarray(y[s:e], dtype=np.float64)
        order = np.argsort(-a[s:e, 0], kind="stable")
        k = len(rel) if top <= 0 else min(top, len(rel))
        plook, val = 1.0, 0.0
        for r in rel[order][:k]:
            val += plook * r
            plook *= (1 - r) * decay
        tot += w[s] * val
        cnt += w[s]
    return tot / max(cnt, 1e-300)


def _per_query(a, y, w, p, c, fn):
    off = _groups(c, len(y))
    tot, cnt = 0.0, 0.0
    for s, e in zip(off[:-1], off[1:]):
        order = np.argsort(-a[s:e, 0], kind="stable")
        tot += w[s] * fn(np.asarray(y[s:e], dtype=np.float64)[order])
        cnt += w[s]
    return tot / max(cnt, 1e-300)


def _map(a, y, w, p, c):
    top, border = int(p.get("top", -1)), float(p.get("border", 0.5))
    def f(rel):
        k = len(rel) if top <= 0 else min(top, len(rel))
        hit = rel[:k] > border
        if not hit.any():
            return 0.0
        prec = np.cumsum(hit) / np.arange(1, k + 1)
        return float(np.sum(prec * hit) / hit.sum())
    return _per_query(a, y, w, p, c, f)


def _mrr(a, y, w, p, c):
    top, border = int(p.get("top", -1)), float(p.get("border", 0.5))
    def f(rel):
        k = len(rel) if top <= 0 else min(top, len(rel))
        nz = np.nonzero(rel[:k] > border)[0]
        return 1.0 / (nz[0] + 1) if len(nz) else 0.0
    return _per_query(a, y, w, p, c, f)


def _precision_at(a, y, w, p, c):
    top, border = int(p.get("top", -1)), float(p.get("border", 0.5))
    def f(rel):
        k = len(rel) if top <= 0 else min(top, len(rel))
        return float(np.mean(rel[:k] > border)) if k else 0.0
    return _per_query(a, y, w, p, c, f)


def _recall_at(a, y, w, p, c):
    top, border = int(p.get("top", -1)), float(p.get("border", 0.5))
    def f(rel):
        k = len(rel) if top <= 0 else min(top, len(rel))
        tot = np.sum(rel > border)
        return float(np.sum(rel[:k] > border) / tot) if tot else 1.0
    return _per_query(a, y, w, p, c, f)


def _avg_gain(a, y, w, p, c):
    top = int(p.get("top", 1))
    return _per_query(a, y, w, p, c, lambda rel: float(np.mean(rel[:max(1, min(top, len(rel)))])))


def _query_rmse(a, y, w, p, c):
    off = _groups(c, len(y))
    tot = 0.0
    for s, e in zip(off[:-1], off[1:]):
        ww = w[s:e]
        shift = np.sum(ww * (y[s:e] - a[s:e, 0])) / ww.sum()
        tot += np.sum(ww * (y[s:e] - a[s:e, 0] - shift) ** 2)
    return math.sqrt(tot / w.sum())


def _query_softmax(a, y, w, p, c):
    off = _groups(c, len(y))
    beta = float(p.get("beta", 1.0))
    tot, cnt = 0.0, 0.0
    for s, e in zip(off[:-1], off[1:]):
        ww, yy = w[s:e], np.asarray(y[s:e], dtype=np.float64)
        x = beta * a[s:e, 0]
        x = x - x.max()
        lse = math.log(np.sum(ww * np.exp(x)))
        sw = np.sum(ww * yy)
        if sw > 0:
            tot -= np.sum(ww * yy * (x - lse))
            cnt += sw
    return tot / max(cnt, 1e-300)


def _query_auc(a, y, w, p, c):
    off = _groups(c, len(y))
    vals = [auc_binary(a[s:e, 0], np.asarray(y[s:e], dtype=np.float64), w[s:e]) for s, e in zip(off[:-1], off[1:])]
    return float(np.mean(vals)) if vals else 0.5


def _make_pairs(y, c):
    pairs = c.get("pairs")
    if pairs is not None:
        pw = c.get("pairs_weight")
        return np.asarray(pairs), (np.ones(len(pairs)) if pw is None else np.asarray(pw, dtype=np.float64))
    off = _groups(c, len(y))
    out = []
    for s, e in zip(off[:-1], off[1:]):
        yy = np.asarray(y[s:e])
        i, j = np.nonzero(yy[:, None] > yy[None, :])
        out.append(np.stack([i + s, j + s], 1))
    pr = np.concatenate(out) if out else np.zeros((0, 2), dtype=np.int64)
    return pr, np.ones(len(pr))


def _pairlogit(a, y, w, p, c):
    pr, pw = _make_pairs(y, c)
    if not len(pr):
        return 0.0
    d = a[pr[:, 0], 0] - a[pr[:, 1], 0]
    return float(np.sum(pw * np.logaddexp(0, -d)) / pw.sum())


def _pair_accuracy(a, y, w, p, c):
    pr, pw = _make_pairs(y, c)
    if not len(pr):
        return 1.0
    return float(np.sum(pw * (a[pr[:, 0], 0] > a[pr[:, 1], 0])) / pw.sum())


# ---- further metrics of the reference (catboost/libs/metrics/metric.cpp) -------------------------------------------
def _rmspe(a, y, w, p, c):
    yy = np.asarray(y, dtype=np.float64)
    return float(math.sqrt(np.sum(w * ((yy - a[:, 0]) / np.maximum(np.abs(yy), 1e-300)) ** 2) / w.sum()))


def _focal(a, y, w, p, c):
    alpha, gamma = float(p.get("focal_alpha", 0.25)), float(p.get("focal_gamma", 2.0))
    pr = np.clip(_sigmoid(a[:, 0]), 1e-15, 1 - 1e-15)
    yy = np.asarray(y, dtype=np.float64)
    pt = np.where(yy > 0.5, pr, 1 - pr)
    at = np.where(yy > 0.5, alpha, 1 - alpha)
    return float(np.sum(w * (-at * (1 - pt) ** gamma * np.log(pt))) / w.sum())


def _f_beta(a, y, w, p, c):
    beta = float(p.get("beta", 1.0))
    tp, fp, fn, _ = _bin_counts(a, y, w, p)
    den = (1 + beta * beta) * tp + beta * beta * fn + fp
    return float((1 + beta * beta) * tp / den) if den > 0 else 0.0


def _wkappa(a, y, w, p, c):
    pred = _classes(a)
    yy = np.asarray(y).astype(np.int64)
    k = int(max(pred.max(), yy.max())) + 1 if len(yy) else 1
    conf = np.zeros((k, k))
    np.add.at(conf, (yy, pred), w)
    n = conf.sum()
    ii, jj = np.meshgrid(np.arange(k), np.arange(k), indexing="ij")
    wt = ((ii - jj) ** 2) / max((k - 1) ** 2, 1)
    exp = np.outer(conf.sum(1), conf.sum(0)) / max(n, 1e-300)
    den = (wt * exp).sum()
    return float(1.0 - (wt * conf).sum() / den) if den > 0 else 0.0


def _loglik_of_prediction(a, y, w, p, c):
    # log-likelihood of the labels under the predicted probabilities relative to the prior (base 2), per document
    yy = np.asarray(y, dtype=np.float64)
    pr = np.clip(_sigmoid(a[:, 0]), 1e-15, 1 - 1e-15)
    prior = np.clip(np.sum(w * yy) / w.sum(), 1e-15, 1 - 1e-15)
    ll = yy * np.log2(pr / prior) + (1 - yy) * np.log2((1 - pr) / (1 - prior))
    return float(np.sum(w * ll) / w.sum())


def _prauc(a, y, w, p, c):
    yy = np.asarray(y, dtype=np.float64) > 0.5
    order = np.argsort(-a[:, 0], kind="stable")
    ws, ys = w[order], yy[order]
    tp = np.cumsum(ws * ys)
    fp = np.cumsum(ws * ~ys)
    # one point per distinct score
    sc = a[order, 0]
    last = np.r_[sc[1:] != sc[:-1], True]
    tp, fp = tp[last], fp[last]
    pos = tp[-1] if len(tp) else 0.0
    if pos <= 0:
        return 0.0
    prec = tp / np.maximum(tp + fp, 1e-300)
    rec = tp / pos
    prev_r = np.r_[0.0, rec[:-1]]
    prev_p = np.r_[1.0, prec[:-1]]
    return float(np.sum((rec - prev_r) * 0.5 * (prec + prev_p)))


def _query_average(a, y, w, p, c):
    top = int(p.get("top", 10 ** 9))
    off = _groups(c, len(y))
    vals = []
    for s, e in zip(off[:-1], off[1:]):
        order = np.argsort(-a[s:e, 0], kind="stable")[:top]
        vals.append(float(np.mean(np.asarray(y[s:e], dtype=np.float64)[order])) if len(order) else 0.0)
    return float(np.mean(vals)) if vals else 0.0


def _filtered_dcg(a, y, w, p, c):
    # DCG over the documents the model keeps (approx > 0), in their stored order inside the query
    exp_num = str(p.get("type", "Base")) == "Exp"
    log_den = str(p.get("denominator", "Position")) != "Position" or True
    off = _groups(c, len(y))
    tot = 0.0
    for s, e in zip(off[:-1], off[1:]):
        keep = a[s:e, 0] > 0
        rel = np.asarray(y[s:e], dtype=np.float64)[keep]
        gain = (2.0 ** rel - 1.0) if exp_num else rel
        pos = np.arange(1, len(rel) + 1)
        tot += float(np.sum(gain / (np.log2(pos + 1.0) if str(p.get("denominator", "LogPosition")) == "LogPosition" else pos)))
    return tot / max(len(off) - 1, 1)


def _err(a, y, w, p, c):
    top = int(p.get("top", 10 ** 9))
    off = _groups(c, len(y))
    vals = []
    for s, e in zip(off[:-1], off[1:]):
        order = np.argsort(-a[s:e, 0], kind="stable")[:top]
        rel = np.clip(np.asarray(y[s:e], dtype=np.float64)[order], 0.0, 1.0)
        look, v = 1.0, 0.0
        for k, r in enumerate(rel):
            v += look * r / (k + 1)
            look *= (1 - r)
        vals.append(v)
    return float(np.mean(vals)) if vals else 0.0


def _multirmse_missing(a, y, w, p, c):
    yy = np.asarray(y, dtype=np.float64).reshape(a.shape[0], -1)
    ok = ~np.isnan(yy)
    d = np.where(ok, yy - a[:, : yy.shape[1]], 0.0)
    tot = 0.0
    for k in range(yy.shape[1]):
        wk = w * ok[:, k]
        tot += np.sum(wk * d[:, k] ** 2) / max(wk.sum(), 1e-300)
    return float(math.sqrt(tot))


def _cox(a, y, w, p, c):
    # partial log-likelihood, larger is better (catboost/libs/metrics/metric.cpp TCoxMetric); |y| = time, y > 0 = event
    # observed, y < 0 = censored
    yy = np.asarray(y, dtype=np.float64)
    t = np.abs(yy)
    order = np.argsort(-t, kind="stable")
    f = a[order, 0]
    m = f.max() if len(f) else 0.0
    lse = m + np.log(np.cumsum(np.exp(f - m)))            # log sum over the risk set (times >= t_i)
    ev = yy[order] > 0
    return float(np.sum((f - lse)[ev]))


def _multi_quantile(a, y, w, p, c):
    alphas = [float(x) for x in str(p.get("alpha", "0.5")).split(",")]
    yy = np.asarray(y, dtype=np.float64)
    tot = 0.0
    for k, al in enumerate(alphas[: a.shape[1]]):
        d = yy - a[:, k]
        tot += np.sum(w * np.where(d >= 0, al * d, (al - 1) * d))
    return float(tot / (w.sum() * max(len(alphas), 1)))


def _survival_aft(a, y, w, p, c):
    # mean distance of exp(approx) from the target interval, 0 inside it (catboost/libs/metrics/metric.cpp
    # TSurvivalAftMetric); an end of -1 is open
    yy = np.asarray(y, dtype=np.float64).reshape(len(a), 2)
    lo = yy[:, 0]
    up = np.where(yy[:, 1] == -1, np.inf, yy[:, 1])
    lo = np.where(lo == -1, np.inf, lo)
    e = np.exp(a[:, 0])
    out = (e <= lo) | (e >= up)
    with np.errstate(invalid="ignore"):
        dist = np.minimum(np.abs(e - lo), np.abs(e - up))
    return float(np.sum(w * np.where(out, dist, 0.0)) / w.sum())


def _group_quantile(a, y, w, p, c):
    # pinball loss of the residual after the weighted mean residual of the document's group is taken out
    alpha = float(p.get("alpha", 0.5))
    off = _groups(c, len(a))
    g = np.repeat(np.arange(len(off) - 1), np.diff(off))
    r = np.asarray(y, dtype=np.float64) - a[:, 0]
    sw = np.bincount(g, weights=w)
    shift = np.bincount(g, weights=w * r) / np.maximum(sw, 1e-300)
    d = r - shift[g]
    return float(np.sum(w * np.where(d >= 0, alpha * d, (alpha - 1) * d)) / w.sum())


_METRICS: Dict[str, tuple] = {
    "SurvivalAft": (_survival_aft, False, ""), "GroupQuantile": (_group_quantile, False, "group"),
    "RMSPE": (_rmspe, False, ""), "Focal": (_focal, False, ""), "F": (_f_beta, True, ""), "WKappa": (_wkappa, True, ""),
    "LogLikelihoodOfPrediction": (_loglik_of_prediction, True, ""), "PRAUC": (_prauc, True, ""),
    "QueryAverage": (_query_average, True, "group"), "FilteredDCG": (_filtered_dcg, True, "group"),
    "ERR": (_err, True, "group"), "MultiRMSEWithMissingValues": (_multirmse_missing, False, ""),
    "Cox": (_cox, True, ""), "MultiQuantile": (_multi_quantile, False, ""),
    # name: (fn, is_max_optimal, needs)
    "RMSE": (_rmse, False, ""), "MAE": (_mae, False, ""), "MAPE": (_mape, False, ""), "SMAPE": (_smape, False, ""),
    "MSLE": (_msle, False, ""), "R2": (_r2, True, ""), "MedianAbsoluteError": (_median_abs, False, ""),
    "Quantile": (_quantile, False, ""), "LogLinQuantile": (_loglinquantile, False, ""), "Poisson": (_poisson, False, ""),
    "Huber": (_huber, False, ""), "Lq": (_lq, False, ""), "Expectile": (_expectile, False, ""),
    "Tweedie": (_tweedie, False, ""), "LogCosh": (_logcosh, False, ""), "FairLoss": (_fair, False, ""),
    "NumErrors": (_numerrors, False, ""), "MultiRMSE": (_multirmse, False, ""),
    "Logloss": (_logloss, False, ""), "CrossEntropy": (_logloss, False, ""), "Accuracy": (_accuracy, True, ""),
    "ZeroOneLoss": (_zero_one, False, ""), "Precision": (_precision, True, ""), "Recall": (_recall, True, ""),
    "F1": (_f1, True, ""), "BalancedAccuracy": (_balanced_accuracy, True, ""),
    "BalancedErrorRate": (_balanced_error, False, ""), "MCC": (_mcc, True, ""), "Kappa": (_kappa, True, ""),
    "BrierScore": (_brier, False, ""), "HingeLoss": (_hinge, False, ""), "CtrFactor": (_ctr_factor, False, ""),
    "NormalizedGini": (_norm_gini, True, ""), "AUC": (_auc, True, ""),
    "MultiClass": (_multiclass, False, ""), "MultiClassOneVsAll": (_multiclass_ova, False, ""),
    "MultiLogloss": (_multilogloss, False, ""), "MultiCrossEntropy": (_multilogloss, False, ""),
    "TotalF1": (_total_f1, True, ""), "HammingLoss": (_hamming, False, ""),
    "NDCG": (_ndcg, True, "group"), "DCG": (_dcg, True, "group"), "PFound": (_pfound, True, "group"),
    "MAP": (_map, True, "group"), "MRR": (_mrr, True, "group"), "PrecisionAt": (_precision_at, True, "group"),
    "RecallAt": (_recall_at, True, "group"), "AverageGain": (_avg_gain, True, "group"),
    "QueryRMSE": (_query_rmse, False, "group"), "QuerySoftMax": (_query_softmax, False, "group"),
    "QueryAUC": (_query_auc, True, "group"), "PairLogit": (_pairlogit, False, "pairs"),
    "PairAccuracy": (_pair_accuracy, True, "pairs"),
    "YetiRank": (_pfound, True, "group"), "YetiRankPairwise": (_pfound, True, "group"),
    "PairLogitPairwise": (_pairlogit, False, "pairs"), "QueryCrossEntropy": (_logloss, False, "group"),
    "LambdaMart": (_ndcg, True, "group"), "StochasticRank": (_ndcg, True, "group"),
    "StochasticFilter": (_filtered_dcg, True, "group"),
    "RMSEWithUncertainty": (lambda a, y, w, p, c: float(np.sum(w * (a[:, 1] + 0.5 * (y - a[:, 0]) ** 2 * np.exp(-2 * a[:, 1])
                                                                 + 0.5 * math.log(2 * math.pi))) / w.sum()), False, ""),
}


def make_metric(desc) -> Metric:
    if isinstance(desc, Metric):
        return desc
    return Metric(str(desc))


def is_max_optimal(desc: str) -> bool:
    return make_metric(desc).is_max_optimal


# ---- metric objects (catboost/python-package/catboost/metrics.py) ----------------------------------------------
# ``metrics.AUC(type='Ranking')``, ``metrics.Quantile(alpha=0.3)``: an object whose string form is the metric description
# accepted everywhere a metric name is (eval_metric, custom_metric, eval_metrics) and that can evaluate itself.
class BuiltinMetric:
    _name = ""

    def __init__(self, **params):
        self._params = {k: v for k, v in params.items() if v is not None}

    def __str__(self):
        if not self._params:
            return self._name
        def fmt(v):
            return str(v).lower() if isinstance(v, bool) else str(v)
        return self._name + ":" + ";".join(f"{k}={fmt(v)}" for k, v in self._params.items())

    __repr__ = __str__

    def set_hints(self, **hints):
        self._params["hints"] = "|".join(f"{k}~{v}" for k, v in hints.items())
        return self

    def is_max_optimal(self):
        return bool(_METRICS[self._name][1])

    def eval(self, label, approx, weight=None, group_id=None, group_weight=None, subgroup_id=None, pairs=None,
             thread_count=-1):
        from ..utils import eval_metric
        return eval_metric(label, approx, str(self), weight, group_id, group_weight, subgroup_id, pairs, thread_count)[0]

    @classmethod
    def params_with_defaults(cls):
        return {}


def _make_metric_classes():
    made = {}
    for _nm in _METRICS:
        made[_nm] = type(_nm, (BuiltinMetric,), {"_name": _nm, "__doc__": f"The {_nm} metric; keyword arguments are its parameters."})
    return made


_METRIC_CLASSES = _make_metric_classes()
globals().update(_METRIC_CLASSES)
