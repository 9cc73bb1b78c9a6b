"""ROC curve and threshold selection helpers (catboost.utils.get_roc_curve / select_threshold)."""
import numpy as np


def roc_curve(model, pool):
    raw = model.predict(pool, prediction_type="RawFormulaVal")
    p = 1.0 / (1.0 + np.exp(-raw))
    y = model._encode_labels(pool.label) > 0.5
    order = np.argsort(-p, kind="stable")
    p, y = p[order], y[order]
    tp = np.cumsum(y)
    fp = np.cumsum(~y)
    distinct = np.r_[np.nonzero(np.diff(p))[0], len(p) - 1]
    tpr = np.r_[0.0, tp[distinct] / max(tp[-1], 1)]
    fpr = np.r_[0.0, fp[distinct] / max(fp[-1], 1)]
    thr = np.r_[1.0, p[distinct]]
    return fpr, tpr, thr


def select_threshold(model, pool, FPR=None, FNR=None):
    fpr, tpr, thr = roc_curve(model, pool)
    if FPR is not None:
        ok = np.nonzero(fpr <= FPR)[0]
        return float(thr[ok[-1]])
    if FNR is not None:
        ok = np.nonzero(1 - tpr <= FNR)[0]
        return float(thr[ok[0]])
    k = int(np.argmin(np.abs(fpr - (1 - tpr))))
    return float(thr[k])
