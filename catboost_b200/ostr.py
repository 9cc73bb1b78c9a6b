"""Object importance: how much every training object influences the loss on other objects (LeafInfluence, Sharchilev
et al. 2018; catboost/private/libs/documents_importance/docs_importance_helpers.cpp).

The tree structures are kept fixed; only the leaf values react to the weight ``w_i`` of a training object.  With the
package's conventions (``der = -dLoss/dF``, ``hess = d2Loss/dF2``) a leaf value is ``lr * D / H`` with
``D = sum w der``, ``H = sum w hess + l2`` over the leaf (``H = sum w + l2`` for the Gradient method), so

    d value_l / d w_i = (lr * dD_l - value_l * dH_l) / H_l
    dD_l = [i in l] der_i  - sum_{j in l} w_j hess_j  J[j]
    dH_l = [i in l] hess_i + sum_{j in l} w_j hess'_j J[j]          (Newton; [i in l] for Gradient)

where ``J[j] = dF(x_j) / dw_i`` accumulated over the earlier trees.  ``AllPoints`` carries J for every training object
(the exact first-order answer), ``SinglePoint`` only for the object itself.  The score of training object i for a test
object k is ``der_k * dF(x_k)/dw_i``: positive when giving i more weight lowers the loss on k.  All removed objects of a
batch are processed together as rows of one matrix, on the GPU when there is one.
"""
from __future__ import annotations

from typing import Optional, Tuple

import numpy as np
import torch

from .data.pool import CatBoostError, Pool


def _point_ders(objective, approx: torch.Tensor, target: torch.Tensor):
    der, hess = objective.der_hess(approx.unsqueeze(0).float(), target, None)
    eps = 1e-3
    _, hp = objective.der_hess((approx + eps).unsqueeze(0).float(), target, None)
    _, hm = objective.der_hess((approx - eps).unsqueeze(0).float(), target, None)
    return der[0].double(), hess[0].double(), ((hp[0] - hm[0]).double() / (2 * eps))


def object_importance(model, objective, params: dict, train_pool: Pool, test_pool: Pool, y_train, y_test,
                      update_method: str = "SinglePoint", device: Optional[str] = None,
                      batch_elements: int = 16_000_000) -> np.ndarray:
    """Scores [n_train, n_test].  ``y_train`` / ``y_test``: targets as the objective sees them (class indices for
    classification)."""
    if model.dims != 1:
        raise CatBoostError("object importance is computed for one-dimensional models")
    if not objective.is_pointwise:
        raise CatBoostError("object importance needs a pointwise loss function")
    kind = update_method.split(":")[0]
    if kind not in ("SinglePoint", "TopKLeaves", "AllPoints"):
        raise CatBoostError(f"unknown update_method {update_method!r}")
    all_points = kind != "SinglePoint"          # TopKLeaves is answered with the exact (AllPoints) update
    dev = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
    lr = float(params.get("learning_rate", 0.03) or 0.03)
    l2 = float(params.get("l2_leaf_reg", 3.0) if params.get("l2_leaf_reg") is not None else 3.0)
    method = params.get("leaf_estimation_method") or "Newton"

    fd, ch = model.pool_arrays(train_pool)
    leaf_tr = torch.from_numpy(model.leaf_indices(fd, ch)).to(dev)                   # [n, T]
    fdt, cht = model.pool_arrays(test_pool)
    leaf_te = torch.from_numpy(model.leaf_indices(fdt, cht)).to(dev)                 # [m, T]
    n, T = leaf_tr.shape
    m = leaf_te.shape[0]
    y = torch.from_numpy(np.asarray(y_train, dtype=np.float32).reshape(n, -1)[:, 0].copy()).to(dev)
    yt = torch.from_numpy(np.asarray(y_test, dtype=np.float32).reshape(m, -1)[:, 0].copy()).to(dev)
    w = torch.ones(n, dtype=torch.float64, device=dev) if train_pool.weight is None else \
        torch.from_numpy(np.asarray(train_pool.weight, dtype=np.float64)).to(dev)
    bias = float(np.ravel(model.bias)[0])
    values = [torch.from_numpy(np.asarray(t.leaf_values, dtype=np.float64)[:, 0] * model.scale).to(dev) for t in model.trees]

    # what the training saw before every tree
    approx = torch.full((n,), bias, dtype=torch.float64, device=dev)
    per_tree = []
    for t in range(T):
        der, hess, hess1 = _point_ders(objective, approx, y)
        L = values[t].shape[0]
        lt = leaf_tr[:, t]
        if method == "Newton":
            H = torch.zeros(L, dtype=torch.float64, device=dev).index_add_(0, lt, w * hess) + l2
        else:
            H = torch.zeros(L, dtype=torch.float64, device=dev).index_add_(0, lt, w) + l2
        per_tree.append((der, hess, hess1, H))
        approx = approx + values[t][lt]
    approx_te = torch.full((m,), bias, dtype=torch.float64, device=dev)
    for t in range(T):
        approx_te = approx_te + values[t][leaf_te[:, t]]
    der_te, _, _ = _point_ders(objective, approx_te, yt)

    out = np.zeros((n, m), dtype=np.float64)
    B = n if not all_points else max(1, min(n, batch_elements // max(n, 1)))
    for b0 in range(0, n, B):
        ids = torch.arange(b0, min(n, b0 + B), device=dev)
        nb = ids.numel()
        rows = torch.arange(nb, device=dev)
        dF_te = torch.zeros((nb, m), dtype=torch.float64, device=dev)
        J = torch.zeros((nb, n), dtype=torch.float64, device=dev) if all_points else \
            torch.zeros(nb, dtype=torch.float64, device=dev)          # SinglePoint: dF(x_i)/dw_i only
        for t in range(T):
            der, hess, hess1, H = per_tree[t]
            lt = leaf_tr[:, t]
            L = H.shape[0]
            own = lt[ids]                                             # the leaf of every removed object
            dD = torch.zeros((nb, L), dtype=torch.float64, device=dev)
            dH = torch.zeros((nb, L), dtype=torch.float64, device=dev)
            dD[rows, own] = der[ids]
            dH[rows, own] = hess[ids] if method == "Newton" else 1.0
            if all_points:
                dD.index_add_(1, lt, -(J * (w * hess)))
                if method == "Newton":
                    dH.index_add_(1, lt, J * (w * hess1))
            else:
                dD[rows, own] -= w[ids] * hess[ids] * J
                if method == "Newton":
                    dH[rows, own] += w[ids] * hess1[ids] * J
            dval = (lr * dD - values[t].unsqueeze(0) * dH) / H.unsqueeze(0)             # [nb, L]
            if all_points:
                J += dval[:, lt]
            else:
                J += dval[rows, own]
            dF_te += dval[:, leaf_te[:, t]]
        out[b0:b0 + nb] = (dF_te * der_te.unsqueeze(0)).cpu().numpy()
    return out


def select(scores: np.ndarray, type: str, top_size: int, sign: str) -> Tuple[np.ndarray, np.ndarray]:
    """Order training objects by |score| (catboost/private/libs/documents_importance/docs_importance.cpp:44-110).
    ``Average``: one list from the mean over the test objects; ``PerObject``: one list per test object."""
    if type not in ("Average", "PerObject"):
        raise CatBoostError("type must be 'Average' or 'PerObject'")
    if sign not in ("All", "Positive", "Negative"):
        raise CatBoostError("importance_values_sign must be 'All', 'Positive' or 'Negative'")
    mat = scores.mean(axis=1, keepdims=True).T if type == "Average" else scores.T           # [lists, n_train]
    idx_out, val_out = [], []
    for row in mat:
        order = np.argsort(-np.abs(row), kind="stable")
        if sign == "Positive":
            order = order[row[order] > 0]
        elif sign == "Negative":
            order = order[row[order] < 0]
        if top_size is not None and top_size >= 0:
            order = order[:top_size]
        idx_out.append(order.astype(np.int64))
        val_out.append(row[order])
    if type == "Average":
        return idx_out[0], val_out[0]
    return idx_out, val_out
