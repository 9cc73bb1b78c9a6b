"""Objectives: derivatives, loss values and starting constants.

``der`` is the negative gradient of the loss with respect to the approx (what the reference calls "der"),
``hess`` the positive second derivative.  Pointwise losses also carry the id of their native implementation
(``ops/cuda/cb_losses.cuh``) so the GPU trainer never leaves the device; the torch versions here drive the
CPU trainer, the multi-dimensional and ranking trainers, and are the oracle of the kernels' tests.
Formulas: catboost/private/libs/algo_helpers/error_functions.h:191-1669,
catboost/cuda/targets/kernel/pointwise_targets.cu, multilogit.cu, query_rmse.cu, query_softmax.cu, pair_logit.cu.
"""
from __future__ import annotations

import math
from typing import Optional

import numpy as np
import torch

from ..data.pool import CatBoostError

NATIVE_LOSS_ID = {"RMSE": 0, "Logloss": 1, "CrossEntropy": 2, "Poisson": 3, "MAE": 4, "Quantile": 5,
                  "LogLinQuantile": 6, "MAPE": 7, "Huber": 8, "Lq": 9, "Expectile": 10, "Tweedie": 11, "LogCosh": 12,
                  "MultiClass": 50}
LOSS_EXTERNAL = 100


class Objective:
    name = "RMSE"
    dims = 1                 # approx dimension
    is_pointwise = True
    needs_groups = False
    needs_pairs = False
    is_classification = False
    is_multiclass = False
    stochastic = False

    def __init__(self, params: Optional[dict] = None):
        self.params = dict(params or {})

    # native pointwise implementation ------------------------------------------------------------
    @property
    def native_id(self) -> Optional[int]:
        """Identifier of the objective's device formula (pointwise losses: cb_losses.cuh; 50 = softmax MultiClass,
        cb_multiclass.cu), None when the derivatives only exist as tensor code."""
        return NATIVE_LOSS_ID.get(self.name)

    def native_params(self):
        return 0.0, 0.0

    # torch implementation ---------------------------------------------------------------------------
    def der_hess(self, approx: torch.Tensor, target: torch.Tensor, weight: Optional[torch.Tensor], ctx=None):
        """approx [dims, n] -> (der [dims, n], hess [dims, n]); both already multiplied by the sample weight."""
        raise NotImplementedError

    def value(self, approx, target, weight, ctx=None) -> float:
        raise NotImplementedError

    def start_constant(self, target: np.ndarray, weight: Optional[np.ndarray]):
        return np.zeros(self.dims)

    def _w(self, x, weight):
        return x if weight is None else x * weight


def _wsum(x, weight):
    return float((x if weight is None else x * weight).sum().item())


def _wtot(n, weight):
    return float(n) if weight is None else float(weight.sum().item())


class _Pointwise(Objective):
    def _point(self, a, y):
        raise NotImplementedError

    def der_hess(self, approx, target, weight, ctx=None):
        d, h, _ = self._point(approx[0], target)
        if weight is not None:
            d, h = d * weight, h * weight
        return d.unsqueeze(0), h.unsqueeze(0)

    def value(self, approx, target, weight, ctx=None):
        _, _, v = self._point(approx[0], target)
        return _wsum(v, weight) / max(_wtot(target.numel(), weight), 1e-300)


class RMSE(_Pointwise):
    name = "RMSE"

    def _point(self, a, y):
        d = y - a
        return d, torch.ones_like(d), d * d

    def value(self, approx, target, weight, ctx=None):
        return math.sqrt(super().value(approx, target, weight))

    def start_constant(self, target, weight):
        return np.array([np.average(target.astype(np.float64), weights=weight)])


class Logloss(_Pointwise):
    name = "Logloss"
    is_classification = True

    def _point(self, a, y):
        p = torch.sigmoid(a)
        v = torch.nn.functional.softplus(a) - y * a
        return y - p, (p * (1 - p)).clamp_min(1e-16), v

    def start_constant(self, target, weight):
        t = np.asarray(target)
        if weight is None:
            p = float(t.sum(dtype=np.float64)) / max(t.size, 1)             # no float64 copy of the target
        else:
            p = float(np.dot(t.astype(np.float64, copy=False), np.asarray(weight, dtype=np.float64)) / np.sum(weight, dtype=np.float64))
        p = min(max(p, 1e-9), 1 - 1e-9)
        return np.array([math.log(p / (1 - p))])


class CrossEntropy(Logloss):
    name = "CrossEntropy"


class Poisson(_Pointwise):
    name = "Poisson"

    def _point(self, a, y):
        e = torch.exp(a)
        return y - e, e, e - y * a


class MAE(_Pointwise):
    name = "MAE"

    def _point(self, a, y):
        d = y - a
        return torch.sign(d), torch.ones_like(d), d.abs()

    def start_constant(self, target, weight):
        return np.array([_weighted_quantile(target, weight, 0.5)])


class Quantile(_Pointwise):
    name = "Quantile"

    def native_params(self):
        return float(self.params.get("alpha", 0.5)), float(self.params.get("delta", 1e-6))

    def _point(self, a, y):
        alpha, delta = self.native_params()
        d = y - a
        up, dn = d > delta, d < -delta
        der = torch.where(up, torch.full_like(d, alpha), torch.where(dn, torch.full_like(d, -(1 - alpha)), torch.zeros_like(d)))
        val = torch.where(up, alpha * d, torch.where(dn, -(1 - alpha) * d, torch.zeros_like(d)))
        return der, torch.ones_like(d), val

    def start_constant(self, target, weight):
        return np.array([_weighted_quantile(target, weight, float(self.params.get("alpha", 0.5)))])


class LogLinQuantile(_Pointwise):
    name = "LogLinQuantile"

    def native_params(self):
        return float(self.params.get("alpha", 0.5)), 0.0

    def _point(self, a, y):
        alpha = self.native_params()[0]
        e = torch.exp(a)
        d = y - e
        der = torch.where(d > 0, alpha * e, -(1 - alpha) * e)
        return der, torch.ones_like(d), torch.where(d > 0, alpha * d, -(1 - alpha) * d)


class MAPE(_Pointwise):
    name = "MAPE"

    def _point(self, a, y):
        d = y - a
        s = 1.0 / y.abs().clamp_min(1.0)
        return torch.sign(d) * s, torch.ones_like(d), d.abs() * s

    def start_constant(self, target, weight):
        w = 1.0 / np.maximum(1.0, np.abs(target))
        return np.array([_weighted_quantile(target, w if weight is None else w * weight, 0.5)])


class Huber(_Pointwise):
    name = "Huber"

    def native_params(self):
        return float(self.params.get("delta", 1.0)), 0.0

    def _point(self, a, y):
        dl = self.native_params()[0]
        d = y - a
        ad = d.abs()
        inside = ad <= dl
        der = torch.where(inside, d, torch.sign(d) * dl)
        hess = torch.where(inside, torch.ones_like(d), torch.full_like(d, 1e-6))
        return der, hess, torch.where(inside, 0.5 * d * d, dl * (ad - 0.5 * dl))


class Lq(_Pointwise):
    name = "Lq"

    def native_params(self):
        return float(self.params.get("q", 2.0)), 0.0

    def _point(self, a, y):
        q = self.native_params()[0]
        d = y - a
        ad = d.abs()
        der = q * ad.pow(q - 1) * torch.sign(d)
        hess = q * (q - 1) * ad.pow(q - 2) if q >= 2 else torch.ones_like(d)
        hess = torch.where(ad == 0, torch.full_like(d, 2.0 if q == 2 else 1.0), hess)
        return der, hess, ad.pow(q)


class Expectile(_Pointwise):
    name = "Expectile"

    def native_params(self):
        return float(self.params.get("alpha", 0.5)), 0.0

    def _point(self, a, y):
        alpha = self.native_params()[0]
        d = y - a
        w = torch.where(d > 0, torch.full_like(d, alpha), torch.full_like(d, 1 - alpha))
        return 2 * w * d, 2 * w, w * d * d


class Tweedie(_Pointwise):
    name = "Tweedie"

    def native_params(self):
        return float(self.params.get("variance_power", 1.5)), 0.0

    def _point(self, a, y):
        p = self.native_params()[0]
        e1, e2 = torch.exp((1 - p) * a), torch.exp((2 - p) * a)
        return y * e1 - e2, (-y * (1 - p) * e1 + (2 - p) * e2).clamp_min(1e-16), -y * e1 / (1 - p) + e2 / (2 - p)


class LogCosh(_Pointwise):
    name = "LogCosh"

    def _point(self, a, y):
        d = y - a
        t = torch.tanh(d)
        ad = d.abs()
        return t, (1 - t * t).clamp_min(1e-6), ad + torch.log1p(torch.exp(-2 * ad)) - math.log(2.0)


# ---- multi-dimensional ----------------------------------------------------------------------------------
class MultiClass(Objective):
    name = "MultiClass"
    is_pointwise = False
    is_classification = True
    is_multiclass = True

    def __init__(self, params=None, n_classes: int = 2):
        super().__init__(params)
        self.dims = int(n_classes)

    def der_hess(self, approx, target, weight, ctx=None):
        p = torch.softmax(approx, dim=0)
        onehot = torch.zeros_like(p)
        onehot.scatter_(0, target.long().unsqueeze(0), 1.0)
        der = onehot - p
        hess = (p * (1 - p)).clamp_min(1e-16)
        if weight is not None:
            der, hess = der * weight, hess * weight
        return der, hess

    def value(self, approx, target, weight, ctx=None):
        lp = torch.log_softmax(approx, dim=0)
        v = -lp.gather(0, target.long().unsqueeze(0))[0]
        return _wsum(v, weight) / max(_wtot(target.numel(), weight), 1e-300)

    def hess_blocks(self, approx, target, weight, idx, n_leaves):
        """Per-leaf K x K Hessian blocks of the negative log-likelihood, [n_leaves, K, K] float64:
        sum over the leaf's documents of w (diag(p) - p p^T)."""
        p = torch.softmax(approx, dim=0).double()                      # [K, n]
        w = torch.ones(p.shape[1], dtype=torch.float64, device=p.device) if weight is None else weight.double()
        K = p.shape[0]
        H = torch.zeros((n_leaves, K, K), dtype=torch.float64, device=p.device)
        pw = p * w
        for k in range(K):
            row = -(pw[k].unsqueeze(0) * p)                            # [K, n]: -w p_k p_j
            row[k] += pw[k]
            H[:, k, :].index_add_(0, idx, row.t())
        return H


class MultiClassOneVsAll(MultiClass):
    hess_blocks = None
    name = "MultiClassOneVsAll"

    def der_hess(self, approx, target, weight, ctx=None):
        p = torch.sigmoid(approx)
        onehot = torch.zeros_like(p)
        onehot.scatter_(0, target.long().unsqueeze(0), 1.0)
        der, hess = onehot - p, (p * (1 - p)).clamp_min(1e-16)
        if weight is not None:
            der, hess = der * weight, hess * weight
        return der, hess

    def value(self, approx, target, weight, ctx=None):
        onehot = torch.zeros_like(approx)
        onehot.scatter_(0, target.long().unsqueeze(0), 1.0)
        v = (torch.nn.functional.softplus(approx) - onehot * approx).sum(0) / approx.shape[0]
        return _wsum(v, weight) / max(_wtot(target.numel(), weight), 1e-300)


class MultiRMSE(Objective):
    name = "MultiRMSE"
    is_pointwise = False

    def __init__(self, params=None, n_targets: int = 1):
        super().__init__(params)
        self.dims = int(n_targets)

    def der_hess(self, approx, target, weight, ctx=None):
        d = target - approx          # target [dims, n]
        h = torch.ones_like(d)
        if weight is not None:
            d, h = d * weight, h * weight
        return d, h

    def value(self, approx, target, weight, ctx=None):
        v = ((target - approx) ** 2).sum(0)
        return math.sqrt(_wsum(v, weight) / max(_wtot(target.shape[1], weight), 1e-300))

    def start_constant(self, target, weight):
        return np.average(target.astype(np.float64), axis=0, weights=weight)


class MultiLogloss(MultiRMSE):
    name = "MultiLogloss"
    is_classification = True

    def der_hess(self, approx, target, weight, ctx=None):
        p = torch.sigmoid(approx)
        d, h = target - p, (p * (1 - p)).clamp_min(1e-16)
        if weight is not None:
            d, h = d * weight, h * weight
        return d, h

    def value(self, approx, target, weight, ctx=None):
        v = (torch.nn.functional.softplus(approx) - target * approx).mean(0)
        return _wsum(v, weight) / max(_wtot(target.shape[1], weight), 1e-300)

    def start_constant(self, target, weight):
        return np.zeros(self.dims)


class MultiCrossEntropy(MultiLogloss):
    name = "MultiCrossEntropy"


class RMSEWithUncertainty(Objective):
    name = "RMSEWithUncertainty"
    is_pointwise = False
    dims = 2

    def der_hess(self, approx, target, weight, ctx=None):
        mu, ls = approx[0], approx[1]          # mean, log std
        # the natural gradient of the Gaussian likelihood (gradient times the inverse Fisher information), as in
        # catboost/private/libs/algo_helpers/error_functions.h TRMSEWithUncertaintyError: the mean's derivative is the
        # plain residual with unit second derivative
        prec = torch.exp(-2 * ls)
        d0 = target - mu
        d1 = (target - mu) ** 2 * prec - 1.0
        h0 = torch.ones_like(mu)
        h1 = (2 * (target - mu) ** 2 * prec).clamp_min(1e-6)
        der, hess = torch.stack([d0, d1]), torch.stack([h0, h1])
        if weight is not None:
            der, hess = der * weight, hess * weight
        return der, hess

    def value(self, approx, target, weight, ctx=None):
        mu, ls = approx[0], approx[1]
        v = ls + 0.5 * (target - mu) ** 2 * torch.exp(-2 * ls) + 0.5 * math.log(2 * math.pi)
        return _wsum(v, weight) / max(_wtot(target.numel(), weight), 1e-300)

    def start_constant(self, target, weight):
        m = float(np.average(target, weights=weight))
        var = float(np.average((target - m) ** 2, weights=weight))
        return np.array([m, 0.5 * math.log(max(var, 1e-12))])


class Focal(_Pointwise):
    """Focal loss for binary classification, -a_t (1 - p_t)^gamma log p_t with p_t the probability of the true class
    (first and second derivatives as in catboost/private/libs/algo_helpers/error_functions.h:1669-1710)."""
    name = "Focal"
    is_classification = True

    def _point(self, a, y):
        alpha = float(self.params.get("focal_alpha", 0.25))
        gamma = float(self.params.get("focal_gamma", 2.0))
        pos = y > 0.5
        p = torch.sigmoid(a).clamp(1e-13, 1.0 - 1e-13)
        pt = torch.where(pos, p, 1.0 - p)
        at = torch.where(pos, torch.full_like(p, alpha), torch.full_like(p, 1.0 - alpha))
        sgn = torch.where(pos, torch.ones_like(p), -torch.ones_like(p))
        lg = torch.log(pt)
        u = at * sgn * (1.0 - pt) ** gamma
        du = -at * sgn * gamma * (1.0 - pt) ** (gamma - 1.0)
        v = gamma * pt * lg + pt - 1.0
        dv = gamma * lg + gamma + 1.0
        der = -(u * v)                                             # ascent direction of -loss
        hess = ((du * v + u * dv) * sgn * (pt * (1.0 - pt))).clamp_min(1e-16)
        return der, hess, -at * (1.0 - pt) ** gamma * lg


class Cox(Objective):
    """Cox proportional hazards: |target| is the time, target > 0 an observed event, target < 0 a censored one.  The
    partial likelihood couples all documents, so the derivatives come from one pass over the documents sorted by time
    (catboost/private/libs/algo_helpers/error_functions.cpp:153-205): with S_i the sum of exp(approx) over documents at
    position >= i, r_i = sum over events e <= i of 1 / S_e and s_i the same sum of 1 / S_e^2,
    der_i = [event_i] - exp(approx_i) r_i and hess_i = exp(approx_i) r_i - exp(approx_i)^2 s_i.  Weights are not used,
    as in the reference."""
    name = "Cox"
    is_pointwise = False

    def _sorted_terms(self, a, target):
        order = torch.sort(target.abs(), stable=True).indices
        e = torch.exp((a - a.max()).double())[order]
        S = torch.flip(torch.cumsum(torch.flip(e, [0]), 0), [0]).clamp_min(1e-300)
        ev = (target[order] > 0).double()
        return order, e, S, ev

    def der_hess(self, approx, target, weight, ctx=None):
        a = approx[0]
        order, e, S, ev = self._sorted_terms(a, target)
        r = torch.cumsum(ev / S, 0)
        s2 = torch.cumsum(ev / (S * S), 0)
        d_s = ev - e * r
        h_s = (e * r - e * e * s2).clamp_min(1e-16)
        der = torch.empty_like(a)
        hess = torch.empty_like(a)
        der[order] = d_s.float()
        hess[order] = h_s.float()
        return der.unsqueeze(0), hess.unsqueeze(0)

    def value(self, approx, target, weight, ctx=None):
        """Negative log partial likelihood (the quantity training minimises)."""
        a = approx[0]
        order, e, S, ev = self._sorted_terms(a, target)
        ll = ((a - a.max()).double()[order] - torch.log(S)) * ev
        return -float(ll.sum().item())


class SurvivalAft(Objective):
    """Accelerated failure time model on interval-censored targets: two label columns [lower, upper], -1 for an open
    end, equal ends for an observed time.  z = (log t - approx) / scale follows the chosen distribution (Normal,
    Logistic or Extreme); derivatives of the log-likelihood with the reference's clipping and its limits for vanishing
    denominators (catboost/private/libs/algo_helpers/error_functions.cpp:360-450, survival_aft_utils.cpp,
    catboost/libs/helpers/distribution_helpers.cpp)."""
    name = "SurvivalAft"
    is_pointwise = False
    target_columns = 2

    def __init__(self, params=None):
        super().__init__(params)
        self.dist = str(self.params.get("dist", "Normal")).capitalize()
        self.scale = float(self.params.get("scale", 1.0))
        if self.dist not in ("Normal", "Logistic", "Extreme"):
            raise CatBoostError(f"SurvivalAft: unknown distribution {self.dist!r}")
        if not self.scale > 0:
            raise CatBoostError("SurvivalAft: scale should be positive")

    # pdf, cdf, pdf', pdf'' of the three distributions ------------------------------------------------
    def _pdf_cdf(self, z):
        if self.dist == "Normal":
            pdf = torch.exp(-0.5 * z * z) * 0.3989422804014327
            cdf = 0.5 + 0.5 * torch.erf(z / math.sqrt(2.0))
            return pdf, cdf, -z * pdf, (z * z - 1.0) * pdf
        ez = torch.exp(z)
        fin = torch.isfinite(ez) & torch.isfinite(ez * ez)
        zero = torch.zeros_like(z)
        if self.dist == "Extreme":
            pdf = torch.where(torch.isfinite(ez), ez * torch.exp(-ez), zero)
            cdf = 1.0 - torch.exp(-ez)
            d1 = torch.where(torch.isfinite(ez), (1.0 - ez) * pdf, zero)
            d2 = torch.where(fin, (ez * ez - 3.0 * ez + 1.0) * pdf, zero)
            return pdf, cdf, d1, d2
        pdf = torch.where(fin, ez / (1.0 + ez) ** 2, zero)
        cdf = torch.where(torch.isfinite(ez), ez / (1.0 + ez), torch.ones_like(z))
        d1 = torch.where(torch.isfinite(ez), pdf * (1.0 - ez) / (1.0 + ez), zero)
        d2 = torch.where(fin, pdf * (ez * ez - 4.0 * ez + 1.0) / (1.0 + ez) ** 2, zero)
        return pdf, cdf, d1, d2

    def _limits(self, order):
        """(min, max) per censoring kind [uncensored / interval, right, left] for a vanishing denominator."""
        s = self.scale
        if order == 1:
            return {"Normal": ((-15.0, 15.0), (-15.0, 0.0), (0.0, 15.0)),
                    "Extreme": ((-15.0, 1.0 / s), (-15.0, 0.0), (0.0, 1.0 / s)),
                    "Logistic": ((-1.0 / s, 1.0 / s), (-1.0 / s, 0.0), (0.0, 1.0 / s))}[self.dist]
        m = 1e-16
        return {"Normal": ((1.0 / s ** 2, 1.0 / s ** 2), (1.0 / s ** 2, m), (m, 1.0 / s ** 2)),
                "Extreme": ((15.0, m), (15.0, m), (m, m)),
                "Logistic": ((m, m), (m, m), (m, m))}[self.dist]

    def der_hess(self, approx, target, weight, ctx=None):
        a = approx[0].double()
        lo, up = target[0].double(), target[1].double()
        s = self.scale
        unc = lo == up
        right = (up == -1) & ~unc
        left = (lo == -1) & ~unc
        zl = (torch.log(lo.clamp_min(1e-300)) - a) / s
        zu = (torch.log(up.clamp_min(1e-300)) - a) / s
        pl, cl, dl, d2l = self._pdf_cdf(zl)
        pu, cu, du, _ = self._pdf_cdf(zu)
        zero, one = torch.zeros_like(a), torch.ones_like(a)
        pu, cu, du = torch.where(right, zero, pu), torch.where(right, one, cu), torch.where(right, zero, du)
        pl_i, cl_i, dl_i = torch.where(left, zero, pl), torch.where(left, zero, cl), torch.where(left, zero, dl)
        n1 = torch.where(unc, dl, pu - pl_i)
        q1 = torch.where(unc, s * pl, s * (cu - cl_i))
        n2 = torch.where(unc, -(pl * d2l - dl * dl), -(cu - cl_i) * (du - dl_i) + (pu - pl_i) ** 2)
        q2 = torch.where(unc, (s * pl) ** 2, (s * (cu - cl_i)) ** 2)
        sign = torch.where(unc, zl > 0, (torch.where(left, zero, zl) > 0) | (torch.where(right, zero, zu) > 0))
        kind = torch.where(right, 1, torch.where(left, 2, 0))

        def guarded(num, den, order):
            r = num / den
            lim = self._limits(order)
            mn = torch.tensor([x[0] for x in lim], dtype=a.dtype, device=a.device)[kind]
            mx = torch.tensor([x[1] for x in lim], dtype=a.dtype, device=a.device)[kind]
            bad = (den < 1e-12) & ~torch.isfinite(r)
            return torch.where(bad, torch.where(sign, mn, mx), r)

        d1 = -guarded(n1, q1, 1).clamp(-15.0, 15.0)
        h = guarded(n2, q2, 2).clamp(1e-16, 15.0)
        return d1.float().unsqueeze(0), h.float().unsqueeze(0)

    def value(self, approx, target, weight, ctx=None):
        """Negative log-likelihood per document."""
        a = approx[0].double()
        lo, up = target[0].double(), target[1].double()
        s = self.scale
        unc = lo == up
        zl = (torch.log(lo.clamp_min(1e-300)) - a) / s
        zu = (torch.log(up.clamp_min(1e-300)) - a) / s
        pl, cl, _, _ = self._pdf_cdf(zl)
        _, cu, _, _ = self._pdf_cdf(zu)
        cu = torch.where(up == -1, torch.ones_like(a), cu)
        cl = torch.where(lo == -1, torch.zeros_like(a), cl)
        lik = torch.where(unc, pl / (s * lo.clamp_min(1e-300)), cu - cl).clamp_min(1e-12)
        v = -torch.log(lik).float()
        return _wsum(v, weight) / max(_wtot(a.numel(), weight), 1e-300)


class MultiQuantile(Objective):
    """One approx dimension per level in ``alpha=a1,a2,...``: the pinball loss of every level
    (catboost/private/libs/algo_helpers/error_functions.cpp TMultiQuantileError::CalcDersMulti)."""
    name = "MultiQuantile"
    is_pointwise = False

    def __init__(self, params=None):
        super().__init__(params)
        al = self.params.get("alpha", 0.5)
        self.alphas = [float(x) for x in str(al).split(",")] if not isinstance(al, (int, float)) else [float(al)]
        self.delta = float(self.params.get("delta", 1e-6))
        self.dims = len(self.alphas)

    def der_hess(self, approx, target, weight, ctx=None):
        al = torch.tensor(self.alphas, dtype=approx.dtype, device=approx.device).unsqueeze(1)
        r = target.unsqueeze(0) - approx
        d = torch.where(r > 0, al.expand_as(r), (al - 1.0).expand_as(r))
        d = torch.where(r.abs() < self.delta, torch.zeros_like(d), d)
        h = torch.ones_like(d)
        if weight is not None:
            d, h = d * weight, h * weight
        return d, h

    def value(self, approx, target, weight, ctx=None):
        al = torch.tensor(self.alphas, dtype=approx.dtype, device=approx.device).unsqueeze(1)
        r = target.unsqueeze(0) - approx
        v = torch.where(r >= 0, al * r, (al - 1.0) * r).sum(0) / self.dims
        return _wsum(v, weight) / max(_wtot(target.numel(), weight), 1e-300)

    def start_constant(self, target, weight):
        return np.array([_weighted_quantile(target, weight, a) for a in self.alphas])


class Combination(Objective):
    """Weighted sum of one-dimensional losses, ``Combination:loss0=Logloss;weight0=1;loss1=QueryRMSE;weight1=0.5``:
    derivatives and second derivatives are the weighted sums of the parts'
    (catboost/cuda/targets/combination_targets_impl.h, catboost/private/libs/options/loss_description.h:176-193);
    parts with weight 0 are left out, the others need a positive weight."""
    name = "Combination"
    is_pointwise = False

    def __init__(self, params=None):
        super().__init__(params)
        count = len(self.params) // 2
        if count < 2:
            raise CatBoostError("Combination loss must have two or more parameters")
        self.parts = []
        for i in range(count):
            lk, wk = f"loss{i}", f"weight{i}"
            if lk not in self.params or wk not in self.params:
                raise CatBoostError(f"Mandatory parameter {lk} or {wk} is missing")
            try:
                w = float(self.params[wk])
            except (TypeError, ValueError):
                raise CatBoostError(f"Value of {wk} must be floating point number, not {self.params[wk]}")
            if w == 0.0:
                continue
            if w < 0.0:
                raise CatBoostError(f"Value of {wk} must be positive, not {w}")
            from ..params import parse_loss
            nm, sub = parse_loss(str(self.params[lk]))
            if nm == "Combination":
                raise CatBoostError("Combination losses do not nest")
            part = make_objective(nm, sub)
            if part.dims != 1:
                raise CatBoostError(f"Combination takes one-dimensional losses; {nm} is not one")
            self.parts.append((part, w))
        if not self.parts:
            raise CatBoostError("Combination loss must have one or more non-zero weights")
        self.needs_groups = any(p.needs_groups for p, _ in self.parts)
        self.needs_pairs = any(p.needs_pairs for p, _ in self.parts)
        self.is_classification = self.parts[0][0].is_classification
        self.stochastic = any(p.stochastic for p, _ in self.parts)

    def der_hess(self, approx, target, weight, ctx=None):
        der = hess = None
        for part, w in self.parts:
            d, h = part.der_hess(approx, target, weight, ctx)
            der = d * w if der is None else der + d * w
            hess = h * w if hess is None else hess + h * w
        return der, hess

    def value(self, approx, target, weight, ctx=None):
        return float(sum(w * part.value(approx, target, weight, ctx) for part, w in self.parts))

    def start_constant(self, target, weight):
        return self.parts[0][0].start_constant(target, weight) if len(self.parts) == 1 else np.zeros(1)


class UserObjective(Objective):
    """Python custom objective with ``calc_ders_range(approxes, targets, weights)`` returning (der, der2) pairs in
    the reference's sign convention (der2 <= 0), see catboost/python-package/catboost/_catboost.pyx trampolines."""
    name = "PythonUserDefinedPerObject"
    is_pointwise = False

    def __init__(self, obj):
        super().__init__({})
        self.obj = obj

    def der_hess(self, approx, target, weight, ctx=None):
        a = approx[0].detach().cpu().numpy().astype(np.float64)
        t = target.detach().cpu().numpy().astype(np.float64)
        w = None if weight is None else weight.detach().cpu().numpy().astype(np.float64)
        res = self.obj.calc_ders_range(a, t, w)
        d = np.array([r[0] for r in res], dtype=np.float32)
        h = -np.array([r[1] for r in res], dtype=np.float32)
        dev = approx.device
        return torch.from_numpy(d).to(dev).unsqueeze(0), torch.from_numpy(h).to(dev).clamp_min(1e-16).unsqueeze(0)

    def value(self, approx, target, weight, ctx=None):
        return float("nan")


class UserMultiObjective(Objective):
    """Python custom objective with ``calc_ders_multi(approxes, target, weight)`` per object, returning the first
    derivatives [dims] and the matrix of second derivatives [dims][dims] in the reference's sign convention
    (catboost/python-package/catboost/_catboost.pyx trampolines); the diagonal of the matrix is used.  The target of an
    object is its row of target columns (multi-target labels) or its class index."""
    name = "PythonUserDefinedMultiTarget"
    is_pointwise = False

    def __init__(self, obj, dims: int, target_is_vector: bool):
        super().__init__({})
        self.obj, self.dims, self.target_is_vector = obj, int(dims), bool(target_is_vector)

    def der_hess(self, approx, target, weight, ctx=None):
        A = approx.detach().t().cpu().numpy().astype(np.float64)                     # [n, dims]
        T = target.detach().cpu().numpy().astype(np.float64)
        T = T.T if self.target_is_vector else T
        w = None if weight is None else weight.detach().cpu().numpy().astype(np.float64)
        n = A.shape[0]
        d = np.empty((n, self.dims), dtype=np.float32)
        h = np.empty((n, self.dims), dtype=np.float32)
        for i in range(n):
            di, hi = self.obj.calc_ders_multi(A[i], T[i], 1.0 if w is None else float(w[i]))
            d[i] = np.asarray(di, dtype=np.float64)
            h[i] = -np.diagonal(np.asarray(hi, dtype=np.float64).reshape(self.dims, self.dims))
        dev = approx.device
        return torch.from_numpy(d.T.copy()).to(dev), torch.from_numpy(h.T.copy()).to(dev).clamp_min(1e-16)

    def value(self, approx, target, weight, ctx=None):
        return float("nan")


def _weighted_quantile(values, weight, alpha):
    v = np.asarray(values, dtype=np.float64)
    order = np.argsort(v, kind="stable")
    v = v[order]
    w = np.ones_like(v) if weight is None else np.asarray(weight, dtype=np.float64)[order]
    cw = np.cumsum(w)
    k = int(np.searchsorted(cw, alpha * cw[-1], side="left"))
    return float(v[min(k, len(v) - 1)])


_POINTWISE = {c.name: c for c in (RMSE, Logloss, CrossEntropy, Poisson, MAE, Quantile, LogLinQuantile, MAPE, Huber,
                                  Lq, Expectile, Tweedie, LogCosh, Focal)}


def make_objective(loss, params: dict, n_classes: Optional[int] = None, n_targets: int = 1) -> Objective:
    if not isinstance(loss, str):
        if hasattr(loss, "calc_ders_multi"):
            vector = n_targets > 1
            return UserMultiObjective(loss, n_targets if vector else int(n_classes or 2), vector)
        return UserObjective(loss)
    if loss in _POINTWISE:
        return _POINTWISE[loss](params)
    if loss == "MultiClass":
        return MultiClass(params, n_classes or 2)
    if loss == "MultiClassOneVsAll":
        return MultiClassOneVsAll(params, n_classes or 2)
    if loss == "MultiRMSE":
        return MultiRMSE(params, n_targets)
    if loss == "MultiLogloss":
        return MultiLogloss(params, n_targets)
    if loss == "MultiCrossEntropy":
        return MultiCrossEntropy(params, n_targets)
    if loss == "RMSEWithUncertainty":
        return RMSEWithUncertainty(params)
    if loss == "Combination":
        return Combination(params)
    if loss == "Cox":
        return Cox(params)
    if loss == "SurvivalAft":
        return SurvivalAft(params)
    if loss == "MultiQuantile":
        return MultiQuantile(params)
    from .ranking import make_ranking_objective
    obj = make_ranking_objective(loss, params)
    if obj is None:
        raise CatBoostError(f"loss function {loss!r} is not implemented")
    return obj
