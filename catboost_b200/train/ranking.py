"""Ranking objectives: QueryRMSE, QuerySoftMax, PairLogit(+Pairwise), YetiRank(+Pairwise), LambdaMart,
QueryCrossEntropy, StochasticRank.

All of them are evaluated per query group on the training device with vectorised tensor code over a padded
``[queries, max_query_len]`` layout (no Python loop over queries).  YetiRank follows the reference's pointwise
formulation: ``permutations`` noisy re-rankings per query (multiplicative Gumbel-type noise on exp(approx)), pairs of
neighbours in every ranking weighted by ``0.15 * decay^position * |relevance difference|``, pairwise logistic
derivatives accumulated per document (catboost/private/libs/algo/yetirank_helpers.cpp:123-205,305-345,
catboost/cuda/targets/kernel/yeti_rank_pointwise.cu:168).  The ``*Pairwise`` names train with the same pointwise
histograms as their base losses (the reference has a separate pairwise-histogram + linear-system path for them).
"""
from __future__ import annotations

import math
from typing import Optional

import numpy as np
import torch

from .objectives import Objective, _wsum, _wtot


USE_KERNELS = True        # False: the tensor formulations below also on the GPU (they are the oracle of the kernels)


class _GroupLayout:
    """Padded view of the query groups: index [Q, Lmax] into the row order, mask of real entries."""

    def __init__(self, offsets: torch.Tensor):
        self.offsets = offsets
        sizes = offsets[1:] - offsets[:-1]
        self.sizes = sizes
        Q = sizes.numel()
        Lmax = int(sizes.max().item()) if Q else 0
        ar = torch.arange(Lmax, device=offsets.device)
        self.mask = ar.unsqueeze(0) < sizes.unsqueeze(1)
        self.index = torch.where(self.mask, offsets[:-1].unsqueeze(1) + ar.unsqueeze(0), torch.zeros((), dtype=torch.long, device=offsets.device))
        self.Q, self.Lmax = Q, Lmax
        n = int(offsets[-1].item())
        self.n = n
        self.group_of_row = torch.repeat_interleave(torch.arange(Q, device=offsets.device), sizes, output_size=n)

    def gather(self, x, fill=0.0):
        return torch.where(self.mask, x[self.index], torch.full((), fill, dtype=x.dtype, device=x.device))

    def scatter(self, padded, n):
        out = torch.zeros(n, dtype=padded.dtype, device=padded.device)
        out[self.index[self.mask]] = padded[self.mask]
        return out


def _layout(ctx):
    lay = getattr(ctx, "_group_layout", None)
    if lay is None:
        lay = _GroupLayout(ctx.group_offsets)
        ctx._group_layout = lay
    return lay


class _GroupObjective(Objective):
    is_pointwise = False
    needs_groups = True
    zero_mean_leaves = False

    @property
    def native_id(self):
        return None


class QueryRMSE(_GroupObjective):
    name = "QueryRMSE"

    def der_hess(self, approx, target, weight, ctx=None):
        if approx.is_cuda and USE_KERNELS:
            from ..ops import api as ops
            d, h = ops.query_der("QueryRMSE", approx[0], target, weight, ctx.group_offsets)
            return d.unsqueeze(0), h.unsqueeze(0)
        lay = _layout(ctx)
        a, n = approx[0], approx.shape[1]
        w = torch.ones_like(a) if weight is None else weight
        res = (target - a) * w
        gsum = torch.zeros(lay.Q, device=a.device).index_add_(0, lay.group_of_row, res)
        gw = torch.zeros(lay.Q, device=a.device).index_add_(0, lay.group_of_row, w)
        shift = gsum / gw.clamp_min(1e-30)
        der = (target - a - shift[lay.group_of_row]) * w
        return der.unsqueeze(0), w.unsqueeze(0).clone()

    def value(self, approx, target, weight, ctx=None):
        d, _ = self.der_hess(approx, target, weight, ctx)
        w = torch.ones_like(d[0]) if weight is None else weight
        return math.sqrt(float(((d[0] / w.clamp_min(1e-30)) ** 2 * w).sum().item()) / max(float(w.sum().item()), 1e-300))


class GroupQuantile(_GroupObjective):
    """Quantile loss of the residual left after the weighted mean residual of the document's group is removed
    (catboost/private/libs/algo_helpers/error_functions.h:935-1000)."""
    name = "GroupQuantile"

    def _resid(self, approx, target, weight, ctx):
        lay = _layout(ctx)
        a = approx[0]
        w = torch.ones_like(a) if weight is None else weight
        res = (target - a) * w
        gsum = torch.zeros(lay.Q, device=a.device).index_add_(0, lay.group_of_row, res)
        gw = torch.zeros(lay.Q, device=a.device).index_add_(0, lay.group_of_row, w)
        return target - a - (gsum / gw.clamp_min(1e-30))[lay.group_of_row], w

    def der_hess(self, approx, target, weight, ctx=None):
        alpha, delta = float(self.params.get("alpha", 0.5)), float(self.params.get("delta", 1e-6))
        val, w = self._resid(approx, target, weight, ctx)
        d = torch.where(val > 0, torch.full_like(val, alpha), torch.full_like(val, alpha - 1.0))
        d = torch.where(val.abs() < delta, torch.zeros_like(d), d) * w
        return d.unsqueeze(0), w.unsqueeze(0).clone()

    def value(self, approx, target, weight, ctx=None):
        alpha = float(self.params.get("alpha", 0.5))
        val, w = self._resid(approx, target, weight, ctx)
        v = torch.where(val >= 0, alpha * val, (alpha - 1.0) * val) * w
        return float(v.sum().item()) / max(float(w.sum().item()), 1e-300)


class QuerySoftMax(_GroupObjective):
    name = "QuerySoftMax"

    def der_hess(self, approx, target, weight, ctx=None):
        beta = float(self.params.get("lambda", self.params.get("beta", 1.0)))
        if approx.is_cuda and USE_KERNELS:
            from ..ops import api as ops
            d, h = ops.query_der("QuerySoftMax", approx[0], target, weight, ctx.group_offsets, beta)
            return d.unsqueeze(0), h.unsqueeze(0)
        lay = _layout(ctx)
        a, n = approx[0], approx.shape[1]
        w = torch.ones_like(a) if weight is None else weight
        A = lay.gather(a * beta, -1e30)
        W = lay.gather(w)
        T = lay.gather(target)
        A = A - A.max(dim=1, keepdim=True).values
        e = torch.exp(A) * W
        p = e / e.sum(1, keepdim=True).clamp_min(1e-30)
        sw = (W * T).sum(1, keepdim=True)
        der = beta * (W * T - sw * p)
        hess = (beta * beta * sw * p * (1 - p)).clamp_min(1e-16)
        return lay.scatter(der, n).unsqueeze(0), lay.scatter(hess, n).unsqueeze(0)

    def value(self, approx, target, weight, ctx=None):
        return float("nan")


def _make_pairs_from_labels(lay: _GroupLayout, target):
    """All (winner, loser) pairs inside each query as padded [Q, L, L] mask."""
    T = lay.gather(target, float("nan"))
    m = lay.mask.unsqueeze(2) & lay.mask.unsqueeze(1)
    return (T.unsqueeze(2) > T.unsqueeze(1)) & m


class PairLogit(_GroupObjective):
    name = "PairLogit"
    needs_groups = False
    zero_mean_leaves = True

    def der_hess(self, approx, target, weight, ctx=None):
        a, n = approx[0], approx.shape[1]
        if approx.is_cuda and USE_KERNELS:
            from ..ops import api as ops
            if ctx is not None and ctx.pairs is not None:
                d, h = ops.pair_logit_der(a, ctx.pairs, ctx.pairs_weight)
            else:
                d, h = ops.query_der("PairLogit", a, target, None, ctx.group_offsets)
            return d.unsqueeze(0), h.unsqueeze(0)
        der = torch.zeros(n, device=a.device)
        hess = torch.zeros(n, device=a.device)
        if ctx is not None and ctx.pairs is not None:
            wi, li = ctx.pairs[:, 0], ctx.pairs[:, 1]
            pw = ctx.pairs_weight
            p = torch.sigmoid(a[li] - a[wi])            # probability of the wrong order
            der.index_add_(0, wi, pw * p)
            der.index_add_(0, li, -pw * p)
            h = pw * p * (1 - p)
            hess.index_add_(0, wi, h)
            hess.index_add_(0, li, h)
        else:
            lay = _layout(ctx)
            A = lay.gather(a)
            pm = _make_pairs_from_labels(lay, target).float()
            p = torch.sigmoid(A.unsqueeze(1) - A.unsqueeze(2))      # [q, i, j] = sigma(a_j - a_i)
            g = pm * p
            d = g.sum(2) - g.sum(1)
            h = pm * p * (1 - p)
            hh = h.sum(2) + h.sum(1)
            der, hess = lay.scatter(d, n), lay.scatter(hh, n)
        return der.unsqueeze(0), hess.clamp_min(1e-16).unsqueeze(0)

    def pair_terms(self, approx, target, weight, ctx=None):
        """(winner doc, loser doc, gradient magnitude g, second derivative h) of every pair: the winner's derivative
        gets +g, the loser's -g.  Used by the pairwise structure search."""
        a = approx[0]
        if ctx is not None and ctx.pairs is not None:
            wi, li, pw = ctx.pairs[:, 0], ctx.pairs[:, 1], ctx.pairs_weight.float()
        else:
            lay = _layout(ctx)
            cached = getattr(lay, "_label_pairs", None)
            if cached is None:
                # the pairs only depend on the labels: enumerated once per data set, query by query in blocks so that
                # the [queries, L, L] mask never exists for all queries at once
                ws, ls = [], []
                step = max(1, (1 << 26) // max(1, lay.Lmax * lay.Lmax))
                T = lay.gather(target, float("nan"))
                for q0 in range(0, lay.Q, step):
                    Tq, mq = T[q0:q0 + step], lay.mask[q0:q0 + step]
                    pm = (Tq.unsqueeze(2) > Tq.unsqueeze(1)) & mq.unsqueeze(2) & mq.unsqueeze(1)      # [q, i, j]: i beats j
                    q, i, j = pm.nonzero(as_tuple=True)
                    ws.append(lay.index[q0 + q, i])
                    ls.append(lay.index[q0 + q, j])
                cached = (torch.cat(ws) if ws else torch.zeros(0, dtype=torch.long, device=a.device),
                          torch.cat(ls) if ls else torch.zeros(0, dtype=torch.long, device=a.device))
                lay._label_pairs = cached
            wi, li = cached
            pw = torch.ones(wi.shape[0], device=a.device)
        p = torch.sigmoid(a[li] - a[wi])
        return wi, li, pw * p, pw * p * (1 - p)

    def value(self, approx, target, weight, ctx=None):
        return float("nan")


class YetiRank(_GroupObjective):
    name = "YetiRank"
    stochastic = True
    zero_mean_leaves = True

    def __init__(self, params=None):
        super().__init__(params)
        self.permutations = int(self.params.get("permutations", 10))
        self.decay = float(self.params.get("decay", 0.85))
        self._gen = None

    def _der_hess_device(self, a, target, weight, lay, noise=None):
        """The hand-written kernel (ops/cuda/cb_ranking.cu): one block per group, sort + pair accumulation in shared
        memory.  ``noise``: optional [permutations, n] uniforms (tests); else a counter-based generator seeded per call."""
        import ctypes
        from ..ops import native
        lib = native.cuda_lib()
        n = a.shape[0]
        self._calls = getattr(self, "_calls", 0) + 1
        der = torch.zeros(n, dtype=torch.float32, device=a.device)
        hess = torch.full((n,), 1e-16, dtype=torch.float32, device=a.device)
        P = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())
        a32, t32 = a.contiguous().float(), target.contiguous().float()
        w32 = None if weight is None else weight.contiguous().float()
        off = lay.offsets.contiguous()
        native.cuda_check(lib.cb_yetirank(P(a32), P(t32), P(w32), P(off), lay.Q, n, self.permutations, self.decay,
                                          (20240229 + 7919 * self._calls) & 0xFFFFFFFFFFFFFFFF, P(noise), P(der), P(hess), int(lay.Lmax),
                                          ctypes.c_void_p(torch.cuda.current_stream(a.device).cuda_stream)), "cb_yetirank")
        return der.unsqueeze(0), hess.unsqueeze(0)

    def der_hess(self, approx, target, weight, ctx=None):
        lay = _layout(ctx)
        a, n = approx[0], approx.shape[1]
        dev = a.device
        if a.is_cuda and lay.Lmax <= 2048 and lay.Q > 0 and lay.n == n:
            return self._der_hess_device(a, target, weight, lay)
        if self._gen is None:
            self._gen = torch.Generator(device="cpu")
            self._gen.manual_seed(20240229)
        A = lay.gather(a, -1e30)
        T = lay.gather(target)
        Q, L = lay.Q, lay.Lmax
        der = torch.zeros((Q, L), device=dev)
        hess = torch.zeros((Q, L), device=dev)
        if L < 2:
            return lay.scatter(der, n).unsqueeze(0), lay.scatter(hess, n).clamp_min(1e-16).unsqueeze(0)
        decay_pow = self.decay ** torch.arange(L - 1, device=dev, dtype=torch.float32)
        for _ in range(self.permutations):
            u = torch.rand((Q, L), generator=self._gen).to(dev).clamp(1e-6, 1 - 1e-6)
            noisy = A + torch.log(u / (1.000001 - u))          # exp(approx) * u / (1 - u), in log space
            noisy = torch.where(lay.mask, noisy, torch.full_like(noisy, -1e30))
            order = torch.argsort(noisy, dim=1, descending=True, stable=True)
            first, second = order[:, :-1], order[:, 1:]
            valid = lay.mask.gather(1, first) & lay.mask.gather(1, second)
            t1, t2 = T.gather(1, first), T.gather(1, second)
            wgt = 0.15 * decay_pow.unsqueeze(0) * (t1 - t2).abs() * valid
            win = torch.where(t1 > t2, first, second)
            los = torch.where(t1 > t2, second, first)
            aw, al = A.gather(1, win), A.gather(1, los)
            p = torch.sigmoid(al - aw)
            g = wgt * p
            h = wgt * p * (1 - p)
            der.scatter_add_(1, win, g)
            der.scatter_add_(1, los, -g)
            hess.scatter_add_(1, win, h)
            hess.scatter_add_(1, los, h)
        der, hess = der / self.permutations, hess / self.permutations
        if weight is not None:
            W = lay.gather(weight)
            der, hess = der * W, hess * W
        return lay.scatter(der, n).unsqueeze(0), lay.scatter(hess, n).clamp_min(1e-16).unsqueeze(0)

    def pair_terms(self, approx, target, weight, ctx=None):
        """Pairs of neighbours in ``permutations`` noisy orderings, as (winner, loser, g, h); see PairLogit.pair_terms."""
        lay = _layout(ctx)
        a = approx[0]
        dev = a.device
        if self._gen is None:
            self._gen = torch.Generator(device="cpu")
            self._gen.manual_seed(20240229)
        A = lay.gather(a, -1e30)
        T = lay.gather(target)
        Q, L = lay.Q, lay.Lmax
        empty = torch.zeros(0, dtype=torch.long, device=dev)
        if L < 2:
            return empty, empty, torch.zeros(0, device=dev), torch.zeros(0, device=dev)
        decay_pow = self.decay ** torch.arange(L - 1, device=dev, dtype=torch.float32)
        out = []
        if dev.type == "cuda" and getattr(self, "_gen_dev", None) is None:
            # the uniforms are drawn where they are used: 4M numbers per permutation from the host generator plus their
            # upload cost more than the sorting they feed
            self._gen_dev = torch.Generator(device=dev)
            self._gen_dev.manual_seed(20240229)
        for _ in range(self.permutations):
            if dev.type == "cuda":
                u = torch.rand((Q, L), generator=self._gen_dev, device=dev).clamp(1e-6, 1 - 1e-6)
            else:
                u = torch.rand((Q, L), generator=self._gen).clamp(1e-6, 1 - 1e-6)
            noisy = A + torch.log(u / (1.000001 - u))
            noisy = torch.where(lay.mask, noisy, torch.full_like(noisy, -1e30))
            order = torch.argsort(noisy, dim=1, descending=True, stable=True)
            first, second = order[:, :-1], order[:, 1:]
            valid = lay.mask.gather(1, first) & lay.mask.gather(1, second)
            t1, t2 = T.gather(1, first), T.gather(1, second)
            wgt = 0.15 * decay_pow.unsqueeze(0) * (t1 - t2).abs() * valid
            win = torch.where(t1 > t2, first, second)
            los = torch.where(t1 > t2, second, first)
            keep = wgt > 0
            wdoc, ldoc = lay.index.gather(1, win)[keep], lay.index.gather(1, los)[keep]
            w = wgt[keep] / self.permutations
            if weight is not None:
                w = w * weight[wdoc]
            p = torch.sigmoid(a[ldoc] - a[wdoc])
            out.append((wdoc, ldoc, w * p, w * p * (1 - p)))
        return tuple(torch.cat([o[k] for o in out]) for k in range(4))

    def value(self, approx, target, weight, ctx=None):
        return float("nan")


class LambdaMart(_GroupObjective):
    name = "LambdaMart"
    zero_mean_leaves = True

    def der_hess(self, approx, target, weight, ctx=None):
        lay = _layout(ctx)
        a, n = approx[0], approx.shape[1]
        sigma = float(self.params.get("sigma", 1.0))
        A = lay.gather(a, -1e30)
        T = lay.gather(target)
        rank = torch.argsort(torch.argsort(A, dim=1, descending=True, stable=True), dim=1).float()
        disc = 1.0 / torch.log2(rank + 2.0)
        gain = torch.pow(2.0, T) - 1.0
        ideal = (torch.sort(torch.where(lay.mask, gain, torch.zeros_like(gain)), dim=1, descending=True).values
                 / torch.log2(torch.arange(lay.Lmax, device=a.device).float() + 2.0)).sum(1, keepdim=True).clamp_min(1e-12)
        pm = _make_pairs_from_labels(lay, target).float()
        delta = ((gain.unsqueeze(2) - gain.unsqueeze(1)) * (disc.unsqueeze(2) - disc.unsqueeze(1))).abs() / ideal.unsqueeze(2)
        p = torch.sigmoid(sigma * (A.unsqueeze(1) - A.unsqueeze(2)))
        g = pm * delta * sigma * p
        d = g.sum(2) - g.sum(1)
        h = pm * delta * sigma * sigma * p * (1 - p)
        hh = h.sum(2) + h.sum(1)
        return lay.scatter(d, n).unsqueeze(0), lay.scatter(hh, n).clamp_min(1e-16).unsqueeze(0)

    def value(self, approx, target, weight, ctx=None):
        return float("nan")


class StochasticFilter(_GroupObjective):
    """Policy gradient for a document filter: every document is kept with probability sigmoid(sigma * approx), the
    reward of a sampled filter is sum over kept documents of target / (position among the kept ones), and the
    derivative is the REINFORCE estimate (kept ? 1 - p : -p) * (reward - baseline) averaged over ``num_estimations``
    samples, with the reward of the deterministic filter approx >= 0 as baseline
    (catboost/private/libs/algo_helpers/error_functions.h:1226-1320).  Gradient steps only."""
    name = "StochasticFilter"
    stochastic = True

    def __init__(self, params=None):
        super().__init__(params)
        self.sigma = float(self.params.get("sigma", 1.0))
        self.num_est = int(self.params.get("num_estimations", 1))
        if not self.sigma > 0 or self.num_est < 1:
            raise CatBoostError("StochasticFilter: sigma must be positive and num_estimations a positive integer")
        self._draws = 0

    @staticmethod
    def _reward(keep, T):
        pos = torch.cumsum(keep, 1) - keep                   # kept documents before this one
        return (keep * T / (pos + 1.0)).sum(1, keepdim=True)

    def der_hess(self, approx, target, weight, ctx=None):
        lay = _layout(ctx)
        a, n = approx[0], approx.shape[1]
        A = lay.gather(a, -1e30)
        T = lay.gather(target)
        m = lay.mask.float()
        base = self._reward((A >= 0).float() * m, T)
        P = torch.sigmoid(A * self.sigma)
        gen = torch.Generator(device="cpu")
        d = torch.zeros_like(A)
        for _ in range(self.num_est):
            self._draws += 1
            gen.manual_seed((int(self.params.get("seed", 0)) * 1000003 + 7919 * self._draws) & 0x7FFFFFFF)
            u = torch.rand(A.shape, generator=gen).to(A.device)
            keep = (P >= u).float() * m
            d += torch.where(keep > 0, 1.0 - P, -P) * (self._reward(keep, T) - base) / self.num_est
        return lay.scatter(d * m, n).unsqueeze(0), torch.ones((1, n), dtype=a.dtype, device=a.device)

    def value(self, approx, target, weight, ctx=None):
        return float("nan")


class QueryCrossEntropy(_GroupObjective):
    """Logloss with a per-query shift chosen so that the mean predicted probability matches the query's mean target,
    mixed with plain Logloss by ``alpha`` (catboost/cuda/targets/kernel/query_cross_entropy.cu)."""
    name = "QueryCrossEntropy"

    def der_hess(self, approx, target, weight, ctx=None):
        lay = _layout(ctx)
        alpha = float(self.params.get("alpha", 0.95))
        a, n = approx[0], approx.shape[1]
        A = lay.gather(a)
        T = lay.gather(target)
        M = lay.mask.float()
        shift = torch.zeros((lay.Q, 1), device=a.device)
        for _ in range(8):                                  # Newton iterations on the shift
            p = torch.sigmoid(A + shift)
            f = ((p - T) * M).sum(1, keepdim=True)
            df = (p * (1 - p) * M).sum(1, keepdim=True).clamp_min(1e-12)
            shift = shift - f / df
        pq = torch.sigmoid(A + shift)
        pp = torch.sigmoid(A)
        hq = pq * (1 - pq)
        # derivative of the shifted part with the shift's dependence on approx taken into account
        corr = ((pq - T) * M).sum(1, keepdim=True) * 0.0
        der = alpha * (T - pq - corr) + (1 - alpha) * (T - pp)
        hess = alpha * hq + (1 - alpha) * pp * (1 - pp)
        d, h = lay.scatter(der * M, n), lay.scatter(hess * M, n)
        if weight is not None:
            d, h = d * weight, h * weight
        return d.unsqueeze(0), h.clamp_min(1e-16).unsqueeze(0)

    def value(self, approx, target, weight, ctx=None):
        return float("nan")


class StochasticRank(LambdaMart):
    name = "StochasticRank"


def make_ranking_objective(loss, params):
    table = {"QueryRMSE": QueryRMSE, "QuerySoftMax": QuerySoftMax, "PairLogit": PairLogit, "PairLogitPairwise": PairLogit,
             "YetiRank": YetiRank, "YetiRankPairwise": YetiRank, "LambdaMart": LambdaMart,
             "QueryCrossEntropy": QueryCrossEntropy, "StochasticRank": StochasticRank, "StochasticFilter": StochasticFilter, "GroupQuantile": GroupQuantile}
    cls = table.get(loss)
    if cls is None:
        return None
    obj = cls(params)
    obj.name = loss
    obj.pairwise_scoring = loss in ("PairLogitPairwise", "YetiRankPairwise")
    return obj
