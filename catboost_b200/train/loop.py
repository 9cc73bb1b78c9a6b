"""The boosting iteration loop for both trainers (device-resident engine and general learner)."""
from __future__ import annotations

import math
import os
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import numpy as np
import torch

from ..data.pool import CatBoostError
from ..ops import api as ops
from .generic import GenericLearner, estimate_leaves
from .snapshot import SnapshotManager


@dataclass
class LoopResult:
    trees: list
    evals_result: Dict[str, Dict[str, List[float]]]
    best_iteration: Optional[int]
    best_score: Dict[str, Dict[str, float]]
    launches_per_iter: int = 0
    train_approx: Optional[np.ndarray] = None


class ObjectiveContext:
    """Per-dataset side information some objectives need (query offsets, pairs) on the training device."""

    def __init__(self, pool, device):
        self.group_offsets = None
        self.pairs = None
        self.pairs_weight = None
        self.device = device
        if pool.group_id is not None:
            self.group_offsets = torch.from_numpy(pool.group_offsets()).to(device)
        if pool.pairs is not None:
            self.pairs = torch.from_numpy(pool.pairs).to(device)
            self.pairs_weight = torch.from_numpy(pool.pairs_weight).to(device)
        self.subgroup_id = pool.subgroup_id


def _parse_monotone(spec, pool) -> dict:
    """monotone_constraints as {float-feature index: +1/-1}.  Accepts a list per feature, a dict by index or name, or
    the strings "(1,0,-1)" / "0:1,3:-1" / "name:1" (catboost/private/libs/options/monotone_constraints.cpp)."""
    per_col = {}
    if isinstance(spec, str):
        body = spec.strip().strip("()[]")
        items = [x.strip() for x in body.split(",") if x.strip()]
        if items and all(":" not in x for x in items):
            per_col = {i: int(float(x)) for i, x in enumerate(items)}
        else:
            for x in items:
                k, v = x.split(":")
                k = k.strip()
                per_col[int(k) if k.lstrip("-").isdigit() else pool.feature_names.index(k)] = int(float(v))
    elif isinstance(spec, dict):
        for k, v in spec.items():
            per_col[pool.feature_names.index(k) if isinstance(k, str) and not k.isdigit() else int(k)] = int(v)
    else:
        per_col = {i: int(v) for i, v in enumerate(spec)}
    out = {}
    for col, c in per_col.items():
        if c == 0:
            continue
        if c not in (-1, 1):
            raise CatBoostError("monotone constraints must be -1, 0 or 1")
        if col not in pool.float_feature_indices:
            raise CatBoostError("monotone constraints apply to numerical features only")
        out[pool.float_feature_indices.index(col)] = c
    return out


def _per_feature_values(spec, pool) -> dict:
    """{external feature index: value} from a list per feature, a dict by index or name, or the strings "(1,0,2)" /
    "0:1.5,3:2" / "name:1" (the forms feature_weights and the penalty options take,
    catboost/private/libs/options/feature_penalties_options.cpp)."""
    out = {}
    if spec is None:
        return out
    key = lambda k: pool.feature_names.index(k) if isinstance(k, str) and not k.strip().lstrip("-").isdigit() else int(k)
    if isinstance(spec, str):
        items = [x.strip() for x in spec.strip().strip("()[]").split(",") if x.strip()]
        if items and all(":" not in x for x in items):
            out = {i: float(x) for i, x in enumerate(items)}
        else:
            for x in items:
                k, v = x.split(":")
                out[key(k.strip())] = float(v)
    elif isinstance(spec, dict):
        out = {key(k): float(v) for k, v in spec.items()}
    else:
        out = {i: float(v) for i, v in enumerate(spec)}
    return {k: v for k, v in out.items() if v != 0.0}


def _flat_penalties(spec, pool, store) -> Optional[np.ndarray]:
    """Per-feature option values laid over the flat features of the store: a quantised float feature and a one-hot
    feature take the value of their source column; features computed from several columns (CTRs) take none."""
    vals = _per_feature_values(spec, pool)
    if not vals:
        return None
    if any(v < 0 for v in vals.values()):
        raise CatBoostError("feature penalties must be non-negative")
    out = np.zeros(store.F, dtype=np.float32)
    for i, f in enumerate(store.features):
        if f.kind == "float" and f.source >= 0:
            out[i] = vals.get(pool.float_feature_indices[f.source], 0.0)
        elif f.kind == "onehot":
            out[i] = vals.get(pool.cat_feature_indices[f.source], 0.0)
    return out


def _has_penalties(o) -> bool:
    return bool(o.first_feature_use_penalties) or bool(o.per_object_feature_penalties)


def _use_fast_engine(o, objective, store, dims) -> bool:
    # objectives without a device formula still use the fused level kernels: their derivatives are computed by the
    # objective's tensor code once per tree, which only allows a single leaf-estimation step
    native = objective.native_id is not None
    external = (not native) and dims == 1 and int(o.leaf_estimation_iterations) == 1
    if dims > 1:
        # MultiClass: K derivative columns through the same level kernels, K x K Newton leaves on the device.  The leaf
        # kernel keeps K + K (K + 1) / 2 + 1 cells per leaf in shared memory and has no step-length control.
        K, L = int(dims), 1 << int(o.depth)
        ok = (native and objective.name == "MultiClass" and 2 <= K <= 16 and L * (K + K * (K + 1) // 2 + 1) * 4 <= 96 * 1024
              and (int(o.leaf_estimation_iterations) == 1 or str(o.leaf_estimation_backtracking) == "No"))
        if not ok:
            return False
    return (store.bins.is_cuda and o.grow_policy == "SymmetricTree" and (native or external)
            and o.boosting_type == "Plain" and o.leaf_estimation_method in ("Newton", "Gradient")
            and float(o.rsm) >= 1.0 and int(o.min_data_in_leaf) <= 1
            and (o.bootstrap_type in ("No", "Bayesian", "Bernoulli", "Poisson") or (o.bootstrap_type == "MVS" and dims == 1))
            and not o.langevin and not o.monotone_constraints and not o.model_shrink_rate
            and str(o.sampling_unit or "Object") == "Object"
            and not _has_penalties(o) and str(o.sampling_frequency or "PerTree") == "PerTree"
            and getattr(objective, "target_columns", 1) == 1          # interval labels stay on the general learner
            and not getattr(objective, "pairwise_scoring", False)       # pairwise systems live in the general learner
            and str(o.random_score_type) != "Gumbel")


class _History:
    def __init__(self, metrics, n_eval, eval_names):
        self.metrics = metrics
        self.names = ["learn"] + eval_names
        self.data = {nm: {str(m): [] for m in metrics} for nm in self.names}
        self.iters: List[int] = []

    def add(self, set_name, metric, value):
        self.data[set_name][str(metric)].append(float(value))


def _eval_names(n):
    return ["validation"] if n == 1 else [f"validation_{k}" for k in range(n)]


def _host_metric(metric, approx_dims_n: torch.Tensor, y, w, pool, loss_dims):
    a = approx_dims_n.detach().t().double().cpu().numpy()
    kw = {}
    if pool is not None:
        if pool.group_id is not None:
            kw["group_offsets"] = pool.group_offsets()
        if pool.pairs is not None:
            kw["pairs"], kw["pairs_weight"] = pool.pairs, pool.pairs_weight
    return metric.eval(a, y, w, **kw)


def run_boosting(o, objective, store, eval_stores, y_train, w_train, base_train, eval_y, eval_w, base_evals,
                 train_pool, eval_pools, metrics, logger, od, ctx, prof, callbacks, plan, ctr_state) -> LoopResult:
    dev = store.bins.device
    dims = objective.dims
    n = store.n
    T = int(o.iterations)
    eval_names = _eval_names(len(eval_stores))
    hist = _History(metrics, len(eval_stores), eval_names)
    snap = SnapshotManager(o, ctx)
    callbacks = list(callbacks or [])
    if o.callback is not None:
        callbacks += list(o.callback) if isinstance(o.callback, (list, tuple)) else [o.callback]

    if _use_fast_engine(o, objective, store, dims):
        return _run_fast(o, objective, store, eval_stores, y_train, w_train, base_train, eval_y, eval_w, base_evals,
                         train_pool, eval_pools, metrics, logger, od, ctx, prof, callbacks, hist, eval_names, snap)

    # ------------------------------------------------------------------ general learner
    f32 = torch.float32
    approx = torch.zeros((dims, store.npad), dtype=f32, device=dev)
    approx[:, :n] = torch.from_numpy(np.ascontiguousarray(base_train)).to(dev, f32)
    multi_target = np.asarray(y_train).ndim == 2
    target = torch.from_numpy(np.ascontiguousarray(np.asarray(y_train).T if multi_target else y_train)).to(dev, f32)
    weight = None if w_train is None else torch.from_numpy(np.asarray(w_train, dtype=np.float32)).to(dev)
    wpad = None
    if weight is not None:
        wpad = torch.zeros(store.npad, dtype=f32, device=dev)
        wpad[:n] = weight
    octx = ObjectiveContext(train_pool, dev)
    eval_approx = [torch.from_numpy(np.ascontiguousarray(b)).to(dev, f32) for b in base_evals]
    learner = GenericLearner(store, o, dims, ctx, seed=int(o.random_seed))
    if str(o.sampling_unit or "Object") == "Group":
        if train_pool.group_id is None:
            raise CatBoostError("sampling_unit='Group' needs group_id")
        off = train_pool.group_offsets()
        learner.group_of_doc = torch.from_numpy(np.repeat(np.arange(len(off) - 1), np.diff(off))).to(dev)
    if _has_penalties(o):
        learner.set_penalties(_flat_penalties(o.first_feature_use_penalties, train_pool, store),
                              _flat_penalties(o.per_object_feature_penalties, train_pool, store),
                              float(o.penalties_coefficient if o.penalties_coefficient is not None else 1.0))
    monotone_flat = None
    if o.monotone_constraints:
        mono = _parse_monotone(o.monotone_constraints, train_pool)
        learner.set_monotone(mono)
        if learner.monotone is not None:
            if o.grow_policy != "SymmetricTree" or dims != 1:
                raise CatBoostError("monotone_constraints need symmetric trees and a one-dimensional model")
            monotone_flat = learner.monotone.cpu().numpy()
    plearner = None
    if getattr(objective, "pairwise_scoring", False) and o.grow_policy == "SymmetricTree":
        from .pairwise import PairwiseKernelLearner, PairwiseLearner
        if store.bins.is_cuda and int(o.depth) <= 6:
            # kernels: pair histograms, per-candidate systems, Cholesky and gain on the device; histograms summed over ranks
            plearner = PairwiseKernelLearner(store, o, seed=int(o.random_seed), ctx=ctx)
        elif not (ctx is not None and ctx.is_distributed):
            plearner = PairwiseLearner(store, o, seed=int(o.random_seed))
    ordered = None
    if o.boosting_type == "Ordered":
        ordered = OrderedState(o, n, train_pool, dev, approx[:, :n], ctx)
    trees = []
    start_iter = 0
    restored = snap.try_load(o)
    if restored is not None:
        trees, hist.data, hist.iters = restored["trees"], restored["hist"], restored["iters"]
        start_iter = len(trees)
        for t in trees:
            _apply_tree_to(store, t, approx, n, dims, dev)
            for es, ea in zip(eval_stores, eval_approx):
                _apply_tree_to(es, t, ea, es.n, dims, dev)
            if learner.has_penalties:
                # features of the restored trees count as used (for every document: the per-document paths of
                # non-symmetric trees are not stored)
                used = t["splits"][:, 0] if t["kind"] == "oblivious" else t["node_split"][:, 0]
                for f in used:
                    if f >= 0:
                        learner.used_feature[int(f)] = True
                        if int(f) in learner.used_by_doc:
                            learner.used_by_doc[int(f)].fill_(True)
        if ordered is not None:
            ordered.approx.copy_(approx[:, :n])      # ordered cursors are not stored; resume from the plain cursor
        learner.gen.manual_seed(int(o.random_seed) + 12345 + start_iter)
        if od is not None:
            for v in hist.data[eval_names[0]][str(metrics[0])]:
                od.add(v)
    best_it, best_val = None, None
    t_loop = time.time()
    stop = False
    shrink_rate = float(o.model_shrink_rate or 0.0)
    if shrink_rate > 0.0:
        approx0 = approx[:, :n].clone()
        eval_approx0 = [ea.clone() for ea in eval_approx]
    for it in range(start_iter, T):
        if shrink_rate > 0.0 and trees:
            # model shrinkage (catboost/private/libs/algo/train.cpp, model_shrink_rate): before every iteration the sum of
            # the trees built so far is multiplied by 1 - rate * learning_rate (Constant) or 1 - rate / iteration
            # (Decreasing); the starting value is left alone
            c = shrink_rate / float(it + 1) if str(o.model_shrink_mode or "Constant") == "Decreasing" \
                else shrink_rate * float(o.learning_rate)
            if not 0.0 <= c < 1.0:
                raise CatBoostError("model_shrink_rate * learning_rate must be in [0, 1)")
            f = 1.0 - c
            approx[:, :n] = approx0 + (approx[:, :n] - approx0) * f
            for ea, ea0 in zip(eval_approx, eval_approx0):
                ea.copy_(ea0 + (ea - ea0) * f)
            for tr_ in trees:
                tr_["values"] = tr_["values"] * f
        with prof.span("derivatives"):
            # ordered boosting: the tree structure is learned from derivatives at the ordered cursor, where the
            # value of a document only comes from documents that precede it in the permutation
            der, hess = objective.der_hess(ordered.approx if ordered is not None else approx[:, :n], target, weight, octx)
            der_p = torch.zeros((dims, store.npad), dtype=f32, device=dev)
            hess_p = torch.zeros((dims, store.npad), dtype=f32, device=dev)
            der_p[:, :n], hess_p[:, :n] = der, hess
            if o.langevin:
                coef = math.sqrt(2.0 / (float(o.learning_rate) * float(o.diffusion_temperature)))
                der_p[:, :n] += learner._randn((dims, n)) * coef
        if plearner is not None:
            # pairwise losses: the split score and the leaf values come from linear systems over all leaves
            with prof.span("structure"):
                wi_, li_, g_, h_ = objective.pair_terms(approx[:, :n], target, weight, octx)
                der1 = torch.zeros(n, dtype=f32, device=dev).index_add_(0, wi_, g_).index_add_(0, li_, -g_)
                tr = plearner.build_tree(wi_, li_, h_, der1, it)
            with prof.span("leaves"):
                vals, wts = plearner.leaf_values(tr.n_leaves, wi_, li_, h_, der1, float(o.learning_rate))
        else:
            with prof.span("structure"):
                tr = learner.build_tree(der_p, hess_p, wpad, it)
            with prof.span("leaves"):
                vals, wts = estimate_leaves(objective, approx, target, weight, tr.leaf, tr.n_leaves, n, o, ctx, octx)
        if monotone_flat is not None and tr.kind == "oblivious":
            from .generic import enforce_monotone_leaves
            vals = enforce_monotone_leaves(vals, wts, tr.splits, monotone_flat)
        tv = torch.from_numpy(vals).to(dev, f32)
        if ordered is not None:
            ordered.update(der, hess, weight, tr.leaf, tr.n_leaves, o)
        approx[:, :n] += tv[tr.leaf[:n].long() & 0xFFFF].t()
        tree = dict(kind=tr.kind, splits=tr.splits, node_split=tr.node_split, leaf_of_node=tr.leaf_of_node, values=vals,
                    weights=wts)
        trees.append(tree)
        with prof.span("eval_apply"):
            for es, ea in zip(eval_stores, eval_approx):
                _apply_tree_to(es, tree, ea, es.n, dims, dev)
        # metrics -----------------------------------------------------------------------------------------
        period = max(1, int(o.metric_period))
        if (it % period == 0) or it == T - 1 or od is not None:
            with prof.span("metrics"):
                hist.iters.append(it)
                for m in metrics:
                    hist.add("learn", m, _dist_metric(m, approx[:, :n], y_train, w_train, train_pool, ctx, objective))
                    for k, (ea, ep) in enumerate(zip(eval_approx, eval_pools)):
                        hist.add(eval_names[k], m, _dist_metric(m, ea, eval_y[k], eval_w[k], ep, ctx, objective))
            if eval_stores:
                v = hist.data[eval_names[0]][str(metrics[0])][-1]
                if best_val is None or (v > best_val if metrics[0].is_max_optimal else v < best_val):
                    best_val, best_it = v, it
                if od is not None and od.add(v):
                    stop = True
            logger.log_iteration(it, T, hist, time.time() - t_loop)
        for cb in callbacks:
            info = _CallbackInfo(it, hist.data)
            if cb.after_iteration(info) is False:
                stop = True
        snap.maybe_save(dict(trees=trees, hist=hist.data, iters=hist.iters), it)
        if stop:
            logger.info(f"Stopped by overfitting detector  ({od.wait} iterations wait)" if od is not None and od.stopped
                        else "Stopped by callback")
            break
    snap.finalize(dict(trees=trees, hist=hist.data, iters=hist.iters))
    return LoopResult(trees, hist.data, best_it, _best_scores(hist, metrics), 0,
                      approx[:, :n].t().double().cpu().numpy())


class OrderedState:
    """Ordered boosting (catboost/cuda/methods/dynamic_boosting.h:75-98,182-232, catboost/private/libs/algo/fold.cpp):
    documents are put in a random permutation and cut into blocks whose sizes grow geometrically
    (``fold_len_multiplier``, first block ``min_fold_size``).  The ordered cursor of a document in block b is only ever
    moved by leaf statistics of blocks < b, so the derivatives that drive the structure search are not fitted to the
    document's own target.  The exported model still gets its leaf values from all documents (plain cursor)."""

    def __init__(self, o, n, pool, dev, approx0, ctx=None):
        self.ctx = ctx if (ctx is not None and ctx.is_distributed) else None
        rank = self.ctx.rank if self.ctx is not None else 0
        rng = np.random.RandomState(int(o.random_seed) + 777 + 7919 * rank)
        n_total = n
        if self.ctx is not None:
            n_total = int(sum(self.ctx.all_gather_object(int(n))))
        bounds = [0]
        size = max(1, min(int(o.min_fold_size), n_total))
        mult = max(1.0001, float(o.fold_len_multiplier))
        while bounds[-1] < n_total:
            bounds.append(min(n_total, bounds[-1] + int(math.ceil(size))))
            size *= mult
        if self.ctx is None:
            if pool.group_id is not None:
                off = pool.group_offsets()
                perm_g = rng.permutation(len(off) - 1)
                order = np.concatenate([np.arange(off[k], off[k + 1]) for k in perm_g]) if len(perm_g) else np.zeros(0, np.int64)
            else:
                order = np.arange(n) if o.has_time else rng.permutation(n)
            block_of_pos = np.zeros(n, dtype=np.int64)
            for b in range(len(bounds) - 1):
                block_of_pos[bounds[b]:bounds[b + 1]] = b
            block = np.zeros(n, dtype=np.int64)
            block[order] = block_of_pos
        else:
            # several ranks: every document (every query) draws a position in the global permutation on its own; the
            # blocks are ranges of global positions, so a rank holds a random part of every block and the per-block leaf
            # statistics are summed over the ranks
            if pool.group_id is not None:
                off = pool.group_offsets()
                ug = rng.random_sample(len(off) - 1)
                u = np.repeat(ug, np.diff(off))
            else:
                u = rng.random_sample(n)
            pos = np.minimum((u * n_total).astype(np.int64), n_total - 1)
            block = np.searchsorted(np.asarray(bounds[1:], dtype=np.int64), pos, side="right")
        self.n_blocks = len(bounds) - 1
        self.block = torch.from_numpy(block).to(dev)
        self.approx = approx0.clone()

    def update(self, der, hess, weight, leaf, n_leaves, o):
        dims, n = der.shape
        idx = leaf[:n].long() & 0xFFFF
        key = self.block * n_leaves + idx
        B, L = self.n_blocks, n_leaves
        sd = torch.zeros((dims, B * L), dtype=torch.float64, device=der.device)
        sh = torch.zeros((dims, B * L), dtype=torch.float64, device=der.device)
        sd.index_add_(1, key, der.double())
        newton = o.leaf_estimation_method == "Newton"
        if newton:
            sh.index_add_(1, key, hess.double())
        else:
            w = torch.ones(n, dtype=torch.float64, device=der.device) if weight is None else weight[:n].double()
            sh.index_add_(1, key, w.unsqueeze(0).expand(dims, n).contiguous())
        if self.ctx is not None:
            self.ctx.all_reduce_sum_(sd)
            self.ctx.all_reduce_sum_(sh)
        sd = sd.view(dims, B, L).cumsum(1)
        sh = sh.view(dims, B, L).cumsum(1)
        val = sd / (sh + float(o.l2_leaf_reg))
        # statistics of blocks < b: shift by one block; the first block learns from itself (it has no history)
        prev = torch.cat([val[:, :1], val[:, :-1]], dim=1)
        inc = prev[:, self.block, idx] * float(o.learning_rate)
        self.approx += inc.float()


class _CallbackInfo:
    def __init__(self, iteration, metrics):
        self.iteration = iteration
        self.metrics = metrics


def _best_scores(hist, metrics):
    out = {}
    for nm, per in hist.data.items():
        out[nm] = {}
        for m in metrics:
            vals = per[str(m)]
            if vals:
                out[nm][str(m)] = max(vals) if m.is_max_optimal else min(vals)
    return out


_Y_CACHE = {}


_GROUP_CACHE = {}


def _device_ndcg(metric, approx, y, w, pool):
    """NDCG / DCG where the approximations live (catboost/cuda/targets/kernel/dcg.cu:17-347 does the same in three
    steps): one stable sort of the documents by (query, descending approximation) -- the hand-written radix sort of
    ops/cuda/cb_sort.cu on a 64-bit key, so ties keep the document order like the host metric --, the position of a
    document inside its query, and a per-query sum of gain / discount; the ideal order is the same with the labels as
    the sort key.  Parameters: top, type (Base / Exp), denominator (LogPosition / Position)."""
    p = dict(getattr(metric, "params", None) or {})
    name = getattr(metric, "name", None)
    if name in ("YetiRank", "YetiRankPairwise"):
        name = "PFound"                       # the value these objectives are logged with
        p = {k: v for k, v in p.items() if k in ("top", "decay")}
    allowed = {"top", "decay"} if name == "PFound" else {"top", "type", "denominator"}
    if set(p) - allowed or pool is None or pool.group_id is None:
        return None
    if not approx.is_cuda or approx.shape[0] != 1 or np.ndim(y) != 1:
        return None
    dev = approx.device
    n = len(y)
    key = (id(pool), str(dev))
    if key not in _GROUP_CACHE:
        if len(_GROUP_CACHE) > 8:
            _GROUP_CACHE.clear()
        off = torch.from_numpy(np.asarray(pool.group_offsets(), dtype=np.int64)).to(dev)
        sizes = off[1:] - off[:-1]
        gid = torch.repeat_interleave(torch.arange(sizes.numel(), device=dev), sizes, output_size=n)
        gw = torch.ones(sizes.numel(), dtype=torch.float64, device=dev) if w is None else \
            torch.from_numpy(np.ascontiguousarray(w, dtype=np.float64)).to(dev)[off[:-1].clamp(max=max(n - 1, 0))]
        _GROUP_CACHE[key] = (pool, off, gid, gw, torch.from_numpy(np.ascontiguousarray(y, dtype=np.float32)).to(dev))
    _, off, gid, gw, yt = _GROUP_CACHE[key]
    Q = off.numel() - 1
    if Q <= 0:
        return None
    top = int(p.get("top", -1))
    exp_num = str(p.get("type", "Base")) == "Exp"
    log_den = str(p.get("denominator", "LogPosition")) == "LogPosition"

    def dcg(values):
        # ascending order of (query, -value): float bits mapped to integers of the same order
        bits = (0.0 - values.float()).contiguous().view(torch.int32).long()          # 0.0 - x: never a negative zero
        ordered = torch.where(bits < 0, bits ^ 0x7FFFFFFF, bits) + (1 << 31)          # in [0, 2^32)
        _, order = ops.sort_pairs((gid << 32) | ordered)
        rank = torch.arange(n, device=dev) - off[gid[order]]
        rel = yt[order].double()
        gain = (torch.pow(2.0, rel) - 1.0) if exp_num else rel
        disc = torch.log2(rank.double() + 2.0) if log_den else (rank.double() + 1.0)
        term = gain / disc
        if top > 0:
            term = torch.where(rank < top, term, torch.zeros_like(term))
        return torch.zeros(Q, dtype=torch.float64, device=dev).index_add_(0, gid[order], term)

    if name == "PFound":
        # sum over the positions of a query of plook_k * r_k with plook_0 = 1, plook_{k+1} = plook_k (1 - r_k) decay: the
        # running product inside a query as an exclusive segmented sum of logarithms (magnitude), with the sign and a
        # "hit zero" flag carried by two more segmented sums
        decay = float(p.get("decay", 0.85))
        bits = (0.0 - approx[0][:n].float()).contiguous().view(torch.int32).long()
        ordered = torch.where(bits < 0, bits ^ 0x7FFFFFFF, bits) + (1 << 31)
        _, order = ops.sort_pairs((gid << 32) | ordered)
        g_sorted = gid[order]
        rank = torch.arange(n, device=dev) - off[g_sorted]
        rel = yt[order].double()
        fac = (1.0 - rel) * decay
        zero, neg = (fac == 0), (fac < 0)
        lg = torch.where(zero, torch.zeros_like(fac), torch.log(fac.abs().clamp_min(1e-300)))

        def excl_seg(v):
            c = torch.cumsum(v, 0)
            first = off[:-1].clamp(max=max(n - 1, 0))
            base = torch.where(off[:-1] < n, c[first] - v[first], torch.zeros_like(c[first]))
            return c - v - base[g_sorted]

        plook = torch.exp(excl_seg(lg))
        plook = torch.where(excl_seg(zero.double()) > 0, torch.zeros_like(plook), plook)
        plook = torch.where((excl_seg(neg.double()).round().long() & 1) == 1, -plook, plook)
        term = plook * rel
        if top > 0:
            term = torch.where(rank < top, term, torch.zeros_like(term))
        got = torch.zeros(Q, dtype=torch.float64, device=dev).index_add_(0, g_sorted, term)
        return float(((got * gw).sum() / gw.sum().clamp_min(1e-300)).item())
    got = dcg(approx[0][:n])
    if name == "NDCG":
        ideal = dcg(yt)
        got = torch.where(ideal > 0, got / ideal.clamp_min(1e-300), torch.ones_like(got))
    return float(((got * gw).sum() / gw.sum().clamp_min(1e-300)).item())


def _device_metric(metric, approx, y, w, pool=None):
    """The common additive metrics evaluated where the approximations live (a host round trip of a 1M x 5 cursor per
    iteration costs more than growing the tree).  Returns None for metrics without a device formula."""
    name = getattr(metric, "name", None)
    if name in ("NDCG", "DCG", "PFound", "YetiRank", "YetiRankPairwise"):
        return _device_ndcg(metric, approx, y, w, pool)
    if name in ("PairLogit", "PairLogitPairwise", "PairAccuracy"):
        # all pairs of a query whose labels differ, or the pool's explicit pairs (ops/cuda/cb_querywise.cu)
        if not approx.is_cuda or approx.shape[0] != 1 or getattr(metric, "params", None) or pool is None or np.ndim(y) != 1:
            return None
        dev = approx.device
        n = len(y)
        if pool.pairs is not None:
            pr = torch.from_numpy(np.ascontiguousarray(pool.pairs, dtype=np.int64)).to(dev)
            pw = None if pool.pairs_weight is None else torch.from_numpy(np.ascontiguousarray(pool.pairs_weight, dtype=np.float32)).to(dev)
            loss, acc = ops.pair_metric(approx[0][:n], None, None, pr, pw)
        elif pool.group_id is not None:
            off = torch.from_numpy(np.asarray(pool.group_offsets(), dtype=np.int64)).to(dev)
            yt = torch.from_numpy(np.ascontiguousarray(y, dtype=np.float32)).to(dev)
            loss, acc = ops.pair_metric(approx[0][:n], yt, off)
        else:
            return None
        return acc if name == "PairAccuracy" else loss
    if name not in ("Logloss", "RMSE", "MAE", "MultiClass", "Accuracy", "AUC", "Precision", "Recall", "F1", "R2") \
            or getattr(metric, "params", None):
        return None
    if not approx.is_cuda or isinstance(y, torch.Tensor) or np.ndim(y) != 1:
        return None
    dev = approx.device
    key = (id(y), str(dev))
    if key not in _Y_CACHE:
        if len(_Y_CACHE) > 8:
            _Y_CACHE.clear()
        _Y_CACHE[key] = (y, torch.from_numpy(np.ascontiguousarray(y, dtype=np.float32)).to(dev))   # keeps y alive
    yt = _Y_CACHE[key][1]
    wt = None if w is None else torch.from_numpy(np.ascontiguousarray(w, dtype=np.float32)).to(dev)
    a = approx.float()
    if name in ("AUC", "Precision", "Recall", "F1", "R2"):
        if a.shape[0] != 1:
            return None
        wd = torch.ones_like(yt, dtype=torch.float64) if wt is None else wt.double()
        if name == "R2":
            mean = (yt.double() * wd).sum() / wd.sum()
            ss_res = (((yt - a[0]).double() ** 2) * wd).sum()
            ss_tot = (((yt.double() - mean) ** 2) * wd).sum()
            return float((1.0 - ss_res / ss_tot.clamp_min(1e-300)).item())
        pos = yt > 0.5
        if name == "AUC":
            # weighted Mann-Whitney statistic with ties counted half (sort on the device, catboost/cuda/targets/auc.cpp)
            order = torch.argsort(a[0], stable=True)
            s_, p_, w_ = a[0][order], pos[order], wd[order]
            wpos, wneg = torch.where(p_, w_, torch.zeros_like(w_)), torch.where(p_, torch.zeros_like(w_), w_)
            _, inv, cnt = torch.unique_consecutive(s_, return_inverse=True, return_counts=True)
            gneg = torch.zeros(cnt.shape[0], dtype=torch.float64, device=dev).index_add_(0, inv, wneg)
            gpos = torch.zeros(cnt.shape[0], dtype=torch.float64, device=dev).index_add_(0, inv, wpos)
            below = torch.cumsum(gneg, 0) - gneg                      # negative weight strictly below each tie group
            num = (gpos * (below + 0.5 * gneg)).sum()
            den = wpos.sum() * wneg.sum()
            return float((num / den.clamp_min(1e-300)).item()) if float(den.item()) > 0 else 0.5
        pred = a[0] > 0
        tp = (wd * (pred & pos)).sum()
        fp = (wd * (pred & ~pos)).sum()
        fn = (wd * (~pred & pos)).sum()
        prec = tp / (tp + fp).clamp_min(1e-300)
        rec = tp / (tp + fn).clamp_min(1e-300)
        if name == "Precision":
            return float(prec.item()) if float((tp + fp).item()) > 0 else 1.0
        if name == "Recall":
            return float(rec.item()) if float((tp + fn).item()) > 0 else 1.0
        return float((2 * prec * rec / (prec + rec).clamp_min(1e-300)).item())
    if name == "Logloss":
        per = torch.nn.functional.softplus(a[0]) - yt * a[0]
    elif name == "RMSE":
        per = (a[0] - yt) ** 2
    elif name == "MAE":
        per = (a[0] - yt).abs()
    elif name == "MultiClass":
        per = torch.logsumexp(a, 0) - a.gather(0, yt.long().unsqueeze(0))[0]
    else:   # Accuracy
        pred = (a[0] > 0).float() if a.shape[0] == 1 else a.argmax(0).float()
        per = (pred == yt).float()
    if wt is None:
        v = per.double().mean()
    else:
        v = (per.double() * wt.double()).sum() / wt.double().sum().clamp_min(1e-300)
    v = float(v.item())
    return math.sqrt(max(v, 0.0)) if name == "RMSE" else v


def _dist_metric(metric, approx, y, w, pool, ctx, objective):
    """Metric value over all ranks (additive metrics are averaged by weight; rank-local otherwise)."""
    v = _device_metric(metric, approx, y, w, pool) if isinstance(approx, torch.Tensor) else None
    if v is None:
        v = _host_metric(metric, approx, y, w, pool, objective.dims)
    if ctx is None or not ctx.is_distributed:
        return v
    wsum = float(len(y)) if w is None else float(np.sum(w))
    parts = ctx.all_gather_object((v, wsum))
    tot = sum(p[1] for p in parts)
    if getattr(metric, "name", "") in ("RMSE", "QueryRMSE", "MultiRMSE"):
        return math.sqrt(sum(p[0] ** 2 * p[1] for p in parts) / tot)
    return sum(p[0] * p[1] for p in parts) / tot


def _apply_tree_to(store, tree, approx, n, dims, dev):
    """approx[:, :n] += leaf values of ``tree`` for the documents of ``store``."""
    vals = torch.from_numpy(np.asarray(tree["values"], dtype=np.float32).reshape(-1, dims)).to(dev)
    if tree["kind"] == "oblivious":
        leaf = ops.leaf_index(store, torch.from_numpy(np.ascontiguousarray(tree["splits"], dtype=np.int32)).to(dev))
        approx[:, :n] += vals[leaf[:n].long() & 0xFFFF].t()
        return
    ns = torch.from_numpy(np.ascontiguousarray(tree["node_split"], dtype=np.int32)).to(dev)
    node = torch.zeros(store.npad, dtype=torch.int16, device=dev)
    depth = _nonsym_depth(tree["node_split"])
    for _ in range(depth):
        ops.update_nodes(store, node, ns)
    lut = torch.from_numpy(np.where(tree["leaf_of_node"] >= 0, tree["leaf_of_node"], 0).astype(np.int64)).to(dev)
    approx[:, :n] += vals[lut[node[:n].long() & 0xFFFF]].t()


def _nonsym_depth(ns) -> int:
    depth = np.zeros(len(ns), dtype=np.int64)
    for k in range(len(ns)):
        if ns[k, 0] >= 0:
            depth[ns[k, 3]] = depth[ns[k, 3] + 1] = depth[k] + 1
    return int(depth.max()) if len(ns) else 0


# ---------------------------------------------------------------------------------------------------------
def _run_fast(o, objective, store, eval_stores, y_train, w_train, base_train, eval_y, eval_w, base_evals, train_pool,
              eval_pools, metrics, logger, od, ctx, prof, callbacks, hist, eval_names, snap) -> LoopResult:
    from .gpu_engine import EvalSet, GpuObliviousEngine
    dev = store.bins.device
    n = store.n
    T = int(o.iterations)
    f32 = torch.float32
    evs = []
    K = int(objective.dims)
    for es, y, w, b in zip(eval_stores, eval_y, eval_w, base_evals):
        if K > 1:
            ap = torch.zeros((K, es.npad), dtype=f32, device=dev)
            ap[:, : es.n] = torch.from_numpy(np.ascontiguousarray(b)).to(dev, f32)
        else:
            ap = torch.zeros(es.npad, dtype=f32, device=dev)
            ap[: es.n] = torch.from_numpy(np.ascontiguousarray(b[0])).to(dev, f32)
        tt = torch.zeros(es.npad, dtype=f32, device=dev)
        tt[: es.n] = torch.from_numpy(np.asarray(y, dtype=np.float32)).to(dev)
        ww = None
        if w is not None:
            ww = torch.zeros(es.npad, dtype=f32, device=dev)
            ww[: es.n] = torch.from_numpy(np.asarray(w, dtype=np.float32)).to(dev)
        evs.append(EvalSet(es, tt, ww, ap))
    boot_p = float(o.bagging_temperature) if o.bootstrap_type == "Bayesian" else float(o.subsample or 1.0)
    btype = o.bootstrap_type
    if btype == "Bayesian" and boot_p == 0:
        btype = "No"
    der_fn = None
    if objective.native_id is None:
        octx = ObjectiveContext(train_pool, dev)
        t_dev = torch.from_numpy(np.asarray(y_train, dtype=np.float32)).to(dev)
        w_dev = None if w_train is None else torch.from_numpy(np.asarray(w_train, dtype=np.float32)).to(dev)
        der_fn = lambda cur: objective.der_hess(cur.unsqueeze(0), t_dev, w_dev, octx)
    with prof.span("engine_setup"):
        eng = GpuObliviousEngine(
            store, torch.from_numpy(np.asarray(y_train, dtype=np.float32)),
            None if w_train is None else torch.from_numpy(np.asarray(w_train, dtype=np.float32)),
            torch.from_numpy(np.ascontiguousarray(base_train if K > 1 else base_train[0], dtype=np.float32)), objective,
            depth=int(o.depth), iterations=T, learning_rate=float(o.learning_rate), l2_leaf_reg=float(o.l2_leaf_reg),
            score_function=o.score_function, random_strength=float(o.random_strength), bootstrap_type=btype,
            bootstrap_param=boot_p, mvs_reg=(None if o.mvs_reg is None else float(o.mvs_reg)),
            leaf_method=o.leaf_estimation_method,
            leaf_iterations=int(o.leaf_estimation_iterations), seed=int(o.random_seed), ctx=ctx,
            reduce=("fused" if o.histogram_reduce in ("fused", None) else "nccl"), eval_sets=evs,
            quantized_hist={"narrow": True, "wide": "wide", "float": False}[o.histogram_cells or "narrow"],
            leaf_backtracking=str(o.leaf_estimation_backtracking or "AnyImprovement"), dims=K,
            der_fn=der_fn, zero_mean_leaves=bool(der_fn is not None and getattr(objective, "zero_mean_leaves", False)))
    phase_timing = os.environ.get("CB200_PHASE_TIMING") == "1" and getattr(eng, "plan", None)
    if phase_timing:
        eng.enable_phase_timing()       # developer aid: per-level phase times of the last tree go to stderr
    # resume from a snapshot: same container and state as the general learner writes (trees + metric history), so either
    # trainer can pick up the other's file
    start = 0
    restored = snap.try_load(o)
    if restored is not None and restored.get("trees"):
        t0 = restored["trees"]
        if any(t.get("kind") != "oblivious" or len(t["splits"]) != int(o.depth) for t in t0):
            raise CatBoostError("the snapshot was written by a run with a different tree shape")
        hist.data, hist.iters = restored["hist"], list(restored["iters"])
        eng.restore_trees(np.stack([np.asarray(t["splits"], dtype=np.int32) for t in t0]),
                          np.stack([np.asarray(t["values"], dtype=np.float32).reshape(-1) for t in t0]),
                          np.stack([np.asarray(t["weights"], dtype=np.float32).reshape(-1) for t in t0]))
        start = len(t0)
        if od is not None and eval_names:
            for v in hist.data.get(eval_names[0], {}).get(str(metrics[0]), []):
                od.add(v)

    def snapshot_state():
        sp_, vals_, wts_ = eng.export_trees()
        return dict(trees=[dict(kind="oblivious", splits=sp_[t], node_split=None, leaf_of_node=None,
                                values=(vals_[t].reshape(-1, K) if K > 1 else vals_[t]), weights=wts_[t])
                           for t in range(len(sp_))], hist=hist.data, iters=hist.iters)

    loss_metric_name = objective.name
    # "cheap" logging: the only tracked metric is the objective itself, which the device already accumulates
    cheap = (len(metrics) == 1 and isinstance(o.loss_function, str) and str(metrics[0]) == o.loss_function
             and der_fn is None)
    need_each = bool(od is not None or callbacks)
    # metrics the caller asked for beyond the objective only exist if they are evaluated along the way (the objective's
    # own curve can be filled from the device history afterwards)
    asked = bool(o.custom_metric) or bool(o.custom_loss)
    want_log = bool(o.verbose) or bool(eval_stores) or (asked and not cheap)
    period = 1 if need_each else (max(1, int(o.metric_period)) if want_log else T)
    done, best_it, best_val, stop = start, None, None, False
    final_loss = None
    t_loop = time.time()
    pinned = torch.zeros(2, dtype=torch.float64).pin_memory()
    pinned_ev = torch.zeros(max(1, 2 * len(evs)), dtype=torch.float64).pin_memory()
    fin = (lambda v: math.sqrt(max(v, 0.0))) if objective.name == "RMSE" else (lambda v: v)
    # Plain per-iteration logging of the objective (no evaluation sets, detector or callbacks): the learn loss after j trees
    # is what iteration j accumulates at its start, so it is read from the device history one iteration behind the
    # launches, on a side stream that only waits for the iteration before the one in flight -- the GPU never idles for
    # the host, and no extra pass over the data is needed.  The last value comes from an explicit pass.
    # (one rank only: with several ranks the value needs a collective, which stays on the main stream)
    lagged = bool(cheap and want_log and period == 1 and not evs and od is None and not callbacks and dev.type == "cuda"
                  and eng.R == 1 and start == 0 and os.environ.get("CB200_LAGGED_LOG", "1") != "0")
    if lagged:
        with prof.span("iterations"):
            side = torch.cuda.Stream(dev)
            main = torch.cuda.current_stream(dev)
            ev_prev, next_log = None, 0

            def read_row(j):
                row = eng.loss_hist[j]
                if eng.R > 1:
                    row = row.clone()
                    ctx.all_reduce_sum_(row)
                pinned.copy_(row, non_blocking=True)

            def emit(idx, value):
                hist.iters.append(idx)
                hist.add("learn", metrics[0], fin(value))
                logger.log_iteration(idx, T, hist, time.time() - t_loop)

            while done < T:
                eng.step(1)
                done += 1
                ev_cur = torch.cuda.Event()
                ev_cur.record(main)
                if ev_prev is not None:
                    with torch.cuda.stream(side):
                        side.wait_event(ev_prev)
                        read_row(done - 2)                    # complete once iteration done-2 has finished
                    side.synchronize()
                    if done - 3 >= next_log:
                        emit(done - 3, float(pinned[0]) / max(float(pinned[1]), 1e-300))
                        next_log = done - 2
                ev_prev = ev_cur
                if eng.arena is not None and (done % 64 == 0):
                    eng.arena.check_status()
                if snap.due() and done < T:
                    snap.maybe_save(snapshot_state, done - 1)
            torch.cuda.synchronize(dev)
            for idx in range(next_log, T - 1):
                read_row(idx + 1)
                torch.cuda.current_stream(dev).synchronize()
                emit(idx, float(pinned[0]) / max(float(pinned[1]), 1e-300))
            emit(T - 1, eng.current_learn_loss(pinned))
            sp, vals, wts = eng.finish()
    with prof.span("iterations"):
        while done < T and not stop:
            k = min(period, T - done)
            if snap.enabled and not want_log and not need_each:
                k = min(k, 64)                       # come up for air so that a due snapshot can be written
            eng.step(k)
            done += k
            if snap.due() and done < T:
                snap.maybe_save(snapshot_state, done - 1)
            if not want_log and not need_each:
                continue
            it = done - 1
            hist.iters.append(it)
            if cheap:
                hist.add("learn", metrics[0], fin(eng.current_learn_loss(pinned)))
                if evs:
                    row = eng.eval_hist[it].clone()
                    if eng.R > 1:
                        ctx.all_reduce_sum_(row)
                    pinned_ev.copy_(row, non_blocking=True)
                    torch.cuda.current_stream(dev).synchronize()
                    for j in range(len(evs)):
                        hist.add(eval_names[j], metrics[0], fin(float(pinned_ev[2 * j]) / max(float(pinned_ev[2 * j + 1]), 1e-300)))
            else:
                torch.cuda.current_stream(dev).synchronize()
                lf_ = eng.leaf[:n].long() & 0xFFFF
                if K > 1:
                    cur = eng.approx[:, :n] + eng.cur_vals.view(eng.L, K)[lf_].t()
                else:
                    cur = (eng.approx[:n] + eng.cur_vals[lf_]).unsqueeze(0)
                for m in metrics:
                    hist.add("learn", m, _dist_metric(m, cur, y_train, w_train, train_pool, ctx, objective))
                    for j, ev in enumerate(evs):
                        ea_ = ev.approx[:, : ev.store.n] if K > 1 else ev.approx[: ev.store.n].unsqueeze(0)
                        hist.add(eval_names[j], m, _dist_metric(m, ea_, eval_y[j], eval_w[j], eval_pools[j], ctx, objective))
            if eng.arena is not None and (it % 64 == 0):
                eng.arena.check_status()
            if evs:
                v = hist.data[eval_names[0]][str(metrics[0])][-1]
                if best_val is None or (v > best_val if metrics[0].is_max_optimal else v < best_val):
                    best_val, best_it = v, it
                if od is not None and od.add(v):
                    stop = True
            logger.log_iteration(it, T, hist, time.time() - t_loop)
            for cb in callbacks:
                if cb.after_iteration(_CallbackInfo(it, hist.data)) is False:
                    stop = True
        if not lagged:
            final_loss = eng.current_learn_loss(pinned) if (not hist.iters and done > 0) else None
            sp, vals, wts = eng.finish()
    if stop and od is not None and od.stopped:
        logger.info(f"Stopped by overfitting detector  ({od.wait} iterations wait)")
    trees = [dict(kind="oblivious", splits=sp[t], node_split=None, leaf_of_node=None,
                  values=(vals[t].reshape(-1, K) if K > 1 else vals[t]), weights=wts[t]) for t in range(done)]
    snap.finalize(dict(trees=trees, hist=hist.data, iters=hist.iters))
    if not hist.iters:
        # nothing was logged during training: fill the learn curve of the objective from the device history
        lh = eng.learn_loss_history()
        name = str(metrics[0]) if (getattr(metrics[0], "name", None) == loss_metric_name and der_fn is None) else None
        if name is not None and len(lh) >= 1 and final_loss is not None:
            vals_l = lh[1:].tolist() + [final_loss]          # row j = loss after j trees; the last one from its own pass
            if objective.name == "RMSE":
                vals_l = [math.sqrt(v) for v in vals_l]
            hist.data["learn"][name] = vals_l
    launches = eng.launches_per_iter
    if phase_timing and ctx.rank == 0:
        import sys
        print("level geometry (grid, slots/pass, smem, threads, chunks, copies, bundle):", eng.level_geo,
              "mean share of the most frequent bin:", round(eng.dominant_bin_share, 3), "skipping:", eng.domw is not None,
              "bins per group:", getattr(eng, "group_bins", None), "feature kinds:",
              "".join(f.kind[0] for f in store.features), file=sys.stderr)
        print("phase us per level [leaf update, histogram, grid wait, reduce + push, score, select]:\n",
              np.round(eng.phase_times_us(), 1), file=sys.stderr)
    train_approx = (eng.approx[:, :n].t().double().cpu().numpy() if K > 1
                    else eng.approx[:n].double().cpu().numpy().reshape(-1, 1))
    eng.close()
    return LoopResult(trees, hist.data, best_it, _best_scores(hist, metrics), launches, train_approx)
