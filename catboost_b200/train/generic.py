"""General tree learner (any objective, any grow policy, CPU or GPU).

Histograms come from the native kernels (``ops.api.hist``: CUDA shared-memory atomics on the GPU, OpenMP on the
CPU); split scoring, leaf selection and leaf estimation are vectorised tensor code that runs on whichever device
holds the store.  The flagship configuration (symmetric trees + pointwise loss on the GPU) does not come through
here: ``gpu_engine.GpuObliviousEngine`` keeps that whole loop on the device.

Reference behaviour reproduced: candidate = (feature, border) with statistics of the ``<=`` side from a bin prefix
sum (catboost/cuda/methods/kernel/split_properties_helpers.cuh:112), score calcers
(catboost/cuda/methods/kernel/score_calcers.cuh), SymmetricTree / Depthwise / Lossguide policies
(catboost/cuda/methods/greedy_subsets_searcher/greedy_search_helper.cpp:320-700,
catboost/private/libs/algo/greedy_tensor_search.cpp:1171,1467,1764), leaf estimation with several
Newton / gradient steps (catboost/private/libs/algo/approx_calcer.cpp,
catboost/cuda/methods/leaves_estimation/descent_helpers.cpp:127-206), exact quantile leaves
(catboost/cuda/methods/kernel/exact_estimation.cu).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional

import numpy as np
import torch

from ..data.quantization import BinnedStore
from ..ops import api as ops


@dataclass
class TreeResult:
    kind: str                                # 'oblivious' | 'nonsymmetric'
    splits: Optional[np.ndarray] = None      # oblivious: int [depth, 4] (feature, bin, _, flags)
    node_split: Optional[np.ndarray] = None  # nonsymmetric: int [nodes, 4] (feature, bin, flags, left_child)
    leaf_of_node: Optional[np.ndarray] = None
    n_leaves: int = 1
    leaf: Optional[torch.Tensor] = None      # int16 [npad] leaf id of every training document


class SplitScorer:
    """Turns histograms [L, S, TB] into per-candidate score terms [L, F, Bmax]."""

    def __init__(self, store: BinnedStore, score_function: str, l2: float):
        self.store = store
        dev = store.bins.device
        F, B = store.F, max(1, store.max_bins)
        off = torch.from_numpy(store.feat_off_host[:-1].astype(np.int64)).to(dev)
        nb = torch.from_numpy(store.feat_nb_host.astype(np.int64)).to(dev)
        ar = torch.arange(B, device=dev)
        self.valid_bin = ar.unsqueeze(0) < nb.unsqueeze(1)                       # [F, B]
        self.idx = torch.where(self.valid_bin, off.unsqueeze(1) + ar.unsqueeze(0), torch.zeros((), dtype=torch.long, device=dev))
        self.onehot = store.feat_onehot.bool().unsqueeze(1)                      # [F, 1]
        ncand = torch.where(self.onehot.squeeze(1), nb, nb - 1)
        self.valid_cand = ar.unsqueeze(0) < ncand.unsqueeze(1)                   # [F, B]
        self.fn = score_function
        self.l2 = float(l2)
        self.F, self.B = F, B

    def sides(self, hist: torch.Tensor):
        """left / right statistics of every candidate: each [L, S, F, B]."""
        H = hist[:, :, self.idx] * self.valid_bin
        cum = H.cumsum(-1)
        total = cum[..., -1:]
        left = torch.where(self.onehot, total - H, cum)      # one-hot: left = "value != v"
        right = total - left
        return left, right, total

    def leaf_terms(self, s, w):
        """(num, den) contribution of one side; s [L, K, F, B] sums, w [L, F, B] weights."""
        w = w.clamp_min(0.0)
        l2 = self.l2
        fn = self.fn
        if fn in ("Cosine", "NewtonCosine"):
            mu = torch.where(w.unsqueeze(1) > 0, s / (w.unsqueeze(1) + l2), torch.zeros_like(s))
            return (s * mu).sum(1), (w.unsqueeze(1) * mu * mu).sum(1)
        if fn in ("L2", "NewtonL2"):
            return torch.where(w.unsqueeze(1) > 1e-20, s * s / (w.unsqueeze(1) + l2), torch.zeros_like(s)).sum(1), None
        if fn == "SolarL2":
            ww = w.unsqueeze(1)
            return torch.where(ww > 1e-20, s * s * (1 + 2 * torch.log(ww + 1)) / ww.clamp_min(1e-20), torch.zeros_like(s)).sum(1), None
        if fn == "LOOL2":
            ww = w.unsqueeze(1)
            adj = torch.where(ww > 1, ww / (ww - 1).clamp_min(1e-20), torch.zeros_like(ww)) ** 2
            return torch.where(ww > 0, adj * s * s / ww.clamp_min(1e-20), torch.zeros_like(s)).sum(1), None
        if fn == "SatL2":
            ww = w.unsqueeze(1)
            adj = torch.where(ww > 2, ww * (ww - 2) / (ww * ww - 3 * ww + 1), torch.zeros_like(ww))
            return torch.where(ww > 0, adj * s * s / ww.clamp_min(1e-20), torch.zeros_like(s)).sum(1), None
        raise ValueError(fn)

    def candidate_terms(self, hist: torch.Tensor, n_sum_stats: int, count_stat: Optional[int] = None):
        """num/den [L, F, B] for every candidate, plus the child document counts when a count statistic exists."""
        left, right, total = self.sides(hist)
        K = n_sum_stats
        nL, dL = self.leaf_terms(left[:, :K], left[:, K])
        nR, dR = self.leaf_terms(right[:, :K], right[:, K])
        num = nL + nR
        den = None if dL is None else dL + dR
        cnt = None
        if count_stat is not None:
            cnt = (left[:, count_stat], right[:, count_stat])
        return num, den, cnt, (left, right, total)

    def finish(self, num, den):
        if den is not None:
            return torch.where(den > 1e-15, num / torch.sqrt(den + 1e-10), torch.full_like(num, -3.0e38))
        return num


class GenericLearner:
    def __init__(self, store: BinnedStore, opts, dims: int, ctx=None, seed: int = 0):
        self.store, self.o, self.dims, self.ctx = store, opts, dims, ctx
        self.dev = store.bins.device
        self.scorer = SplitScorer(store, opts.score_function, float(opts.l2_leaf_reg))
        self.gen = torch.Generator(device="cpu")
        self.gen.manual_seed(int(seed) + 12345)
        self.leaf = torch.zeros(store.npad, dtype=torch.int16, device=self.dev)
        self.use_count = int(opts.min_data_in_leaf) > 1
        self._onehot_host = store.feat_onehot.cpu().numpy().astype(bool)        # read on the host by the growth loops
        self.monotone = None          # float tensor [F] in {-1, 0, +1} per flat feature, set by set_monotone()
        self.group_of_doc = None      # int64 [n] query number of every document: set for sampling_unit='Group'
        # feature penalties (set_penalties): the score of a candidate loses coef * first_use[f] while feature f is in no
        # tree yet, and coef * per_object[f] * (documents of the leaf that have not met f on their path in any tree)
        self.pen_first = None         # float tensor [F] or None
        self.pen_object = None        # float tensor [F] or None
        self.pen_coef = 1.0
        self.used_feature = torch.zeros(store.F, dtype=torch.bool, device=self.dev)
        self.used_by_doc = {}         # flat feature -> bool [n], only for features with a per-object penalty
        self._resample = None         # set by build_tree when the bootstrap is redrawn at every level
        self.n_total = store.n
        if ctx is not None and ctx.is_distributed:
            t = torch.tensor([store.n], dtype=torch.float64, device=self.dev)
            ctx.all_reduce_sum_(t)
            self.n_total = int(t.item())


    # -- feature penalties (catboost/private/libs/algo/feature_penalties_calcer.cpp) ------------------------
    def set_penalties(self, first_use, per_object, coef: float):
        """first_use / per_object: float arrays [F] over the flat features of the store (zeros = no penalty)."""
        to = lambda v: None if v is None or not np.any(v) else torch.from_numpy(np.asarray(v, dtype=np.float32)).to(self.dev)
        self.pen_first, self.pen_object, self.pen_coef = to(first_use), to(per_object), float(coef)
        if self.pen_object is not None:
            for f in torch.nonzero(self.pen_object).flatten().tolist():
                self.used_by_doc[int(f)] = torch.zeros(self.store.n, dtype=torch.bool, device=self.dev)

    @property
    def has_penalties(self) -> bool:
        return self.pen_first is not None or self.pen_object is not None

    def _penalty(self, node_ids=None):
        """Penalty [L, F] (L = 1 for symmetric trees, where a level splits every leaf) to subtract from the scores."""
        if not self.has_penalties:
            return None
        L = 1 if node_ids is None else len(node_ids)
        pen = torch.zeros((L, self.store.F), dtype=torch.float32, device=self.dev)
        if self.pen_first is not None:
            pen += (self.pen_first * (~self.used_feature).float()).unsqueeze(0)
        if self.pen_object is not None:
            n = self.store.n
            row = None
            if node_ids is not None:
                lut = torch.full((max(int(max(node_ids)) + 1, 1),), -1, dtype=torch.long, device=self.dev)
                lut[torch.tensor(list(node_ids), device=self.dev)] = torch.arange(L, device=self.dev)
                node = self.leaf[:n].long() & 0xFFFF
                row = torch.where(node < lut.numel(), lut[node.clamp_max(lut.numel() - 1)], torch.full_like(node, -1))
            for f, seen in self.used_by_doc.items():
                fresh = ~seen
                if row is None:
                    cnt = fresh.sum().view(1).float()
                else:
                    sel = fresh & (row >= 0)
                    cnt = torch.bincount(row[sel], minlength=L).float()
                if self.ctx is not None and self.ctx.is_distributed:
                    cnt = cnt.double()
                    self.ctx.all_reduce_sum_(cnt)
                    cnt = cnt.float()
                pen[:, f] += self.pen_object[f] * cnt
        return pen * self.pen_coef

    def _mark_used(self, tr: "TreeResult"):
        """After a tree: the features it splits on count as used; per-object flags follow the path of every document."""
        if not self.has_penalties:
            return
        n = self.store.n
        if tr.kind == "oblivious":
            for f in tr.splits[:, 0]:
                if f >= 0:
                    self.used_feature[int(f)] = True
                    if int(f) in self.used_by_doc:
                        self.used_by_doc[int(f)].fill_(True)
            return
        ns = tr.node_split
        on_path = {0: frozenset()}
        for node in range(len(ns)):
            f, left = int(ns[node, 0]), int(ns[node, 3])
            if f >= 0:
                self.used_feature[f] = True
                on_path[left] = on_path[left + 1] = on_path[node] | {f}
        leaf_doc = self.leaf[:n].long() & 0xFFFF
        for f, seen in self.used_by_doc.items():
            leaves = [int(tr.leaf_of_node[node]) for node, fs in on_path.items() if f in fs and tr.leaf_of_node[node] >= 0]
            if leaves:
                seen |= torch.isin(leaf_doc, torch.tensor(leaves, device=self.dev))

    # -- helpers ---------------------------------------------------------------------------------------
    def _rand(self, shape):
        return torch.rand(shape, generator=self.gen).to(self.dev)

    def _randn(self, shape):
        return torch.randn(shape, generator=self.gen).to(self.dev)

    def _score_noise(self, shape):
        """Unit noise added to split scores: standard normal, or standard Gumbel for random_score_type='Gumbel'."""
        if str(self.o.random_score_type) == "Gumbel":
            u = torch.rand(shape, generator=self.gen).clamp_(1e-12, 1.0 - 1e-7)
            return (-torch.log(-torch.log(u))).to(self.dev)
        return self._randn(shape)

    def bootstrap_weights(self, der: torch.Tensor) -> Optional[torch.Tensor]:
        o, n = self.o, self.store.n
        bt = o.bootstrap_type
        if bt == "No":
            return None
        if self.group_of_doc is not None and bt in ("Bayesian", "Bernoulli", "Poisson"):
            # sampling_unit='Group' (catboost/private/libs/algo/bootstrap? fold sampling by query): one draw per
            # query, shared by its documents
            ng = int(self.group_of_doc.max().item()) + 1 if n else 0
            if bt == "Bayesian":
                t = float(o.bagging_temperature)
                if t == 0:
                    return None
                g = (-torch.log(self._rand(ng).clamp_min(1e-20))) ** t
            elif bt == "Bernoulli":
                g = (self._rand(ng) < float(o.subsample)).float()
            else:
                g = torch.poisson(torch.full((ng,), float(o.subsample)), generator=self.gen).to(self.dev)
            return g[self.group_of_doc]
        if bt == "Bayesian":
            t = float(o.bagging_temperature)
            if t == 0:
                return None
            e = -torch.log(self._rand(n).clamp_min(1e-20))
            return e if t == 1.0 else e ** t
        if bt == "Bernoulli":
            return (self._rand(n) < float(o.subsample)).float()
        if bt == "Poisson":
            return torch.poisson(torch.full((n,), float(o.subsample)), generator=self.gen).to(self.dev)
        if bt == "MVS":
            # minimal-variance sampling (catboost/private/libs/algo/mvs.cpp): keep probability ~ |gradient|
            g = torch.sqrt((der * der).sum(0)[:n] + (float(o.mvs_reg) if o.mvs_reg is not None else (der.abs().mean().item() ** 2)))
            rate = float(o.subsample)
            if rate >= 1.0:
                return None
            # the threshold mu solves sum_i min(1, g_i / mu) = rate * n; the left side falls monotonically in mu, so 40
            # bisection steps on it give mu to float precision without sorting the gradients (the device kernel
            # ops/cuda/cb_mvs.cu does the same per block of 8192 documents)
            target = rate * n
            lo, hi = 0.0, max(float(g.sum().item()) / max(target, 1e-30), 1e-30)
            while float(torch.clamp(g / hi, max=1.0).sum().item()) > target:
                hi *= 2.0
            for _ in range(40):
                mid = 0.5 * (lo + hi)
                if float(torch.clamp(g / mid, max=1.0).sum().item()) > target:
                    lo = mid
                else:
                    hi = mid
            mu = torch.tensor(max(hi, 1e-30), dtype=g.dtype, device=g.device)
            p = (g / mu).clamp(max=1.0)
            keep = self._rand(n) < p
            return torch.where(keep, 1.0 / p.clamp_min(1e-12), torch.zeros_like(p))
        raise ValueError(bt)

    def _hist(self, stats, slot_table, nslots):
        h = ops.hist(self.store, self.leaf, stats, slot_table, nslots)
        if self.ctx is not None and self.ctx.is_distributed:
            self.ctx.all_reduce_sum_(h)
        return h

    def _noise_std(self, der, iteration):
        rs = float(self.o.random_strength)
        if rs <= 0:
            return 0.0
        n = self.store.n
        ss = (der[:, :n] ** 2).sum().double()
        if self.ctx is not None and self.ctx.is_distributed:
            ss = ss.reshape(1)
            self.ctx.all_reduce_sum_(ss)
            ss = ss[0]
        N = max(self.n_total, 1)
        sd = math.sqrt(float(ss.item()) / N)
        m = math.exp(math.log(N) - iteration * float(self.o.learning_rate))
        return rs * sd * m / (1 + m)

    def _feature_mask(self):
        fw = self.store.feat_weight > 0
        rsm = float(self.o.rsm)
        if rsm < 1.0 and self.store.F > 1:
            keep = self._rand(self.store.F) < rsm
            if not bool((keep & fw).any()):
                keep[int(torch.randint(0, self.store.F, (1,), generator=self.gen))] = True
            fw = fw & keep
        return fw

    # -- structure search ------------------------------------------------------------------------------
    def build_tree(self, der: torch.Tensor, hess: torch.Tensor, weight: Optional[torch.Tensor], iteration: int) -> TreeResult:
        """der/hess: [dims, npad] (already multiplied by the sample weights)."""
        o, n, npad = self.o, self.store.n, self.store.npad
        newton = o.score_function.startswith("Newton")
        K = self.dims
        rows = K + 1 + (1 if self.use_count else 0)
        wcol = hess[:, :n].sum(0) / K if newton else (torch.ones(n, device=self.dev) if weight is None else weight[:n])

        def make_stats():
            bw = self.bootstrap_weights(der)
            st = torch.zeros((rows, npad), dtype=torch.float32, device=self.dev)
            if bw is not None:
                st[:K, :n] = der[:, :n] * bw
                st[K, :n] = wcol * bw
            else:
                st[:K, :n] = der[:, :n]
                st[K, :n] = wcol
            if self.use_count:
                st[K + 1, :n] = 1.0
            return st

        stats = make_stats()
        # sampling_frequency='PerTreeLevel' (catboost/private/libs/algo/greedy_tensor_search.cpp: the bootstrap runs before
        # every level's candidate scoring): the growers call this for fresh weights at every level after the first
        self._resample = make_stats if (str(o.sampling_frequency or "PerTree") == "PerTreeLevel"
                                        and o.bootstrap_type != "No") else None
        self.leaf.zero_()
        noise_std = self._noise_std(der, iteration)
        fmask = self._feature_mask()
        if o.grow_policy == "SymmetricTree":
            tr = self._grow_symmetric(stats, K, noise_std, fmask)
        elif o.grow_policy in ("Depthwise", "Region"):
            tr = self._grow_depthwise(stats, K, noise_std, fmask)
        else:
            tr = self._grow_lossguide(stats, K, noise_std, fmask)
        self._mark_used(tr)
        return tr

    def set_monotone(self, per_float_feature: dict):
        """``per_float_feature``: {float-feature index: +1 / -1}.  A candidate on a constrained feature is only allowed
        when in every leaf the value of the right child is not below (+1) / above (-1) the value of the left child;
        finished trees are repaired by ``enforce_monotone_leaves`` (catboost/private/libs/algo/monotonic_constraint_utils.cpp)."""
        c = np.zeros(self.store.F, dtype=np.float32)
        for f, ff in enumerate(self.store.features):
            if ff.kind == "float" and int(ff.source) in per_float_feature:
                c[f] = float(per_float_feature[int(ff.source)])
        self.monotone = torch.from_numpy(c).to(self.dev) if np.any(c != 0) else None

    def _monotone_ok(self, left, right, K):
        """[F, B] mask of the candidates that respect the constraints (single-dimension models)."""
        l2 = self.scorer.l2
        vl = left[:, 0] / (left[:, K].clamp_min(0) + l2 + 1e-20)             # [L, F, B]
        vr = right[:, 0] / (right[:, K].clamp_min(0) + l2 + 1e-20)
        diff = (vr - vl) * self.monotone.view(1, -1, 1)
        empty = (left[:, K] <= 0) | (right[:, K] <= 0)
        return ((diff >= 0) | empty).all(0)

    def _cand_mask(self, fmask, cnt):
        m = self.scorer.valid_cand & fmask.unsqueeze(1)
        return m

    def _grow_symmetric(self, stats, K, noise_std, fmask) -> TreeResult:
        depth = int(self.o.depth)
        sc = self.scorer
        splits = np.full((depth, 4), 0, dtype=np.int32)
        splits[:, 0] = -1
        cstat = K + 1 if self.use_count else None
        fw = self.store.feat_weight
        h_prev, small_right = None, None
        for level in range(depth):
            L = 1 << level
            if level and self._resample is not None:
                stats, h_prev = self._resample(), None       # new weights: the parent histograms no longer apply
            if h_prev is None:
                table = torch.arange(L, dtype=torch.int16, device=self.dev)
                h = self._hist(stats, table, L)
            else:
                # sibling subtraction: only the lighter child of every parent is accumulated, the other one is the
                # parent's histogram minus it (catboost/cuda/methods/pointwise_kernels.cpp:70-92)
                half = L >> 1
                ar = torch.arange(L, device=self.dev)
                parent, bit = ar & (half - 1), ar >> (level - 1)
                is_small = bit == small_right[parent].long()
                table = torch.where(is_small, parent, torch.full_like(parent, -1)).to(torch.int16)
                h_small = self._hist(stats, table, half)
                h_big = h_prev - h_small
                h = torch.where(is_small.view(L, 1, 1), h_small[parent], h_big[parent])
            native_scores = (USE_NATIVE_CPU_SCORES and self.dev.type == "cpu" and cstat is None and self.monotone is None
                             and sc.fn in ("Cosine", "NewtonCosine", "L2", "NewtonL2") and h.dtype == torch.float32)
            if native_scores:
                # host: one native pass per feature over the level's histograms (ops/cpu/cb_cpu.cpp cbc_symmetric_scores)
                score, cnt, sides_ = self._native_symmetric_scores(h, K), None, None
            else:
                num, den, cnt, sides_ = sc.candidate_terms(h, K, cstat)
                score = sc.finish(num.sum(0), None if den is None else den.sum(0))          # [F, B]
            if noise_std > 0:
                score = score + self._score_noise(score.shape) * noise_std
            score = score * fw.unsqueeze(1)
            pen = self._penalty()
            if pen is not None:
                score = score - pen[0].unsqueeze(1)
            mask = self._cand_mask(fmask, cnt)
            if self.monotone is not None and K == 1:
                mask = mask & self._monotone_ok(sides_[0], sides_[1], K)
            if cnt is not None:
                mdl = int(self.o.min_data_in_leaf)
                ok = ((cnt[0] >= mdl) | (cnt[0] == 0)).all(0) & ((cnt[1] >= mdl) | (cnt[1] == 0)).all(0)
                mask = mask & ok
            score = torch.where(mask, score, torch.full_like(score, -float("inf")))
            best = int(torch.argmax(score.reshape(-1)).item())
            f, b = best // sc.B, best % sc.B
            if not math.isfinite(float(score[f, b].item())):
                break
            onehot = bool(self._onehot_host[f])
            splits[level] = (f, b, 0, 1 if onehot else 0)
            ops.update_leaf(self.store, self.leaf, f, b, onehot, level)
            # which child of every leaf is the lighter one (by the weight column) decides what the next level accumulates
            if sides_ is not None:
                small_right = sides_[1][:, K, f, b] < sides_[0][:, K, f, b]
            else:
                o0, nbf = int(self.store.feat_off_host[f]), int(self.store.feat_nb_host[f])
                wrow = h[:, K, o0:o0 + nbf]
                wl = (wrow.sum(1) - wrow[:, b]) if onehot else wrow[:, :b + 1].sum(1)
                small_right = (wrow.sum(1) - wl) < wl
            h_prev = h
        return TreeResult("oblivious", splits=splits, n_leaves=1 << depth, leaf=self.leaf)

    def _native_symmetric_scores(self, h, K):
        import ctypes
        from ..ops import native
        st = self.store
        L, S, TB = int(h.shape[0]), int(h.shape[1]), int(h.shape[2])
        hc = h.contiguous()
        out = torch.empty((st.F, self.scorer.B), dtype=torch.float32)
        cache = self.__dict__.get("_native_score_args")
        if cache is None:
            cache = (np.ascontiguousarray(st.feat_off_host[:-1], dtype=np.int32), np.ascontiguousarray(st.feat_nb_host, dtype=np.int32),
                     np.ascontiguousarray(self._onehot_host, dtype=np.uint8))
            self.__dict__["_native_score_args"] = cache
        off, nb, oh = cache
        P = lambda a: a.ctypes.data_as(ctypes.c_void_p)
        native.cpu_lib().cbc_symmetric_scores(
            ctypes.c_void_p(hc.data_ptr()), L, S, int(K), TB, int(st.F), P(off), P(nb), P(oh),
            0 if self.scorer.fn in ("Cosine", "NewtonCosine") else 1, ctypes.c_double(self.scorer.l2), int(self.scorer.B),
            ctypes.c_void_p(out.data_ptr()))
        return out

    def _per_leaf_best(self, h, K, noise_std, fmask, node_ids=None):
        if self.has_penalties:
            return self._per_leaf_best_tensor(h, K, noise_std, fmask, self._penalty(node_ids if node_ids is not None
                                                                                  else range(h.shape[0])))
        if self.dev.type == "cuda" and self.monotone is None:
            # device search: one warp per (leaf, feature) + one warp per leaf, 16 bytes per leaf read back
            self._search_calls = getattr(self, "_search_calls", 0) + 1
            if node_ids is None:
                lid = None
            else:
                ids = list(node_ids)
                if len(ids) <= 4 or ids == list(range(ids[0], ids[0] + len(ids))):
                    # consecutive node numbers (the two children of a split, a whole level): made on the device
                    lid = torch.arange(ids[0], ids[0] + len(ids), dtype=torch.int32, device=self.dev) \
                        if ids == list(range(ids[0], ids[0] + len(ids))) else torch.tensor(ids, dtype=torch.int32, device=self.dev)
                else:
                    lid = torch.tensor(ids, dtype=torch.int32, device=self.dev)
            score, feat, bins, gain = ops.leaf_search(
                self.store, h, K, self.scorer.l2, self.o.score_function, noise_std,
                (int(self.o.random_seed) * 1000003 + self._search_calls * 7919) & 0x7FFFFFFFFFFFFFFF, lid, fmask.float(),
                float(self.o.min_data_in_leaf) if self.use_count else 0.0)
            best = np.where(feat >= 0, feat.astype(np.int64) * self.scorer.B + bins, 0)
            return best, np.where(feat >= 0, score, -np.inf), gain
        return self._per_leaf_best_tensor(h, K, noise_std, fmask)

    def _per_leaf_best_tensor(self, h, K, noise_std, fmask, penalty=None):
        """The same search as tensor code (CPU path, monotone constraints, and the oracle of the device kernel)."""
        sc = self.scorer
        cstat = K + 1 if self.use_count else None
        num, den, cnt, (left, right, total) = sc.candidate_terms(h, K, cstat)
        score = sc.finish(num, den)                                                   # [L, F, B]
        # gain over not splitting (L2 form), used for leaf priority and for "no useful split" detection
        w_tot = total[:, K, :, 0].clamp_min(0)
        s_tot = total[:, :K, :, 0]
        parent = (s_tot * s_tot / (w_tot.unsqueeze(1) + sc.l2)).sum(1)                 # [L, F]
        l2num = (left[:, :K] ** 2 / (left[:, K].clamp_min(0).unsqueeze(1) + sc.l2)).sum(1) + \
                (right[:, :K] ** 2 / (right[:, K].clamp_min(0).unsqueeze(1) + sc.l2)).sum(1)
        gain = l2num - parent.unsqueeze(-1)
        if noise_std > 0:
            score = score + self._score_noise(score.shape) * noise_std
        score = score * self.store.feat_weight.view(1, -1, 1)
        if penalty is not None:
            score = score - penalty.unsqueeze(-1)
        mask = (sc.valid_cand & fmask.unsqueeze(1)).unsqueeze(0).expand_as(score)
        nonempty = (left[:, K] > 0) & (right[:, K] > 0)
        mask = mask & nonempty
        if cnt is not None:
            mdl = int(self.o.min_data_in_leaf)
            mask = mask & (cnt[0] >= mdl) & (cnt[1] >= mdl)
        score = torch.where(mask, score, torch.full_like(score, -float("inf")))
        flat = score.reshape(score.shape[0], -1)
        best = torch.argmax(flat, dim=1)
        bscore = flat.gather(1, best.unsqueeze(1)).squeeze(1)
        bgain = gain.reshape(gain.shape[0], -1).gather(1, best.unsqueeze(1)).squeeze(1)
        return best.cpu().numpy(), bscore.cpu().numpy(), bgain.cpu().numpy()

    def _grow_depthwise(self, stats, K, noise_std, fmask) -> TreeResult:
        depth = int(self.o.depth)
        B = self.scorer.B
        node_split: List[List[int]] = [[-1, 0, 0, -1]]
        frontier = [0]
        for level in range(depth):
            if not frontier:
                break
            if level and self._resample is not None:
                stats = self._resample()
            table = torch.full((len(node_split),), -1, dtype=torch.int16, device=self.dev)
            table[torch.tensor(frontier, device=self.dev)] = torch.arange(len(frontier), dtype=torch.int16, device=self.dev)
            h = self._hist(stats, table, len(frontier))
            best, bscore, _ = self._per_leaf_best(h, K, noise_std, fmask, frontier)
            new_frontier = []
            for j, node in enumerate(frontier):
                if not math.isfinite(float(bscore[j])):
                    continue
                f, b = int(best[j]) // B, int(best[j]) % B
                left = len(node_split)
                node_split.append([-1, 0, 0, -1])
                node_split.append([-1, 0, 0, -1])
                node_split[node] = [f, b, 1 if bool(self._onehot_host[f]) else 0, left]
                new_frontier += [left, left + 1]
            if not new_frontier:
                break
            ops.update_nodes(self.store, self.leaf, torch.tensor(node_split, dtype=torch.int32, device=self.dev))
            frontier = new_frontier
        return self._finish_nonsymmetric(node_split)

    def _grow_lossguide(self, stats, K, noise_std, fmask) -> TreeResult:
        max_leaves, max_depth = int(self.o.max_leaves), int(self.o.depth)
        B = self.scorer.B
        node_split: List[List[int]] = [[-1, 0, 0, -1]]
        node_depth = [0]
        cand = {}        # node -> (gain, feature, bin)

        cuda = self.dev.type == "cuda"
        # slot table over all nodes the tree can have, kept on the device and edited in place (no upload per split)
        table_all = torch.full((2 * max_leaves + 1,), -1, dtype=torch.int16, device=self.dev)

        def evaluate(nodes):
            nonlocal stats
            if nodes != [0] and self._resample is not None:
                stats = self._resample()
            table_all.fill_(-1)
            for j, node in enumerate(nodes):
                table_all[node] = j                       # scalar writes: kernel arguments, not host-to-device copies
            h = self._hist(stats, table_all[: len(node_split)], len(nodes))
            best, bscore, bgain = self._per_leaf_best(h, K, noise_std, fmask, nodes)
            for j, node in enumerate(nodes):
                if math.isfinite(float(bscore[j])) and node_depth[node] < max_depth:
                    cand[node] = (float(bgain[j]), int(best[j]) // B, int(best[j]) % B)

        evaluate([0])
        n_leaves = 1
        while n_leaves < max_leaves and cand:
            node = max(cand, key=lambda k: cand[k][0])
            _, f, b = cand.pop(node)
            left = len(node_split)
            node_split += [[-1, 0, 0, -1], [-1, 0, 0, -1]]
            node_depth += [node_depth[node] + 1] * 2
            node_split[node] = [f, b, 1 if bool(self._onehot_host[f]) else 0, left]
            if cuda:
                ops.update_one_node(self.store, self.leaf, node, f, b, bool(self._onehot_host[f]), left)
            else:
                step = [[-1, 0, 0, -1]] * len(node_split)
                step[node] = node_split[node]
                ops.update_nodes(self.store, self.leaf, torch.tensor(step, dtype=torch.int32, device=self.dev))
            n_leaves += 1
            if n_leaves < max_leaves:
                evaluate([left, left + 1])
        return self._finish_nonsymmetric(node_split)

    def _finish_nonsymmetric(self, node_split) -> TreeResult:
        ns = np.array(node_split, dtype=np.int32)
        leaf_of_node = np.full(len(ns), -1, dtype=np.int32)
        terminal = np.nonzero(ns[:, 0] < 0)[0]
        leaf_of_node[terminal] = np.arange(len(terminal), dtype=np.int32)
        # relabel documents: node id -> leaf id
        lut = torch.from_numpy(np.where(leaf_of_node >= 0, leaf_of_node, 0).astype(np.int16)).to(self.dev)
        n = self.store.n
        self.leaf[:n] = lut[self.leaf[:n].long() & 0xFFFF]
        return TreeResult("nonsymmetric", node_split=ns, leaf_of_node=leaf_of_node, n_leaves=len(terminal), leaf=self.leaf)


# ---------------------------------------------------------------------------------------------------------
def enforce_monotone_leaves(vals: np.ndarray, wts: np.ndarray, splits: np.ndarray, monotone_flat: np.ndarray) -> np.ndarray:
    """Repair the leaf values of an oblivious tree so that, for every level that splits a constrained feature, the leaf
    on the right of that split is not below (+1) / above (-1) its mirror leaf on the left: violating pairs are replaced
    by their weighted mean (pool-adjacent-violators on two elements), repeated until nothing moves."""
    vals = np.array(vals, dtype=np.float64, copy=True)
    w = np.maximum(np.asarray(wts, dtype=np.float64), 1e-12)
    levels = [(k, float(monotone_flat[int(splits[k, 0])])) for k in range(splits.shape[0])
              if splits[k, 0] >= 0 and monotone_flat[int(splits[k, 0])] != 0]
    if not levels:
        return vals
    idx = np.arange(vals.shape[0])
    for _ in range(4 * len(levels) + 4):
        moved = False
        for k, c in levels:
            lo = idx[(idx >> k) & 1 == 0]
            hi = lo | (1 << k)
            bad = c * (vals[hi, 0] - vals[lo, 0]) < -1e-15
            if bad.any():
                a, b = lo[bad], hi[bad]
                mean = (vals[a, 0] * w[a] + vals[b, 0] * w[b]) / (w[a] + w[b])
                vals[a, 0] = mean
                vals[b, 0] = mean
                moved = True
        if not moved:
            break
    return vals


_LANGEVIN_DRAWS = [0]
USE_LEAF_KERNEL = True        # False: the tensor formulation below also on the GPU (the oracle of the kernel path)
USE_NATIVE_CPU_LEAVES = True  # False: the tensor formulation also on the CPU (the oracle of cbc_leaf_newton)
USE_NATIVE_CPU_SCORES = True  # False: SplitScorer's tensor code scores symmetric levels on the CPU too (the oracle)


def estimate_leaves(objective, approx, target, weight, leaf, n_leaves, n, opts, ctx=None, obj_ctx=None,
                    total_weight: Optional[float] = None):
    """Leaf values [n_leaves, dims] (already multiplied by the learning rate) and leaf weights [n_leaves]."""
    method, iters = opts.leaf_estimation_method, int(opts.leaf_estimation_iterations)
    l2, lr = float(opts.l2_leaf_reg), float(opts.learning_rate)
    dims = approx.shape[0]
    dev = approx.device
    idx = leaf[:n].long() & 0xFFFF
    if method == "Exact":
        return _exact_leaves(objective, approx, target, weight, idx, n_leaves, n, lr, ctx)
    if (USE_LEAF_KERNEL and approx.is_cuda and dims == 1 and method in ("Newton", "Gradient") and objective.native_id is not None
            and not (ctx is not None and ctx.is_distributed) and not getattr(opts, "langevin", False)
            and not getattr(objective, "zero_mean_leaves", False) and leaf.dtype == torch.int16 and n_leaves <= 4096):
        # one-dimensional losses with a device formula: every step of the estimation in one cooperative launch, the same
        # kernel the symmetric-tree trainer uses (per-leaf sums in shared cells, the step taken on the device)
        p0, p1 = (float(x) for x in objective.native_params())
        out = ops.leaf_newton(int(objective.native_id), p0, p1, approx[0], target, None if weight is None else weight[:n],
                              leaf, n, n_leaves, max(1, iters), method == "Newton", l2, lr,
                              str(getattr(opts, "leaf_estimation_backtracking", None) or "No"))
        if out is not None:
            return out[0].double().unsqueeze(1).cpu().numpy(), out[1].cpu().numpy()
    if (USE_NATIVE_CPU_LEAVES and not approx.is_cuda and dims == 1 and method in ("Newton", "Gradient")
            and objective.native_id in (0, 1, 2, 3) and type(objective).__name__ in ("RMSE", "Logloss", "CrossEntropy", "Poisson")
            and not (ctx is not None and ctx.is_distributed) and not getattr(opts, "langevin", False)
            and not getattr(objective, "zero_mean_leaves", False) and leaf.dtype == torch.int16
            and str(getattr(opts, "leaf_estimation_backtracking", None) or "No") in ("No", "AnyImprovement", "Armijo")
            and approx.dtype == torch.float32 and target.dtype == torch.float32 and target.dim() == 1):
        # host losses with a closed formula: all steps in one native call (ops/cpu/cb_cpu.cpp cbc_leaf_newton)
        import ctypes
        from ..ops import native
        a0 = approx[0, :n].contiguous()
        tg = target[:n].contiguous()
        wt = None if weight is None else weight[:n].contiguous().float()
        lf = leaf[:n].contiguous()
        dl = np.zeros(n_leaves, dtype=np.float64)
        lw = np.zeros(n_leaves, dtype=np.float64)
        P = lambda t: ctypes.c_void_p(t.data_ptr())
        rc = native.cpu_lib().cbc_leaf_newton(
            ctypes.c_int(int(objective.native_id)), P(a0), P(tg), None if wt is None else P(wt), P(lf), ctypes.c_longlong(n),
            ctypes.c_int(int(n_leaves)), ctypes.c_int(max(1, iters)), ctypes.c_int(1 if method == "Newton" else 0),
            ctypes.c_double(l2),
            ctypes.c_int({"No": 0, "AnyImprovement": 1, "Armijo": 2}[str(getattr(opts, "leaf_estimation_backtracking", None) or "No")]),
            dl.ctypes.data_as(ctypes.c_void_p), lw.ctypes.data_as(ctypes.c_void_p))
        if rc == 0:
            return (dl * lr).reshape(-1, 1), lw
    delta = torch.zeros((n_leaves, dims), dtype=torch.float32, device=dev)
    wcol = torch.ones(n, dtype=torch.float32, device=dev) if weight is None else weight[:n]
    leaf_w = None
    # Step-length control (catboost/cuda/methods/leaves_estimation/descent_helpers.cpp:127-206, step_estimator.cpp): every
    # pass evaluates the loss at the point it takes its derivatives at; a point that fails the condition is dropped and
    # the next pass tries half the step from the last accepted point.  A rejected try uses up one iteration.
    mode = str(getattr(opts, "leaf_estimation_backtracking", None) or "No")
    wvec = weight if weight is None else weight[:n]
    backtrack = mode in ("AnyImprovement", "Armijo") and max(1, iters) > 1
    base, direction, f_base, dirgrad, cur_step = delta, torch.zeros_like(delta), None, 0.0, 1.0
    for it in range(max(1, iters)):
        a = approx[:, :n] if it == 0 else approx[:, :n] + delta[idx].t()
        if backtrack:
            v = _loss_sum(objective, a, target, wvec, obj_ctx, ctx)
            if v is None:
                backtrack = False
            elif it > 0 and not (v <= f_base - (1e-5 * cur_step * dirgrad if mode == "Armijo" else 0.0)):
                cur_step *= 0.5
                delta = base + cur_step * direction
                continue
        der, hess = objective.der_hess(a, target, wvec, obj_ctx)
        cols = torch.cat([der, hess, wcol.unsqueeze(0)], 0)
        sums = ops.leaf_sums(leaf, cols, n_leaves, n)
        if ctx is not None and ctx.is_distributed:
            ctx.all_reduce_sum_(sums)
        sd, sh, sw = sums[:, :dims], sums[:, dims:2 * dims], sums[:, 2 * dims]
        if leaf_w is None:
            leaf_w = sw.clone()
        if getattr(opts, "langevin", False) and float(opts.diffusion_temperature or 0.0) > 0.0:
            # Langevin boosting also perturbs the per-leaf derivative sums (catboost/private/libs/algo_helpers/
            # langevin_utils.cpp:79-142): rate * sqrt(|sum of second derivatives| + l2) for Newton steps,
            # rate * sqrt(leaf weight + l2) for gradient steps, rate = sqrt(2 / learning rate / temperature); leaves
            # without weight are left alone.  Every rank draws the same numbers (seeded by the iteration state).
            rate = math.sqrt(2.0 / lr / float(opts.diffusion_temperature))
            gen = torch.Generator(device="cpu")
            _LANGEVIN_DRAWS[0] += 1                       # the same sequence on every rank: they call in lockstep
            gen.manual_seed((int(opts.random_seed) * 1000003 + 7919 * _LANGEVIN_DRAWS[0]) & 0x7FFFFFFF)
            z = torch.randn((n_leaves, dims), generator=gen).to(dev)
            scale = torch.sqrt((sh.abs() if method == "Newton" else sw.unsqueeze(1).expand_as(sd)) + l2)
            sd = sd + torch.where(sw.unsqueeze(1) >= 1e-9, rate * scale * z, torch.zeros_like(sd)).to(sd.dtype)
        blocks = getattr(objective, "hess_blocks", None) if (method == "Newton" and dims > 1) else None
        if blocks is not None:
            # the K x K Hessian block of every leaf (catboost/cuda/methods/leaves_estimation/descent_helpers.cpp:91-117):
            # (H + l2 I) step = gradient
            H = blocks(a, target, wvec, idx, n_leaves)
            if ctx is not None and ctx.is_distributed:
                ctx.all_reduce_sum_(H)
            H = H + l2 * torch.eye(dims, dtype=H.dtype, device=H.device)
            step = torch.linalg.solve(H, sd.double().unsqueeze(-1)).squeeze(-1).float()
        else:
            den = (sh if method == "Newton" else sw.unsqueeze(1).expand_as(sd)) + l2
            step = torch.where(den > 0, sd / den, torch.zeros_like(sd)).float()
        if backtrack:
            base, direction, f_base, cur_step = delta, step, v, 1.0
            dirgrad = float((sd.double() * step.double()).sum().item())
        delta = delta + step
    if getattr(objective, "zero_mean_leaves", False):
        tot = leaf_w.sum().clamp_min(1e-30)
        delta = delta - ((delta.double() * leaf_w.unsqueeze(1)).sum(0) / tot).float()
    return (delta * lr).double().cpu().numpy(), leaf_w.cpu().numpy()


def _loss_sum(objective, a, target, weight, obj_ctx, ctx):
    """Weighted sum of the loss over all ranks at approx ``a`` (None when the objective has no finite value)."""
    import math
    try:
        if hasattr(objective, "_point") and a.shape[0] == 1:
            v = objective._point(a[0], target)[2]
            s = float((v if weight is None else v * weight).double().sum().item())
        else:
            wt = float(target.shape[-1] if weight is None else weight.sum().item())
            s = float(objective.value(a, target, weight, obj_ctx)) * wt
    except (NotImplementedError, RuntimeError, TypeError, IndexError):
        return None
    if not math.isfinite(s):
        return None
    if ctx is not None and ctx.is_distributed:
        t = torch.tensor([s], dtype=torch.float64, device=a.device)
        ctx.all_reduce_sum_(t)
        s = float(t.item())
    return s


def _exact_leaves(objective, approx, target, weight, idx, n_leaves, n, lr, ctx):
    """Weighted alpha-quantile of the residuals inside each leaf (MAE / Quantile / MAPE)."""
    alpha = float(objective.params.get("alpha", 0.5)) if objective.name == "Quantile" else 0.5
    res = (target - approx[0, :n]).double()
    w = torch.ones_like(res) if weight is None else weight[:n].double()
    if objective.name == "MAPE":
        w = w / target.abs().clamp_min(1.0).double()
    if ctx is not None and ctx.is_distributed:
        import torch.distributed as dist
        parts = ctx.all_gather_object((res.cpu(), w.cpu(), idx.cpu()))
        res = torch.cat([p[0] for p in parts]).to(approx.device)
        w = torch.cat([p[1] for p in parts]).to(approx.device)
        idx = torch.cat([p[2] for p in parts]).to(approx.device)
    if res.is_cuda:
        # one stable radix sort (ops/cuda/cb_sort.cu) by (leaf, residual): the residual's float32 bits mapped to integers
        # of the same order sit below the leaf number in a 64-bit key (catboost/cuda/methods/kernel/exact_estimation.cu
        # sorts per-leaf segments for the same purpose)
        bits = (res.float() + 0.0).contiguous().view(torch.int32).long()
        ordered = torch.where(bits < 0, bits ^ 0x7FFFFFFF, bits) + (1 << 31)
        _, order = ops.sort_pairs((idx.long() << 32) | ordered)
    else:
        order = torch.argsort(res, stable=True)
        order = order[torch.argsort(idx[order], stable=True)]
    li, r, ww = idx[order], res[order], w[order]
    cw = torch.cumsum(ww, 0)
    tot = torch.zeros(n_leaves, dtype=torch.float64, device=approx.device).index_add_(0, li, ww)
    counts = torch.bincount(li, minlength=n_leaves)
    starts = torch.cumsum(counts, 0) - counts
    base = torch.where(starts > 0, cw[(starts - 1).clamp_min(0)], torch.zeros_like(tot))
    thr = base + alpha * tot
    pos = torch.searchsorted(cw, thr, right=False)
    pos = torch.minimum(pos, (starts + counts - 1).clamp_min(0))
    vals = torch.where(counts > 0, r[pos.clamp(max=max(len(r) - 1, 0))], torch.zeros_like(tot))
    return (vals * lr).unsqueeze(1).cpu().numpy(), tot.cpu().numpy()
