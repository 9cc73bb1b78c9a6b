"""Pairwise structure search and leaf values for ``PairLogitPairwise`` / ``YetiRankPairwise``.

The pointwise losses score a split from per-leaf sums.  The pairwise ones score it from a quadratic model over ALL
leaves of the candidate tree at once (catboost/private/libs/algo/pairwise_scoring.cpp:123-260,
catboost/private/libs/algo_helpers/pairwise_leaves_calculation.cpp:9-60,
catboost/cuda/methods/pairwise_oblivious_trees/*): with pair weights ``h_p`` (second derivative of the pair loss) and
document derivatives ``d_i`` the gain of leaf values ``x`` is ``x.d - x'Mx / 2``, ``M`` the Laplacian of the pair graph
contracted to the leaves,  ``M = sum_p h_p (e_a - e_b)(e_a - e_b)'``  (a, b = leaves of the two documents of the pair).
For a candidate border every leaf splits in two, so each candidate has its own 2L x 2L system; the best ``x`` solves
``(M + reg) x = d`` with the last unknown pinned to zero (the system is singular along the constant vector) and is
shifted to zero mean afterwards.

Pairwise histograms.  For one feature the child of a document under border t is decided by ``bin > t``, so as t grows a
pair passes through three configurations: both right (t < lo), the document with the smaller bin left and the other
right (lo <= t < hi), both left (t >= hi) with lo / hi the smaller / larger bin of the pair.  Each configuration is a
range of borders, so the off-diagonal weights of all candidates of the feature are three range-updates per pair into a
difference array ``[borders + 1, 2L, 2L]`` followed by a prefix sum over the borders -- the same role as the reference's
pairwise histograms (4 values per bin, feature and leaf pair).  The systems of a feature are solved as one batch.

``PairwiseLearner`` is tensor code (batched solves through the framework, single rank): the CPU path and the oracle.
``PairwiseKernelLearner`` runs the same search as hand-written kernels (``ops/cuda/cb_pairwise.cu``: four pair histograms
per (feature, bin, leaf pair), bin prefix sums, one block per candidate that assembles the system, factorises it and
scores it) and sums the histograms over the ranks, so pairwise losses train on several GPUs.
"""
from __future__ import annotations

from typing import Optional, Tuple

import numpy as np
import torch

from .generic import TreeResult


def _solve_pairwise(M: torch.Tensor, d: torch.Tensor, l2: float, prior: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """Leaf values and gain of every system of a batch.  M [..., S, S] (Laplacian), d [..., S]; float64."""
    S = M.shape[-1]
    cell = 1.0 / S
    non_diag = -prior * cell
    diag = prior * (1.0 - cell) + l2
    A = M[..., :-1, :-1] + non_diag
    eye = torch.eye(S - 1, dtype=M.dtype, device=M.device)
    A = A + eye * (diag - non_diag + 1e-9)
    rhs = d[..., :-1].unsqueeze(-1)
    x = torch.linalg.solve(A, rhs).squeeze(-1)
    x = torch.cat([x, torch.zeros_like(x[..., :1])], -1)
    x = x - x.mean(-1, keepdim=True)
    gain = (x * d).sum(-1) - 0.5 * (x * (M @ x.unsqueeze(-1)).squeeze(-1)).sum(-1)
    return x, gain


class PairwiseLearner:
    """Symmetric trees for pairwise losses on one rank."""

    def __init__(self, store, opts, seed: int = 0):
        self.store, self.o = store, opts
        self.dev = store.bins.device
        F, n = store.F, store.n
        self.bins = torch.stack([store.column(f)[:n].long() for f in range(F)]) if F else torch.zeros((0, n), dtype=torch.long)
        self.nb = torch.from_numpy(store.feat_nb_host.astype(np.int64)).to(self.dev)
        self.onehot = store.feat_onehot.bool()
        self.leaf = torch.zeros(store.npad, dtype=torch.int16, device=self.dev)
        self.l2 = float(opts.l2_leaf_reg)
        self.prior = float(opts.bayesian_matrix_reg if opts.bayesian_matrix_reg is not None else 0.1)
        self.gen = torch.Generator(device="cpu")
        self.gen.manual_seed(int(seed) + 4242)

    # ------------------------------------------------------------------------------------------------------
    def _feature_scores(self, f: int, leaf: torch.Tensor, L: int, wi, li, h, der) -> torch.Tensor:
        """Gain of every border of feature f: [nb - 1] float64."""
        dev = self.dev
        nbf = int(self.nb[f].item())
        if bool(self.onehot[f].item()):
            return self._onehot_scores(f, leaf, L, wi, li, h, der, nbf)
        T = nbf - 1                                  # candidate borders t = 0 .. T-1, right child iff bin > t
        if T <= 0:
            return torch.zeros(0, dtype=torch.float64, device=dev)
        S = 2 * L
        b = self.bins[f]
        bi, bj = b[wi], b[li]
        lw, ll = leaf[wi], leaf[li]
        lo, hi = torch.minimum(bi, bj), torch.maximum(bi, bj)
        hd = h.double()
        off = torch.zeros((T + 1) * S * S, dtype=torch.float64, device=dev)

        def add_range(t0, t1, ca, cb, w):
            # +w on borders [t0, t1) of cell (ca, cb)
            t0c, t1c = t0.clamp(max=T), t1.clamp(max=T)
            cell = ca * S + cb
            off.index_add_(0, t0c * (S * S) + cell, w)
            off.index_add_(0, t1c * (S * S) + cell, -w)

        zero = torch.zeros_like(lo)
        # both right: t < lo
        add_range(zero, lo, lw + L, ll + L, hd)
        # split: lo <= t < hi; the document with the smaller bin has gone left
        i_left = bi < bj
        ca = torch.where(i_left, lw, lw + L)
        cb = torch.where(i_left, ll + L, ll)
        add_range(lo, hi, ca, cb, hd)
        # both left: t >= hi
        add_range(hi, torch.full_like(hi, T), lw, ll, hd)
        W = off.view(T + 1, S, S)[:T].cumsum(0)
        W = W + W.transpose(1, 2)
        M = torch.diag_embed(W.sum(-1)) - W
        # derivative sums of the children
        dd = torch.zeros((T + 1) * S, dtype=torch.float64, device=dev)
        n = der.shape[0]
        lf = leaf[:n]
        bd = b.clamp(max=T)
        derd = der.double()
        dd.index_add_(0, lf + L, derd)                          # t = 0: everything with bin > 0 ... start all right
        dd.index_add_(0, bd * S + lf + L, -derd)                # from t = bin on the document is left
        dd.index_add_(0, bd * S + lf, derd)
        D = dd.view(T + 1, S)[:T].cumsum(0)
        _, gain = _solve_pairwise(M, D, self.l2, self.prior)
        return gain

    def _onehot_scores(self, f, leaf, L, wi, li, h, der, nbf) -> torch.Tensor:
        """Gain of every value of a one-hot feature (right child iff bin == value), one system per value."""
        S = 2 * L
        b = self.bins[f]
        n = der.shape[0]
        gains = []
        for v in range(nbf):
            child = leaf[:n] + (b[:n] == v).long() * L
            W = torch.zeros(S * S, dtype=torch.float64, device=self.dev)
            W.index_add_(0, child[wi] * S + child[li], h.double())
            W = W.view(S, S)
            W = W + W.t()
            M = torch.diag(W.sum(-1)) - W
            D = torch.zeros(S, dtype=torch.float64, device=self.dev).index_add_(0, child, der.double())
            gains.append(_solve_pairwise(M, D, self.l2, self.prior)[1])
        return torch.stack(gains) if gains else torch.zeros(0, dtype=torch.float64, device=self.dev)

    def build_tree(self, wi, li, h, der, iteration: int, random_strength: float = 0.0) -> TreeResult:
        """wi / li: winner / loser document of every pair; h: pair weights; der: per-document derivative [n]."""
        o = self.o
        depth = int(o.depth)
        n = self.store.n
        F = self.store.F
        splits = np.full((depth, 4), 0, dtype=np.int32)
        splits[:, 0] = -1
        leaf = torch.zeros(n, dtype=torch.long, device=self.dev)
        fw = self.store.feat_weight
        for level in range(depth):
            L = 1 << level
            best = (-float("inf"), -1, -1)
            for f in range(F):
                if float(fw[f].item()) <= 0:
                    continue
                gain = self._feature_scores(f, leaf, L, wi, li, h, der)
                if gain.numel() == 0:
                    continue
                if random_strength > 0:
                    gain = gain + torch.randn(gain.shape, generator=self.gen, dtype=torch.float64).to(self.dev) * random_strength
                gain = gain * float(fw[f].item())
                v, t = torch.max(gain, 0)
                if float(v.item()) > best[0]:
                    best = (float(v.item()), f, int(t.item()))
            if best[1] < 0 or not np.isfinite(best[0]):
                break
            _, f, t = best
            oh = bool(self.onehot[f].item())
            splits[level] = (f, t, 0, 1 if oh else 0)
            leaf = leaf + ((self.bins[f] == t) if oh else (self.bins[f] > t)).long() * L
        self.leaf.zero_()
        self.leaf[:n] = leaf.to(torch.int16)
        return TreeResult("oblivious", splits=splits, n_leaves=1 << depth, leaf=self.leaf)

    def leaf_values(self, leaf_count: int, wi, li, h, der, lr: float):
        """Pairwise leaf values of the finished tree (already multiplied by the learning rate) and leaf weights."""
        n = self.store.n
        lf = self.leaf[:n].long() & 0xFFFF
        S = leaf_count
        W = torch.zeros(S * S, dtype=torch.float64, device=self.dev)
        W.index_add_(0, lf[wi] * S + lf[li], h.double())
        W = W.view(S, S)
        W = W + W.t()
        M = torch.diag(W.sum(-1)) - W
        d = torch.zeros(S, dtype=torch.float64, device=self.dev).index_add_(0, lf, der.double())
        cnt = torch.bincount(lf, minlength=S).double()
        if S < 2:
            return np.zeros((S, 1)), cnt.cpu().numpy()
        x, _ = _solve_pairwise(M, d, self.l2, self.prior)
        return (x * lr).unsqueeze(1).cpu().numpy(), cnt.cpu().numpy()


class PairwiseKernelLearner(PairwiseLearner):
    """The same search on the GPU with the kernels of ``cb_pairwise.cu``; histograms are summed over the ranks (queries
    are never split between ranks, so every pair is local to one of them).  Leaf values of the finished tree come from
    one more system over the final leaves, assembled from a pair histogram without a feature dimension."""

    H_BUDGET_BYTES = 1 << 30
    USE_SORTED_PAIRS = True        # False: deep levels through global atomics (the oracle of the sorted-pair kernel)

    def __init__(self, store, opts, seed: int = 0, ctx=None):
        self.store, self.o = store, opts
        self.dev = store.bins.device
        self.ctx = ctx
        self.leaf = torch.zeros(store.npad, dtype=torch.int16, device=self.dev)
        self.l2 = float(opts.l2_leaf_reg)
        self.prior = float(opts.bayesian_matrix_reg if opts.bayesian_matrix_reg is not None else 0.1)
        self.gen = torch.Generator(device="cpu")
        self.gen.manual_seed(int(seed) + 4242)
        self.onehot = store.feat_onehot.bool()
        self.bins = None                                 # the kernels read the packed store directly
        self.B = max(4, (store.max_bins + 3) // 4 * 4)

    def _reduce(self, t):
        if self.ctx is not None and self.ctx.is_distributed:
            self.ctx.all_reduce_sum_(t)

    def level_gains(self, L: int, wi, li, h, der_pad) -> torch.Tensor:
        """Gain of every candidate of the level: float32 [F_padded_to_groups, B] (-inf where there is none)."""
        import ctypes
        from ..ops import native
        lib, st = native.cuda_lib(), self.store
        G, B = st.G, self.B
        per_group = 4 * B * L * L * 4 * 4
        ng_max = max(1, min(G, self.H_BUDGET_BYTES // per_group))
        gains = torch.full((G * 4, B), -float("inf"), dtype=torch.float32, device=self.dev)
        stream = ctypes.c_void_p(torch.cuda.current_stream(self.dev).cuda_stream)
        p = lambda t: ctypes.c_void_p(t.data_ptr())
        grid = 148 * 8
        wi32, li32 = wi.to(torch.int32).contiguous(), li.to(torch.int32).contiguous()
        h32 = h.to(torch.float32).contiguous()
        # the largest pair weight scales the fixed-point cells of the shared-memory histogram kernel (shallow levels)
        wmax = float(h32.abs().max().item()) if h32.numel() else 0.0
        if lib.cb_pair_solve_smem_bytes(L) > 227 * 1024:
            raise RuntimeError("too many leaves for the pairwise solve kernel")
        # Deep levels (the L x L cells of a feature group no longer fit in shared memory): the pairs are sorted by leaf pair once
        # per level (the hand-written radix sort) and cut into chunks that share one cell, see cb_pair_hist_sorted_kernel
        sorted_pairs = None
        if wmax > 0.0 and 4 * B * L * L * 16 > 96 * 1024 and B <= 256 and wi32.numel() > 0 and self.USE_SORTED_PAIRS:
            from ..ops import api as ops
            key = self.leaf[wi].long() * L + self.leaf[li].long()
            _, order = ops.sort_pairs(key)
            counts = torch.bincount(key, minlength=L * L).cpu().numpy()
            chunk = int(lib.cb_pair_chunk_pairs())
            rows, begin = [], 0
            for cell, c in enumerate(counts.tolist()):
                for b in range(0, c, chunk):
                    rows.append((begin + b, begin + min(c, b + chunk), cell, 0))
                begin += c
            table = torch.tensor(rows, dtype=torch.int32, device=self.dev).contiguous()
            sorted_pairs = (wi32[order].contiguous(), li32[order].contiguous(), h32[order].contiguous(), table)
        for g0 in range(0, G, ng_max):
            ng = min(ng_max, G - g0)
            H = torch.zeros(ng * 4 * B * L * L * 4, dtype=torch.float32, device=self.dev)
            D = torch.zeros(ng * 4 * B * L, dtype=torch.float32, device=self.dev)
            if sorted_pairs is not None:
                ws, ls, hs, table = sorted_pairs
                native.cuda_check(lib.cb_pair_hist_sorted(ctypes.c_void_p(st.handle), p(ws), p(ls), p(hs), int(ws.numel()),
                                                          p(table), int(table.shape[0]), L, B, g0, ng, p(H), wmax, stream),
                                  "cb_pair_hist_sorted")
            # (with sorted pairs only the derivative histograms are left for this call)
            native.cuda_check(lib.cb_pair_hist(ctypes.c_void_p(st.handle), p(self.leaf), p(wi32), p(li32), p(h32),
                                               0 if sorted_pairs is not None else int(wi32.numel()), p(der_pad), L, B, g0, ng,
                                               p(H), p(D), wmax, grid, stream), "cb_pair_hist")
            self._reduce(H)
            self._reduce(D)
            native.cuda_check(lib.cb_pair_scan(ctypes.c_void_p(st.handle), g0 * 4, ng * 4, L, B, p(H), p(D), grid, stream),
                              "cb_pair_scan")
            nf = min(ng * 4, st.F - g0 * 4)
            out = gains[g0 * 4: g0 * 4 + nf]
            native.cuda_check(lib.cb_pair_solve(ctypes.c_void_p(st.handle), p(H), p(D), g0 * 4, nf, L, B, self.l2, self.prior,
                                                p(out), stream), "cb_pair_solve")
            del H, D
        return gains[: st.F]

    def build_tree(self, wi, li, h, der, iteration: int, random_strength: float = 0.0) -> TreeResult:
        from ..ops import api as ops
        depth = int(self.o.depth)
        st = self.store
        splits = np.full((depth, 4), 0, dtype=np.int32)
        splits[:, 0] = -1
        self.leaf.zero_()
        der_pad = torch.zeros(st.npad, dtype=torch.float32, device=self.dev)
        der_pad[: st.n] = der.float()
        for level in range(depth):
            gains = self.level_gains(1 << level, wi, li, h, der_pad)
            if random_strength > 0:
                noise = torch.randn(gains.shape, generator=self.gen, dtype=torch.float32).to(self.dev) * random_strength
                gains = torch.where(torch.isfinite(gains), gains + noise * st.feat_weight.unsqueeze(1), gains)
            flat = int(torch.argmax(gains.reshape(-1)).item())
            f, t = flat // gains.shape[1], flat % gains.shape[1]
            if not np.isfinite(float(gains[f, t].item())):
                break
            oh = bool(self.onehot[f].item())
            splits[level] = (f, t, 0, 1 if oh else 0)
            ops.update_leaf(st, self.leaf, f, t, oh, level)
        return TreeResult("oblivious", splits=splits, n_leaves=1 << depth, leaf=self.leaf)

    def leaf_values(self, leaf_count: int, wi, li, h, der, lr: float):
        n = self.store.n
        lf = self.leaf[:n].long() & 0xFFFF
        S = leaf_count
        W = torch.zeros(S * S, dtype=torch.float64, device=self.dev)
        W.index_add_(0, lf[wi] * S + lf[li], h.double())
        d = torch.zeros(S, dtype=torch.float64, device=self.dev).index_add_(0, lf, der.double())
        cnt = torch.bincount(lf, minlength=S).double()
        self._reduce(W)
        self._reduce(d)
        self._reduce(cnt)
        W = W.view(S, S)
        W = W + W.t()
        M = torch.diag(W.sum(-1)) - W
        if S < 2:
            return np.zeros((S, 1)), cnt.cpu().numpy()
        x, _ = _solve_pairwise(M, d, self.l2, self.prior)
        return (x * lr).unsqueeze(1).cpu().numpy(), cnt.cpu().numpy()
