"""Device-resident trainer for symmetric (oblivious) trees with a one-dimensional pointwise objective.

One boosting iteration is a fixed sequence of launches with no host read anywhere, captured once in a CUDA graph
and replayed:

    derivatives (+ cursor update by the previous tree, + bootstrap weights)
    depth x fused level kernel  (leaf update -> histograms -> cross-GPU reduce-scatter -> score -> argmax)
    final leaf update
    leaf_estimation_iterations x leaf pass (per-leaf sums -> cross-GPU sum -> Newton / gradient step)
    evaluation sets: apply the new tree + metric sums
    bookkeeping (learn loss history, iteration counter)

The reference drives the same steps from the host with two blocking device->host reads per level
(catboost/cuda/methods/oblivious_tree_doc_parallel_structure_searcher.cpp:63-164) and bounces every
leaf-estimation step through the CPU (leaves_estimation/descent_helpers.cpp:127-206).

Multi-GPU: doc-parallel; each rank holds a row shard and all features.  ``reduce='fused'`` uses the in-kernel
peer-store reduce-scatter; ``reduce='nccl'`` is the baseline (stand-alone kernels + NCCL all-reduce).
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional

import numpy as np
import torch

from ..data.quantization import BinnedStore
from ..ops import native
from ..parallel.runtime import ArenaLayout, DistContext, PeerArena, split_columns

SCORE_FN = {"Cosine": (0, 0), "L2": (1, 0), "NewtonCosine": (0, 1), "NewtonL2": (1, 1), "SolarL2": (2, 0),
            "LOOL2": (3, 0), "SatL2": (4, 0)}
BOOTSTRAP = {"No": 0, "Bayesian": 1, "Bernoulli": 2, "Poisson": 3, "MVS": 0}      # MVS: its own kernel after the gradients


def _p(t):
    if t is None:
        return None
    return ctypes.c_void_p(t.data_ptr())


class EvalSet:
    def __init__(self, store: BinnedStore, target: torch.Tensor, weight: Optional[torch.Tensor], approx0: torch.Tensor):
        self.store, self.target, self.weight = store, target, weight
        self.approx = approx0


class GpuObliviousEngine:
    def __init__(self, store: BinnedStore, target: torch.Tensor, weight: Optional[torch.Tensor], approx0: torch.Tensor,
                 objective, *, depth: int, iterations: int, learning_rate: float,
                 l2_leaf_reg: float, score_function: str = "Cosine", random_strength: float = 1.0,
                 bootstrap_type: str = "Bayesian", bootstrap_param: float = 1.0, leaf_method: str = "Newton",
                 leaf_iterations: int = 1, seed: int = 0, ctx: Optional[DistContext] = None, reduce: str = "fused",
                 eval_sets: Optional[List[EvalSet]] = None, use_graph: bool = True, threads: int = 512,
                 ext_der: Optional[torch.Tensor] = None, ext_hess: Optional[torch.Tensor] = None,
                 timeout_s: float = 20.0, quantized_hist: bool = True, dynamic_work: bool = True,
                 der_fn=None, zero_mean_leaves: bool = False, max_bundle: int = 8,
                 fused_leaf_steps: bool = True, mvs_reg=None, leaf_backtracking: str = "AnyImprovement",
                 fuse_leaf_update: bool = True, dims: int = 1, skip_dominant_bin: bool = True):
        assert store.bins.is_cuda, "GpuObliviousEngine needs a CUDA store"
        if depth > 16:
            raise ValueError("depth must be <= 16")
        self.lib = native.cuda_lib()
        self.store = store
        self.dev = store.bins.device
        self.ctx = ctx or DistContext(0, 1, self.dev)
        self.ctx.device = self.dev
        self.R, self.rank = self.ctx.world, self.ctx.rank
        self.depth, self.iterations = depth, iterations
        self.lr, self.l2 = float(learning_rate), float(l2_leaf_reg)
        self.score_fn, self.newton_stats = SCORE_FN[score_function]
        self.random_strength = float(random_strength)
        self.boot_type, self.boot_p = BOOTSTRAP[bootstrap_type], float(bootstrap_param)
        # minimal-variance sampling: sampling weights from the finished derivatives, block by block (ops/cuda/cb_mvs.cu)
        self.mvs = bootstrap_type == "MVS" and float(bootstrap_param) < 1.0
        self.mvs_reg = -1.0 if mvs_reg is None else float(mvs_reg)
        if self.mvs and dims > 1:
            raise ValueError("MVS sampling on the device trainer covers one-dimensional losses")
        self.leaf_newton = 1 if leaf_method == "Newton" else 0
        self.leaf_iterations = max(1, int(leaf_iterations))
        self.objective = objective
        self.loss_id = int(objective.native_id) if objective.native_id is not None else 100
        self.p0, self.p1 = (float(x) for x in objective.native_params())
        self.seed = (int(seed) * 0x9E3779B97F4A7C15 + 0x1234567 * (self.rank + 1)) & 0xFFFFFFFFFFFFFFFF
        self.score_seed = (int(seed) * 0xD1B54A32D192ED03 + 77) & 0xFFFFFFFFFFFFFFFF
        self.reduce = reduce if self.R > 1 else "fused"
        if self.R > 1 and self.reduce == "fused" and not self.ctx.single_host:
            self.reduce = "nccl"          # ranks on several machines: no peer-mapped arena, histograms go through NCCL
        self.use_graph = use_graph
        # False: fp32 shared atomics; "wide": 23-bit fixed point in two int32 cells; True / "narrow": one int32 cell
        self.quantized_hist = bool(quantized_hist)
        self.narrow_hist = self.quantized_hist and quantized_hist != "wide"
        self.max_bundle = int(max_bundle)
        self.dynamic_work = bool(dynamic_work)
        self.threads = threads
        self.eval_sets = eval_sets or []
        self.ext_der, self.ext_hess = ext_der, ext_hess
        # Objectives without a device formula (query-wise ranking losses, Python objectives): der_fn(cursor[n]) returns
        # (der[n], hess[n]) device tensors; they are written into the external-derivative rows before every tree.  The
        # iteration then contains framework ops, so it is not captured into a graph.
        self.der_fn = der_fn
        self.zero_mean_leaves = bool(zero_mean_leaves)
        if der_fn is not None:
            self.loss_id = 100
            self.use_graph = False
            self.ext_der = torch.zeros(store.npad, dtype=torch.float32, device=self.dev)
            self.ext_hess = torch.zeros(store.npad, dtype=torch.float32, device=self.dev)
        n, npad, dev = store.n, store.npad, self.dev
        self.n, self.npad = n, npad
        # K > 1: MultiClass.  K derivative columns + one weight column drive the same level kernels; the cursor, the leaf
        # values and the model rows get K entries per document / leaf
        self.K = K = int(dims)
        if K > 1:
            if K > int(self.lib.cb_mc_max_classes()):
                raise ValueError("too many classes for the device trainer")
            if der_fn is not None or ext_der is not None:
                raise ValueError("external derivatives are one-dimensional")
            if not self.quantized_hist:
                self.quantized_hist, self.narrow_hist = True, False       # no fp32-atomic path for K + 1 statistics
        self.S = K + 1
        self.L = 1 << depth
        f32, i32, i64, f64 = torch.float32, torch.int32, torch.int64, torch.float64
        if K > 1:
            self.approx = torch.zeros((K, npad), dtype=f32, device=dev)
            self.approx[:, :n] = approx0.to(dev, f32).reshape(K, n)
        else:
            self.approx = torch.zeros(npad, dtype=f32, device=dev)
            self.approx[:n] = approx0.to(dev, f32).reshape(-1)
        self.target = torch.zeros(npad, dtype=f32, device=dev)
        self.target[:n] = target.to(dev, f32)
        self.weight = None
        self.weight_max = 1.0          # largest document weight over all ranks (scale of the fixed-point leaf cells)
        if weight is not None:
            self.weight = torch.zeros(npad, dtype=f32, device=dev)
            self.weight[:n] = weight.to(dev, f32)
            wm = self.weight.max().reshape(1).double()
            if ctx is not None and ctx.is_distributed:
                import torch.distributed as dist
                dist.all_reduce(wm, op=dist.ReduceOp.MAX, group=ctx.group)
            self.weight_max = max(float(wm.item()), 1e-30)
        self.leaf = torch.zeros(npad, dtype=torch.int16, device=dev)
        self.leaf_vmax = torch.zeros(2, dtype=f32, device=dev)
        self.leaf_grid = None
        self.fused_leaf_steps = bool(fused_leaf_steps)
        self.leaf_backtracking = {"No": 0, "AnyImprovement": 1, "Armijo": 2}[str(leaf_backtracking or "AnyImprovement")]
        self.fuse_leaf_update = bool(fuse_leaf_update)
        self._check_each = os.environ.get("CB200_CHECK") == "1"      # invariants after every iteration (slow, debugging)
        self.skip_dominant_bin = bool(skip_dominant_bin) and os.environ.get("CB200_SKIP_DOMINANT", "1") != "0"
        self.stats = torch.zeros((self.S, npad), dtype=f32, device=dev)
        self.scal = torch.zeros(4, dtype=f64, device=dev)
        self.iter_ptr = torch.zeros(1, dtype=i32, device=dev)
        cap = max(1, iterations)
        self.loss_hist = torch.zeros((cap, 2), dtype=f64, device=dev)
        self.splits = torch.full((cap * depth, 4), 0, dtype=i32, device=dev)
        self.splits[:, 0] = -1
        self.model_vals = torch.zeros((cap, self.L * K), dtype=f32, device=dev)
        self.model_wts = torch.zeros((cap, self.L), dtype=f32, device=dev)
        self.cur_vals = torch.zeros(self.L * K, dtype=f32, device=dev)
        self.delta = torch.zeros(self.L * K, dtype=f32, device=dev)
        self.leaf_w = torch.zeros(self.L, dtype=f32, device=dev)
        # three rotating copies of the per-leaf (der, hess, weight) sums + the loss sum
        self.sums = torch.zeros(max(self.L * 9, int(self.lib.cb_leaf_newton_sums_doubles(self.L)),
                                    int(self.lib.cb_mc_leaf_sums_doubles(K, self.L)) if K > 1 else 0), dtype=f64, device=dev)
        self.sums_combined = torch.zeros_like(self.sums) if K > 1 else None
        self.counter = torch.zeros(1, dtype=i32, device=dev)
        self.best_key = torch.zeros(1, dtype=i64, device=dev)
        self.cur_loss = torch.zeros(2, dtype=f64, device=dev)
        self.statmax = torch.zeros(self.S, dtype=f32, device=dev)
        msg_bytes = self.lib.cb_select_msg_bytes()
        self.msg_local = torch.zeros((max(self.R, 1), msg_bytes // 8 + 1), dtype=i64, device=dev)
        self.msg_all = torch.zeros((max(self.R, 1), msg_bytes // 8 + 1), dtype=i64, device=dev)
        self.mask = [torch.zeros(1024, dtype=i32, device=dev) for _ in range(2)]
        n_eval = len(self.eval_sets)
        self.eval_scal = torch.zeros(max(1, 2 * n_eval), dtype=f64, device=dev)
        self.eval_hist = torch.zeros((cap, max(1, 2 * n_eval)), dtype=f64, device=dev)
        # geometry ---------------------------------------------------------------------------------------
        TB = store.TB
        self.TB = TB
        self.B = max(4, (store.max_bins + 3) // 4 * 4)
        slots_max = 1 if depth <= 1 else 1 << (depth - 2)
        self.slots_max = slots_max
        if self.R > 1 and self.reduce == "fused":
            fb, cb = split_columns(store.feat_off_host, self.R)
        else:
            fb, cb = [0] + [store.F] * self.R, [0] + [TB] * self.R
            if self.R == 1:
                fb, cb = [0, store.F], [0, TB]
        self.feat_bounds, self.col_bounds = fb, cb
        if self.R > 1 and self.reduce == "fused":
            self.Wmax = max(4, max(cb[r + 1] - cb[r] for r in range(self.R)))
        else:
            self.Wmax = TB
        hl = 1 if depth <= 1 else 1 << (depth - 2)      # leaves kept for the sibling subtraction
        self.hbuf = [torch.zeros((hl * 2, self.S, self.Wmax), dtype=f32, device=dev) for _ in range(2)]
        # several ranks: the slots hold tagged 8-byte words (value + level tag), so twice the floats; a mailbox slot must
        # hold the largest tagged message (split key + lighter-child mask, or the per-leaf sums of a Newton step)
        slot_floats = slots_max * self.S * self.Wmax * (2 if self.R > 1 else 1)
        select_words = 2 + max(1, (1 << max(depth - 1, 0)) // 32)
        mbox_bytes = max(msg_bytes, 256, 8 * select_words,
                         int(self.lib.cb_leaf_newton_msg_bytes(self.L)) if self.L <= 4096 else 0,
                         int(self.lib.cb_mc_leaf_msg_bytes(K, self.L)) if (K > 1 and self.L <= 1024) else 0)
        self.arena = (PeerArena(self.ctx, ArenaLayout(self.R, mbox_bytes, slot_floats), timeout_s=timeout_s)
                      if self.reduce == "fused" else None)
        if self.reduce == "fused":
            self.slots = self.arena.local_slots_tensor()
            self.partial = None
            self.priv = None
            self._make_plan()
        else:
            self.partial = torch.zeros((slots_max * self.S, TB), dtype=f32, device=dev)
            self.slots = None
            self.plan = None
            # leaf sums across ranks go through NCCL in this mode
        sm = ctypes.c_int(0)
        smem = ctypes.c_int(0)
        native.cuda_check(self.lib.cb_device_info(ctypes.byref(sm), ctypes.byref(smem)), "cb_device_info")
        self.sm_count, self.max_smem = sm.value, smem.value
        self.grid_stream = self.sm_count * 8
        self.graph = None
        self.done = 0
        self._warmed = False
        self.launches_per_iter = 0

    # ------------------------------------------------------------------------------------------------------
    def _make_plan(self):
        R = self.R
        arr = ctypes.c_void_p * R
        local_slots = arr(*[self.arena.local_slot_ptr(r) for r in range(R)])
        own = (ctypes.c_int * (R + 1))(*self.col_bounds)
        partial_ptr = None
        self.plan = self.lib.cb_fused_create(
            ctypes.c_void_p(self.store.handle), ctypes.c_void_p(self.arena.handle), _p(self.leaf), _p(self.stats),
            self.S, self.B, partial_ptr, local_slots, _p(self.hbuf[0]), _p(self.hbuf[1]), own, self.Wmax,
            _p(self.mask[0]), _p(self.mask[1]), _p(self.splits), self.depth, self.l2, self.score_fn,
            self.random_strength, _p(self.scal), _p(self.iter_ptr), self.score_seed, self.lr, _p(self.best_key),
            _p(self.msg_local), _p(self.msg_all), self.msg_all.stride(0), self.threads)
        if not self.plan:
            raise RuntimeError("cb_fused_create failed")
        self.lib.cb_fused_set_features(ctypes.c_void_p(self.plan), self.feat_bounds[self.rank],
                                       self.feat_bounds[self.rank + 1])
        # fixed-point accumulation is on: statmax must be known to the geometry (it doubles the tile size)
        self.lib.cb_fused_set_priv(ctypes.c_void_p(self.plan), None, _p(self.statmax) if self.quantized_hist else None)
        self.lib.cb_fused_set_narrow(ctypes.c_void_p(self.plan), 1 if self.narrow_hist else 0, self.max_bundle)
        if os.environ.get("CB200_UNIFORM_BINS") != "1":
            # bins of the widest feature of every group: bundles of narrow columns (CTR, one-hot, binary) get small tiles
            nbp = np.full(self.store.G * 4, 4, dtype=np.int64)
            nbp[: self.store.F] = (np.asarray(self.store.feat_nb_host, dtype=np.int64) + 3) // 4 * 4
            gbins = np.ascontiguousarray(np.maximum(4, nbp.reshape(-1, 4).max(1)).astype(np.int32))
            self.lib.cb_fused_set_group_bins(ctypes.c_void_p(self.plan), gbins.ctypes.data_as(ctypes.c_void_p), int(len(gbins)))
            self.group_bins = gbins
        self.lib.cb_fused_set_fuse_leaf(ctypes.c_void_p(self.plan), 1 if self.fuse_leaf_update else 0)
        # columns where one bin holds a large share of the documents (sparse data): most lanes of a warp would add to
        # the same histogram cell, so such data gets up to 8 replicas of every cell instead of 2 (measured on 60 % zeros:
        # 6.8 -> 4.9 ms per iteration; on dense data more replicas cost about 1 %)
        self.dominant_bin_share, self.domw = self._dominant_bins()
        if not (self.narrow_hist and self.S == 2 and self.skip_dominant_bin):
            self.domw = None
        gate = float(os.environ.get("CB200_DOMINANT_GATE", "0.25"))
        if self.domw is not None and self.dominant_bin_share > gate:
            # sparse data: most (document, feature) pairs would hit one hot cell per feature; those are skipped and the
            # cell is restored from per-slot totals
            self.lib.cb_fused_set_dominant(ctypes.c_void_p(self.plan), _p(self.domw))
        else:
            self.domw = None
            if self.dominant_bin_share > gate:
                self.lib.cb_fused_set_max_copies(ctypes.c_void_p(self.plan), 8)
        self.work = torch.zeros(self.store.G + 1, dtype=torch.int32, device=self.dev)
        if self.dynamic_work:
            self.lib.cb_fused_set_work(ctypes.c_void_p(self.plan), _p(self.work))
        self.level_geo = []
        for level in range(self.depth):
            spp, smem, thr, nk, cp, bd = (ctypes.c_int(0) for _ in range(6))
            grid = self.lib.cb_fused_geometry(ctypes.c_void_p(self.plan), level, ctypes.byref(spp), ctypes.byref(smem),
                                              ctypes.byref(thr), ctypes.byref(nk), ctypes.byref(cp), ctypes.byref(bd))
            if grid <= 0:
                raise RuntimeError(f"no cooperative launch geometry for level {level}")
            self.level_geo.append((grid, spp.value, smem.value, thr.value, nk.value, cp.value, bd.value))
        # private tiles: one region per (chunk, group) work item, sized for the largest level
        G = self.store.G
        need = 0
        for level, geo in enumerate(self.level_geo):
            nslots = 1 if level == 0 else 1 << (level - 1)
            need = max(need, G * geo[4] * nslots * self.S * 4 * self.B)
        self.priv = torch.empty(need, dtype=torch.float32, device=self.dev)
        self.lib.cb_fused_set_priv(ctypes.c_void_p(self.plan), _p(self.priv),
                                   _p(self.statmax) if self.quantized_hist else None)

    def enable_phase_timing(self):
        """Record globaltimer stamps of the fused kernel's phases (block 0) for every level of the latest tree."""
        self.phase_ts = torch.zeros(self.depth * 8 + 2 * 4096 + self.depth * 4, dtype=torch.int64, device=self.dev)
        self.lib.cb_fused_set_phase_ts(ctypes.c_void_p(self.plan), _p(self.phase_ts))

    def phase_times_us(self):
        """[depth][6] microseconds: leaf update, histogram, wait for grid, reduce+push(+peer wait), score, select."""
        t = self.phase_ts[: self.depth * 8].view(self.depth, 8).cpu().numpy().astype(np.float64)
        return (t[:, 1:7] - t[:, 0:6]) / 1000.0

    def score_phase_times_us(self):
        """[depth][3] microseconds inside the score phase of block 0: noise scale, first accumulate, until its end."""
        t = self.phase_ts[: self.depth * 8].view(self.depth, 8).cpu().numpy().astype(np.float64)
        s = self.phase_ts[self.depth * 8 + 8192:].view(self.depth, 4).cpu().numpy().astype(np.float64)
        return np.stack([s[:, 0] - t[:, 4], s[:, 1] - s[:, 0], s[:, 2] - s[:, 1]], 1) / 1000.0

    def block_finish_times(self):
        """(histogram end time relative to the level start in us, SM id) per block at level depth-2."""
        raw = self.phase_ts.cpu().numpy()
        grid = self.level_geo[self.depth - 2][0]
        t0 = raw[(self.depth - 2) * 8 + 1]
        blk = raw[self.depth * 8: self.depth * 8 + 2 * grid].reshape(grid, 2)
        return (blk[:, 0] - t0) / 1000.0, blk[:, 1]

    def _stream(self):
        return ctypes.c_void_p(torch.cuda.current_stream(self.dev).cuda_stream)

    # ------------------------------------------------------------------------------------------------------
    def _grad(self):
        chk = native.cuda_check
        if self.K > 1:
            chk(self.lib.cb_mc_grad(_p(self.approx), _p(self.target), _p(self.weight), _p(self.leaf), _p(self.cur_vals),
                                    self.n, self.npad, self.K, _p(self.stats), self.newton_stats, self.boot_type, self.boot_p,
                                    self.seed, _p(self.iter_ptr), _p(self.scal), _p(self.statmax), self.grid_stream,
                                    self._stream()), "cb_mc_grad")
            self.launches_per_iter += 1
            return
        chk(self.lib.cb_grad_pointwise(self.loss_id, self.p0, self.p1, _p(self.approx), _p(self.target), _p(self.weight),
                                       _p(self.leaf), _p(self.cur_vals), self.n, self.npad, _p(self.stats),
                                       self.newton_stats, self.boot_type, self.boot_p, self.seed, _p(self.iter_ptr),
                                       _p(self.scal), _p(self.ext_der), _p(self.ext_hess), _p(self.statmax),
                                       self.grid_stream, self._stream()), "cb_grad_pointwise")
        self.launches_per_iter += 1
        if self.mvs:
            chk(self.lib.cb_mvs_sample(_p(self.stats), self.npad, self.n, self.boot_p, self.mvs_reg, self.seed,
                                       _p(self.iter_ptr), _p(self.statmax) if self.quantized_hist else None, None,
                                       self._stream()), "cb_mvs_sample")
            self.launches_per_iter += 1

    def _dominant_bins(self, sample: int = 65536):
        """(mean share of the most frequent bin over the features, packed dominant bins per feature group or None).

        Counted on a strided sample of this rank's rows and summed over the ranks, so every rank takes the same
        decision.  A feature gets a dominant bin when at least 30 % of the sampled documents share one bin; the packed
        word of a group holds 255 for its other features."""
        st = self.store
        if st.n <= 0 or st.F <= 0:
            return 0.0, None
        G = st.bins.shape[0]
        step = max(1, st.n // sample)
        rows = st.bins[:, : st.n: step].contiguous()
        m = rows.shape[1]
        b = rows.view(torch.uint8).view(G, m, 4).permute(0, 2, 1).reshape(G * 4, m)
        idx = b.long() + (torch.arange(G * 4, device=b.device) * 256).unsqueeze(1)
        cnt = torch.bincount(idx.reshape(-1), minlength=G * 4 * 256).view(G * 4, 256).double()
        tot = torch.tensor([float(m)], dtype=torch.float64, device=b.device)
        if self.ctx is not None and self.ctx.is_distributed:
            self.ctx.all_reduce_sum_(cnt)
            self.ctx.all_reduce_sum_(tot)
        top, arg = cnt.max(1)
        share = top / tot.clamp_min(1.0)
        mean_share = float(share[: st.F].mean().item())
        dom = torch.where(share >= 0.30, arg, torch.full_like(arg, 255))
        dom[st.F:] = 255
        if st.max_bins >= 256 or not bool((dom != 255).any()):
            return mean_share, None
        d = dom.view(G, 4).to(torch.int64)
        packed = (d[:, 0] | (d[:, 1] << 8) | (d[:, 2] << 16) | (d[:, 3] << 24))
        packed = torch.where(packed >= 2 ** 31, packed - 2 ** 32, packed).to(torch.int32).contiguous()
        return mean_share, packed

    def _level_fused(self, level: int):
        grid, spp, smem, thr, nk, cp, bd = self.level_geo[level]
        hprev, hcur = self.hbuf[(level + 1) & 1], self.hbuf[level & 1]
        hcur_ptr = _p(hcur) if level < self.depth - 1 else None
        native.cuda_check(self.lib.cb_fused_launch(ctypes.c_void_p(self.plan), level, _p(hprev), hcur_ptr,
                                                   _p(self.mask[level & 1]), _p(self.mask[(level + 1) & 1]), grid, spp,
                                                   smem, thr, nk, cp, bd, self._stream()), "cb_level_fused")
        self.launches_per_iter += 1

    def _level_unfused(self, level: int):
        chk, lib, st = native.cuda_check, self.lib, self.store
        nslots = 1 if level == 0 else 1 << (level - 1)
        rows = nslots * self.S
        if level > 0:
            chk(lib.cb_update_leaf(ctypes.c_void_p(st.handle), _p(self.leaf), _p(self.splits), _p(self.iter_ptr),
                                   self.depth, level - 1, self.grid_stream, self._stream()), "cb_update_leaf")
        self.partial[:rows].zero_()
        per_slot = self.S * 4 * self.B * 4
        spp = max(1, min(nslots, (self.max_smem - 2048) // per_slot))
        grid = self.sm_count * max(1, min(4, (200 * 1024) // max(1, spp * per_slot)))
        chk(lib.cb_hist(ctypes.c_void_p(st.handle), _p(self.leaf), _p(self.stats), self.S, level,
                        _p(self.mask[level & 1]), None, 0, spp, self.B, _p(self.partial), grid, self.threads,
                        self._stream()), "cb_hist")
        if self.R > 1:
            import torch.distributed as dist
            dist.all_reduce(self.partial[:rows], group=self.ctx.group)
        hprev, hcur = self.hbuf[(level + 1) & 1], self.hbuf[level & 1]
        hcur_ptr = _p(hcur) if level < self.depth - 1 else None
        src = (ctypes.c_void_p * 1)(self.partial.data_ptr())
        chk(lib.cb_score(ctypes.c_void_p(st.handle), src, 1, _p(hprev), hcur_ptr, self.TB, 0, 0, st.F, level, self.S,
                         _p(self.mask[level & 1]), self.l2, self.score_fn, self.random_strength, _p(self.scal),
                         _p(self.iter_ptr), self.score_seed, self.lr, _p(self.best_key), self._stream()), "cb_score")
        chk(lib.cb_select_local_launch(ctypes.c_void_p(st.handle), hcur_ptr, self.TB, 0, level, self.S,
                                       _p(self.best_key), _p(self.msg_local), self._stream()), "cb_select_local")
        chk(lib.cb_select_final_launch(ctypes.c_void_p(st.handle), _p(self.msg_local), 1, self.msg_local.stride(0) * 8,
                                       level, _p(self.splits), _p(self.iter_ptr), self.depth,
                                       _p(self.mask[(level + 1) & 1]), _p(self.best_key), self._stream()),
            "cb_select_final")
        self.launches_per_iter += 5 + (1 if level > 0 else 0)

    def _leaves(self):
        chk, lib = native.cuda_check, self.lib
        chk(lib.cb_update_leaf(ctypes.c_void_p(self.store.handle), _p(self.leaf), _p(self.splits), _p(self.iter_ptr),
                               self.depth, self.depth - 1, self.grid_stream, self._stream()), "cb_update_leaf")
        self.launches_per_iter += 1
        comm = ctypes.c_void_p(self.arena.handle) if (self.arena is not None and self.R > 1) else None
        if self.K > 1:
            if self.R > 1 and comm is None:
                raise RuntimeError("MultiClass on several ranks needs the peer arena (histogram_reduce='fused')")
            for it in range(self.leaf_iterations):
                first, last = (1 if it == 0 else 0), (1 if it == self.leaf_iterations - 1 else 0)
                chk(lib.cb_mc_leaf_step(_p(self.approx), _p(self.target), _p(self.weight), _p(self.leaf), self.n, self.npad,
                                        self.K, self.L, _p(self.delta), _p(self.sums), _p(self.sums_combined), _p(self.leaf_w),
                                        first, last, self.leaf_newton, self.l2, self.lr, _p(self.cur_vals), _p(self.model_vals),
                                        _p(self.model_wts), self.L, _p(self.iter_ptr), comm, self.weight_max, self.sm_count * 4,
                                        self._stream()), "cb_mc_leaf_step")
                self.launches_per_iter += 2
            return
        if self.R > 1 and comm is None:
            # NCCL baseline: sums are all-reduced between two kernels
            for it in range(self.leaf_iterations):
                self._leaf_pass_nccl(it)
            return
        if self.leaf_grid is None:
            self.leaf_grid = int(lib.cb_leaf_newton_max_grid(self.L)) if self.der_fn is None and self.loss_id != 100 else 0
        if self.leaf_grid > 0 and self.fused_leaf_steps:
            # all steps of the leaf estimation in one cooperative launch
            rc = lib.cb_leaf_newton(self.loss_id, self.p0, self.p1, _p(self.approx), _p(self.target), _p(self.weight),
                                   _p(self.leaf), self.n, self.L, _p(self.delta), _p(self.sums), _p(self.counter),
                                   _p(self.leaf_vmax),
                                   self.leaf_iterations, self.leaf_newton, self.l2, self.lr, _p(self.cur_vals),
                                   _p(self.model_vals), _p(self.model_wts), self.L, _p(self.iter_ptr), _p(self.leaf_w),
                                   comm, self.leaf_backtracking, self.leaf_grid, self._stream())
            if rc != -2:
                chk(rc, "cb_leaf_newton")
                self.launches_per_iter += 1
                return
            self.leaf_grid = 0          # too many leaves for one mailbox message: one launch per step instead
        for it in range(self.leaf_iterations):
            last = 1 if it == self.leaf_iterations - 1 else 0
            chk(lib.cb_leaf_pass_q(self.loss_id, self.p0, self.p1, _p(self.approx), _p(self.target), _p(self.weight),
                                   _p(self.leaf), _p(self.ext_der), _p(self.ext_hess), self.n, self.L, _p(self.delta),
                                   _p(self.sums), _p(self.counter), 1 if it == 0 else 0, last, self.leaf_newton,
                                   self.l2, self.lr, _p(self.cur_vals), _p(self.model_vals), _p(self.model_wts), self.L,
                                   _p(self.iter_ptr), _p(self.leaf_w), comm,
                                   _p(self.leaf_vmax) if self.quantized_hist and self.leaf_iterations > 1 else None,
                                   self.sm_count * 2, self._stream()), "cb_leaf_pass")
            self.launches_per_iter += 1

    def _leaf_pass_nccl(self, it):
        # baseline path only: torch ops + NCCL all-reduce of the per-leaf sums
        import torch.distributed as dist
        n = self.n
        leaf = self.leaf[:n].long() & 0xFFFF
        ap = self.approx[:n] + (self.delta[leaf] if it > 0 else 0)
        if self.der_fn is not None:
            d, h = self.ext_der[:n].unsqueeze(0), self.ext_hess[:n].unsqueeze(0)
        else:
            d, h = self.objective.der_hess(ap.unsqueeze(0), self.target[:n],
                                           None if self.weight is None else self.weight[:n])
        w = torch.ones_like(ap) if self.weight is None else self.weight[:n]
        sums = torch.zeros((3, self.L), dtype=torch.float64, device=self.dev)
        sums[0].index_add_(0, leaf, d[0].double())
        sums[1].index_add_(0, leaf, h[0].double())
        sums[2].index_add_(0, leaf, w.double())
        dist.all_reduce(sums, group=self.ctx.group)
        den = (sums[1] if self.leaf_newton else sums[2]) + self.l2
        step = torch.where(den > 0, sums[0] / den, torch.zeros_like(den)).float()
        if it == 0:
            self.delta.copy_(step)
        else:
            self.delta.add_(step)
        if it == self.leaf_iterations - 1:
            self.cur_vals.copy_(self.delta * self.lr)
            self.model_vals.index_copy_(0, self.iter_ptr.long(), self.cur_vals.unsqueeze(0))
            self.model_wts.index_copy_(0, self.iter_ptr.long(), sums[2].float().unsqueeze(0))

    def _evals(self):
        chk, lib = native.cuda_check, self.lib
        for k, ev in enumerate(self.eval_sets):
            chk(lib.cb_apply_tree_bins(ctypes.c_void_p(ev.store.handle), _p(ev.approx), ev.store.npad, _p(self.splits),
                                       _p(self.iter_ptr), self.depth, _p(self.cur_vals), self.K, self.grid_stream,
                                       self._stream()), "cb_apply_tree_bins")
            if self.K > 1:
                chk(lib.cb_mc_metric(_p(ev.approx), _p(ev.target), _p(ev.weight), ev.store.n, ev.store.npad, self.K, None,
                                     None, ctypes.c_void_p(self.eval_scal.data_ptr() + 16 * k), self.grid_stream,
                                     self._stream()), "cb_mc_metric")
                self.launches_per_iter += 2
                continue
            chk(lib.cb_metric_sum(self.loss_id, self.p0, self.p1, _p(ev.approx), _p(ev.target), _p(ev.weight),
                                  ev.store.n, None, None, ctypes.c_void_p(self.eval_scal.data_ptr() + 16 * k),
                                  self.grid_stream, self._stream()), "cb_metric_sum")
            self.launches_per_iter += 2

    def _external_derivatives(self):
        n = self.n
        cur = self.approx[:n] + self.cur_vals[self.leaf[:n].long() & 0xFFFF]
        d, h = self.der_fn(cur)
        self.ext_der[:n] = d.reshape(-1)
        self.ext_hess[:n] = h.reshape(-1)

    def _center_leaves(self):
        # ranking losses are invariant to a shift of the scores: keep the weighted mean of the tree's leaves at zero
        it = self.iter_ptr.long()
        w = self.model_wts.index_select(0, it)[0].double()
        mean = ((self.cur_vals.double() * w).sum() / w.sum().clamp_min(1e-30)).float()
        self.cur_vals.sub_(mean)
        self.model_vals.index_copy_(0, it, self.cur_vals.unsqueeze(0))

    def _iteration(self):
        self.launches_per_iter = 0
        if self.der_fn is not None:
            self._external_derivatives()
        self._grad()
        for level in range(self.depth):
            if self.reduce == "fused":
                self._level_fused(level)
            else:
                self._level_unfused(level)
        self._leaves()
        if self.zero_mean_leaves:
            self._center_leaves()
        self._evals()
        n_extra = 2 * len(self.eval_sets)
        native.cuda_check(self.lib.cb_iter_end(_p(self.iter_ptr), _p(self.scal), _p(self.loss_hist), _p(self.eval_scal),
                                               _p(self.eval_hist), n_extra, _p(self.statmax), self.S, self._stream()),
                          "cb_iter_end")
        self.launches_per_iter += 1

    # ------------------------------------------------------------------------------------------------------
    def _capture(self):
        torch.cuda.synchronize(self.dev)
        self.ctx.barrier()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, capture_error_mode="relaxed"):
            self._iteration()
        self.graph = g

    def step(self, count: int = 1):
        """Run ``count`` boosting iterations (asynchronously).  The first one runs eagerly (module loading,
        function attributes), the second call captures the CUDA graph that all later iterations replay."""
        if self.done + count > self.iterations:
            raise RuntimeError("more iterations requested than the engine was sized for")
        graph_ok = self.use_graph and not (self.R > 1 and self.reduce != "fused")
        for _ in range(count):
            if not graph_ok or not self._warmed:
                self._iteration()
                self._warmed = True
            else:
                if self.graph is None:
                    self._capture()
                self.graph.replay()
            self.done += 1
            if self._check_each:
                self.check_invariants()

    def current_learn_loss(self, pinned: Optional[torch.Tensor] = None) -> float:
        """Mean learn loss including the newest tree (one streaming kernel + a 16-byte device->host read),
        summed over ranks."""
        self.cur_loss.zero_()
        if self.K > 1:
            native.cuda_check(self.lib.cb_mc_metric(_p(self.approx), _p(self.target), _p(self.weight), self.n, self.npad,
                                                    self.K, _p(self.leaf), _p(self.cur_vals), _p(self.cur_loss),
                                                    self.grid_stream, self._stream()), "cb_mc_metric")
        else:
            native.cuda_check(self.lib.cb_metric_sum(self.loss_id, self.p0, self.p1, _p(self.approx), _p(self.target),
                                                     _p(self.weight), self.n, _p(self.leaf), _p(self.cur_vals),
                                                     _p(self.cur_loss), self.grid_stream, self._stream()), "cb_metric_sum")
        if self.R > 1:
            self.ctx.all_reduce_sum_(self.cur_loss)
        if pinned is not None:
            pinned.copy_(self.cur_loss, non_blocking=True)
            torch.cuda.current_stream(self.dev).synchronize()
            v = pinned
        else:
            v = self.cur_loss.cpu()
        return float(v[0]) / max(float(v[1]), 1e-300)

    def finish(self):
        """Apply the last tree to the training cursor and return (splits, leaf values, leaf weights) on the host."""
        torch.cuda.synchronize(self.dev)
        if self.arena is not None:
            self.arena.check_status()
        n = self.n
        leaf = self.leaf[:n].long() & 0xFFFF
        if self.K > 1:
            self.approx[:, :n] += self.cur_vals.view(self.L, self.K)[leaf].t()
        else:
            self.approx[:n] += self.cur_vals[leaf]
        self.cur_vals.zero_()
        self.leaf.zero_()
        T = self.done
        sp = self.splits[: T * self.depth].cpu().numpy().reshape(T, self.depth, 4)
        return sp, self.model_vals[:T].cpu().numpy(), self.model_wts[:T].cpu().numpy()

    # ------------------------------------------------------------------------------------------------------
    def check_invariants(self):
        """Checks of the device state after the latest iteration (a debugging aid in the place of a race detector: a lost
        update, a stale read across ranks or an out-of-range write shows up here long before it shows up in the loss).
        Synchronises the device.  Raises RuntimeError with the first violated invariant.  ``CB200_CHECK=1`` makes the
        training loop call it after every iteration."""
        torch.cuda.synchronize(self.dev)
        if self.arena is not None:
            self.arena.check_status()                       # a bounded device wait that ran out of time
        T, n, F = self.done, self.n, self.store.F
        if T == 0:
            return
        sp = self.splits[(T - 1) * self.depth: T * self.depth]
        feat, bins = sp[:, 0], sp[:, 1]
        if bool(((feat < -1) | (feat >= F)).any()):
            raise RuntimeError(f"invariant: split feature outside [-1, {F}) in tree {T - 1}: {feat.tolist()}")
        nb = self.store.feat_nb.to(self.dev)
        ok = feat >= 0
        if bool(ok.any()) and bool((bins[ok] >= nb[feat[ok].long()]).any() or (bins[ok] < 0).any()):
            raise RuntimeError(f"invariant: split bin outside its feature's bins in tree {T - 1}")
        leaf = self.leaf[:n].long() & 0xFFFF
        if bool((leaf >= self.L).any()):
            raise RuntimeError("invariant: a document's leaf index is outside the tree")
        if not bool(torch.isfinite(self.approx).all()):
            raise RuntimeError("invariant: a non-finite approximation")
        if not bool(torch.isfinite(self.model_vals[T - 1]).all()):
            raise RuntimeError("invariant: a non-finite leaf value")
        # the leaf weights of the newest tree are the document weights, summed over all ranks
        w_local = float(n) if self.weight is None else float(self.weight[:n].double().sum().item())
        tot = torch.tensor([w_local], dtype=torch.float64, device=self.dev)
        if self.ctx is not None and self.ctx.is_distributed:
            self.ctx.all_reduce_sum_(tot)
        got = float(self.model_wts[T - 1].double().sum().item())
        if abs(got - float(tot.item())) > 1e-4 * max(1.0, float(tot.item())):
            raise RuntimeError(f"invariant: leaf weights of tree {T - 1} sum to {got}, the data weighs {float(tot.item())}")
        # every rank holds the same tree
        if self.ctx is not None and self.ctx.is_distributed:
            mine = sp[:, :2].contiguous().long()
            ref = mine.clone()
            import torch.distributed as dist
            dist.broadcast(ref, src=0, group=self.ctx.group)
            if not bool(torch.equal(mine, ref)):
                raise RuntimeError(f"invariant: rank {self.ctx.rank} holds a different tree {T - 1} than rank 0")

    def export_trees(self):
        """(splits [T, depth, 4], leaf values [T, L], leaf weights [T, L]) of the finished iterations, on the host.
        Unlike ``finish`` this leaves the engine ready to continue (used for snapshots)."""
        torch.cuda.synchronize(self.dev)
        T = self.done
        return (self.splits[: T * self.depth].cpu().numpy().reshape(T, self.depth, 4),
                self.model_vals[:T].cpu().numpy(), self.model_wts[:T].cpu().numpy())

    def restore_trees(self, splits: np.ndarray, vals: np.ndarray, wts: np.ndarray):
        """Continue a run from ``T0 = len(splits)`` finished trees: the trees go back into the device-side model, the
        training and evaluation cursors are rebuilt by applying the trees in their original order (the same fp32
        additions the uninterrupted run made, so the continuation is bit-identical), and the iteration counter --
        which also drives the counter-based random numbers of the bootstrap and of the score noise -- is set to T0.
        The reference restores the same way: models are stored, cursors are recomputed
        (catboost/cuda/methods/doc_parallel_boosting.h:500-512)."""
        if self.done != 0:
            raise RuntimeError("restore_trees must be called before the first step")
        T0 = int(len(splits))
        if T0 == 0:
            return
        if T0 > self.iterations:
            raise RuntimeError("the snapshot holds more trees than this run asks for")
        sp = torch.from_numpy(np.ascontiguousarray(splits, dtype=np.int32).reshape(T0 * self.depth, 4)).to(self.dev)
        self.splits[: T0 * self.depth] = sp
        self.model_vals[:T0] = torch.from_numpy(np.ascontiguousarray(vals, dtype=np.float32)).to(self.dev)
        self.model_wts[:T0] = torch.from_numpy(np.ascontiguousarray(wts, dtype=np.float32)).to(self.dev)
        chk, lib = native.cuda_check, self.lib
        sets = [(self.store, self.approx)] + [(ev.store, ev.approx) for ev in self.eval_sets]
        for t in range(T0):
            sp_ptr = ctypes.c_void_p(self.splits.data_ptr() + t * self.depth * 16)
            v_ptr = ctypes.c_void_p(self.model_vals.data_ptr() + t * self.L * self.K * 4)
            for st, ap in sets:
                chk(lib.cb_apply_tree_bins(ctypes.c_void_p(st.handle), _p(ap), st.npad, sp_ptr, None, self.depth, v_ptr, self.K,
                                           self.grid_stream, self._stream()), "cb_apply_tree_bins")
        self.iter_ptr.fill_(T0)
        self.cur_vals.zero_()
        self.leaf.zero_()
        self.done = T0
        self._resumed = True
        torch.cuda.synchronize(self.dev)

    def learn_loss_history(self) -> np.ndarray:
        """Mean learn loss seen at the start of every finished iteration (summed over ranks)."""
        h = self.loss_hist[: self.done].clone()
        if self.R > 1:
            self.ctx.all_reduce_sum_(h)
        h = h.cpu().numpy()
        return h[:, 0] / np.maximum(h[:, 1], 1e-300)

    def eval_loss_history(self) -> np.ndarray:
        n_eval = len(self.eval_sets)
        if not n_eval:
            return np.zeros((self.done, 0))
        h = self.eval_hist[: self.done].clone()
        if self.R > 1:
            self.ctx.all_reduce_sum_(h)
        h = h.cpu().numpy().reshape(self.done, n_eval, 2)
        return h[:, :, 0] / np.maximum(h[:, :, 1], 1e-300)

    def close(self):
        if getattr(self, "plan", None):
            self.lib.cb_fused_destroy(ctypes.c_void_p(self.plan))
            self.plan = None
        if getattr(self, "arena", None) is not None:
            self.arena.close()
