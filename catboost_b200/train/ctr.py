"""CTR engine: permutation-ordered target statistics for categorical features and their combinations.

For every *projection* (one categorical feature, or a combination of up to ``max_ctr_complexity`` of them) and every
CTR description (type + prior) a float feature is produced and binarised with its own borders:

* training rows: statistics of the rows that precede the row in a random permutation and share its category
  (exclusive prefix inside the category, in permutation order) -- ``(good + prior) / (total + 1)`` for the target-class
  types (``Borders``, ``Buckets``, ``BinarizedTargetMeanValue``), the category count so far is NOT used for the counter types:
  ``Counter`` / ``FeatureFreq`` use the count of the category in the whole learn set (they do not look at the target);
* evaluation rows and the final model: statistics of the whole learn set.

Behaviour follows catboost/cuda/ctrs/ctr_calcers.h:122-160, ctr_bins_builder.h:137-245 (equal keys contiguous in
permutation order, segmented exclusive scan, divide with priors), catboost/private/libs/algo/online_ctr.cpp and the
prior defaults of catboost/private/libs/options/cat_feature_options.cpp:118-140.  The device path is a stable (hand-written radix) sort by
category of the rows taken in permutation order, a segmented exclusive scan, and a scatter back.
Combination hashes use the model's hash rule (catboost/libs/model/hash.h:11-14) so that the stored tables can be
looked up at apply time from raw categorical hashes.
"""
from __future__ import annotations

import itertools
import os
import re
from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import numpy as np
import torch

from ..data.pool import CatBoostError, Pool
from ..data.quantization import FlatFeature, select_borders
from ..models.ctr import CtrFeature, projection_hash

TARGET_CTRS = ("Borders", "Buckets", "BinarizedTargetMeanValue", "FloatTargetMeanValue")
COUNT_CTRS = ("Counter", "FeatureFreq")


@dataclass
class CtrSpec:
    cat_features: Tuple[int, ...]
    ctr_type: str
    prior_num: float
    prior_denom: float = 1.0
    target_border_idx: int = 0
    border_count: int = 15


@dataclass
class CtrPlan:
    specs: List[CtrSpec]
    target_borders: np.ndarray          # thresholds that binarise the target into classes
    n_target_classes: int


@dataclass
class CtrState:
    flat_features: List[FlatFeature]
    train_bins: torch.Tensor            # uint8 [n_ctr, n_train] on the training device
    eval_bins: List[torch.Tensor]
    model_ctrs: List[CtrFeature]
    permutation: np.ndarray = field(default=None)


def _parse_ctr_description(desc: str, default_priors):
    """'Borders:TargetBorderCount=1:Prior=0/1:Prior=0.5/1' -> (type, target_border_count, [(num, denom)], border_count)."""
    parts = desc.split(":")
    ctype = parts[0]
    priors, tbc, bc = [], 1, None
    for p in parts[1:]:
        k, _, v = p.partition("=")
        if k == "Prior":
            a, _, b = v.partition("/")
            priors.append((float(a), float(b) if b else 1.0))
        elif k == "TargetBorderCount":
            tbc = int(v)
        elif k == "CtrBorderCount":
            bc = int(v)
    return ctype, tbc, priors or list(default_priors), bc


def plan_ctrs(o, pool: Pool, ctr_cats: List[int], ctx) -> CtrPlan:
    gpu = o.task_type == "GPU"
    simple = o.simple_ctr if o.simple_ctr is not None else o.ctr_description
    if simple is None:
        simple = ["Borders", "Counter"]          # FeatureFreq is the reference's GPU name for the count-based CTR
    if isinstance(simple, str):
        simple = [simple]
    combos = o.combinations_ctr if o.combinations_ctr is not None else simple
    if isinstance(combos, str):
        combos = [combos]
    tbc_max = 1
    specs: List[CtrSpec] = []

    def add(projection, descs):
        nonlocal tbc_max
        for d in descs:
            ctype, tbc, priors, bc = _parse_ctr_description(
                d, [(0.0, 1.0), (0.5, 1.0), (1.0, 1.0)] if d.split(":")[0] in TARGET_CTRS else [(0.0, 1.0)])
            if ctype not in TARGET_CTRS + COUNT_CTRS:
                raise CatBoostError(f"unknown CTR type {ctype!r}")
            if o.ctr_target_border_count:
                tbc = int(o.ctr_target_border_count)
            tbc_max = max(tbc_max, tbc)
            for num, den in priors:
                if ctype in TARGET_CTRS:
                    for tb in range(tbc):
                        specs.append(CtrSpec(tuple(projection), ctype, num, den, tb, bc or int(o.ctr_border_count)))
                else:
                    specs.append(CtrSpec(tuple(projection), ctype, num, den, 0, bc or int(o.ctr_border_count)))

    # per_feature_ctr: "<categorical feature (dataset column)>:<CTR description>", several entries per feature allowed
    per_feature = {}
    for item in ([o.per_feature_ctr] if isinstance(o.per_feature_ctr, str) else list(o.per_feature_ctr or [])):
        fid, _, desc = str(item).partition(":")
        if not desc or not fid.strip().lstrip("-").isdigit():
            raise CatBoostError(f"per_feature_ctr entry {item!r}: expected '<feature index>:<CTR description>'")
        if int(fid) not in list(pool.cat_feature_indices):
            raise CatBoostError(f"per_feature_ctr: feature {int(fid)} is not categorical")
        per_feature.setdefault(int(fid), []).append(desc)
    for c in ctr_cats:
        add((c,), per_feature.get(int(pool.cat_feature_indices[c]), simple))
    complexity = int(o.max_ctr_complexity)
    if complexity >= 2 and len(ctr_cats) >= 2:
        # Static combinations: pairs (and triples when asked) among the categorical features of lowest cardinality.
        # The reference discovers combinations greedily while a tree grows (tree CTRs, feature-parallel only);
        # here they are enumerated up front under a fixed budget so that training stays doc-parallel.
        card = {c: len(pool.cat_distinct_values(c)) for c in ctr_cats}
        if ctx is not None and ctx.is_distributed:          # every rank must enumerate the same combinations
            all_cards = ctx.all_gather_object(card)
            card = {c: max(d[c] for d in all_cards) for c in ctr_cats}
        ranked = sorted(ctr_cats, key=lambda c: card[c])
        budget = 24
        top = ranked[: 8]
        for k in range(2, min(complexity, 3) + 1):
            for proj in itertools.combinations(top, k):
                if budget <= 0:
                    break
                add(tuple(sorted(proj)), combos)
                budget -= 1
    return CtrPlan(specs, np.zeros(0), 2)


def _target_classes(plan: CtrPlan, y: np.ndarray, codec, n_borders: int):
    """Binarise the target into ``n_borders + 1`` classes (MinEntropy-like equal-frequency borders for regression,
    the class index for classification)."""
    y = np.asarray(y, dtype=np.float64).reshape(len(y), -1)[:, 0]
    if codec is not None and (codec.is_binclass or codec.is_multiclass):
        cls = y.astype(np.int64)
        k = int(cls.max()) + 1 if len(cls) else 2
        return cls, max(k, 2), np.arange(k - 1) + 0.5
    srt = np.sort(y)
    borders, _ = select_borders(srt.reshape(-1, 1).astype(np.float32), n_borders, "MinEntropy")
    b = borders[0].astype(np.float64)
    if len(b) == 0:
        b = np.array([float(np.mean(y))])
    cls = np.searchsorted(b, y, side="left")
    return cls.astype(np.int64), len(b) + 1, b


def _projection_keys(pool: Pool, projection, device):
    """Dense category ids of the projection for the rows of ``pool`` + the 64-bit projection hash per row."""
    h = projection_hash([pool.cat_hashes[c] for c in projection])
    return h


_MAGIC_I64 = 0x4906BA494954CB65        # models.ctr.MAGIC_MULT; below 2^63, so the same bits as a signed constant


def _cat_column_t(pool: Pool, c: int, device) -> torch.Tensor:
    """Sign-extended 32-bit category hashes of one categorical feature as an int64 device tensor (cached on the pool)."""
    cache = pool.__dict__.setdefault("_cat_hash_tensors", {})
    key = (c, str(device))
    if key not in cache:
        col = np.ascontiguousarray(pool.cat_hashes[c], dtype=np.uint32).view(np.int32)
        cache[key] = torch.from_numpy(col).to(device).long()            # widened (sign-extended) on the device
    return cache[key]


def projection_hash_t(cols) -> torch.Tensor:
    """models.ctr.projection_hash on the device: 64-bit wrap-around arithmetic, returned as int64 (same bits)."""
    res = torch.zeros_like(cols[0])
    for b in cols:
        res = (res + b * _MAGIC_I64) * _MAGIC_I64
    return res


def _stable_sort(keys: torch.Tensor):
    """(sorted keys, order): the hand-written radix sort on the GPU (ops/cuda/cb_sort.cu), the framework's stable sort on
    the CPU."""
    from ..ops import api as ops
    if keys.dtype != torch.int64:
        return torch.sort(keys, stable=True)
    return ops.sort_pairs(keys)


def _group_rows(h: torch.Tensor, order_t: torch.Tensor):
    """One stable sort of the projection hashes taken in permutation order: rows of equal hash become contiguous and
    keep the permutation order inside their group.  Returns (rows, seg_id, first_idx, uniq): the row id at every sorted
    position, the dense group number of every sorted position, the first sorted position of every group, and the
    distinct hashes in (signed) increasing order."""
    n = h.shape[0]
    sorted_h, srt = _stable_sort(h[order_t])
    rows = order_t[srt]
    start = torch.ones(n, dtype=torch.bool, device=h.device)
    if n > 1:
        start[1:] = sorted_h[1:] != sorted_h[:-1]
    seg_id = torch.cumsum(start, 0, dtype=torch.int64) - 1
    first_idx = torch.nonzero(start).squeeze(1)
    return rows, seg_id, first_idx, sorted_h[first_idx]


def _segment_stats(cols, rows, seg_id, first_idx, want_prefix: bool):
    """``cols``: list of 0/1 indicator vectors [n] (int32).  Per column: the total inside every group [U] and, if asked,
    the exclusive running count inside the group in permutation order, aligned with the original rows [n].  Integer
    running sums: exact for any row count."""
    n = rows.shape[0]
    last_idx = torch.cat([first_idx[1:], first_idx.new_tensor([n])]) - 1
    totals, prefix = [], []
    for col in cols:
        vals = col[rows]
        cs = torch.cumsum(vals, 0, dtype=torch.int32)
        base = cs[first_idx] - vals[first_idx]
        totals.append((cs[last_idx] - base).float())
        if want_prefix:
            out = torch.empty(n, dtype=torch.float32, device=rows.device)
            out[rows] = (cs - vals - base[seg_id]).float()
            prefix.append(out)
    return torch.stack(totals), (torch.stack(prefix) if want_prefix else None)


class _TensorGroup:
    """Grouping, ordered statistics and bucketing of one projection as tensor operations (host training, and the
    oracle of the device kernels)."""

    def __init__(self, h, order_t, cls_t, need_tb, want_prefix):
        n = h.shape[0]
        rows_t, seg_id, first_idx, self.uniq_t = _group_rows(h, order_t)
        self.keys_t = torch.empty(n, dtype=torch.int64, device=h.device)       # dense group number of every row
        self.keys_t[rows_t] = seg_id
        cols = [torch.ones(n, dtype=torch.int32, device=h.device)] + [(cls_t > tb).int() for tb in need_tb]
        self.totals, self.prefix = _segment_stats(cols, rows_t, seg_id, first_idx, want_prefix)

    def _values(self, d):
        kind, ci, pn, pd, denom = d
        if kind == 0:
            return (self.prefix[ci] + pn) / (self.prefix[0] + pd)
        return ((self.totals[0] + pn) / denom)[self.keys_t]

    def value_ranges(self, descs):
        out = []
        for d in descs:
            v = self._values(d)
            out.append((np.float32(v.min().item()), np.float32(v.max().item())))
        return out

    def sample_values(self, d, sample_idx):
        v = self._values(d)
        return v if sample_idx is None else v[sample_idx]

    def binarize(self, descs, borders, lo_row, n_local):
        dev = self.keys_t.device
        return [torch.searchsorted(torch.from_numpy(b).to(dev), self._values(d).contiguous(), right=False)
                .to(torch.uint8)[lo_row:lo_row + n_local] for d, b in zip(descs, borders)]


class _KernelGroup:
    """The same through the hand-written kernels of ops/cuda/cb_ctr.cu: one library sort, then segmented scans, value
    range and bucketing without materialising a CTR value in memory."""

    def __init__(self, h, order_t, cls_u8, need_tb, want_prefix):
        from ..ops import api as ops
        self.ops = ops
        sorted_h, srt = _stable_sort(h[order_t])
        self.rows_t = order_t[srt]
        self.n = int(h.shape[0])
        self.excl, self.seg_id, self.uniq_t, self.totals_i = ops.ctr_scan(sorted_h, self.rows_t, cls_u8, need_tb)
        self.totals = self.totals_i.float()
        self._keys = None

    def value_ranges(self, descs):
        out = []
        for k in range(0, len(descs), self.ops.CTR_MAX_SPECS):
            out += self.ops.ctr_minmax(descs[k:k + self.ops.CTR_MAX_SPECS], self.excl, self.totals_i, self.seg_id)
        return out

    def sample_values(self, d, sample_idx):
        kind, ci, pn, pd, denom = d
        assert kind == 1
        if self._keys is None:
            self._keys = torch.empty(self.n, dtype=torch.int32, device=self.rows_t.device)
            self._keys[self.rows_t] = self.seg_id
        keys = self._keys if sample_idx is None else self._keys[sample_idx]
        return ((self.totals[0] + pn) / denom)[keys.long()]

    def binarize(self, descs, borders, lo_row, n_local):
        out = []
        for k in range(0, len(descs), self.ops.CTR_MAX_SPECS):
            m = self.ops.ctr_binarize(descs[k:k + self.ops.CTR_MAX_SPECS], borders[k:k + self.ops.CTR_MAX_SPECS], self.excl,
                                      self.totals_i, self.seg_id, self.rows_t, lo_row, n_local)
            out += [m[j] for j in range(m.shape[0])]
        return out


_STAGE_TIMES = {}          # developer aid (CB200_CTR_TIMING=1): seconds per stage of the CTR computation, rank 0 prints them


class _Stage:
    def __init__(self, name, dev):
        self.name, self.dev, self.on = name, dev, os.environ.get("CB200_CTR_TIMING") == "1"

    def __enter__(self):
        if self.on:
            import time
            if self.dev.type == "cuda":
                torch.cuda.synchronize(self.dev)
            self.t0 = time.perf_counter()

    def __exit__(self, *exc):
        if self.on:
            import time
            if self.dev.type == "cuda":
                torch.cuda.synchronize(self.dev)
            _STAGE_TIMES[self.name] = _STAGE_TIMES.get(self.name, 0.0) + time.perf_counter() - self.t0


class _ShardedGroup:
    """One projection on several ranks without mirroring the categorical data: every category belongs to the rank its
    hash maps to.  A rank sends (hash, permutation position, target class) of its rows to the owners (one all-to-all),
    the owner groups, scans and buckets its categories with the single-rank code (all rows of a category are with it),
    and the bucket numbers travel back the same way.  Only the tables the model keeps (distinct hashes and their totals)
    and a few scalars (value ranges, border samples) are exchanged in full.  The reference mirrors categorical columns
    on every device of a host (catboost/cuda/gpu_data/feature_parallel_dataset_builder.cpp); at 45M rows x 26 columns
    on 8 GPUs this path keeps one eighth of the sort and scan work and no copy of the other ranks' columns."""

    def __init__(self, ctx, h, pos, cls, need_tb, want_prefix, sample_pos):
        import torch.distributed as dist
        self.ctx, self.dist = ctx, dist
        dev = h.device
        R = ctx.world
        with _Stage("shard: owner sort", dev):
            owner = (((h >> 20) ^ h) & 0x7FFFFFFF) % R
            _, self.perm = torch.sort(owner, stable=True)
            send = torch.bincount(owner, minlength=R)
            recv = torch.empty_like(send)
            dist.all_to_all_single(recv, send, group=ctx.group)
            self.send_counts, self.recv_counts = [int(v) for v in send.tolist()], [int(v) for v in recv.tolist()]
        self.n_local = int(h.shape[0])
        with _Stage("shard: forward exchange", dev):
            h_r, pos_r, cls_r = self._forward(h[self.perm]), self._forward(pos[self.perm]), self._forward(cls[self.perm])
        self.m = int(h_r.shape[0])
        self.inner = None
        ncols = 1 + len(need_tb)
        if self.m:
            with _Stage("shard: position sort", dev):
                order_t = torch.argsort(pos_r)
            with _Stage("shard: group (sort + scan)", dev):
                self.inner = (_KernelGroup(h_r, order_t, cls_r.to(torch.uint8), need_tb, want_prefix) if dev.type == "cuda"
                              else _TensorGroup(h_r, order_t, cls_r, need_tb, want_prefix))
            uniq_l, totals_l = self.inner.uniq_t, self.inner.totals.float()
        else:
            uniq_l = torch.zeros(0, dtype=torch.int64, device=dev)
            totals_l = torch.zeros((ncols, 0), dtype=torch.float32, device=dev)
        # the model's table = the owners' tables side by side (their hash sets are disjoint), sorted by hash; padded
        # tensor collectives on the training device, no pickling of arrays that can have one entry per document
        t_tables = _Stage("shard: table gather", dev)
        t_tables.__enter__()
        sizes = [int(v) for v in ctx.all_gather_object(int(uniq_l.shape[0]))]
        cap = max(max(sizes), 1)
        ubuf = torch.zeros(cap, dtype=torch.int64, device=dev)
        ubuf[: uniq_l.shape[0]] = uniq_l
        tbuf = torch.zeros((ncols, cap), dtype=torch.float32, device=dev)
        tbuf[:, : uniq_l.shape[0]] = totals_l
        uall = [torch.empty_like(ubuf) for _ in sizes]
        tall = [torch.empty_like(tbuf) for _ in sizes]
        dist.all_gather(uall, ubuf, group=ctx.group)
        dist.all_gather(tall, tbuf, group=ctx.group)
        uniq = torch.cat([u[:c] for u, c in zip(uall, sizes)])
        totals = torch.cat([t[:, :c] for t, c in zip(tall, sizes)], dim=1)
        del uall, tall, ubuf, tbuf
        self.uniq_t, o_ = torch.sort(uniq)
        self.totals = totals[:, o_].contiguous()
        t_tables.__exit__()
        # items of this owner that belong to the border sample (given as permutation positions)
        self.sample_items = None
        if sample_pos is not None:
            with _Stage("shard: sample membership", dev):
                self.sample_items = torch.nonzero(torch.isin(pos_r, sample_pos)).squeeze(1)

    def _exchange(self, t, send_counts, recv_counts, width=1):
        out = torch.empty((sum(recv_counts) * width,), dtype=t.dtype, device=t.device)
        self.dist.all_to_all_single(out, t.contiguous().view(-1), [c * width for c in recv_counts],
                                    [c * width for c in send_counts], group=self.ctx.group)
        return out

    def _forward(self, t):
        return self._exchange(t, self.send_counts, self.recv_counts)

    def value_ranges(self, descs):
        local = self.inner.value_ranges(descs) if self.inner is not None else [(np.float32(np.inf), np.float32(-np.inf))] * len(descs)
        parts = self.ctx.all_gather_object([(float(a), float(b)) for a, b in local])
        return [(np.float32(min(p_[k][0] for p_ in parts)), np.float32(max(p_[k][1] for p_ in parts)))
                for k in range(len(descs))]

    def sample_values(self, d, sample_idx):
        if self.inner is not None:
            v = self.inner.sample_values(d, self.sample_items).cpu().numpy()
        else:
            v = np.zeros(0, np.float32)
        parts = self.ctx.all_gather_object(v)
        return torch.from_numpy(np.concatenate(parts))

    def binarize(self, descs, borders, lo_row, n_local):
        k = len(descs)
        dev = self.perm.device
        if self.inner is not None:
            cols = self.inner.binarize(descs, borders, 0, self.m)
            mat = torch.stack(cols, 1).contiguous()                     # [m, k]: the k buckets of an item travel together
        else:
            mat = torch.zeros((0, k), dtype=torch.uint8, device=dev)
        back = self._exchange(mat, self.recv_counts, self.send_counts, width=k).view(self.n_local, k)
        out = torch.empty((self.n_local, k), dtype=torch.uint8, device=dev)
        out[self.perm] = back
        return [out[:, j].contiguous() for j in range(k)]


def _all_gather_rows(ctx, t: torch.Tensor, counts) -> torch.Tensor:
    """Concatenation over the ranks (in rank order) of per-rank vectors of different lengths."""
    import torch.distributed as dist
    m = max(counts)
    buf = torch.zeros(m, dtype=t.dtype, device=t.device)
    buf[: t.shape[0]] = t
    outs = [torch.empty_like(buf) for _ in counts]
    dist.all_gather(outs, buf, group=ctx.group)
    return torch.cat([o_[:c] for o_, c in zip(outs, counts)])


def compute_ctr_features(plan: CtrPlan, o, train_pool: Pool, y_train, w_train, eval_pools, device, ctx, codec) -> CtrState:
    """Several ranks: the statistics of a category must come from all rows, not from the rows of one rank.  Every rank
    draws the same global permutation; the categories are then dealt to the ranks by hash (``_ShardedGroup``) and the
    targets (one float column) are all-gathered.  ``CB200_CTR_GATHER=1`` selects the older scheme instead, in which the
    categorical columns are all-gathered and every rank computes every table (kept as the oracle of the sharded one)."""
    dev = torch.device(device)
    n_local = train_pool.num_row()
    dist_mode = ctx is not None and ctx.is_distributed
    sharded = dist_mode and os.environ.get("CB200_CTR_GATHER") != "1"
    if os.environ.get("CB200_CTR_SHARDED") == "1" and ctx is not None and not dist_mode:
        import torch.distributed as dist
        sharded = dist.is_available() and dist.is_initialized()       # the sharded code on a group of one rank (profiling)
    if dist_mode:
        counts = [int(c) for c in ctx.all_gather_object(n_local)]
        lo_row = sum(counts[: ctx.rank])
        n = sum(counts)
        gather = lambda t: _all_gather_rows(ctx, t, counts)
        y_train = gather(torch.from_numpy(np.ascontiguousarray(y_train, dtype=np.float32)).to(dev)).cpu().numpy()
    else:
        lo_row, n = 0, n_local
        gather = lambda t: t
    rng = np.random.RandomState(int(o.random_seed) + 101)
    if o.has_time:
        order = np.arange(n)
    else:
        # block-wise shuffle like the reference (fold_permutation_block), groups stay together
        blk = int(o.fold_permutation_block or 1)
        if train_pool.group_id is not None:
            off = train_pool.group_offsets()
            if dist_mode:
                sizes = np.concatenate(ctx.all_gather_object(np.diff(off)))
                off = np.concatenate([[0], np.cumsum(sizes)])
            g = rng.permutation(len(off) - 1)
            order = np.concatenate([np.arange(off[k], off[k + 1]) for k in g]) if len(g) else np.zeros(0, np.int64)
        elif blk > 1:
            nb = (n + blk - 1) // blk
            order = np.concatenate([np.arange(b * blk, min(n, (b + 1) * blk)) for b in rng.permutation(nb)])
        else:
            order = rng.permutation(n)
    order_t = torch.from_numpy(order.astype(np.int64)).to(dev)
    tbc = max([s.target_border_idx for s in plan.specs if s.ctr_type in TARGET_CTRS] + [0]) + 1
    cls, n_cls, tborders = _target_classes(plan, y_train, codec, tbc)
    plan.target_borders, plan.n_target_classes = tborders, n_cls
    cls_t = torch.from_numpy(cls).to(dev)
    cls_u8 = cls_t.to(torch.uint8)

    flat, train_cols, eval_cols, model_ctrs = [], [], [[] for _ in eval_pools], []
    sample_idx = None          # rows the CTR borders are chosen from (one draw for all CTR features)
    if n > 200000:
        sample_idx = torch.from_numpy(np.random.default_rng(int(o.random_seed) + 7).choice(
            n, 200000, replace=False, shuffle=False)).to(dev)
    if sharded:
        inv = np.empty(n, dtype=np.int64)
        inv[order] = np.arange(n, dtype=np.int64)
        pos_local = torch.from_numpy(inv[lo_row:lo_row + n_local].copy()).to(dev)
        cls_local = cls_t[lo_row:lo_row + n_local].contiguous()
        sample_pos = torch.from_numpy(np.sort(inv[sample_idx.cpu().numpy()])).to(dev) if sample_idx is not None else None
        del inv
    cat_cache = {}

    def gathered_cat(c):
        if c not in cat_cache:
            cat_cache[c] = gather(_cat_column_t(train_pool, c, dev))
        return cat_cache[c]

    by_proj = {}
    for s in plan.specs:
        by_proj.setdefault(s.cat_features, []).append(s)
    for proj, specs in by_proj.items():
        # hashing, grouping and look-ups stay on the training device (a host sort of 45M 64-bit keys per projection
        # would dominate the whole fit)
        # indicators: class > border k  (Borders), one column per needed target border + the count column
        need_tb = sorted({s.target_border_idx for s in specs if s.ctr_type in TARGET_CTRS})
        want_prefix = any(s.ctr_type in TARGET_CTRS for s in specs)
        if sharded:
            with _Stage("hash", dev):
                h_train_t = projection_hash_t([_cat_column_t(train_pool, c, dev) for c in proj])
            grp = _ShardedGroup(ctx, h_train_t, pos_local, cls_local, need_tb, want_prefix, sample_pos)
        else:
            with _Stage("hash", dev):
                h_train_t = projection_hash_t([gathered_cat(c) for c in proj])
            with _Stage("group (sort + scan)", dev):
                if dev.type == "cuda":
                    grp = _KernelGroup(h_train_t, order_t, cls_u8, need_tb, want_prefix)
                else:
                    grp = _TensorGroup(h_train_t, order_t, cls_t, need_tb, want_prefix)
        uniq_t, totals = grp.uniq_t, grp.totals
        U = int(uniq_t.numel())
        t_host = _Stage("tables to host", dev)
        t_host.__enter__()
        # model tables want the hashes in unsigned order: the signed-sorted list is that order rotated
        rot = int((uniq_t < 0).sum().item())
        uniq_s = uniq_t.cpu().numpy().view(np.uint64)
        uniq = np.concatenate([uniq_s[rot:], uniq_s[:rot]])
        totals_s = totals.cpu().numpy()
        totals_np = np.concatenate([totals_s[:, rot:], totals_s[:, :rot]], axis=1)
        max_count = float(totals_np[0].max()) if U else 1.0
        t_host.__exit__()
        eval_keys = []
        for ep in eval_pools:
            he_t = projection_hash_t([_cat_column_t(ep, c, dev) for c in proj])
            if U:
                pos = torch.searchsorted(uniq_t, he_t).clamp(max=U - 1)
                ok = uniq_t[pos] == he_t
            else:
                pos = torch.zeros_like(he_t)
                ok = torch.zeros(he_t.shape, dtype=torch.bool, device=dev)
            eval_keys.append((pos, ok))
        # every CTR of the projection as (kind, numerator column, prior numerator, prior denominator, denominator)
        descs = []
        for s in specs:
            if s.ctr_type in TARGET_CTRS:
                descs.append((0, 1 + need_tb.index(s.target_border_idx), float(s.prior_num), float(s.prior_denom), 1.0))
            elif s.ctr_type == "Counter":
                descs.append((1, 0, float(s.prior_num), float(s.prior_denom), max_count + s.prior_denom))
            else:   # FeatureFreq
                descs.append((1, 0, float(s.prior_num), float(s.prior_denom), float(n) + s.prior_denom))
        target_pos = [k for k, d in enumerate(descs) if d[0] == 0]
        with _Stage("value ranges", dev):
            ranges = dict(zip(target_pos, grp.value_ranges([descs[k] for k in target_pos]))) if target_pos else {}
        all_borders = []
        t_b = _Stage("count-type borders", dev)
        t_b.__enter__()
        for k, (s, d) in enumerate(zip(specs, descs)):
            if d[0] == 0:
                # Uniform grid between the smallest and largest learn value (same arithmetic as the host routine:
                # float32, lo + (hi - lo) * k / (count + 1))
                lo_v, hi_v = ranges[k]
                if hi_v > lo_v:
                    kk = np.arange(1, s.border_count + 1, dtype=np.float32)
                    b = np.unique((lo_v + (hi_v - lo_v) * kk / np.float32(s.border_count + 1)).astype(np.float32))
                else:
                    b = np.zeros(0, dtype=np.float32)
            else:
                sample = grp.sample_values(d, sample_idx)
                borders, _ = select_borders(sample.cpu().numpy().reshape(-1, 1), s.border_count, "GreedyLogSum")
                b = np.asarray(borders[0], dtype=np.float32)
            all_borders.append(b)
        t_b.__exit__()
        keep = [k for k, b in enumerate(all_borders) if len(b)]
        with _Stage("bucketing", dev):
            cols_out = grp.binarize([descs[k] for k in keep], [all_borders[k] for k in keep], lo_row, n_local) if keep else []
        t_m = _Stage("eval columns + model tables", dev)
        t_m.__enter__()
        for k, col in zip(keep, cols_out):
            s, d, b = specs[k], descs[k], all_borders[k]
            train_cols.append(col)
            if d[0] == 0:
                full = (totals[d[1]] + s.prior_num) / (totals[0] + s.prior_denom)
                unseen = s.prior_num / s.prior_denom
            else:
                full = (totals[0] + s.prior_num) / d[4]
                unseen = s.prior_num / d[4]
            bt = torch.from_numpy(b).to(dev)
            for e, (pos, ok) in enumerate(eval_keys):
                ev = torch.where(ok, full[pos] if U else torch.zeros_like(ok, dtype=torch.float32),
                                 torch.full((len(ok),), float(unseen), device=dev))
                eval_cols[e].append(torch.searchsorted(bt, ev.contiguous(), right=False).to(torch.uint8))
            ctr_index = len(model_ctrs)
            if d[0] == 0:
                good = totals_np[d[1]]
                model_ctrs.append(CtrFeature(list(proj), s.ctr_type, s.prior_num, s.prior_denom, s.target_border_idx,
                                             uniq.copy(), good.astype(np.float64), totals_np[0].astype(np.float64), 0.0))
            else:
                model_ctrs.append(CtrFeature(list(proj), s.ctr_type, s.prior_num, s.prior_denom, 0, uniq.copy(),
                                             totals_np[0].astype(np.float64), totals_np[0].astype(np.float64),
                                             max_count if s.ctr_type == "Counter" else float(n)))
            flat.append(FlatFeature("ctr", ctr_index, borders=b, n_bins=len(b) + 1, ctr=s))
        t_m.__exit__()
    if _STAGE_TIMES and (ctx is None or ctx.rank == 0):
        import sys
        print("CTR stages (s):", {k: round(v, 3) for k, v in _STAGE_TIMES.items()}, "projections:", len(by_proj), file=sys.stderr)
        _STAGE_TIMES.clear()
    train_bins = torch.stack(train_cols) if train_cols else torch.zeros((0, n_local), dtype=torch.uint8, device=dev)
    eval_bins = [torch.stack(c) if c else torch.zeros((0, ep.num_row()), dtype=torch.uint8, device=dev)
                 for c, ep in zip(eval_cols, eval_pools)]
    return CtrState(flat, train_bins, eval_bins, model_ctrs, order)
