"""In-memory model: tree ensembles over float / one-hot / CTR splits, and their evaluation.

Structure follows the reference's ``TFullModel`` / ``TModelTrees`` (catboost/libs/model/model.h,
flatbuffers/model.fbs:16-53): a global list of *binary features* (every (float feature, border), every
(one-hot feature, value), every (ctr, border)), trees that reference them by index, oblivious trees stored as
``depth`` split indices + ``2^depth * dims`` leaf values where bit ``d`` of the leaf index is the outcome of
split ``d``; non-symmetric trees stored as step nodes.  Leaf values are doubles; prediction =
``scale * sum(leaf values) + bias``.
"""
from __future__ import annotations

import ctypes
import json
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import numpy as np

from ..data.pool import CatBoostError, Pool
from ..ops import native


@dataclass
class FloatFeatureInfo:
    flat_index: int                  # column in the user's data
    feature_index: int               # index among the float features
    borders: np.ndarray
    nan_mode: str = "Min"            # Min | Max | Forbidden
    has_nans: bool = False
    name: str = ""


@dataclass
class CatFeatureInfo:
    flat_index: int
    feature_index: int
    name: str = ""


@dataclass
class OneHotFeatureInfo:
    cat_feature_index: int
    values: np.ndarray               # uint32 hashes; bin k (k >= 1) means "value == values[k-1]"
    string_values: List[str] = field(default_factory=list)


@dataclass
class Split:
    kind: str                        # 'float' | 'onehot' | 'ctr'
    feature: int                     # float feature index / cat feature index / ctr index
    border: float = 0.0              # float & ctr: go right when value > border
    value: int = 0                   # one-hot: go right when hash == value

    def key(self):
        return (self.kind, self.feature, float(self.border), int(self.value))


@dataclass
class ObliviousTree:
    splits: List[int]                # indices into Model.splits, level 0 first (bit 0 of the leaf index)
    leaf_values: np.ndarray          # [2^depth, dims] float64
    leaf_weights: np.ndarray         # [2^depth] float64


@dataclass
class NonSymmetricTree:
    split_of_node: np.ndarray        # int32 [nodes]; -1 for a leaf
    left: np.ndarray                 # int32 [nodes] child taken when the condition is false
    right: np.ndarray                # int32 [nodes]
    leaf_of_node: np.ndarray         # int32 [nodes]; leaf id for terminal nodes
    leaf_values: np.ndarray          # [leaves, dims]
    leaf_weights: np.ndarray


class Model:
    def __init__(self):
        self.float_features: List[FloatFeatureInfo] = []
        self.cat_features: List[CatFeatureInfo] = []
        self.one_hot: Dict[int, OneHotFeatureInfo] = {}
        self.ctrs: list = []               # CtrFeature objects (models/ctr.py)
        self.splits: List[Split] = []
        self.trees: list = []
        self.dims: int = 1
        self.scale: float = 1.0
        self.bias: np.ndarray = np.zeros(1)
        self.params: dict = {}
        self.info: Dict[str, str] = {}
        self.class_names: Optional[list] = None
        self.loss_name: str = "RMSE"
        self.feature_names: List[str] = []
        self.n_features: int = 0
        self.cat_hash_to_string: Dict[int, str] = {}

    # ------------------------------------------------------------------ construction helpers
    def split_index(self, sp: Split) -> int:
        cache = self.__dict__.get("_split_cache")
        if cache is None or len(cache) != len(self.splits):
            cache = self.__dict__["_split_cache"] = {s.key(): i for i, s in enumerate(self.splits)}
        k = sp.key()
        if k not in cache:
            cache[k] = len(self.splits)
            self.splits.append(sp)
        return cache[k]

    @property
    def tree_count(self) -> int:
        return len(self.trees)

    def is_oblivious(self) -> bool:
        return all(isinstance(t, ObliviousTree) for t in self.trees)

    def shrink(self, ntree_end: int, ntree_start: int = 0):
        self.trees = self.trees[ntree_start:ntree_end]

    def copy(self) -> "Model":
        import copy
        m = copy.copy(self)
        m.trees = list(self.trees)
        m.splits = list(self.splits)
        m.__dict__.pop("_split_cache", None)
        m.bias = self.bias.copy()
        return m

    # ------------------------------------------------------------------ evaluation
    def _split_outcomes_block(self, float_data: np.ndarray, cat_hashes: Optional[np.ndarray], ctr_values=None):
        """bool [n_splits, n]: outcome of every binary feature for the rows (generic path)."""
        n = float_data.shape[0] if float_data.size or cat_hashes is None else cat_hashes.shape[1]
        out = np.zeros((len(self.splits), n), dtype=bool)
        nan_max = {f.feature_index: (f.nan_mode == "Max") for f in self.float_features}
        for i, sp in enumerate(self.splits):
            if sp.kind == "float":
                col = float_data[:, sp.feature]
                r = col > sp.border
                nanm = np.isnan(col)
                if nanm.any():
                    r = np.where(nanm, nan_max.get(sp.feature, False), r)
                out[i] = r
            elif sp.kind == "onehot":
                out[i] = cat_hashes[sp.feature] == np.uint32(sp.value)
            else:
                out[i] = ctr_values[sp.feature] > sp.border
        return out

    def _float_only_oblivious(self) -> bool:
        return self.is_oblivious() and all(s.kind == "float" for s in self.splits) and len(self.trees) > 0

    def _packed_oblivious(self):
        """Arrays for the native batch evaluators (float-only oblivious models)."""
        cache = self.__dict__.get("_packed")
        if cache is not None and cache["T"] == len(self.trees):
            return cache
        used = sorted({s.feature for s in self.splits})
        fmap = {f: u for u, f in enumerate(used)}
        finfo = {f.feature_index: f for f in self.float_features}
        borders, boff = [], [0]
        for f in used:
            b = np.asarray(finfo[f].borders, dtype=np.float32)
            borders.append(b)
            boff.append(boff[-1] + len(b))
        borders_cat = np.concatenate(borders) if borders else np.zeros(1, np.float32)
        depth = np.array([len(t.splits) for t in self.trees], dtype=np.int32)
        soff = np.zeros(len(self.trees), dtype=np.int32)
        soff[1:] = np.cumsum(depth)[:-1]
        sfeat = np.zeros(int(depth.sum()), dtype=np.uint16)
        sbin = np.zeros(int(depth.sum()), dtype=np.uint8)
        k = 0
        for t in self.trees:
            for si in t.splits:
                sp = self.splits[si]
                b = np.asarray(finfo[sp.feature].borders, dtype=np.float32)
                # bin > idx  <=>  value > borders[idx]
                idx = int(np.searchsorted(b, np.float32(sp.border)))
                if idx >= len(b) or b[idx] != np.float32(sp.border):
                    idx = int(np.argmin(np.abs(b - sp.border)))
                sfeat[k] = fmap[sp.feature]
                sbin[k] = idx
                k += 1
        leaves = np.array([t.leaf_values.shape[0] for t in self.trees], dtype=np.int64)
        loff = np.zeros(len(self.trees), dtype=np.int64)
        loff[1:] = np.cumsum(leaves)[:-1]
        vals = np.concatenate([t.leaf_values.reshape(-1, self.dims) for t in self.trees]).astype(np.float64)
        nanmax = np.array([1 if finfo[f].nan_mode == "Max" else 0 for f in used], dtype=np.uint8)
        cache = dict(T=len(self.trees), used=np.array(used, dtype=np.int32), borders=borders_cat,
                     boff=np.array(boff, dtype=np.int32), depth=depth, soff=soff, sfeat=sfeat, sbin=sbin, loff=loff,
                     vals=np.ascontiguousarray(vals), nanmax=nanmax)
        self.__dict__["_packed"] = cache
        return cache

    def predict_raw(self, float_data: np.ndarray, cat_hashes: Optional[np.ndarray] = None, ntree_start: int = 0,
                    ntree_end: int = 0, task_type: str = "CPU", device: Optional[str] = None,
                    thread_count: int = -1) -> np.ndarray:
        """Raw formula values [n, dims] (float64)."""
        T = len(self.trees)
        ntree_end = T if ntree_end in (0, None) or ntree_end > T else ntree_end
        n = float_data.shape[0] if (float_data.size or cat_hashes is None or not cat_hashes.size) else cat_hashes.shape[1]
        if ntree_start == 0 and ntree_end == T and self._float_only_oblivious() and n > 0:
            if task_type == "GPU":
                from .gpu_apply import predict_oblivious_gpu
                return predict_oblivious_gpu(self, float_data, device)
            return self._predict_native_cpu(float_data, thread_count)
        return self._predict_generic(float_data, cat_hashes, ntree_start, ntree_end)

    def _predict_native_cpu(self, X: np.ndarray, thread_count: int = -1) -> np.ndarray:
        p = self._packed_oblivious()
        X = np.ascontiguousarray(X, dtype=np.float32)
        n = X.shape[0]
        out = np.zeros((self.dims, n), dtype=np.float64)
        lib = native.cpu_lib()
        if thread_count and thread_count > 0:
            lib.cbc_set_num_threads(int(thread_count))
        P = lambda a: a.ctypes.data_as(ctypes.c_void_p)
        bias = np.ascontiguousarray(np.broadcast_to(self.bias, (self.dims,)), dtype=np.float64)
        lib.cbc_predict_oblivious(P(X), ctypes.c_longlong(n), ctypes.c_longlong(X.strides[0] // 4), P(p["used"]),
                                  P(p["borders"]), P(p["boff"]), P(p["nanmax"]), ctypes.c_int(len(p["used"])),
                                  P(p["depth"]), P(p["soff"]), P(p["sfeat"]), P(p["sbin"]), P(p["loff"]), P(p["vals"]),
                                  ctypes.c_int(p["T"]), ctypes.c_int(self.dims), ctypes.c_double(self.scale), P(bias),
                                  P(out))
        return out.T.copy()

    def _ctr_values(self, cat_hashes):
        if not self.ctrs:
            return None
        return [c.apply(cat_hashes) for c in self.ctrs]

    def _predict_generic(self, float_data, cat_hashes, ntree_start, ntree_end, block: int = 65536) -> np.ndarray:
        n = float_data.shape[0] if (float_data.size or cat_hashes is None or not cat_hashes.size) else cat_hashes.shape[1]
        out = np.zeros((n, self.dims), dtype=np.float64)
        for r0 in range(0, n, block):
            r1 = min(n, r0 + block)
            fd = float_data[r0:r1]
            ch = None if cat_hashes is None else cat_hashes[:, r0:r1]
            ctrv = self._ctr_values(ch)
            oc = self._split_outcomes_block(fd, ch, ctrv)
            acc = np.zeros((r1 - r0, self.dims), dtype=np.float64)
            for t in self.trees[ntree_start:ntree_end]:
                acc += t.leaf_values[self.leaf_indices_of_tree(t, oc)]
            out[r0:r1] = acc
        return out * self.scale + np.broadcast_to(self.bias, (self.dims,))

    @staticmethod
    def leaf_indices_of_tree(t, outcomes: np.ndarray) -> np.ndarray:
        n = outcomes.shape[1]
        if isinstance(t, ObliviousTree):
            idx = np.zeros(n, dtype=np.int64)
            for d, si in enumerate(t.splits):
                idx |= outcomes[si].astype(np.int64) << d
            return idx
        node = np.zeros(n, dtype=np.int64)
        for _ in range(len(t.split_of_node)):
            sp = t.split_of_node[node]
            active = sp >= 0
            if not active.any():
                break
            go_right = np.zeros(n, dtype=bool)
            go_right[active] = outcomes[sp[active], np.nonzero(active)[0]]
            node = np.where(active, np.where(go_right, t.right[node], t.left[node]), node)
        return t.leaf_of_node[node].astype(np.int64)

    def leaf_indices(self, float_data, cat_hashes=None, ntree_start=0, ntree_end=0) -> np.ndarray:
        T = len(self.trees)
        ntree_end = T if ntree_end in (0, None) or ntree_end > T else ntree_end
        oc = self._split_outcomes_block(float_data, cat_hashes, self._ctr_values(cat_hashes))
        return np.stack([self.leaf_indices_of_tree(t, oc) for t in self.trees[ntree_start:ntree_end]], axis=1)

    def staged_raw(self, float_data, cat_hashes=None, ntree_start=0, ntree_end=0, eval_period=1, at_iterations=False):
        """Raw predictions of growing prefixes of the ensemble.  Staged prediction yields after every ``eval_period``
        trees (and after the last one); metric evaluation (``at_iterations``) yields at the iterations
        ntree_start, ntree_start + eval_period, ... and the last one, where iteration i is the model of i + 1 trees
        (catboost/private/libs/algo/plot.cpp)."""
        T = len(self.trees)
        ntree_end = T if ntree_end in (0, None) or ntree_end > T else ntree_end
        oc = self._split_outcomes_block(float_data, cat_hashes, self._ctr_values(cat_hashes))
        acc = np.zeros((oc.shape[1], self.dims), dtype=np.float64)
        bias = np.broadcast_to(self.bias, (self.dims,))
        for k, t in enumerate(self.trees[ntree_start:ntree_end], start=ntree_start):
            acc += t.leaf_values[self.leaf_indices_of_tree(t, oc)]
            if (k + (0 if at_iterations else 1) - ntree_start) % eval_period == 0 or k + 1 == ntree_end:
                yield acc * self.scale + bias

    # ------------------------------------------------------------------ pool plumbing
    def pool_arrays(self, pool: Pool) -> Tuple[np.ndarray, Optional[np.ndarray]]:
        """Map a pool's columns onto the model's float / cat feature indexing."""
        est = getattr(self, "estimators", None)
        if est is not None and (getattr(pool, "text_data", None) or getattr(pool, "embedding_data", None)):
            pool = pool.with_estimated(est.transform(pool), est.names)
        if pool.n_features < self.n_features:
            raise CatBoostError(f"the model needs {self.n_features} features, the data has {pool.n_features}")
        want_f = [f.flat_index for f in self.float_features]
        have_f = {c: j for j, c in enumerate(pool.float_feature_indices)}
        want_c = [c.flat_index for c in self.cat_features]
        have_c = {c: j for j, c in enumerate(pool.cat_feature_indices)}
        for c in want_c:
            if c not in have_c:
                raise CatBoostError(f"feature {c} is categorical in the model but not in the data")
        if want_f == list(pool.float_feature_indices):
            fd = pool.float_data
        else:
            fd = np.full((pool.num_row(), len(want_f)), np.nan, dtype=np.float32)
            for j, c in enumerate(want_f):
                if c in have_f:
                    fd[:, j] = pool.float_data[:, have_f[c]]
                else:
                    raise CatBoostError(f"feature {c} is numeric in the model but categorical in the data")
        ch = None
        if want_c:
            ch = np.stack([pool.cat_hashes[have_c[c]] for c in want_c]) if want_c else None
        return fd, ch
