"""In-memory dataset (``Pool``) and file loaders.

Mirrors the user-facing behaviour of ``catboost.Pool`` (catboost/python-package/catboost/core.py:624) and the
dsv / column-description / libsvm loaders (catboost/libs/data/cb_dsv_loader.cpp, libsvm_loader.cpp,
catboost/libs/column_description/cd_parser.cpp): float features are kept as a float32 row-major matrix,
categorical features as hashed uint32 columns (plus the original strings for the hash -> string map that
``.cbm`` files carry), labels / weights / groups / pairs / baselines as numpy arrays.
"""
from __future__ import annotations

import os
from typing import Iterable, Optional, Sequence

import numpy as np

from .cat_hash import hash_cat_values

try:  # pandas is optional
    import pandas as _pd
except Exception:  # pragma: no cover
    _pd = None


class CatBoostError(Exception):
    """Raised for every user-visible error of the framework (name kept for drop-in compatibility)."""


def _is_str_like(v) -> bool:
    return isinstance(v, (str, bytes))


def _column_roles_from_cd(path: str, n_cols: Optional[int] = None):
    """Parse a column-description file: ``index<TAB>type[<TAB>name]`` per line."""
    roles, names = {}, {}
    with open(path) as fh:
        for line in fh:
            line = line.rstrip("\n")
            if not line.strip():
                continue
            parts = line.split("\t")
            idx = int(parts[0])
            roles[idx] = parts[1].strip()
            if len(parts) > 2 and parts[2].strip():
                names[idx] = parts[2].strip()
    return roles, names


_CD_ALIASES = {"Target": "Label", "DocId": "SampleId", "QueryId": "GroupId"}


def read_dsv(path: str, column_description: Optional[str] = None, delimiter: str = "\t", has_header: bool = False,
             ignore_csv_quoting: bool = False):
    """Load a delimiter-separated file.  Columns without a role are numeric features (``Num``)."""
    roles, names = ({}, {})
    if column_description:
        roles, names = _column_roles_from_cd(column_description)
    rows = []
    header = None
    with open(path) as fh:
        for li, line in enumerate(fh):
            line = line.rstrip("\r\n")
            if not line:
                continue
            parts = line.split(delimiter)
            if li == 0 and has_header:
                header = parts
                continue
            rows.append(parts)
    if not rows:
        raise CatBoostError(f"empty dataset file {path}")
    ncol = len(rows[0])
    if not roles:
        roles = {0: "Label"}
    num_idx, cat_idx = [], []
    label_idx, weight_idx, group_idx, subgroup_idx, baseline_idx, gw_idx, ts_idx = [], None, None, None, [], None, None
    feature_names = []
    for c in range(ncol):
        role = _CD_ALIASES.get(roles.get(c, "Num"), roles.get(c, "Num"))
        if role == "Num":
            num_idx.append(c)
        elif role == "Categ":
            cat_idx.append(c)
        elif role == "Label":
            label_idx.append(c)
        elif role == "Weight":
            weight_idx = c
        elif role == "GroupId":
            group_idx = c
        elif role == "SubgroupId":
            subgroup_idx = c
        elif role == "Baseline":
            baseline_idx.append(c)
        elif role == "GroupWeight":
            gw_idx = c
        elif role == "Timestamp":
            ts_idx = c
        elif role in ("Auxiliary", "SampleId", "Text", "NumVector"):
            continue
        else:
            raise CatBoostError(f"unknown column type {role!r} in column description")
        if role in ("Num", "Categ"):
            feature_names.append(names.get(c, header[c] if header else str(len(feature_names))))
    feat_cols = sorted(num_idx + cat_idx)
    n = len(rows)
    data = np.empty((n, len(feat_cols)), dtype=object)
    for j, c in enumerate(feat_cols):
        col = [r[c] for r in rows]
        if c in cat_idx:
            data[:, j] = col
        else:
            data[:, j] = [float(v) if v not in ("", "NaN", "nan", "N/A", "NA", "None", "-") else np.nan for v in col]
    cat_features = [feat_cols.index(c) for c in cat_idx]
    def _col(c, conv=float):
        return np.array([conv(r[c]) for r in rows])
    label = None
    if label_idx:
        try:
            label = np.stack([_col(c) for c in label_idx], axis=1)
        except ValueError:
            label = np.stack([_col(c, str) for c in label_idx], axis=1)
        if label.shape[1] == 1:
            label = label[:, 0]
    return dict(
        data=data, label=label, cat_features=cat_features,
        weight=_col(weight_idx) if weight_idx is not None else None,
        group_id=_col(group_idx, str) if group_idx is not None else None,
        subgroup_id=_col(subgroup_idx, str) if subgroup_idx is not None else None,
        group_weight=_col(gw_idx) if gw_idx is not None else None,
        timestamp=_col(ts_idx) if ts_idx is not None else None,
        baseline=np.stack([_col(c) for c in baseline_idx], axis=1) if baseline_idx else None,
        feature_names=feature_names,
    )


def read_libsvm(path: str):
    """``label [qid:G] index:value ...`` per line; feature indices start from 1 and grow along the line
    (catboost/libs/data/libsvm_loader.cpp:230-300); a ``qid`` field is the group id.  Missing entries are zeros."""
    labels, rows, groups, maxf = [], [], [], 0
    with open(path) as fh:
        for ln, line in enumerate(fh, 1):
            parts = line.split()
            if not parts:
                continue
            labels.append(float(parts[0]))
            row = {}
            for tok in parts[1:]:
                k, _, v = tok.partition(":")
                if k == "qid":
                    groups.append(int(v))
                    continue
                idx = int(k)
                if idx < 1:
                    raise CatBoostError(f"{path}:{ln}: libsvm feature indices start from 1")
                row[idx - 1] = float(v)
                maxf = max(maxf, idx)
            rows.append(row)
    if groups and len(groups) != len(rows):
        raise CatBoostError(f"{path}: some lines have a 'qid' field and some do not")
    X = np.zeros((len(rows), maxf), dtype=np.float32)
    for i, row in enumerate(rows):
        for k, v in row.items():
            X[i, k] = v
    out = dict(data=X, label=np.array(labels))
    if groups:
        out["group_id"] = np.array(groups)
    return out


def read_pairs(path: str):
    pairs, weights = [], []
    with open(path) as fh:
        for line in fh:
            p = line.split()
            if len(p) >= 2:
                pairs.append((int(p[0]), int(p[1])))
                weights.append(float(p[2]) if len(p) > 2 else 1.0)
    return np.array(pairs, dtype=np.int64).reshape(-1, 2), np.array(weights, dtype=np.float32)


class _ColumnView:
    """A list of equally long 1-D arrays that indexes like the object matrix ``data[:, c]`` the Pool constructor uses."""
    ndim = 2
    dtype = np.dtype(object)

    def __init__(self, cols):
        self.cols = cols
        self.shape = (len(cols[0]) if cols else 0, len(cols))

    def __getitem__(self, key):
        rows, c = key
        return self.cols[c][rows]


class Pool:
    """Dataset container accepted by ``fit`` / ``predict`` / ``cv``.

    Parameters follow ``catboost.Pool``: ``data`` may be a numpy array, a pandas DataFrame, a list of rows,
    another Pool, or a path to a dsv / ``libsvm://`` file (with ``column_description``).
    """

    def __init__(self, data, label=None, cat_features: Optional[Sequence] = None, text_features=None,
                 embedding_features=None, column_description: Optional[str] = None, pairs=None, delimiter: str = "\t",
                 has_header: bool = False, ignore_csv_quoting: bool = False, weight=None, group_id=None,
                 group_weight=None, subgroup_id=None, pairs_weight=None, baseline=None, timestamp=None,
                 feature_names: Optional[Sequence[str]] = None, feature_tags=None, thread_count: int = -1,
                 log_cout=None, log_cerr=None, data_can_be_none: bool = False):
        if isinstance(data, Pool):
            self.__dict__.update({k: (v.copy() if isinstance(v, np.ndarray) else v) for k, v in data.__dict__.items()})
            return
        if isinstance(data, (str, os.PathLike)):
            path = os.fspath(data)
            if path.startswith("quantized://"):
                self.__dict__.update(Pool.load_quantized(path[len("quantized://"):]).__dict__)
                return
            if path.startswith("libsvm://"):
                loaded = read_libsvm(path[len("libsvm://"):])
            else:
                if path.startswith("dsv://"):
                    path = path[len("dsv://"):]
                loaded = read_dsv(path, column_description, delimiter, has_header, ignore_csv_quoting)
            data = loaded.pop("data")
            label = loaded.get("label") if label is None else label
            cat_features = loaded.get("cat_features") if cat_features is None else cat_features
            weight = loaded.get("weight") if weight is None else weight
            group_id = loaded.get("group_id") if group_id is None else group_id
            subgroup_id = loaded.get("subgroup_id") if subgroup_id is None else subgroup_id
            group_weight = loaded.get("group_weight") if group_weight is None else group_weight
            baseline = loaded.get("baseline") if baseline is None else baseline
            timestamp = loaded.get("timestamp") if timestamp is None else timestamp
            feature_names = loaded.get("feature_names") if feature_names is None else feature_names
            if isinstance(pairs, (str, os.PathLike)):
                pairs, pw = read_pairs(os.fspath(pairs))
                pairs_weight = pw if pairs_weight is None else pairs_weight
        names = None
        if type(data).__name__ == "FeaturesData" and hasattr(data, "columns") and hasattr(data, "get_feature_names"):
            if cat_features is not None:
                raise CatBoostError("cat_features must not be given with FeaturesData: it knows its categorical columns")
            fcols, cat_features = data.columns()
            if feature_names is None:
                feature_names = data.get_feature_names()
            data = _ColumnView(fcols)
        if _pd is not None and isinstance(data, _pd.DataFrame):
            names = [str(c) for c in data.columns]
            if cat_features is None:
                cat_features = [i for i, dt in enumerate(data.dtypes) if str(dt) in ("object", "category", "string", "str")]
            if len(cat_features or []) or text_features or embedding_features:
                # keep the columns in their own dtypes: integer categorical columns are hashed by the native routine
                # from their distinct values, float columns are copied without a detour through Python objects
                frame_cols = [data.iloc[:, c].to_numpy() for c in range(data.shape[1])]
                data = _ColumnView(frame_cols)
            else:
                data = data.to_numpy()
        elif _pd is not None and isinstance(data, _pd.Series):
            data = data.to_numpy().reshape(-1, 1)
        if data is None:
            if not data_can_be_none:
                raise CatBoostError("data is None")
            data = np.zeros((0, 0), dtype=np.float32)
        if hasattr(data, "tocsr") and hasattr(data, "toarray"):
            # scipy.sparse matrices: the binned store is dense one-byte columns either way, so the values are laid out
            # as a dense float32 matrix here (missing entries = 0)
            if cat_features or text_features or embedding_features:
                raise CatBoostError("sparse matrices carry numerical features only; pass categorical data as a DataFrame")
            data = np.asarray(data.toarray(), dtype=np.float32)
        if not isinstance(data, (np.ndarray, _ColumnView)):
            try:
                import torch
                if isinstance(data, torch.Tensor):
                    data = data.detach().cpu().numpy()
            except Exception:  # pragma: no cover
                pass
        if not isinstance(data, (np.ndarray, _ColumnView)):
            data = np.asarray(data, dtype=object if (cat_features or text_features or embedding_features) else None)
        if data.ndim == 1:
            data = data.reshape(-1, 1)
        if data.ndim != 2:
            raise CatBoostError("data must be two-dimensional")
        n, ncol = data.shape
        if feature_names is not None:
            names = [str(x) for x in feature_names]
            if len(names) != ncol:
                raise CatBoostError("feature_names length does not match the number of columns")
        cat_idx = self._resolve_feature_indices(cat_features, names, ncol)
        self.cat_feature_indices = cat_idx
        self.feature_names = names if names is not None else [str(i) for i in range(ncol)]
        self.n_features = ncol
        text_idx = self._resolve_feature_indices(text_features, names, ncol)
        emb_idx = self._resolve_feature_indices(embedding_features, names, ncol)
        self.text_feature_indices, self.embedding_feature_indices = text_idx, emb_idx
        self.text_data = [np.array(["" if v is None else str(v) for v in data[:, c]], dtype=object) for c in text_idx]
        self.embedding_data = []
        for c in emb_idx:
            try:
                self.embedding_data.append(np.stack([np.asarray(v, dtype=np.float32).reshape(-1) for v in data[:, c]]))
            except ValueError:
                raise CatBoostError(f"embedding feature {c}: all rows must hold vectors of the same length")
        special = set(cat_idx) | set(text_idx) | set(emb_idx)
        float_idx = [c for c in range(ncol) if c not in special]
        self.float_feature_indices = float_idx
        # float matrix
        if not cat_idx and data.dtype == np.float32 and data.flags.c_contiguous:
            self.float_data = data
        elif not cat_idx and data.dtype != object:
            self.float_data = np.ascontiguousarray(data, dtype=np.float32)
        else:
            fcols = []
            for c in float_idx:
                col = data[:, c]
                try:
                    fcols.append(np.ascontiguousarray(col, dtype=np.float32))
                except (ValueError, TypeError):
                    fcols.append(np.array([np.nan if (v is None or v == "") else float(v) for v in col], dtype=np.float32))
            fd = np.empty((n, len(float_idx)), dtype=np.float32)
            if fcols and n:
                import ctypes
                from ..ops import native
                ptrs = (ctypes.c_void_p * len(fcols))(*[f.ctypes.data for f in fcols])
                native.cpu_lib().cbc_interleave_f32(ptrs, ctypes.c_int(len(fcols)), ctypes.c_longlong(n),
                                                    fd.ctypes.data_as(ctypes.c_void_p))
            self.float_data = fd
        # categorical columns: hashed + string dictionary
        self.cat_hashes = np.empty((len(cat_idx), n), dtype=np.uint32)
        self.cat_strings = []
        self._cat_distinct = {}
        for j, c in enumerate(cat_idx):
            col = data[:, c]
            h, strs, distinct = hash_cat_values(col)
            self.cat_hashes[j] = h
            self.cat_strings.append(strs)
            self._cat_distinct[j] = distinct
        self.label = self._prep_label(label, n)
        self.weight = self._prep_vec(weight, n, "weight")
        self.group_weight = self._prep_vec(group_weight, n, "group_weight")
        if self.group_weight is not None and self.weight is None:
            self.weight = self.group_weight
        self.baseline = None if baseline is None else np.asarray(baseline, dtype=np.float64).reshape(n, -1)
        self.timestamp = None if timestamp is None else np.asarray(timestamp)
        self.group_id = None
        self.subgroup_id = None if subgroup_id is None else np.asarray(subgroup_id)
        if group_id is not None:
            self.set_group_id(group_id)
        self.pairs = None
        self.pairs_weight = None
        if pairs is not None:
            self.set_pairs(pairs, pairs_weight)
        self.thread_count = thread_count
        self._quantized = None

    # ------------------------------------------------------------------ helpers
    @staticmethod
    def _resolve_feature_indices(spec, names, ncol):
        if spec is None:
            return []
        out = []
        for s in spec:
            if isinstance(s, (int, np.integer)):
                out.append(int(s))
            else:
                if names is None or str(s) not in names:
                    raise CatBoostError(f"unknown feature name {s!r}")
                out.append(names.index(str(s)))
        if any(i < 0 or i >= ncol for i in out):
            raise CatBoostError("feature index out of range")
        return sorted(set(out))

    @staticmethod
    def _prep_vec(v, n, what):
        if v is None:
            return None
        a = np.asarray(v, dtype=np.float32).reshape(-1)
        if a.shape[0] != n:
            raise CatBoostError(f"length of {what} ({a.shape[0]}) differs from the number of rows ({n})")
        return a

    @staticmethod
    def _prep_label(label, n):
        if label is None:
            return None
        if _pd is not None and isinstance(label, (_pd.Series, _pd.DataFrame)):
            label = label.to_numpy()
        a = np.asarray(label)
        if a.ndim == 2 and a.shape[1] == 1:
            a = a[:, 0]
        if a.shape[0] != n:
            raise CatBoostError(f"length of label ({a.shape[0]}) differs from the number of rows ({n})")
        return a

    # ------------------------------------------------------------------ public API (catboost.Pool compatible)
    def num_row(self) -> int:
        return int(self.float_data.shape[0]) if self.float_data.size or not len(self.cat_feature_indices) else int(self.cat_hashes.shape[1])

    def num_col(self) -> int:
        return int(self.n_features)

    @property
    def shape(self):
        return (self.num_row(), self.num_col())

    def get_label(self):
        return None if self.label is None else self.label.copy()

    def get_weight(self):
        return np.ones(self.num_row(), dtype=np.float32) if self.weight is None else self.weight.copy()

    def get_baseline(self):
        return None if self.baseline is None else self.baseline.copy()

    def get_cat_feature_indices(self):
        return list(self.cat_feature_indices)

    def get_text_feature_indices(self):
        return list(getattr(self, "text_feature_indices", None) or [])

    def get_embedding_feature_indices(self):
        return list(getattr(self, "embedding_feature_indices", None) or [])

    def num_pairs(self) -> int:
        return 0 if self.pairs is None else int(len(self.pairs))

    def get_feature_names(self):
        return list(self.feature_names)

    def get_group_id_hash(self):
        return None if self.group_id is None else self.group_id.copy()

    def get_features(self):
        out = np.empty((self.num_row(), self.n_features), dtype=np.float32)
        for j, c in enumerate(self.float_feature_indices):
            out[:, c] = self.float_data[:, j]
        for j, c in enumerate(self.cat_feature_indices):
            out[:, c] = self.cat_hashes[j].astype(np.float32)
        return out

    def is_empty_(self):
        return self.num_row() == 0

    def is_quantized(self) -> bool:
        return self._quantized is not None

    def set_weight(self, weight):
        self.weight = self._prep_vec(weight, self.num_row(), "weight")

    def set_baseline(self, baseline):
        self.baseline = None if baseline is None else np.asarray(baseline, dtype=np.float64).reshape(self.num_row(), -1)

    def set_feature_names(self, names):
        names = [str(x) for x in names]
        if len(names) != self.n_features:
            raise CatBoostError("feature_names length does not match the number of columns")
        self.feature_names = names

    def set_group_id(self, group_id):
        g = np.asarray(group_id)
        if g.shape[0] != self.num_row():
            raise CatBoostError("length of group_id differs from the number of rows")
        # groups must be contiguous (the reference requires grouped input)
        change = np.ones(len(g), dtype=bool)
        if len(g) > 1:
            change[1:] = g[1:] != g[:-1]
        ids = np.cumsum(change) - 1
        uniq_first = {}
        for k, v in zip(ids[change], g[change]):
            if v in uniq_first:
                raise CatBoostError("queries (groups) must be stored contiguously in the dataset")
            uniq_first[v] = k
        self.group_id = ids.astype(np.int64)

    def set_subgroup_id(self, subgroup_id):
        self.subgroup_id = np.asarray(subgroup_id)

    def set_group_weight(self, group_weight):
        self.group_weight = self._prep_vec(group_weight, self.num_row(), "group_weight")
        self.weight = self.group_weight

    def set_timestamp(self, timestamp):
        ts = np.asarray(timestamp)
        if len(ts) != self.num_row():
            raise CatBoostError("timestamp length does not match the number of rows")
        self.timestamp = ts

    def train_eval_split(self, has_time=False, is_classification=False, eval_fraction=0.2, save_eval_pool=True,
                         random_seed=0):
        """(train pool, eval pool): the last ``eval_fraction`` of the rows when ``has_time`` (or of the time order given
        by ``timestamp``), a random subset otherwise; whole query groups stay together; stratified by label for
        classification."""
        n = self.num_row()
        if not 0.0 < eval_fraction < 1.0:
            raise CatBoostError("eval_fraction must be inside (0, 1)")
        rng = np.random.default_rng(random_seed)
        if self.group_id is not None:
            off = self.group_offsets()
            g = np.arange(len(off) - 1)
            if not has_time:
                rng.shuffle(g)
            k = max(1, int(round(len(g) * eval_fraction)))
            ev_groups = np.sort(g[-k:])
            is_eval = np.zeros(n, dtype=bool)
            for q in ev_groups:
                is_eval[off[q]:off[q + 1]] = True
        else:
            if has_time:
                order = np.argsort(self.timestamp, kind="stable") if self.timestamp is not None else np.arange(n)
                k = max(1, int(round(n * eval_fraction)))
                is_eval = np.zeros(n, dtype=bool)
                is_eval[order[-k:]] = True
            elif is_classification and self.label is not None:
                is_eval = np.zeros(n, dtype=bool)
                lab = np.asarray(self.label).reshape(n, -1)[:, 0]
                for c in np.unique(lab):
                    idx = np.nonzero(lab == c)[0]
                    rng.shuffle(idx)
                    is_eval[idx[: max(1, int(round(len(idx) * eval_fraction)))]] = True
            else:
                is_eval = np.zeros(n, dtype=bool)
                is_eval[rng.permutation(n)[: max(1, int(round(n * eval_fraction)))]] = True
        train = self.slice(np.nonzero(~is_eval)[0])
        return train, (self.slice(np.nonzero(is_eval)[0]) if save_eval_pool else None)

    def set_pairs(self, pairs, pairs_weight=None):
        p = np.asarray(pairs, dtype=np.int64).reshape(-1, 2)
        if p.size and (p.min() < 0 or p.max() >= self.num_row()):
            raise CatBoostError("pair index out of range")
        self.pairs = p
        self.pairs_weight = (np.ones(len(p), dtype=np.float32) if pairs_weight is None
                             else np.asarray(pairs_weight, dtype=np.float32))

    def set_pairs_weight(self, pairs_weight):
        self.pairs_weight = np.asarray(pairs_weight, dtype=np.float32)

    def cat_distinct_values(self, j: int) -> np.ndarray:
        """Sorted distinct hashes of categorical feature ``j`` (position in ``cat_feature_indices``); known from the
        hashing pass for a pool built from raw columns, computed on demand otherwise."""
        cache = self.__dict__.setdefault("_cat_distinct", {})
        if j not in cache:
            cache[j] = np.unique(self.cat_hashes[j])
        return cache[j]

    def group_offsets(self):
        """Start offsets of the query groups (length n_groups + 1); one group per row when ungrouped."""
        n = self.num_row()
        if self.group_id is None:
            return np.arange(n + 1, dtype=np.int64)
        change = np.ones(n, dtype=bool)
        change[1:] = self.group_id[1:] != self.group_id[:-1]
        return np.concatenate([np.nonzero(change)[0], [n]]).astype(np.int64)

    def with_estimated(self, extra: np.ndarray, names):
        """A pool whose text / embedding columns are replaced by numeric columns computed from them (appended after the
        original feature positions, so the other features keep their indices)."""
        out = Pool.__new__(Pool)
        out.__dict__.update(self.__dict__)
        extra = np.ascontiguousarray(extra, dtype=np.float32)
        out.float_data = np.ascontiguousarray(np.concatenate([self.float_data, extra], 1), dtype=np.float32)
        out.float_feature_indices = list(self.float_feature_indices) + [self.n_features + k for k in range(extra.shape[1])]
        out.feature_names = list(self.feature_names) + [str(x) for x in names]
        out.n_features = self.n_features + extra.shape[1]
        out.text_data, out.embedding_data = [], []
        out.text_feature_indices, out.embedding_feature_indices = [], []
        out.__dict__.pop("_cat_hash_tensors", None)
        return out

    def slice(self, rindex):
        """New Pool with the given rows (order preserved)."""
        idx = np.asarray(rindex, dtype=np.int64)
        out = Pool.__new__(Pool)
        out.__dict__.update(self.__dict__)
        out.float_data = np.ascontiguousarray(self.float_data[idx])
        out.cat_hashes = np.ascontiguousarray(self.cat_hashes[:, idx])
        out._cat_distinct = {}
        out.__dict__.pop("_cat_hash_tensors", None)
        out.text_data = [t[idx] for t in getattr(self, "text_data", [])]
        out.embedding_data = [e[idx] for e in getattr(self, "embedding_data", [])]
        for k in ("label", "weight", "group_weight", "baseline", "timestamp", "group_id", "subgroup_id"):
            v = getattr(self, k)
            setattr(out, k, None if v is None else v[idx])
        if self.pairs is not None:
            pos = -np.ones(self.num_row(), dtype=np.int64)
            pos[idx] = np.arange(len(idx))
            keep = (pos[self.pairs[:, 0]] >= 0) & (pos[self.pairs[:, 1]] >= 0)
            out.pairs = pos[self.pairs[keep]]
            out.pairs_weight = self.pairs_weight[keep]
        out._quantized = None
        return out

    def slice_range(self, begin: int, end: int):
        """New Pool with rows [begin, end) as VIEWS of this pool's arrays (no copy; used by the multi-GPU launcher, whose
        workers map the parent's arrays from shared memory and keep only their own rows in sight)."""
        begin, end = int(begin), int(end)
        out = Pool.__new__(Pool)
        out.__dict__.update(self.__dict__)
        out.float_data = self.float_data[begin:end]
        out.cat_hashes = self.cat_hashes[:, begin:end]
        out._cat_distinct = {}
        out.__dict__.pop("_cat_hash_tensors", None)
        out.text_data = [t[begin:end] for t in getattr(self, "text_data", [])]
        out.embedding_data = [e[begin:end] for e in getattr(self, "embedding_data", [])]
        for k in ("label", "weight", "group_weight", "baseline", "timestamp", "group_id", "subgroup_id"):
            v = getattr(self, k)
            setattr(out, k, None if v is None else v[begin:end])
        if self.pairs is not None:
            keep = ((self.pairs[:, 0] >= begin) & (self.pairs[:, 0] < end) & (self.pairs[:, 1] >= begin) & (self.pairs[:, 1] < end))
            out.pairs = self.pairs[keep] - begin
            out.pairs_weight = self.pairs_weight[keep]
        out._quantized = None
        return out

    def quantize(self, ignored_features=None, per_float_feature_quantization=None, border_count=None,
                 max_bin=None, feature_border_type=None, nan_mode=None, input_borders=None, task_type=None,
                 used_ram_limit=None, random_seed=None, **kwargs):
        """Pre-compute borders and bins (kept on the host); later fits reuse them."""
        from .quantization import build_quantization
        bc = border_count if border_count is not None else (max_bin if max_bin is not None else 254)
        self._quantized = build_quantization(self, bc, feature_border_type or "GreedyLogSum", nan_mode or "Min",
                                             per_float_feature_quantization, input_borders)
        return self

    # ---- quantized pool files ---------------------------------------------------------------------------------
    # The role of the reference's quantized pool (catboost/private/libs/quantized_pool/serialization.cpp,
    # ``Pool.save`` / ``Pool("quantized://...")``): a data set is stored as one byte per (document, float feature) plus
    # the border grids instead of four-byte floats.  The container is this framework's own (label line + a plain-data
    # stream, utils/plainser.py), not the reference's flatbuffers layout.
    _QUANTIZED_LABEL = b"catboost_b200_quantized_pool_v1\n"

    def _save_quantized(self, fname: str):
        """Write a quantized pool to ``fname`` (``save`` comes here for quantized pools)."""
        from ..utils import plainser
        q = self._quantized
        X = self.float_data
        n, F = X.shape
        bins = np.empty((n, F), dtype=np.uint8)
        for f in range(F):
            col = X[:, f]
            b = np.searchsorted(np.asarray(q.borders[f], dtype=np.float32), col, side="left").astype(np.int64)
            # value > border goes right: bin = number of borders strictly below the value
            nanmask = np.isnan(col)
            if nanmask.any():
                b[nanmask] = len(q.borders[f]) if q.nan_is_max[f] else 0
            bins[:, f] = b
        state = dict(bins=bins, borders=[np.asarray(b, dtype=np.float32) for b in q.borders],
                     nan_is_max=np.asarray(q.nan_is_max), has_nan=np.asarray(q.has_nan), border_type=q.border_type,
                     nan_mode=q.nan_mode, cat_hashes=self.cat_hashes, label=self.label, weight=self.weight,
                     group_id=self.group_id, subgroup_id=None if self.subgroup_id is None or self.subgroup_id.dtype.kind not in "iuf" else self.subgroup_id,
                     group_weight=self.group_weight, baseline=self.baseline, pairs=self.pairs, pairs_weight=self.pairs_weight,
                     feature_names=list(self.feature_names), n_features=int(self.n_features),
                     float_feature_indices=list(self.float_feature_indices), cat_feature_indices=list(self.cat_feature_indices))
        with open(fname, "wb") as fh:
            fh.write(self._QUANTIZED_LABEL + plainser.dumps(state))

    @classmethod
    def load_quantized(cls, fname: str) -> "Pool":
        """Read a file written by ``save``.  Every float value comes back as a representative of its bin (a point
        strictly between the bin's borders), so quantising the pool again with the stored grid reproduces the stored
        bins exactly and training sees the same data set; the grid is attached, so ``fit`` does not rebuild it."""
        from ..utils import plainser
        from .quantization import FeatureQuantization
        with open(fname, "rb") as fh:
            blob = fh.read()
        if not blob.startswith(cls._QUANTIZED_LABEL):
            raise CatBoostError(f"{fname} is not a quantized pool of this framework")
        try:
            st = plainser.loads(blob[len(cls._QUANTIZED_LABEL):])
        except plainser.PlainDataError as e:
            raise CatBoostError(f"{fname} is damaged: {e}") from e
        bins = st["bins"]
        n, F = bins.shape
        X = np.empty((n, F), dtype=np.float32)
        for f in range(F):
            b = np.asarray(st["borders"][f], dtype=np.float32)
            if len(b) == 0:
                X[:, f] = 0.0
                continue
            # representatives: below the first border, between neighbours, above the last one
            rep = np.empty(len(b) + 1, dtype=np.float32)
            rep[0] = np.nextafter(b[0], np.float32(-np.inf))
            rep[1:-1] = np.nextafter(b[:-1], np.float32(np.inf)) if len(b) > 1 else rep[1:-1]
            rep[-1] = np.nextafter(b[-1], np.float32(np.inf))
            X[:, f] = rep[np.minimum(bins[:, f], len(b))]
        pool = cls.__new__(cls)
        cat_idx, float_idx = list(st["cat_feature_indices"]), list(st["float_feature_indices"])
        pool.__dict__.update(dict(
            cat_feature_indices=cat_idx, float_feature_indices=float_idx, feature_names=list(st["feature_names"]),
            n_features=int(st["n_features"]), text_feature_indices=[], embedding_feature_indices=[], text_data=[],
            embedding_data=[], float_data=X, cat_hashes=st["cat_hashes"], cat_strings=[], _cat_distinct={},
            label=st["label"], weight=st["weight"], group_weight=st["group_weight"], baseline=st["baseline"], timestamp=None,
            group_id=st["group_id"], subgroup_id=st["subgroup_id"], pairs=st["pairs"], pairs_weight=st["pairs_weight"],
            thread_count=-1))
        pool._quantized = FeatureQuantization([np.asarray(b, dtype=np.float32) for b in st["borders"]],
                                              np.asarray(st["nan_is_max"]), np.asarray(st["has_nan"]), st["border_type"],
                                              st["nan_mode"])
        return pool

    def save_quantization_borders(self, path: str):
        if self._quantized is None:
            raise CatBoostError("pool is not quantized")
        with open(path, "w") as fh:
            for f, b in enumerate(self._quantized.borders):
                for v in b:
                    fh.write(f"{f}\t{float(v):.9g}\n")

    def save(self, fname: str):
        """A quantized pool is written in the binary quantized form (read back with ``Pool("quantized://" + fname)``);
        a raw pool as a tab-separated file with the label in column 0 (plus ``fname + '.cd'``)."""
        if self._quantized is not None:
            return self._save_quantized(fname)
        n = self.num_row()
        feats = self.get_features().astype(object)
        for j, c in enumerate(self.cat_feature_indices):
            inv = {h: s for s, h in self.cat_strings[j].items()}
            feats[:, c] = [inv.get(int(h), str(int(h))) for h in self.cat_hashes[j]]
        with open(fname, "w") as fh:
            for i in range(n):
                lab = "" if self.label is None else str(self.label[i])
                fh.write("\t".join([lab] + [str(v) for v in feats[i]]) + "\n")
        with open(fname + ".cd", "w") as fh:
            fh.write("0\tLabel\n")
            for c in self.cat_feature_indices:
                fh.write(f"{c + 1}\tCateg\n")

    def __len__(self):
        return self.num_row()


def to_pool(data, label=None, **kw) -> Pool:
    if isinstance(data, Pool):
        if label is not None:
            raise CatBoostError("label must be None when data is a Pool")
        return data
    return Pool(data, label, **kw)
