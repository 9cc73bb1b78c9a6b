"""Float-feature quantisation and the binned feature store.

Borders are chosen on the host from a bounded random sample (the reference also builds borders on the CPU
from at most 200 000 rows: catboost/libs/data/quantization.cpp, library/cpp/grid_creator/binarization.cpp);
the binning itself runs on the training device (hand-written kernel ``cb_quantize`` on the GPU, OpenMP on the
CPU) and writes the packed group store directly.

Binned store layout (replaces the reference's compressed index, catboost/cuda/gpu_data/compressed_index.h):
``bins`` is int32 ``[G][npad]`` (uint32 payload): byte ``j`` of word ``[g][i]`` is the bin of flat feature
``4g+j`` for document ``i``.  A level of tree search streams each group row once with 16-byte loads.
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass, field
from typing import List, Optional

import numpy as np
import torch

from ..ops import native
from .pool import CatBoostError

BORDER_TYPES = {"Median": 0, "GreedyLogSum": 1, "Uniform": 2, "UniformAndQuantiles": 3, "MinEntropy": 4,
                "MaxLogSum": 5, "GreedyMinEntropy": 6}
MAX_SAMPLE_FOR_BORDERS = 200_000


def _ptr(a):
    if a is None:
        return None
    if isinstance(a, torch.Tensor):
        return ctypes.c_void_p(a.data_ptr())
    return a.ctypes.data_as(ctypes.c_void_p)


@dataclass
class FeatureQuantization:
    """Borders of every float feature of a pool (index = position among the float features)."""
    borders: List[np.ndarray]
    nan_is_max: np.ndarray          # uint8 per float feature
    has_nan: np.ndarray             # uint8 per float feature
    border_type: str = "GreedyLogSum"
    nan_mode: str = "Min"

    def n_features(self):
        return len(self.borders)


def select_borders(sample: np.ndarray, border_count: int, border_type: str = "GreedyLogSum"):
    """Borders for every column of a float32 row-major sample."""
    if border_type not in BORDER_TYPES:
        raise CatBoostError(f"unknown feature_border_type {border_type!r}")
    if not (1 <= border_count <= 255):
        raise CatBoostError("border_count must be in [1, 255] (one-byte bins)")
    sample = np.ascontiguousarray(sample, dtype=np.float32)
    n, F = sample.shape
    out = np.zeros((F, border_count), dtype=np.float32)
    counts = np.zeros(F, dtype=np.int32)
    has_nan = np.zeros(F, dtype=np.uint8)
    if n and F:
        lib = native.cpu_lib()
        # Launchers that start one process per GPU pin OMP_NUM_THREADS to 1; border selection runs on one rank while
        # the others wait for it, so it takes the cores this process may run on, whatever the variable says
        old = int(lib.cbc_num_threads())
        try:
            cores = len(os.sched_getaffinity(0))
        except (AttributeError, OSError):
            cores = os.cpu_count() or 1
        want = max(old, min(cores, 64))
        if want != old:
            lib.cbc_set_num_threads(want)
        lib.cbc_select_borders_matrix(_ptr(sample), ctypes.c_longlong(n), ctypes.c_int(F),
                                                   ctypes.c_longlong(sample.strides[0] // 4),
                                                   ctypes.c_int(border_count), ctypes.c_int(BORDER_TYPES[border_type]),
                                                   _ptr(out), _ptr(counts), _ptr(has_nan))
        if want != old:
            lib.cbc_set_num_threads(old)
    return [out[f, :counts[f]].copy() for f in range(F)], has_nan


def _border_sample(X: np.ndarray, seed: int, ctx=None):
    """Rows the float borders are chosen from, and per-feature NaN flags over ALL rows.

    One process: every row, or a seeded subsample of MAX_SAMPLE_FOR_BORDERS rows.  Several ranks: the same rule applied
    to the concatenation of the ranks' shards in rank order -- every rank draws the same global row numbers, picks the
    ones it holds, and the pieces are gathered on rank 0 (which returns the sample; the others return None).  The
    borders therefore do not depend on how the rows are split over the ranks, and a NaN that only occurs on one rank
    is seen (the reference builds its grid from the whole learn set, catboost/libs/data/quantization.cpp)."""
    n = X.shape[0]
    if ctx is None or not ctx.is_distributed:
        if n > MAX_SAMPLE_FOR_BORDERS:
            # Floyd's sampler of the Generator API: O(sample), where RandomState.choice permutes all n rows
            rng = np.random.default_rng(seed)
            idx = np.sort(rng.choice(n, MAX_SAMPLE_FOR_BORDERS, replace=False, shuffle=False))
            return X[idx], None
        return X, None
    counts = ctx.all_gather_object(int(n))
    total, off = int(sum(counts)), int(sum(counts[: ctx.rank]))
    if total > MAX_SAMPLE_FOR_BORDERS:
        rng = np.random.default_rng(seed)
        idx = np.sort(rng.choice(total, MAX_SAMPLE_FOR_BORDERS, replace=False, shuffle=False))
        mine = idx[(idx >= off) & (idx < off + n)] - off
        part = X[mine]
    else:
        part = X
    # a NaN anywhere in a column sets its flag (one pass over the shard, blocked to keep the temporary small)
    nan_local = np.zeros(X.shape[1], dtype=bool)
    for r0 in range(0, n, 1 << 18):
        nan_local |= np.isnan(X[r0:r0 + (1 << 18)]).any(0)
    flags = ctx.all_gather_object(nan_local)
    has_nan_all = np.logical_or.reduce(flags) if flags else nan_local
    sample = ctx.gather_rows(np.ascontiguousarray(part, dtype=np.float32), 0)
    return sample, has_nan_all


def build_quantization(pool, border_count: int = 254, border_type: str = "GreedyLogSum", nan_mode: str = "Min",
                       per_float_feature_quantization=None, input_borders=None, seed: int = 0,
                       ctx=None) -> FeatureQuantization:
    """Float border grids.  With a distributed ``ctx`` this is a collective call: the grid is built on rank 0 from a
    sample of all ranks' rows and broadcast."""
    X = pool.float_data
    n, F = X.shape
    if nan_mode not in ("Min", "Max", "Forbidden"):
        raise CatBoostError(f"unknown nan_mode {nan_mode!r}")
    sample, has_nan_all = _border_sample(X, seed, ctx)
    if ctx is not None and ctx.is_distributed:
        q = None
        if ctx.rank == 0:
            class _Rows:
                float_data = sample
            q = build_quantization(_Rows, border_count, border_type, nan_mode, per_float_feature_quantization,
                                   input_borders, seed)
            q.has_nan = np.asarray(has_nan_all).astype(np.uint8)
        q = ctx.broadcast_object(q, 0)
        if nan_mode == "Forbidden" and np.asarray(has_nan_all).any():
            raise CatBoostError("NaN values are present but nan_mode is Forbidden")
        return q
    borders, has_nan = select_borders(sample, min(border_count, 255), border_type)
    if nan_mode == "Forbidden" and has_nan.any():
        raise CatBoostError("NaN values are present but nan_mode is Forbidden")
    if per_float_feature_quantization:
        specs = per_float_feature_quantization
        if isinstance(specs, str):
            specs = [specs]
        for spec in specs:
            parts = str(spec).split(":")
            f = int(parts[0])
            kw = dict(p.split("=") for p in parts[1:])
            bc = int(kw.get("border_count", border_count))
            bt = kw.get("border_type", border_type)
            b, _ = select_borders(sample[:, f:f + 1], min(bc, 255), bt)
            borders[f] = b[0]
    if input_borders is not None:
        per = {}
        if isinstance(input_borders, str):
            with open(input_borders) as fh:
                for line in fh:
                    p = line.split()
                    if len(p) >= 2:
                        per.setdefault(int(p[0]), []).append(float(p[1]))
        else:
            per = {int(k): list(v) for k, v in dict(input_borders).items()}
        for f, b in per.items():
            borders[f] = np.array(sorted(set(b)), dtype=np.float32)[:255]
    nan_is_max = np.full(F, 1 if nan_mode == "Max" else 0, dtype=np.uint8)
    return FeatureQuantization(borders, nan_is_max, has_nan, border_type, nan_mode)


@dataclass
class FlatFeature:
    """One column of the binned store and what it means for the model."""
    kind: str                         # 'float' | 'onehot' | 'ctr'
    source: int                       # float-feature index / cat-feature index / ctr index
    borders: Optional[np.ndarray] = None    # float & ctr features
    values: Optional[np.ndarray] = None     # one-hot: hash value per bin
    ctr: object = None                # CtrDescriptor for 'ctr'
    n_bins: int = 1


@dataclass
class BinnedStore:
    bins: torch.Tensor                # int32 [G][npad]
    n: int
    npad: int
    features: List[FlatFeature]
    feat_off: torch.Tensor            # int32 [F+1] on device
    feat_nb: torch.Tensor             # int32 [F]
    feat_onehot: torch.Tensor         # uint8 [F]
    feat_weight: torch.Tensor         # float32 [F]
    feat_off_host: np.ndarray = field(default=None)
    feat_nb_host: np.ndarray = field(default=None)
    handle: int = 0                   # native CbData* (CUDA only)

    @property
    def F(self):
        return len(self.features)

    @property
    def G(self):
        return (self.F + 3) // 4

    @property
    def TB(self):
        return int(self.feat_off_host[-1])

    @property
    def device(self):
        return self.bins.device

    @property
    def max_bins(self):
        return int(self.feat_nb_host.max()) if len(self.feat_nb_host) else 1

    def column(self, f: int) -> torch.Tensor:
        """uint8 bins of one flat feature (for tests and the generic paths)."""
        w = self.bins[f // 4, : self.n]
        return ((w >> (8 * (f % 4))) & 255).to(torch.uint8)

    def refresh_handle(self):
        if self.bins.is_cuda:
            lib = native.cuda_lib()
            if self.handle:
                lib.cb_data_destroy(ctypes.c_void_p(self.handle))
            self.handle = lib.cb_data_create(_ptr(self.bins), self.npad, self.n, self.F, _ptr(self.feat_off),
                                             _ptr(self.feat_nb), _ptr(self.feat_onehot), _ptr(self.feat_weight),
                                             self.TB)
            if not self.handle:
                raise RuntimeError("cb_data_create failed")

    def __del__(self):  # pragma: no cover
        try:
            if self.handle:
                native.cuda_lib().cb_data_destroy(ctypes.c_void_p(self.handle))
        except Exception:
            pass


def pad_rows(n: int) -> int:
    return max(256, (n + 255) // 256 * 256)


def make_store(features: List[FlatFeature], n: int, device, feature_weights=None) -> BinnedStore:
    """Allocate an all-zero store for the given flat features."""
    F = len(features)
    G = max(1, (F + 3) // 4)
    npad = pad_rows(n)
    nb = np.array([f.n_bins for f in features], dtype=np.int32) if F else np.zeros(0, np.int32)
    if F and nb.max() > 256:
        raise CatBoostError("a feature has more than 256 bins")
    off = np.zeros(F + 1, dtype=np.int32)
    for i in range(F):
        off[i + 1] = off[i] + (int(nb[i]) + 3) // 4 * 4
    onehot = np.array([1 if f.kind == "onehot" else 0 for f in features], dtype=np.uint8)
    fw = np.ones(F, dtype=np.float32) if feature_weights is None else np.asarray(feature_weights, dtype=np.float32)
    dev = torch.device(device)
    store = BinnedStore(
        bins=torch.zeros((G, npad), dtype=torch.int32, device=dev), n=n, npad=npad, features=features,
        feat_off=torch.from_numpy(off).to(dev), feat_nb=torch.from_numpy(nb).to(dev),
        feat_onehot=torch.from_numpy(onehot).to(dev), feat_weight=torch.from_numpy(fw).to(dev),
        feat_off_host=off, feat_nb_host=nb)
    store.refresh_handle()
    return store


LAST_QUANTIZE = {"kernel": None}       # which device kernel the latest quantize_floats_into call used


def quantize_floats_into(store: BinnedStore, X: np.ndarray, quant: FeatureQuantization, flat_begin: int = 0,
                         float_subset: Optional[List[int]] = None, chunk_rows: int = 0, pinned: bool = True):
    """Bin the float columns of ``X`` (host, float32 row-major) into flat features
    ``flat_begin .. flat_begin + len(subset)`` of the store.  ``flat_begin`` must be a multiple of 4 unless the
    CPU path is used; the float features always come first in practice (flat_begin == 0).
    Returns the number of bytes copied host -> device."""
    n, Ftot = X.shape
    subset = list(range(Ftot)) if float_subset is None else list(float_subset)
    F = len(subset)
    if F == 0 or n == 0:
        return 0
    if flat_begin % 4 != 0:
        raise CatBoostError("float features must start at a group boundary")
    borders = np.concatenate([quant.borders[f] for f in subset]).astype(np.float32) if F else np.zeros(0, np.float32)
    boff = np.zeros(F + 1, dtype=np.int32)
    boff[1:] = np.cumsum([len(quant.borders[f]) for f in subset])
    nanmax = np.ascontiguousarray(quant.nan_is_max[subset])
    if float_subset is not None and subset != list(range(Ftot)):
        X = np.ascontiguousarray(X[:, subset])
    ld = X.strides[0] // 4
    dev = store.bins.device
    g0 = flat_begin // 4
    if dev.type == "cpu":
        if len(borders) == 0:
            borders = np.zeros(1, np.float32)
        native.cpu_lib().cbc_quantize(_ptr(X), ctypes.c_longlong(n), ctypes.c_int(F), ctypes.c_longlong(ld),
                                      _ptr(borders), _ptr(boff), _ptr(nanmax), _ptr(store.bins[g0:]),
                                      ctypes.c_longlong(store.npad), ctypes.c_longlong(0))
        return 0
    lib = native.cuda_lib()
    d_borders = torch.from_numpy(borders if len(borders) else np.zeros(1, np.float32)).to(dev)
    d_boff = torch.from_numpy(boff).to(dev)
    d_nan = torch.from_numpy(nanmax).to(dev)
    if chunk_rows <= 0:
        chunk_rows = max(1, (256 << 20) // max(1, 4 * ld))     # ~256 MiB staging chunks
    stream = torch.cuda.current_stream(dev)
    copied = 0
    use_tma = os.environ.get("CB200_QUANTIZE_TMA", "1") != "0"
    used_tma = False
    d_status = torch.zeros(1, dtype=torch.int32, device=dev)
    xt = torch.from_numpy(X)
    for r0 in range(0, n, chunk_rows):
        r1 = min(n, r0 + chunk_rows)
        src = xt[r0:r1]
        if pinned and not src.is_pinned():
            try:
                src = src.pin_memory()
            except RuntimeError:
                pass
        d_chunk = src.to(dev, non_blocking=True)
        copied += (r1 - r0) * ld * 4
        rc = -2
        if use_tma:
            # tiled bulk copies into shared memory (needs a 16-byte aligned base and row pitch)
            rc = lib.cb_quantize_tma(_ptr(d_chunk), r1 - r0, F, d_chunk.stride(0), _ptr(d_borders), _ptr(d_boff),
                                     _ptr(d_nan), _ptr(store.bins[g0:]), store.npad, r0, _ptr(d_status),
                                     ctypes.c_void_p(stream.cuda_stream))
            if rc not in (0, -2):
                native.cuda_check(rc, "cb_quantize_tma")
        if rc == -2:
            native.cuda_check(lib.cb_quantize(_ptr(d_chunk), r1 - r0, F, d_chunk.stride(0), _ptr(d_borders),
                                              _ptr(d_boff), _ptr(d_nan), _ptr(store.bins[g0:]), store.npad, r0,
                                              ctypes.c_void_p(stream.cuda_stream)), "cb_quantize")
        else:
            used_tma = True
        d_chunk.record_stream(stream)
    LAST_QUANTIZE["kernel"] = "tma" if used_tma else "plain"
    if used_tma and int(d_status.item()) != 0:
        raise RuntimeError(f"cb_quantize_tma: a bulk copy did not arrive in time (status {int(d_status.item()):#x})")
    return copied


def pack_columns_into(store: BinnedStore, cols: torch.Tensor, flat_begin: int):
    """Write already-binned uint8 columns ``[F][n]`` (on the store's device) as flat features
    ``flat_begin ..``."""
    F, n = cols.shape
    if F == 0:
        return
    cols = cols.contiguous()
    if store.bins.device.type == "cpu":
        native.cpu_lib().cbc_pack_bins(_ptr(cols), ctypes.c_longlong(n), ctypes.c_longlong(cols.stride(0)),
                                       ctypes.c_int(F), ctypes.c_int(flat_begin), _ptr(store.bins),
                                       ctypes.c_longlong(store.npad), ctypes.c_longlong(0))
    else:
        stream = torch.cuda.current_stream(store.bins.device)
        native.cuda_check(native.cuda_lib().cb_pack_bins(_ptr(cols), n, cols.stride(0), F, flat_begin,
                                                         _ptr(store.bins), store.npad, 0,
                                                         ctypes.c_void_p(stream.cuda_stream)), "cb_pack_bins")
