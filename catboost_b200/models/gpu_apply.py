"""GPU batch apply of float-only oblivious models (``predict(..., task_type='GPU')``).

The reference's GPU evaluator quantises into an intermediate uchar4 buffer and evaluates in a second kernel
(catboost/libs/model/cuda/evaluator.cu:85-343, float-only / oblivious / one-dimensional only).  Here one kernel
(``cb_predict_kernel``) stages the bins of a tile of rows in shared memory (32 features at a time, their borders in
shared memory, a warp reading one row's values as one contiguous piece) and walks all trees; models with up
to 8 output dimensions are supported.  Rows are streamed from pinned host memory in chunks so that any dataset
size fits; when the caller's matrix already lives in pinned memory the chunks are copied straight from it.  With
several devices the rows are cut into one contiguous range per device and every range is streamed by its own host
thread (the reference's GPU evaluator is single-device: catboost/libs/model/cuda/evaluator.cu).
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from ..ops import native


_COPY_POOL = None


def _parallel_copy(dst: np.ndarray, src: np.ndarray, threads: int = 8):
    """dst[...] = src with several host threads (numpy releases the interpreter lock while it copies): the copy of
    pageable rows into a pinned staging buffer is what limits apply from host memory, and one thread moves about a
    third of what the memory system can."""
    global _COPY_POOL
    n = dst.shape[0]
    if n < 65536 or threads <= 1:
        np.copyto(dst, src)
        return
    if _COPY_POOL is None:
        from concurrent.futures import ThreadPoolExecutor
        _COPY_POOL = ThreadPoolExecutor(max_workers=8, thread_name_prefix="cb200-copy")
    cuts = [n * k // threads for k in range(threads + 1)]
    futs = [_COPY_POOL.submit(np.copyto, dst[cuts[k]:cuts[k + 1]], src[cuts[k]:cuts[k + 1]]) for k in range(threads)]
    for f in futs:
        f.result()


class GpuPredictor:
    """Model arrays resident on one GPU; ``predict`` may be called repeatedly (its staging buffers are kept between
    calls when they are below 1 GiB of pinned memory)."""

    # used features one launch of the quantising kernel can hold (one byte per feature and row of a 256-row block plus the
    # staged borders, within 224 KB of shared memory); models above it are evaluated as a sum of tree ranges
    MAX_USED = 700

    @staticmethod
    def _slice_packed(p, t0, t1):
        """The packed arrays of trees [t0, t1) as a model of their own: only the features those trees use."""
        depth = np.asarray(p["depth"])[t0:t1]
        s0 = int(np.asarray(p["soff"])[t0])
        s1 = s0 + int(depth.sum())
        sfeat_old = np.asarray(p["sfeat"], dtype=np.int64)[s0:s1]
        keep = np.unique(sfeat_old)                                   # positions in the full model's used list
        remap = np.full(len(p["used"]), -1, dtype=np.int64)
        remap[keep] = np.arange(len(keep))
        boff = np.asarray(p["boff"], dtype=np.int64)
        borders = np.asarray(p["borders"], dtype=np.float32)
        nb = (boff[keep + 1] - boff[keep]) if len(keep) else np.zeros(0, dtype=np.int64)
        new_boff = np.zeros(len(keep) + 1, dtype=np.int32)
        new_boff[1:] = np.cumsum(nb)
        new_borders = np.concatenate([borders[boff[k]:boff[k + 1]] for k in keep]) if len(keep) else np.zeros(1, np.float32)
        l0 = int(np.asarray(p["loff"])[t0])
        leaves = (1 << depth.astype(np.int64))
        loff = np.zeros(len(depth), dtype=np.int64)
        loff[1:] = np.cumsum(leaves)[:-1]
        soff = np.zeros(len(depth), dtype=np.int32)
        soff[1:] = np.cumsum(depth)[:-1]
        return dict(T=int(t1 - t0), used=np.asarray(p["used"])[keep].astype(np.int32), borders=new_borders, boff=new_boff,
                    depth=depth.astype(np.int32), soff=soff, sfeat=remap[sfeat_old].astype(np.uint16),
                    sbin=np.asarray(p["sbin"])[s0:s1], loff=loff,
                    vals=np.ascontiguousarray(np.asarray(p["vals"])[l0:l0 + int(leaves.sum())]),
                    nanmax=np.asarray(p["nanmax"])[keep])

    def __init__(self, model, device=None, packed=None, with_bias=True):
        p = packed if packed is not None else model._packed_oblivious()
        self.dev = torch.device(device if device is not None else "cuda")
        if self.dev.index is None:
            self.dev = torch.device("cuda", torch.cuda.current_device())
        t = lambda a, dt=None: torch.from_numpy(np.ascontiguousarray(a if dt is None else a.astype(dt))).to(self.dev)
        self.used, self.borders, self.boff = t(p["used"]), t(p["borders"]), t(p["boff"])
        self.nanmax = t(p["nanmax"])
        self.depth, self.soff = t(p["depth"]), t(p["soff"])
        self.sfeat, self.sbin, self.loff = t(p["sfeat"]), t(p["sbin"]), t(p["loff"])
        self.vals = t(p["vals"], np.float32)
        self.T, self.dims, self.U = p["T"], model.dims, len(p["used"])
        boff = np.asarray(p["boff"], dtype=np.int64)
        self.max_borders = int(np.diff(boff).max()) if len(boff) > 1 else 1
        self.scale = float(model.scale)
        self.bias = t(np.broadcast_to(model.bias if with_bias else np.zeros(1), (model.dims,)), np.float32)
        if self.dims > 8:
            raise ValueError("GPU apply supports up to 8 prediction dimensions")
        self.lib = native.cuda_lib()
        # Models that use many features are evaluated from the raw values (cb_predict_wide.cu): split = (column, border).
        # Chosen when the binary searches of the quantising kernel (7 reads per used feature and row) would outnumber
        # the reads of the tree walk itself (one per split and row), and the row tile fits in shared memory.
        used, boff = np.asarray(p["used"], dtype=np.int64), np.asarray(p["boff"], dtype=np.int64)
        sfeat, sbin = np.asarray(p["sfeat"], dtype=np.int64), np.asarray(p["sbin"], dtype=np.int64)
        self.S = int(len(sfeat))
        self.F_stage = int(used.max()) + 1 if len(used) else 0
        self.total_leaf_floats = int(np.asarray(p["vals"]).size)
        self.wide = None
        self.status = torch.zeros(1, dtype=torch.int32, device=self.dev)     # set by a device wait that ran out of time
        import os
        mode = os.environ.get("CB200_PREDICT_WIDE", "auto")
        want = mode == "1" or (mode == "auto" and 7 * self.U > self.S and self.U > 200)
        if want and self.S > 0 and self.lib.cb_predict_wide_fits(self.F_stage, self.S, self.T, self.dims, self.total_leaf_floats):
            nanmax_col = np.zeros(self.F_stage, dtype=np.uint8)
            nanmax_col[used] = np.asarray(p["nanmax"], dtype=np.uint8)
            self.wide = dict(col=t(used[sfeat], np.int32), border=t(np.asarray(p["borders"], dtype=np.float32)[boff[sfeat] + sbin]),
                             nanmax=t(nanmax_col) if nanmax_col.any() else None)
        # Too many used features for one launch of either kernel (2000 columns: the raw-value kernel's row tile does not
        # fit either): consecutive tree ranges that each use at most MAX_USED features, outputs summed.
        self.parts = None
        if self.wide is None and self.U > self.MAX_USED:
            ranges, t0, seen = [], 0, set()
            soff_h, depth_h = np.asarray(p["soff"], dtype=np.int64), np.asarray(p["depth"], dtype=np.int64)
            for tr in range(self.T):
                feats = set(sfeat[soff_h[tr]:soff_h[tr] + depth_h[tr]].tolist())
                if len(seen | feats) > self.MAX_USED and tr > t0:
                    ranges.append((t0, tr))
                    t0, seen = tr, set()
                seen |= feats
            ranges.append((t0, self.T))
            self.parts = [GpuPredictor(model, self.dev, packed=self._slice_packed(p, a, b), with_bias=(k == 0))
                          for k, (a, b) in enumerate(ranges)]

    def predict_device(self, X: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
        """X: float32 [n, F] on the device (row stride arbitrary).  Returns float32 [dims, n]."""
        n = X.shape[0]
        if out is None:
            out = torch.empty((self.dims, n), dtype=torch.float32, device=self.dev)
        if self.parts is not None:
            self.parts[0].predict_device(X, out)
            tmp = torch.empty_like(out)
            for part in self.parts[1:]:
                out += part.predict_device(X, tmp)
            return out
        P = lambda a: ctypes.c_void_p(a.data_ptr()) if a is not None else None
        st = ctypes.c_void_p(torch.cuda.current_stream(self.dev).cuda_stream)
        if self.wide is not None and X.shape[1] >= self.F_stage and X.stride(1) == 1:
            w = self.wide
            native.cuda_check(self.lib.cb_predict_oblivious_wide(
                P(X), n, X.stride(0), self.F_stage, P(w["nanmax"]), P(self.depth), P(self.soff), P(w["col"]), P(w["border"]),
                P(self.loff), P(self.vals), self.T, self.S, self.dims, self.total_leaf_floats, self.scale, P(self.bias),
                P(out), P(self.status), st), "cb_predict_oblivious_wide")
            return out
        native.cuda_check(self.lib.cb_predict_oblivious(P(X), n, X.stride(0), P(self.used), P(self.borders), P(self.boff),
                                                        P(self.nanmax), self.U, P(self.depth), P(self.soff),
                                                        P(self.sfeat), P(self.sbin), P(self.loff), P(self.vals), self.T,
                                                        self.dims, self.scale, P(self.bias), P(out), self.max_borders,
                                                        self.total_leaf_floats, st),
                          "cb_predict_oblivious")
        return out

    def predict(self, X: np.ndarray, chunk_rows: int = 0, out: np.ndarray = None) -> np.ndarray:
        """Rows from host memory, in chunks through two pinned staging buffers and two streams: while one chunk is
        copied to the device and evaluated, the host fills the other buffer, and results come back asynchronously."""
        X = np.ascontiguousarray(X, dtype=np.float32)
        n, F = X.shape
        res = np.empty((n, self.dims), dtype=np.float64) if out is None else out
        if n == 0:
            return res
        if chunk_rows <= 0:
            # about 256 MB of floats per buffer; one geometry for every batch above 64K rows, so that the buffers kept
            # from the previous call fit the next one whatever its length
            chunk_rows = max(4096, (64 << 20) // max(F, 1)) if n > 65536 else n
        xt = torch.from_numpy(X)
        src_pinned = bool(xt.is_pinned())            # the caller's rows are page-locked: no staging copy needed
        with torch.cuda.device(self.dev):
            nbuf = 2 if n > 65536 or n > chunk_rows else 1
            key = (chunk_rows, F, src_pinned, nbuf)
            bufs = self.__dict__.setdefault("_bufs", {}).get(key)
            if bufs is None:
                stage = [None if src_pinned else torch.empty((chunk_rows, F), dtype=torch.float32).pin_memory()
                         for _ in range(nbuf)]
                back = [torch.empty((self.dims, chunk_rows), dtype=torch.float32).pin_memory() for _ in range(nbuf)]
                dbuf = [torch.empty((chunk_rows, F), dtype=torch.float32, device=self.dev) for _ in range(nbuf)]
                dout = [torch.empty((self.dims, chunk_rows), dtype=torch.float32, device=self.dev) for _ in range(nbuf)]
                streams = [torch.cuda.Stream(self.dev) for _ in range(nbuf)]
                bufs = (stage, back, dbuf, dout, streams)
                pinned = nbuf * chunk_rows * (self.dims + (0 if src_pinned else F)) * 4
                if pinned <= (1 << 30):
                    while len(self._bufs) >= 2:                   # at most two geometries are kept (a small and a large one)
                        self._bufs.pop(next(iter(self._bufs)))
                    self._bufs[key] = bufs
            stage, back, dbuf, dout, streams = bufs
            pending = [None] * nbuf                          # (event, r0, r1) of the chunk in flight on every buffer
            cur = torch.cuda.current_stream(self.dev)
            for st in streams:
                st.wait_stream(cur)

            def drain(k):
                if pending[k] is not None:
                    ev, r0, r1, h_out = pending[k]
                    ev.synchronize()
                    res[r0:r1] = h_out.t().numpy()
                    pending[k] = None

            for c, r0 in enumerate(range(0, n, chunk_rows)):
                k = c % nbuf
                r1 = min(n, r0 + chunk_rows)
                m = r1 - r0
                drain(k)
                if not src_pinned:
                    _parallel_copy(stage[k][:m].numpy(), X[r0:r1])
                h_src = xt[r0:r1] if src_pinned else stage[k][:m]
                # a short last chunk uses the front of the buffers as a dense [dims, m] block
                d_out = dout[k].view(-1)[: self.dims * m].view(self.dims, m)
                h_out = back[k].view(-1)[: self.dims * m].view(self.dims, m)
                with torch.cuda.stream(streams[k]):
                    dbuf[k][:m].copy_(h_src, non_blocking=True)
                    self.predict_device(dbuf[k][:m], d_out)
                    h_out.copy_(d_out, non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(streams[k])
                pending[k] = (ev, r0, r1, h_out)
            for k in range(nbuf):
                drain(k)
            cur.wait_stream(streams[0])
            self.check_status()
        return res

    def check_status(self):
        """Raise if a bounded device wait of an apply kernel ran out of time (the results of that call are not valid)."""
        code = int(self.status.item())
        if code:
            self.status.zero_()
            raise RuntimeError(f"GPU apply: a device wait timed out (status 0x{code:x})")


class MultiGpuPredictor:
    """The same model resident on several GPUs of this machine; a batch is cut into one contiguous row range per device
    and the ranges are evaluated concurrently, each by its own host thread (copies and launches release the interpreter
    lock, so the threads overlap)."""

    def __init__(self, model, devices):
        self.devices = [torch.device("cuda", int(d)) for d in devices]
        self.parts = [GpuPredictor(model, d) for d in self.devices]
        self.T, self.dims = self.parts[0].T, self.parts[0].dims

    def predict(self, X: np.ndarray, chunk_rows: int = 0) -> np.ndarray:
        import threading
        X = np.ascontiguousarray(X, dtype=np.float32)
        n = X.shape[0]
        res = np.empty((n, self.dims), dtype=np.float64)
        R = len(self.parts)
        if n < 4096 * R or R == 1:
            return self.parts[0].predict(X, chunk_rows, res)
        bounds = [n * r // R for r in range(R + 1)]
        errors = []

        def work(r):
            try:
                self.parts[r].predict(X[bounds[r]:bounds[r + 1]], chunk_rows, res[bounds[r]:bounds[r + 1]])
            except Exception as e:          # surfaced on the calling thread
                errors.append(e)

        threads = [threading.Thread(target=work, args=(r,)) for r in range(R)]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        if errors:
            raise errors[0]
        return res


def predict_oblivious_gpu(model, X: np.ndarray, device=None) -> np.ndarray:
    """``device``: None (current device), a device / ordinal, or a CatBoost devices string ('0-3', '0:2') or list:
    several devices shard the rows."""
    devs = None
    if isinstance(device, (list, tuple)):
        devs = [int(d) for d in device]
    elif isinstance(device, str) and not device.startswith("cuda"):
        from ..params import parse_devices
        devs = parse_devices(device, torch.cuda.device_count())
    if devs is not None and len(devs) > 1:
        key = "_gpu_predictor_multi"
        pred = model.__dict__.get(key)
        if pred is None or pred.T != len(model.trees) or [d.index for d in pred.devices] != devs:
            pred = MultiGpuPredictor(model, devs)
            model.__dict__[key] = pred
        return pred.predict(X)
    if devs is not None:
        device = torch.device("cuda", devs[0])
    key = "_gpu_predictor"
    pred = model.__dict__.get(key)
    if pred is None or pred.T != len(model.trees) or (device is not None and torch.device(device) != pred.dev
                                                      and torch.device(device).index is not None):
        pred = GpuPredictor(model, device)
        model.__dict__[key] = pred
    return pred.predict(X)
