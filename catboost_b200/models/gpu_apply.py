"""GPU batch apply of float-only oblivious models (``predict(..., task_type='GPU')``).

The reference's GPU evaluator quantises into an intermediate uchar4 buffer and evaluates in a second kernel
(catboost/libs/model/cuda/evaluator.cu:85-343, float-only / oblivious / one-dimensional only).  Here one kernel
(``cb_predict_kernel``) stages the bins of a 256-row tile in shared memory and walks all trees; models with up
to 8 output dimensions are supported.  Rows are streamed from pinned host memory in chunks so that any dataset
size fits.
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from ..ops import native


class GpuPredictor:
    """Model arrays resident on one GPU; ``predict`` may be called repeatedly."""

    def __init__(self, model, device=None):
        p = model._packed_oblivious()
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
        self.scale = float(model.scale)
        self.bias = t(np.broadcast_to(model.bias, (model.dims,)), np.float32)
        if self.dims > 8:
            raise ValueError("GPU apply supports up to 8 prediction dimensions")
        self.lib = native.cuda_lib()

    def predict_device(self, X: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
        """X: float32 [n, F] on the device (row stride arbitrary).  Returns float32 [dims, n]."""
        n = X.shape[0]
        if out is None:
            out = torch.empty((self.dims, n), dtype=torch.float32, device=self.dev)
        P = lambda a: ctypes.c_void_p(a.data_ptr())
        st = ctypes.c_void_p(torch.cuda.current_stream(self.dev).cuda_stream)
        native.cuda_check(self.lib.cb_predict_oblivious(P(X), n, X.stride(0), P(self.used), P(self.borders), P(self.boff),
                                                        P(self.nanmax), self.U, P(self.depth), P(self.soff),
                                                        P(self.sfeat), P(self.sbin), P(self.loff), P(self.vals), self.T,
                                                        self.dims, self.scale, P(self.bias), P(out), st),
                          "cb_predict_oblivious")
        return out

    def predict(self, X: np.ndarray, chunk_rows: int = 1 << 22) -> np.ndarray:
        X = np.ascontiguousarray(X, dtype=np.float32)
        n = X.shape[0]
        res = np.empty((n, self.dims), dtype=np.float64)
        xt = torch.from_numpy(X)
        with torch.cuda.device(self.dev):
            for r0 in range(0, n, chunk_rows):
                r1 = min(n, r0 + chunk_rows)
                src = xt[r0:r1]
                try:
                    src = src.pin_memory()
                except RuntimeError:
                    pass
                d = src.to(self.dev, non_blocking=True)
                o = self.predict_device(d)
                res[r0:r1] = o.t().double().cpu().numpy()
        return res


def predict_oblivious_gpu(model, X: np.ndarray, device=None) -> np.ndarray:
    key = "_gpu_predictor"
    pred = model.__dict__.get(key)
    if pred is None or pred.T != len(model.trees):
        pred = GpuPredictor(model, device)
        model.__dict__[key] = pred
    return pred.predict(X)
