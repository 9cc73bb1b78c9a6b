"""Labelled wall-clock spans around stages of training (the role of TCudaProfiler,
catboost/cuda/cuda_lib/cuda_profiler.h:132-227).  With ``sync=True`` the device is synchronised at span
boundaries so that times are attributable (the reference's ImplicitLabelSync mode)."""
from __future__ import annotations

import contextlib
import time
from collections import OrderedDict


class Profiler:
    def __init__(self, enabled=True, sync=False):
        self.enabled, self.sync = enabled, sync
        self.acc = OrderedDict()
        self.count = OrderedDict()

    @contextlib.contextmanager
    def span(self, label: str):
        if not self.enabled:
            yield
            return
        if self.sync:
            self._sync()
        nvtx = self._nvtx()
        if nvtx is not None:
            nvtx.range_push(label)                # shows up as a named range in Nsight traces
        t0 = time.perf_counter()
        try:
            yield
        finally:
            if nvtx is not None:
                nvtx.range_pop()
            if self.sync:
                self._sync()
            self.acc[label] = self.acc.get(label, 0.0) + time.perf_counter() - t0
            self.count[label] = self.count.get(label, 0) + 1

    @staticmethod
    def _nvtx():
        try:
            import torch
            if torch.cuda.is_available():
                return torch.cuda.nvtx
        except Exception:
            pass
        return None

    @staticmethod
    def _sync():
        try:
            import torch
            if torch.cuda.is_available():
                torch.cuda.synchronize()
        except Exception:
            pass

    def report(self):
        return dict(self.acc)

    def table(self) -> str:
        rows = sorted(self.acc.items(), key=lambda kv: -kv[1])
        return "\n".join(f"{k:<24s}{v * 1000:12.2f} ms  x{self.count[k]}" for k, v in rows)
