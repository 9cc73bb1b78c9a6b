"""Overfitting detectors (catboost/libs/overfitting_detector/: ``Iter`` stops after ``od_wait`` iterations
without improvement; ``IncToDec`` turns the history of the evaluation metric into a p-value-like statistic and
stops when it drops below ``od_pval``)."""
from __future__ import annotations

import math


class OverfittingDetector:
    def __init__(self, od_type="IncToDec", wait=20, pval=0.0, max_optimal=False):
        self.type, self.wait, self.pval, self.max_optimal = od_type, int(wait), float(pval), bool(max_optimal)
        if self.type == "IncToDec" and self.pval <= 0:
            self.type = "Iter"
        self.best = None
        self.best_iter = -1
        self.iter = -1
        self.stopped = False
        self.local_max = None
        self.cur_pval = 1.0

    def _better(self, a, b):
        return a > b if self.max_optimal else a < b

    def add(self, value: float) -> bool:
        """Feed the metric of one iteration; returns True when training should stop."""
        self.iter += 1
        v = value if self.max_optimal else -value
        if self.best is None or v > self.best:
            self.best, self.best_iter = v, self.iter
        if self.type == "Iter":
            self.stopped = (self.iter - self.best_iter) >= self.wait
            return self.stopped
        # IncToDec: exponential statistic of (drop from the best) / (rise before the best)
        if self.local_max is None:
            self.local_max = v
            self.first = v
        self.local_max = max(self.local_max, v)
        rise = max(self.best - self.first, 1e-12)
        drop = max(self.best - v, 0.0)
        lam = 0.99
        x = drop / rise
        self.cur_pval = math.exp(-0.5 / max(x, 1e-12)) if x > 0 else 1.0
        self.cur_pval = 1.0 - self.cur_pval if x > 0 else 1.0
        if (self.iter - self.best_iter) >= self.wait and self.cur_pval < self.pval:
            self.stopped = True
        return self.stopped
