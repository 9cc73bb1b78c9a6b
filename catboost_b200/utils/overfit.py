"""Overfitting detectors (catboost/libs/overfitting_detector/overfitting_detector.cpp).

All three types watch the evaluation metric after its last local optimum:

* ``IncToDec`` keeps an exponentially forgotten estimate of the largest increase the metric has shown (forgetting factor
  0.99 per iteration over the last 2000 values) and, once ``od_wait`` iterations have passed since the optimum, turns the
  ratio expected increase / drop since the optimum into ``p = exp(-0.5 / ratio)``; training stops when ``p < od_pval``.
* ``Iter`` is ``IncToDec`` with threshold 1: it stops ``od_wait`` iterations after the optimum.
* ``Wilcoxon`` collects the per-iteration deteriorations since the optimum and stops when the signed-rank test says
  they are systematically positive (two-sided p-value from the normal approximation of the rank statistic below
  ``od_pval``), again only after ``od_wait`` of them.
"""
from __future__ import annotations

import math
from collections import deque

LAMBDA_FORGET = 0.99
ITERATION_FORGET = 2000
LAMBDA_SCALE = 0.5
EPS = 1e-10


def wilcoxon_signed_rank_pvalue(deltas) -> float:
    """Two-sided p-value of the signed-rank statistic of ``deltas`` (zeros dropped, average ranks for ties, normal
    approximation); 0.5 when nothing is left, like the reference's ``NStatistics::Wilcoxon``."""
    v = [d for d in deltas if d != 0]
    n = len(v)
    if n == 0:
        return 0.5
    order = sorted(range(n), key=lambda i: abs(v[i]))
    ranks = [0.0] * n
    i = 0
    while i < n:
        j = i
        while j + 1 < n and abs(v[order[j + 1]]) == abs(v[order[i]]):
            j += 1
        r = 0.5 * (i + j) + 1.0
        for k in range(i, j + 1):
            ranks[order[k]] = r
        i = j + 1
    w = sum(r if v[k] > 0 else -r for k, r in enumerate(ranks))
    sigma = math.sqrt(n * (n + 1) * (2 * n + 1) / 6.0)
    z = abs(w) / max(sigma, 1e-300)
    return max(0.0, min(1.0, math.erfc(z / math.sqrt(2.0))))


class OverfittingDetector:
    def __init__(self, od_type="IncToDec", wait=20, pval=0.0, max_optimal=False):
        self.type, self.wait, self.max_optimal = od_type, int(wait), bool(max_optimal)
        self.pval = float(pval)
        if self.type == "Iter" or (self.type == "IncToDec" and self.pval <= 0):
            self.type, self.pval = "Iter", 1.0          # threshold 1: any p-value below 1 stops
        self.empty = True
        self.local_max = 0.0
        self.last = 0.0
        self.expected_inc = 0.0
        self.from_local_max = 0
        self.errors = deque()
        self.deltas = []
        self.cur_pval = 1.0
        self.stopped = False
        self.iter = -1
        self.best_iter = -1

    def add(self, value: float) -> bool:
        """Feed the metric of one iteration; returns True when training should stop."""
        self.iter += 1
        err = value if self.max_optimal else -value
        if self.type == "Wilcoxon":
            if self.empty or err > self.local_max:
                self.empty = False
                self.deltas = []
                self.local_max = err
                self.best_iter = self.iter
            else:
                self.deltas.append(self.last - err)
            self.last = err
            self.cur_pval = wilcoxon_signed_rank_pvalue(self.deltas) if len(self.deltas) >= self.wait else 1.0
        else:
            if self.empty or err > self.local_max:
                if self.empty:
                    self.empty = False
                    self.expected_inc = 0.0
                self.local_max = err
                self.from_local_max = 0
                self.best_iter = self.iter
            else:
                self.from_local_max += 1
            self.errors.appendleft(err)
            if len(self.errors) > ITERATION_FORGET:
                self.errors.pop()
            self.expected_inc *= LAMBDA_FORGET
            mult = 1.0
            for e in self.errors:
                self.expected_inc = max(self.expected_inc, mult * (err - e))
                mult *= LAMBDA_FORGET
                if mult < 1e-9:
                    break
            self.last = err
            if self.from_local_max >= self.wait:
                ratio = self.expected_inc / max(self.local_max - self.last, EPS)
                self.cur_pval = math.exp(-LAMBDA_SCALE / max(ratio, EPS))
            else:
                self.cur_pval = 1.0
        self.stopped = (not self.empty) and self.cur_pval < self.pval
        return self.stopped
