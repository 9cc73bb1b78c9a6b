"""Training loggers: console lines, ``learn_error.tsv`` / ``test_error.tsv`` / ``time_left.tsv`` and
``catboost_training.json`` under ``train_dir`` (catboost/libs/loggers/logger.h, catboost_logger_helpers.cpp).
TensorBoard event files are not written."""
from __future__ import annotations

import json
import os
import sys
import time


class TrainLogger:
    def __init__(self, o, metric_names, n_eval, log_cout=None, enabled=True):
        self.o = o
        self.enabled = enabled
        self.out = log_cout if log_cout is not None else sys.stdout
        self.verbose = bool(o.verbose) and enabled
        v = o.verbose
        self.print_period = int(v) if (not isinstance(v, bool) and isinstance(v, int) and v > 1) else 1
        self.metric_names = metric_names
        self.n_eval = n_eval
        self.files = {}
        self.json_iters = []
        self.dir = None
        if enabled and o.allow_writing_files and o.train_dir:
            try:
                os.makedirs(o.train_dir, exist_ok=True)
                self.dir = o.train_dir
                self.files["learn"] = open(os.path.join(self.dir, "learn_error.tsv"), "w")
                self.files["learn"].write("iter\t" + "\t".join(metric_names) + "\n")
                if n_eval:
                    self.files["test"] = open(os.path.join(self.dir, "test_error.tsv"), "w")
                    self.files["test"].write("iter\t" + "\t".join(metric_names) + "\n")
                self.files["time"] = open(os.path.join(self.dir, "time_left.tsv"), "w")
                self.files["time"].write("iter\tPassed\tRemaining\n")
            except OSError:
                self.dir = None
                self.files = {}

    def info(self, msg):
        if self.verbose:
            print(msg, file=self.out)

    def log_value(self, it, total, name, value, elapsed):
        if self.verbose and (it % self.print_period == 0 or it == total - 1):
            print(f"{it}:\t{name}: {value:.7f}\ttotal: {elapsed:.3g}s", file=self.out)

    def log_iteration(self, it, total, hist, elapsed):
        if not self.enabled:
            return
        remaining = elapsed / max(it + 1, 1) * (total - it - 1)
        names = hist.names
        first = self.metric_names[0]
        if self.verbose and (it % self.print_period == 0 or it == total - 1):
            parts = [f"{it}:", f"learn: {hist.data['learn'][first][-1]:.7f}"]
            for nm in names[1:]:
                vals = hist.data[nm][first]
                if vals:
                    parts.append(f"test{'' if len(names) == 2 else nm[10:]}: {vals[-1]:.7f}")
            parts.append(f"total: {_fmt(elapsed)}\tremaining: {_fmt(remaining)}")
            print("\t".join(parts), file=self.out)
        if self.files:
            self.files["learn"].write(f"{it}\t" + "\t".join(f"{hist.data['learn'][m][-1]:.9g}" for m in self.metric_names) + "\n")
            if "test" in self.files and len(names) > 1:
                self.files["test"].write(f"{it}\t" + "\t".join(f"{hist.data[names[1]][m][-1]:.9g}" for m in self.metric_names) + "\n")
            self.files["time"].write(f"{it}\t{int(elapsed * 1000)}\t{int(remaining * 1000)}\n")
            rec = {"iteration": it, "passed_time": elapsed, "remaining_time": remaining,
                   "learn": [hist.data["learn"][m][-1] for m in self.metric_names]}
            if len(names) > 1:
                rec["test"] = [hist.data[names[1]][m][-1] for m in self.metric_names]
            self.json_iters.append(rec)

    def close(self):
        for f in self.files.values():
            try:
                f.close()
            except Exception:
                pass
        if self.dir:
            meta = {"meta": {"iteration_count": int(self.o.iterations), "name": self.o.name,
                             "learn_metrics": [{"name": m} for m in self.metric_names],
                             "test_metrics": [{"name": m} for m in self.metric_names] if self.n_eval else [],
                             "launch_mode": "Train"},
                    "iterations": self.json_iters}
            try:
                with open(os.path.join(self.dir, "catboost_training.json"), "w") as fh:
                    json.dump(meta, fh)
            except OSError:
                pass
        self.files = {}


def _fmt(sec):
    if sec < 1:
        return f"{sec * 1000:.0f}ms"
    if sec < 60:
        return f"{sec:.2f}s"
    m, s = divmod(int(sec), 60)
    if m < 60:
        return f"{m}m {s}s"
    h, m = divmod(m, 60)
    return f"{h}h {m}m {s}s"
