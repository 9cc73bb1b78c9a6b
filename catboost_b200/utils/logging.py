"""Training loggers: console lines, ``learn_error.tsv`` / ``test_error.tsv`` / ``time_left.tsv`` and
``catboost_training.json`` under ``train_dir`` (catboost/libs/loggers/logger.h, catboost_logger_helpers.cpp), and
TensorBoard scalar event files ``learn/events.out.tfevents`` / ``test/events.out.tfevents``
(catboost/libs/loggers/tensorboard_logger.cpp)."""
from __future__ import annotations

import json
import os
import sys
import time


def _crc32c_table():
    tab = []
    for i in range(256):
        c = i
        for _ in range(8):
            c = (c >> 1) ^ 0x82F63B78 if c & 1 else c >> 1
        tab.append(c)
    return tab


_CRC_TAB = _crc32c_table()


def _masked_crc32c(data: bytes) -> int:
    c = 0xFFFFFFFF
    for b in data:
        c = _CRC_TAB[(c ^ b) & 0xFF] ^ (c >> 8)
    c ^= 0xFFFFFFFF
    return ((((c >> 15) | (c << 17)) & 0xFFFFFFFF) + 0xA282EAD8) & 0xFFFFFFFF


def _varint(v: int) -> bytes:
    out = bytearray()
    v &= (1 << 64) - 1
    while True:
        b = v & 0x7F
        v >>= 7
        if v:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


class TensorBoardWriter:
    """Scalar summaries in the TFRecord / Event protobuf layout, written without any TensorFlow dependency:
    record = length (8 bytes LE), masked CRC-32C of the length, payload, masked CRC-32C of the payload;
    payload = Event{wall_time = 1 (double), step = 2 (int64), file_version = 3 / summary = 5};
    Summary{value = 1: {tag = 1 (string), simple_value = 2 (float)}}."""

    def __init__(self, directory: str):
        import struct
        self._struct = struct
        os.makedirs(directory, exist_ok=True)
        self.fh = open(os.path.join(directory, "events.out.tfevents"), "wb")
        self._record(self._event(time.time(), 0, version="brain.Event:2"))

    def _event(self, wall, step, version=None, tag=None, value=None) -> bytes:
        st = self._struct
        ev = b"\x09" + st.pack("<d", wall) + b"\x10" + _varint(step)
        if version is not None:
            v = version.encode()
            ev += b"\x1a" + _varint(len(v)) + v
        if tag is not None:
            t = tag.encode()
            val = b"\x0a" + _varint(len(t)) + t + b"\x15" + st.pack("<f", float(value))
            summ = b"\x0a" + _varint(len(val)) + val
            ev += b"\x2a" + _varint(len(summ)) + summ
        return ev

    def _record(self, payload: bytes):
        st = self._struct
        head = st.pack("<Q", len(payload))
        self.fh.write(head + st.pack("<I", _masked_crc32c(head)) + payload + st.pack("<I", _masked_crc32c(payload)))

    def add_scalar(self, tag: str, value: float, step: int):
        self._record(self._event(time.time(), int(step), tag=tag, value=value))

    def close(self):
        try:
            self.fh.close()
        except Exception:
            pass


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
        self.tb = {}
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
                self.tb = {"learn": TensorBoardWriter(os.path.join(self.dir, "learn"))}
                if n_eval:
                    self.tb["test"] = TensorBoardWriter(os.path.join(self.dir, "test"))
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
            for m in self.metric_names:
                if "learn" in self.tb:
                    self.tb["learn"].add_scalar(m, hist.data["learn"][m][-1], it)
                if "test" in self.tb and len(names) > 1 and hist.data[names[1]][m]:
                    self.tb["test"].add_scalar(m, hist.data[names[1]][m][-1], it)
            rec = {"iteration": it, "passed_time": elapsed, "remaining_time": remaining,
                   "learn": [hist.data["learn"][m][-1] for m in self.metric_names]}
            if len(names) > 1:
                rec["test"] = [hist.data[names[1]][m][-1] for m in self.metric_names]
            self.json_iters.append(rec)

    def close(self):
        for w in self.tb.values():
            w.close()
        self.tb = {}
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
