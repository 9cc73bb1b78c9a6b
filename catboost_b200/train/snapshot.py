"""Training snapshots: periodic save of the boosting progress and resume.

The reference stores models + metric history (not cursors) and re-applies the ensemble on restore
(catboost/cuda/methods/boosting_progress_tracker.cpp:189-260, doc_parallel_boosting.h:500-512); the file is
written to a temporary name and renamed atomically (catboost/libs/helpers/progress_helper.h:40-89).  The same
contract is kept here.  File layout: label line, 32 hex digits md5 of the body, body = a plain-data stream
(``utils/plainser.py``: little-endian PODs with ui32 size prefixes in the manner of the reference's ysaveload
streams) holding the options fingerprint and the state (trees as arrays, metric history, iteration list).  Reading
a snapshot never executes anything stored in it.
"""
from __future__ import annotations

import hashlib
import os
import time

from ..data.pool import CatBoostError
from ..utils import plainser

LABEL = b"catboost_b200_snapshot_v1\n"
_FINGERPRINT_KEYS = ("loss_function", "depth", "learning_rate", "l2_leaf_reg", "border_count", "grow_policy",
                     "random_seed", "bootstrap_type", "score_function", "leaf_estimation_method",
                     "leaf_estimation_iterations", "task_type")


def fingerprint(o) -> str:
    return hashlib.md5(repr([(k, str(o.get(k))) for k in _FINGERPRINT_KEYS]).encode()).hexdigest()


class SnapshotManager:
    def __init__(self, o, ctx=None):
        self.enabled = bool(o.save_snapshot) and (ctx is None or ctx.rank == 0)
        self.read_enabled = bool(o.save_snapshot)
        name = o.snapshot_file or "experiment.cbsnapshot"
        self.path = name if os.path.isabs(name) else os.path.join(o.train_dir or ".", name)
        self.interval = float(o.snapshot_interval)
        self.last = time.time()
        self.fp = fingerprint(o)

    def try_load(self, o):
        if not self.read_enabled or not os.path.exists(self.path):
            return None
        with open(self.path, "rb") as fh:
            blob = fh.read()
        if not blob.startswith(LABEL):
            raise CatBoostError(f"{self.path} is not a catboost_b200 snapshot")
        digest, body = blob[len(LABEL):len(LABEL) + 32], blob[len(LABEL) + 32:]
        if hashlib.md5(body).hexdigest().encode() != digest:
            raise CatBoostError(f"snapshot {self.path} is corrupted (checksum mismatch)")
        try:
            payload = plainser.loads(body)
        except (plainser.PlainDataError, UnicodeDecodeError) as e:
            raise CatBoostError(f"snapshot {self.path} is unreadable: {e}") from e
        if not isinstance(payload, dict) or payload.get("fingerprint") != self.fp:
            raise CatBoostError("snapshot was written with different training parameters")
        return payload["state"]

    def _write(self, state):
        body = plainser.dumps({"fingerprint": self.fp, "state": state})
        os.makedirs(os.path.dirname(os.path.abspath(self.path)), exist_ok=True)
        tmp = self.path + ".tmp"
        with open(tmp, "wb") as fh:
            fh.write(LABEL + hashlib.md5(body).hexdigest().encode() + body)
        os.replace(tmp, self.path)

    def due(self) -> bool:
        """True when this rank writes snapshots and the interval since the last one has passed (callers whose state is
        expensive to collect -- a device -> host copy -- ask before collecting it)."""
        return self.enabled and (time.time() - self.last >= self.interval)

    def maybe_save(self, state, iteration):
        if self.due():
            self._write(state() if callable(state) else state)
            self.last = time.time()

    def finalize(self, state):
        if self.enabled:
            self._write(state() if callable(state) else state)
