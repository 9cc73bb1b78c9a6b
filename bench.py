#!/usr/bin/env python
"""Headline benchmark: seconds per 1000 boosting iterations (device-timed, max over ranks).

    python bench.py --gpus N --steps K --warmup W [--config higgs|epsilon|small] [--impl reference]

Default config ``higgs`` is the dense numeric binary-classification workload: 10.5M rows x 28 float32 features
(21 ~N(0,1) + 7 non-linear derived), Logloss, symmetric trees depth 6, border_count 128, learning_rate 0.1,
doc-parallel over N GPUs (strong scaling: the row count is fixed, each rank holds rows/N).
A "step" is one boosting iteration.  Two numbers are reported:

* ``value``     -- K iterations of the device-resident trainer, each bracketed by CUDA events (L2 flushed between
                   iterations with a 512 MiB write that is not timed), max over ranks.
* ``e2e.value`` -- the same metric through the public API: wall seconds of one ``CatBoostClassifier.fit`` of 1000
                   iterations on host data, including the host->device upload of the feature matrix from pinned
                   memory, border selection, quantisation, and a device->host read of the learn loss every iteration.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

BASELINE_S_PER_1000 = {"higgs": 55.601, "epsilon": 44.971, "small": None, "criteo": None, "ranking": None, "sparse": None,
                       "airline": 485.825, "msrank": 11.057, "synthetic": 36.658, "synthetic5k": 28.014}
CONFIGS = {
    # rows, float features, depth, border_count
    "higgs": dict(rows=10_500_000, features=28, depth=6, border_count=128, model="Logloss symmetric depth6 10.5Mx28"),
    "epsilon": dict(rows=400_000, features=2000, depth=6, border_count=128, model="Logloss symmetric depth6 400Kx2000"),
    "small": dict(rows=200_000, features=28, depth=6, border_count=128, model="Logloss symmetric depth6 200Kx28"),
    # the feature matrix of the ranking workload (60 % exact zeros, 64 borders) under Logloss: isolates the level kernels
    "sparse": dict(rows=2_000_000, features=700, depth=6, border_count=64, model="Logloss symmetric depth6 2Mx700 60% zeros"),
    # categorical workload (13 numeric + 26 categorical columns, CTR features); end-to-end fit() only.  The named
    # reference config has 45M rows: pass --rows 45000000 for the full size.
    # learning to rank: 2M documents x 700 features in groups of about 100, YetiRank, 64 borders; end-to-end fit() only
    "ranking": dict(rows=2_000_000, features=700, depth=6, border_count=64, model="YetiRank symmetric depth6 2Mx700"),
    "criteo": dict(rows=45_000_000, features=39, depth=8, border_count=128, model="Logloss symmetric depth8 13num+26cat CTR"),
    # the other shapes of the reference's training_speed benchmark (catboost/benchmarks/training_speed/README.md:207-228),
    # as synthetic matrices of those sizes under Logloss
    "airline": dict(rows=115_000_000, features=13, depth=6, border_count=128, model="Logloss symmetric depth6 115Mx13"),
    "msrank": dict(rows=1_200_000, features=137, depth=6, border_count=128, model="Logloss symmetric depth6 1.2Mx137"),
    "synthetic": dict(rows=10_000_000, features=100, depth=6, border_count=128, model="Logloss symmetric depth6 10Mx100"),
    "synthetic5k": dict(rows=100_000, features=5000, depth=6, border_count=128, model="Logloss symmetric depth6 100Kx5000"),
    # the CPU plumbing config: 100K x 50, 200 iterations, task_type CPU; runs without a GPU (wall time of fit())
    "cpu": dict(rows=100_000, features=50, depth=6, border_count=128, model="Logloss symmetric depth6 100Kx50 on CPU"),
}


def make_data(config: str, rows: int, features: int, rank: int, world: int, seed: int = 0):
    """Seeded synthetic shard of the named shape (rows/world rows for this rank)."""
    lo, hi = rows * rank // world, rows * (rank + 1) // world
    n = hi - lo
    rng = np.random.default_rng(seed * 1000 + rank)
    if config == "sparse":
        X = rng.random((n, features), dtype=np.float32)
        for r0 in range(0, n, 250_000):
            blk = X[r0:r0 + 250_000]
            blk[rng.random(blk.shape, dtype=np.float32) < 0.6] = 0.0
        w = np.random.default_rng(seed + 3).standard_normal(features).astype(np.float32) / np.sqrt(features)
        s_ = X @ w + 0.15 * rng.standard_normal(n, dtype=np.float32)
        return X, (s_ > np.median(s_[: min(n, 200_000)])).astype(np.float32)
    if config == "epsilon":
        X = rng.standard_normal((n, features), dtype=np.float32)
        X /= np.linalg.norm(X, axis=1, keepdims=True)
        w = np.random.default_rng(seed + 7).standard_normal(features).astype(np.float32)
        y = ((X @ w + 0.1 * rng.standard_normal(n, dtype=np.float32)) > 0).astype(np.float32)
        return X, y
    base = features * 3 // 4
    X = np.empty((n, features), dtype=np.float32)
    X[:, :base] = rng.standard_normal((n, base), dtype=np.float32)
    r2 = np.random.default_rng(seed + 11)
    for j in range(base, features):
        a, b = r2.integers(0, base, 2)
        kind = (j - base) % 3
        X[:, j] = X[:, a] * X[:, b] if kind == 0 else (np.abs(X[:, a] - X[:, b]) if kind == 1 else X[:, a] ** 2)
    f = np.zeros(n, dtype=np.float32)
    for _ in range(8):
        a, b, c = r2.integers(0, features, 3)
        f += r2.standard_normal() * X[:, a] + 0.5 * r2.standard_normal() * X[:, b] * X[:, c]
    f = f / max(float(f.std()), 1e-6) + 0.12
    y = (rng.random(n, dtype=np.float32) < 1.0 / (1.0 + np.exp(-f))).astype(np.float32)
    return X, y


def make_criteo_like(rows: int, rank: int, world: int, seed: int = 0):
    """The categorical workload: 13 numeric columns (integer counts from a log-normal distribution, 20 % missing) and 26
    categorical columns whose cardinalities are drawn log-uniformly from [10, 1e6] and whose values follow Zipf(s = 1.1);
    about 25 % positives from a logistic model over per-category random effects.  Every rank draws the same
    cardinalities and effect tables (seeded by ``seed``) and its own rows (seeded by the rank)."""
    import pandas as pd
    lo, hi = rows * rank // world, rows * (rank + 1) // world
    n = hi - lo
    rng = np.random.default_rng(seed * 1000 + rank)
    tab_rng = np.random.default_rng(seed + 5)
    cards = np.unique(np.round(np.exp(tab_rng.uniform(np.log(10.0), np.log(1e6), 26))).astype(np.int64))
    while len(cards) < 26:
        cards = np.unique(np.concatenate([cards, np.round(np.exp(tab_rng.uniform(np.log(10.0), np.log(1e6), 26 - len(cards)))).astype(np.int64)]))
    cards = tab_rng.permutation(cards)[:26]
    cols = {}
    f = np.zeros(n, dtype=np.float32)
    for j in range(13):
        v = np.floor(np.exp(rng.normal(1.0, 1.5, n))).astype(np.float32)
        if j < 4:
            f += (0.25 - 0.1 * j) * np.log1p(v) - 0.3
        v[rng.random(n) < 0.2] = np.nan
        cols[f"n{j}"] = v
    for j, card in enumerate(cards):
        # Zipf(1.1) truncated to the cardinality: inversion of the continuous power law x^-1.1 on [1, card + 1), floored
        # (P(k) proportional to k^-0.1 - (k + 1)^-0.1, which is k^-1.1 up to a slowly varying factor)
        top = float(card + 1) ** -0.1
        c = (np.floor((1.0 - rng.random(n, dtype=np.float32) * np.float32(1.0 - top)) ** np.float32(-10.0)).astype(np.int64) - 1)
        c = np.clip(c, 0, int(card) - 1).astype(np.int32)
        effect = (tab_rng.standard_normal(int(card)) * 0.35).astype(np.float32)
        f += effect[c]
        cols[f"c{j}"] = c
    # intercept for about 25 % positives (bisection on a sample of this rank; the ranks agree to within sampling noise)
    fs = f[: min(n, 200_000)].astype(np.float64)
    a, b = -20.0, 20.0
    for _ in range(40):
        mid = 0.5 * (a + b)
        if np.mean(1.0 / (1.0 + np.exp(-(fs + mid)))) > 0.25:
            b = mid
        else:
            a = mid
    f += np.float32(0.5 * (a + b))
    y = (rng.random(n, dtype=np.float32) < 1.0 / (1.0 + np.exp(-f))).astype(np.float32)
    return pd.DataFrame(cols), y, [f"c{j}" for j in range(26)]


def bench_ranking(args, cfg, rank, world, dev):
    """End-to-end fit() of the ranking workload: YetiRank derivatives by the per-group kernel, trees by the fused level
    kernels; the per-iteration time is the wall time of the iterations phase."""
    import torch
    import catboost_b200 as cb
    n, F = cfg["rows"] // world, cfg["features"]
    rng = np.random.default_rng(17 + rank)
    # 60 % exact zeros, the rest U(0, 1); queries of 5 .. 200 documents; relevance 0 .. 4 from quantiles of a latent
    # linear score plus noise
    X = rng.random((n, F), dtype=np.float32)
    for r0 in range(0, n, 250_000):
        blk = X[r0:r0 + 250_000]
        blk[rng.random(blk.shape, dtype=np.float32) < 0.6] = 0.0
    wv = np.random.default_rng(3).standard_normal(F).astype(np.float32) / np.sqrt(F)
    score = X @ wv + 0.15 * rng.standard_normal(n, dtype=np.float32)
    rel = np.digitize(score, np.quantile(score[: min(n, 200000)], [0.5, 0.8, 0.93, 0.98])).astype(np.float32)
    sizes = rng.integers(5, 201, size=n // 5 + 1)
    gid = np.repeat(np.arange(len(sizes)), sizes)[:n]
    iters = args.e2e_iters if args.e2e_iters > 0 else max(args.steps + args.warmup, 50)
    model = cb.CatBoostRanker(loss_function="YetiRank", iterations=iters, depth=cfg["depth"], border_count=cfg["border_count"],
                              learning_rate=0.1, task_type="GPU", random_seed=0, allow_writing_files=False, verbose=False)
    torch.cuda.synchronize(dev)
    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    t0 = time.perf_counter()
    model.fit(X, rel, group_id=gid)
    torch.cuda.synchronize(dev)
    fit_s = time.perf_counter() - t0
    clocks = sampler.stop()
    tm = model._train_info.get("timings", {})
    it_s = float(tm.get("iterations", float("nan")))
    # batch apply of the trained model: rows already on the device (kernel throughput) and rows from host memory
    # through the public predict call (staging, copies and the read-back included)
    apply = None
    if rank == 0:
        from catboost_b200.models.gpu_apply import GpuPredictor
        pred = GpuPredictor(model._model, dev)
        n_dev = min(n, 1_000_000)
        Xd = torch.from_numpy(X[:n_dev]).to(dev)
        out = torch.empty((pred.dims, n_dev), dtype=torch.float32, device=dev)
        for _ in range(3):
            pred.predict_device(Xd, out)
        reps = max(1, 100_000_000 // n_dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(dev)
        e0.record()
        for _ in range(reps):
            pred.predict_device(Xd, out)
        e1.record()
        torch.cuda.synchronize(dev)
        dev_s = e0.elapsed_time(e1) / 1000.0
        n_host = min(n, 2_000_000)
        model.predict(X[:100_000], prediction_type="RawFormulaVal", task_type="GPU")
        t1 = time.perf_counter()
        model.predict(X[:n_host], prediction_type="RawFormulaVal", task_type="GPU")
        host_s = time.perf_counter() - t1
        apply = {"trees": iters, "features": F, "device_rows": n_dev * reps, "device_rows_per_s": n_dev * reps / dev_s,
                 "tree_rows_per_s": n_dev * reps * iters / dev_s, "host_rows": n_host, "host_rows_per_s": n_host / host_s,
                 "note": "device: 100M rows as repeated passes over 1M resident rows; host: predict() from pageable memory"}
        del Xd, out
    n_ev = int(np.searchsorted(gid, gid[min(n, 200000) - 1]))           # whole queries only
    ev_pool = cb.Pool(X[:n_ev], rel[:n_ev], group_id=gid[:n_ev])
    ndcg = [model.eval_metrics(ev_pool, ["NDCG"], ntree_end=1)["NDCG"][-1], model.eval_metrics(ev_pool, ["NDCG"], eval_period=iters)["NDCG"][-1]]
    if rank == 0:
        print(json.dumps({"metric": "sec/1000 iters (wall time of the iterations phase of fit())", "value": it_s / iters * 1000.0,
                          "unit": "s/1000iter", "n_gpus": world, "steps": iters, "warmup": 0, "ms_per_step": it_s / iters * 1000.0,
                          "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "fp32",
                          "data": "synthetic", "impl": "ours",
                          "config": {"model": cfg["model"], "global_batch": cfg["rows"], "seq_len": F,
                                     "parallelism": f"doc-parallel dp{world}", "depth": cfg["depth"], "group_size": "uniform 5..200"},
                          "e2e": {"value": fit_s / iters * 1000.0, "unit": "s/1000iter", "fit_seconds": fit_s,
                                  "fit_breakdown_s": {k: round(float(v), 4) for k, v in tm.items()}},
                          "clocks": clocks, "ndcg_first_last": [float(ndcg[0]), float(ndcg[-1])], "apply": apply,
                          "gpu_launches": int(model._train_info.get("launches_per_iter", 0)) * iters}))
    return 0


def bench_cpu(args):
    """Config 1: binary Logloss on the CPU trainer, 100K x 50, depth 6, 128 borders, learning rate 0.1, l2 3, 200
    iterations; the metric is the wall time of the iterations phase of fit() scaled to 1000 iterations."""
    import catboost_b200 as cb
    cfg = CONFIGS["cpu"]
    n, F = (args.rows or cfg["rows"]), cfg["features"]
    rng = np.random.default_rng(1)
    X = rng.standard_normal((n, F)).astype(np.float32)
    w = rng.standard_normal(F) / np.sqrt(F)
    y = (rng.random(n) < 1.0 / (1.0 + np.exp(-(X @ w + 0.5 * rng.standard_normal(n))))).astype(np.float32)
    iters = args.e2e_iters if args.e2e_iters > 0 else 200
    m = cb.CatBoostClassifier(loss_function="Logloss", iterations=iters, depth=6, border_count=128, learning_rate=0.1,
                              l2_leaf_reg=3.0, task_type="CPU", random_seed=0, allow_writing_files=False, verbose=False)
    t0 = time.perf_counter()
    m.fit(X, y)
    fit_s = time.perf_counter() - t0
    tm = m._train_info.get("timings", {})
    # the general learner reports its iteration phase in parts
    parts = [tm[k] for k in ("derivatives", "structure", "leaves", "eval_apply", "metrics") if k in tm]
    it_s = float(tm["iterations"]) if "iterations" in tm else (float(sum(parts)) if parts else fit_s)
    acc = float((m.predict(X) == y).mean())
    print(json.dumps({"metric": "sec/1000 iters (wall time of the iterations phase of fit(), CPU trainer)",
                      "value": it_s / iters * 1000.0, "unit": "s/1000iter", "n_gpus": 0, "steps": iters, "warmup": 0,
                      "ms_per_step": it_s / iters * 1000.0, "higher_is_better": False, "scaling": "strong",
                      "vs_baseline": None, "dtype": "fp32", "data": "synthetic", "impl": "ours",
                      "config": {"model": cfg["model"], "global_batch": n, "seq_len": F, "parallelism": "one process, OpenMP"},
                      "e2e": {"value": fit_s / iters * 1000.0, "unit": "s/1000iter", "fit_seconds": fit_s,
                              "fit_breakdown_s": {k: round(float(v), 4) for k, v in tm.items()}},
                      "learn_accuracy": acc, "gpu_launches": 0}))
    return 0


def bench_criteo(args, cfg, rank, world, dev):
    """End-to-end fit() on the categorical workload; the per-iteration time is the wall time of the iterations phase."""
    import torch
    import catboost_b200 as cb
    df, y, cats = make_criteo_like(cfg["rows"], rank, world)
    iters = args.e2e_iters if args.e2e_iters > 0 else max(args.steps + args.warmup, 50)
    model = cb.CatBoostClassifier(loss_function="Logloss", iterations=iters, depth=cfg["depth"], border_count=cfg["border_count"],
                                  learning_rate=0.1, task_type="GPU", random_seed=0, allow_writing_files=False,
                                  max_ctr_complexity=int(args.ctr_complexity), verbose=False)
    torch.cuda.synchronize(dev)
    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    t0 = time.perf_counter()
    model.fit(df, y, cat_features=cats)
    torch.cuda.synchronize(dev)
    fit_s = time.perf_counter() - t0
    clocks = sampler.stop()
    tm = model._train_info.get("timings", {})
    it_s = float(tm.get("iterations", float("nan")))
    if rank == 0:
        print(json.dumps({"metric": "sec/1000 iters (wall time of the iterations phase of fit())", "value": it_s / iters * 1000.0,
                          "unit": "s/1000iter", "n_gpus": world, "steps": iters, "warmup": 0, "ms_per_step": it_s / iters * 1000.0,
                          "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "fp32",
                          "data": "synthetic", "impl": "ours",
                          "config": {"model": cfg["model"], "global_batch": cfg["rows"], "seq_len": 39,
                                     "parallelism": f"doc-parallel dp{world}", "depth": cfg["depth"],
                                     "ctr": f"simple_ctr defaults, max_ctr_complexity={int(args.ctr_complexity)}",
                                     "generator": "13 log-normal counts with 20% NaN + 26 Zipf(1.1) categoricals, "
                                                  "cardinalities log-uniform in [10, 1e6], ~25% positives"},
                          "e2e": {"value": fit_s / iters * 1000.0, "unit": "s/1000iter", "fit_seconds": fit_s,
                                  "fit_breakdown_s": {k: round(float(v), 4) for k, v in tm.items()}},
                          "clocks": clocks, "features_in_store": model._train_info.get("h2d_bytes"),
                          "gpu_launches": int(model._train_info.get("launches_per_iter", 0)) * iters}))
    return 0


class ClockSampler:
    """nvidia-smi samples of SM clock / throttle reasons during the timed region (reading only)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.idx)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        if not self.lines:
            # a timed region shorter than the sampling period: take one reading right away (clocks take longer than
            # that to fall back after the last kernel)
            try:
                one = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-i",
                                      str(self.idx)], capture_output=True, text=True, timeout=10)
                self.lines += [ln.strip() for ln in one.stdout.splitlines() if ln.strip()]
            except (OSError, subprocess.SubprocessError):
                pass
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            p = [x.strip() for x in ln.split(",")]
            if len(p) < 9:
                continue
            try:
                sm.append(float(p[1])); mx.append(float(p[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        top = sorted(sm)[len(sm) // 2:] if sm else []
        return {"sm_mhz": statistics.median(top) if top else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm(args):
    """The unmodified reference through its own public API (``CatBoostClassifier(task_type='GPU').fit``), when an
    installed copy exists under ``baseline/_ref``; nothing of this package is imported on this path.  Without an
    installed copy the arm prints why: the reference's CMake tree cannot be configured with the tool chain of this image
    (its global flags are clang-only and the base library needs the ragel and yasm generators, none of which is
    installed and none of which can be fetched offline)."""
    ref_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "_ref")
    sys.path.insert(0, ref_dir)
    try:
        import catboost as ref                      # noqa: F401  (the reference's python package, if it was built)
    except Exception as e:                          # ImportError, or a broken native module
        print(json.dumps({"impl": "reference",
                          "unavailable": "no installed reference under baseline/_ref (" + type(e).__name__ + "): its CMake "
                                         "configure stops at the clang-only flags of cmake/global_flags.compiler.gnu.cmake "
                                         "under gcc, and util/ needs ragel + yasm; clang, ragel, yasm, swig and conan are "
                                         "not in the image and cannot be fetched offline"}))
        return 0
    import torch
    cfg = dict(CONFIGS[args.config])
    if args.rows:
        cfg["rows"] = args.rows
    if args.config in ("criteo", "ranking"):
        print(json.dumps({"impl": "reference", "unavailable": f"reference arm is wired for the dense configs, not {args.config}"}))
        return 0
    K, W = args.steps, max(3, args.warmup)
    X, y = make_data(args.config, cfg["rows"], cfg["features"], 0, 1)
    devices = "0" if args.gpus <= 1 else f"0-{args.gpus - 1}"
    common = dict(loss_function="Logloss", depth=cfg["depth"], border_count=cfg["border_count"], learning_rate=0.1,
                  l2_leaf_reg=3.0, task_type="GPU", devices=devices, random_seed=0, allow_writing_files=False, verbose=False)
    # the reference has no per-iteration device timer in its public API: time fit() at W and at W + K iterations and
    # take the difference (data loading and quantisation cancel out)
    def fit_seconds(iters):
        m = ref.CatBoostClassifier(iterations=iters, **common)
        t0 = time.perf_counter()
        m.fit(X, y)
        return time.perf_counter() - t0
    fit_seconds(W)
    sampler = ClockSampler(0)
    sampler.start()
    t_small, t_big = fit_seconds(W), fit_seconds(W + K)
    clocks = sampler.stop()
    ms = max(t_big - t_small, 0.0) / K * 1000.0
    t0 = time.perf_counter()
    ref.CatBoostClassifier(iterations=1000, **common).fit(X, y)
    e2e_s = time.perf_counter() - t0
    print(json.dumps({"metric": "sec/1000 iters (difference of two fit() wall times)", "value": ms, "unit": "s/1000iter",
                      "n_gpus": args.gpus, "steps": K, "warmup": W, "ms_per_step": ms, "higher_is_better": False,
                      "scaling": "strong", "vs_baseline": None, "dtype": "fp32", "data": "synthetic", "impl": "reference",
                      "config": {"model": cfg["model"], "global_batch": cfg["rows"], "seq_len": cfg["features"],
                                 "parallelism": f"reference doc-parallel devices={devices}"},
                      "clocks": clocks, "e2e": {"value": e2e_s, "unit": "s/1000iter", "h2d_bytes_per_step": int(X.nbytes // 1000),
                                                "d2h_bytes_per_step": 0}, "gpu_launches": None}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--config", default="higgs", choices=sorted(CONFIGS))
    ap.add_argument("--rows", type=int, default=0)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--reduce", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--cells", default="narrow", choices=["narrow", "wide", "float"],
                    help="shared-memory histogram cells: one int32, hi/lo int32 pair, or fp32")
    ap.add_argument("--single-cells", action="store_true", help="time only the cell type given by --cells")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--e2e-iters", type=int, default=0,
                    help="boosting iterations of the end-to-end fit() (default 1000: the metric's own iteration count)")
    ap.add_argument("--ctr-complexity", type=int, default=2, help="max_ctr_complexity of the categorical config")
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--apply-100m", action="store_true", help="stream 100M rows through predict() (repeated passes over the host matrix)")
    ap.add_argument("--phases", action="store_true", help="print per-phase times of the fused level kernel")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.config == "cpu":
        return bench_cpu(args)
    if args.warmup < 3:
        args.warmup = 3
    if args.gpus > 1 and "RANK" not in os.environ:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29541", os.path.abspath(__file__)] + sys.argv[1:]
        return subprocess.call(cmd)

    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)

    import catboost_b200 as cb
    from catboost_b200.data.pool import Pool
    from catboost_b200.params import resolve_options
    from catboost_b200.parallel.runtime import DistContext
    from catboost_b200.train.boosting import build_store, plan_features
    from catboost_b200.train.gpu_engine import GpuObliviousEngine
    from catboost_b200.train.objectives import make_objective

    cfg = dict(CONFIGS[args.config])
    if args.rows:
        cfg["rows"] = args.rows
    K, W = args.steps, args.warmup
    if args.config == "criteo":
        return bench_criteo(args, cfg, rank, world, dev)
    if args.config == "ranking":
        return bench_ranking(args, cfg, rank, world, dev)
    X, y = make_data(args.config, cfg["rows"], cfg["features"], rank, world)
    params = dict(loss_function="Logloss", iterations=K + W, depth=cfg["depth"], border_count=cfg["border_count"],
                  learning_rate=0.1, l2_leaf_reg=3.0, task_type="GPU", random_seed=0, allow_writing_files=False,
                  histogram_reduce=args.reduce, histogram_cells=args.cells)

    # ---------------- device-timed trainer steps -------------------------------------------------------------
    ctx = DistContext.current(dev)
    pool = Pool(X, y)
    o = resolve_options(params, "Logloss", n_rows=cfg["rows"])
    plan = plan_features(o, pool, ctx, None)
    store, h2d = build_store(plan, pool, dev)
    obj = make_objective("Logloss", {})
    p1 = float(y.mean())
    bias = float(np.log(p1 / (1 - p1)))
    flush = None if args.no_flush else torch.empty(512 << 20, dtype=torch.uint8, device=dev)

    def make_engine(cells, reduce, iterations):
        return GpuObliviousEngine(store, torch.from_numpy(y), None, torch.full((len(y),), bias), obj, depth=cfg["depth"],
                                  iterations=iterations, learning_rate=0.1, l2_leaf_reg=3.0, score_function=o.score_function,
                                  random_strength=float(o.random_strength), bootstrap_type=o.bootstrap_type,
                                  bootstrap_param=float(o.bagging_temperature or 1.0), leaf_method=o.leaf_estimation_method,
                                  leaf_iterations=int(o.leaf_estimation_iterations), seed=0, ctx=ctx, reduce=reduce,
                                  leaf_backtracking=str(o.leaf_estimation_backtracking or "AnyImprovement"),
                                  quantized_hist={"narrow": True, "wide": "wide", "float": False}[cells])

    def timed_run(cells, with_clocks):
        """K timed iterations (CUDA events around each, L2 flushed before each, max over ranks of the sum)."""
        eng = make_engine(cells, args.reduce, K + W)
        if args.phases and eng.plan:
            eng.enable_phase_timing()
        eng.step(W)
        torch.cuda.synchronize(dev)
        ctx.barrier()
        sampler = ClockSampler(local) if with_clocks else None
        if sampler:
            sampler.start()
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K)]
        for k in range(K):
            if flush is not None:
                flush.fill_(k & 0xFF)
            if world > 1:
                dist.barrier(device_ids=[local])
            evs[k][0].record()
            eng.step(1)
            evs[k][1].record()
        torch.cuda.synchronize(dev)
        ctx.barrier()
        clocks = sampler.stop() if sampler else None
        t = torch.tensor([sum(a.elapsed_time(b) for a, b in evs)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        res = dict(total_ms=float(t.item()), clocks=clocks, launches=eng.launches_per_iter * K,
                   loss_curve=eng.learn_loss_history(), splits=eng.splits[: 5 * cfg["depth"]].clone(),
                   vals=eng.model_vals[:5].clone())
        if args.phases and eng.plan and rank == 0:
            np.set_printoptions(precision=1, suppress=True, linewidth=160)
            print('phase us per level [leaf_update, hist, grid_wait, reduce_push, score, select]:\n', eng.phase_times_us(), file=sys.stderr)
            print('inside score (block 0) [noise scale, first accumulate, rest]:\n', eng.score_phase_times_us(), file=sys.stderr)
            bt, sm = eng.block_finish_times()
            order = np.argsort(bt)
            print('hist end per block (us) pct 0/10/50/90/100:', np.percentile(bt, [0, 10, 50, 90, 100]), file=sys.stderr)
            print('slowest blocks (block, sm, us):', [(int(b), int(sm[b]), float(bt[b])) for b in order[-8:]], file=sys.stderr)
        eng.finish()
        if eng.arena is not None:
            eng.arena.check_status()
        eng.close()
        del eng
        return res

    main_run = timed_run(args.cells, True)
    total_ms, clocks, launches, loss_curve = (main_run[k] for k in ("total_ms", "clocks", "launches", "loss_curve"))
    # the same steps with the other cell type (exact 24-bit hi/lo pairs when the headline run uses single int32 cells)
    other_cells = "wide" if args.cells == "narrow" else "narrow"
    other_run = None if args.single_cells else timed_run(other_cells, False)
    # multi-GPU self-check after the timed region: the first trees are the same on every rank, and the same as those of
    # the path that reduces the histograms with NCCL instead of the in-kernel peer stores
    consistency = None
    if world > 1:
        sp = main_run["splits"].contiguous()
        gathered = [torch.empty_like(sp) for _ in range(world)]
        dist.all_gather(gathered, sp)
        same_ranks = all(bool(torch.equal(g, gathered[0])) for g in gathered)
        vl = main_run["vals"].contiguous()
        gv = [torch.empty_like(vl) for _ in range(world)]
        dist.all_gather(gv, vl)
        same_vals = all(bool(torch.equal(g, gv[0])) for g in gv)
        base = make_engine(args.cells, "nccl", 3)
        base.step(3)
        torch.cuda.synchronize(dev)
        nb = 3 * cfg["depth"]
        match = (base.splits[:nb, :2] == sp[:nb, :2]).all(1).float().mean()
        leaf_diff = (base.model_vals[:3] - vl[:3]).abs().max()
        base.finish()
        base.close()
        del base
        consistency = {"first_5_trees_identical_on_all_ranks": bool(same_ranks and same_vals),
                       "first_3_trees_splits_equal_to_nccl_path": float(match.item()),
                       "first_3_trees_max_leaf_value_diff_vs_nccl_path": float(leaf_diff.item())}
    del store
    torch.cuda.empty_cache()

    # ---------------- end to end through the public API -----------------------------------------------------------
    e2e = None
    if not args.no_e2e:
        Xp = torch.from_numpy(X).pin_memory().numpy() if hasattr(torch.Tensor, "pin_memory") else X
        e2e_iters = args.e2e_iters if args.e2e_iters > 0 else (1000 if args.config != "small" else 200)
        params_e2e = dict(params, iterations=e2e_iters)
        model = cb.CatBoostClassifier(**params_e2e, verbose=True, metric_period=1)
        devnull = open(os.devnull, "w")
        torch.cuda.synchronize(dev)
        ctx.barrier()
        t0 = time.perf_counter()
        model.fit(Xp, y, log_cout=devnull)
        torch.cuda.synchronize(dev)
        t1 = time.perf_counter()
        e2e_s = torch.tensor([t1 - t0], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)
        iters = e2e_iters
        e2e = {"value": float(e2e_s.item()) / iters * 1000.0, "unit": "s/1000iter",
               "h2d_bytes_per_step": int(X.nbytes * world // iters), "d2h_bytes_per_step": 16,
               "fit_seconds": float(e2e_s.item()), "iterations": iters,
               "fit_breakdown_s": {k: round(float(v), 4) for k, v in model._train_info.get("timings", {}).items()},
               "note": "whole fit(): pinned upload + quantisation + iterations with a per-iteration learn-loss read"}
    apply_info = None
    if not args.no_e2e and rank == 0:
        # batch apply of the model just trained: device-resident rows, quantisation fused into the tree walk
        from catboost_b200.models.gpu_apply import GpuPredictor
        pred = GpuPredictor(model._model, dev)
        rows = min(len(X), 4_000_000)
        xd = torch.from_numpy(X[:rows]).to(dev)
        out = torch.empty((model._model.dims, rows), dtype=torch.float32, device=dev)
        for _ in range(2):
            pred.predict_device(xd, out)
        torch.cuda.synchronize(dev)
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 5
        a0.record()
        for _ in range(reps):
            pred.predict_device(xd, out)
        a1.record()
        torch.cuda.synchronize(dev)
        ms = a0.elapsed_time(a1) / reps
        apply_info = {"rows_per_s": rows / (ms * 1e-3), "rows": rows, "trees": model.tree_count_, "ms": ms,
                      "tree_rows_per_s": rows * model.tree_count_ / (ms * 1e-3), "n_gpus": 1,
                      "note": "kernel only: rows resident on one device"}
        del xd, out, pred
        torch.cuda.empty_cache()
        # the public call on all GPUs of the run: rows streamed from pinned host memory (H2D of every row and D2H of every
        # prediction inside the timed region), one contiguous row range per device
        devs = list(range(world))
        model.predict(Xp[:200_000], prediction_type="RawFormulaVal", task_type="GPU", devices=devs)      # warm-up
        reps_h = max(1, 100_000_000 // len(Xp)) if args.apply_100m else 1
        t0 = time.perf_counter()
        for _ in range(reps_h):
            model.predict(Xp, prediction_type="RawFormulaVal", task_type="GPU", devices=devs)
        dt = time.perf_counter() - t0
        apply_info["host"] = {"rows_per_s": len(Xp) * reps_h / dt, "rows": len(Xp) * reps_h, "n_gpus": world,
                              "seconds": dt, "h2d_bytes": int(Xp.nbytes) * reps_h,
                              "note": "predict(task_type='GPU', devices=all) from pinned host memory; every pass copies "
                                      "all rows to the devices again"}
    if rank == 0:
        ms_per_step = total_ms / K
        value = ms_per_step          # ms per iteration == seconds per 1000 iterations
        base = BASELINE_S_PER_1000.get(args.config)
        out = {"metric": "sec/1000 iters (device-timed, max over ranks)", "value": value, "unit": "s/1000iter",
               "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms_per_step, "higher_is_better": False,
               "scaling": "strong", "vs_baseline": (value / base) if base else None,
               "dtype": {"narrow": "fp32 statistics, histogram cells int32 fixed point (13-16 bit addends, exact integer sums)",
                         "wide": "fp32 statistics, histogram cells 24-bit fixed point in int32 hi/lo pairs (exact integer sums)",
                         "float": "fp32"}[args.cells],
               "data": "synthetic", "impl": "ours",
               "config": {"model": cfg["model"], "global_batch": cfg["rows"], "seq_len": cfg["features"],
                          "parallelism": f"doc-parallel dp{world}", "loss": "Logloss", "depth": cfg["depth"],
                          "border_count": cfg["border_count"], "learning_rate": 0.1, "histogram_reduce": args.reduce, "histogram_cells": args.cells,
                          "l2_policy": ("flush: 512 MiB write between timed iterations" if flush is not None
                                        else "inputs larger than L2")},
               "clocks": clocks, "e2e": e2e, "apply": apply_info, "gpu_launches": launches,
               "other_cells": (None if other_run is None else
                               {"histogram_cells": other_cells, "value": other_run["total_ms"] / K, "unit": "s/1000iter",
                                "learn_loss_last": float(other_run["loss_curve"][-1])}),
               "multi_gpu_consistency": consistency,
               "learn_loss_first_last": [float(loss_curve[1]) if len(loss_curve) > 1 else None, float(loss_curve[-1])]}
        print(json.dumps(out))
    if world > 1:
        dist.barrier(device_ids=[local])
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
