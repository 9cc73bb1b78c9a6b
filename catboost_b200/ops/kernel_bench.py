"""Per-kernel timing and roofline report.

    python -m catboost_b200.ops.kernel_bench [--rows N] [--features F] [--kernel name] [--reps R]

Every kernel is timed in isolation with CUDA events (3 warm-up launches, an L2 flush between timed launches) and
reported as algorithmic bytes / time against a copy bandwidth given with ``--peak-gbs`` (the number a STREAM-style
copy reaches on the machine; default 6650 GB/s).  The same entry point is what the committed ncu summaries were taken on.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys

import numpy as np
import torch


def _time(fn, reps, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for k in range(reps):
        flush.fill_(k & 0xFF)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    return total / reps


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=4_000_000)
    ap.add_argument("--features", type=int, default=28)
    ap.add_argument("--depth", type=int, default=6)
    ap.add_argument("--trees", type=int, default=100)
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--kernel", default="all")
    ap.add_argument("--peak-gbs", type=float, default=0.0, help="measured copy bandwidth of the GPU in GB/s")
    ap.add_argument("--peak-tflops", type=float, default=0.0, help="measured bf16 GEMM throughput of the GPU in TFLOP/s")
    ap.add_argument("--knn-queries", type=int, default=65536)
    ap.add_argument("--knn-cloud", type=int, default=131072)
    ap.add_argument("--knn-dim", type=int, default=128)
    ap.add_argument("--knn-candidates", type=int, default=8, choices=(8, 16), help="length of a candidate list")
    args = ap.parse_args(argv)
    from ..data.pool import Pool
    from ..data.quantization import build_quantization, make_store, quantize_floats_into, FlatFeature
    from ..models.gpu_apply import GpuPredictor
    from ..params import resolve_options
    from ..parallel.runtime import DistContext
    from ..train.boosting import build_store, plan_features
    from ..train.gpu_engine import GpuObliviousEngine
    from ..train.objectives import make_objective
    from . import api as ops
    from . import native

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    lib = native.cuda_lib()
    hbm, src = (args.peak_gbs, "given") if args.peak_gbs > 0 else (6650.0, "default")
    n, F = args.rows, args.features
    rng = np.random.default_rng(0)
    X = rng.standard_normal((n, F), dtype=np.float32)
    y = (X[:, 0] + 0.5 * X[:, 1] * X[:, 2] > 0).astype(np.float32)
    pool = Pool(X, y)
    o = resolve_options(dict(task_type="GPU", border_count=128), "Logloss", n)
    plan = plan_features(o, pool, DistContext(0, 1, dev), None)
    store, _ = build_store(plan, pool, dev)
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    P = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())
    st = lambda: ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    sm = torch.cuda.get_device_properties(dev).multi_processor_count
    out = []

    def report(name, ms, nbytes, note=""):
        gbs = nbytes / (ms * 1e-3) / 1e9
        rec = {"kernel": name, "rows": n, "features": F, "ms": round(ms, 4), "algorithmic_MB": round(nbytes / 1e6, 1),
               "GBps": round(gbs, 1), "frac_of_hbm_peak": round(gbs / hbm, 3), "peak_source": f"{src} {hbm} GB/s",
               "note": note}
        out.append(rec)
        print(json.dumps(rec))

    want = lambda k: args.kernel in ("all", k)
    obj = make_objective("Logloss", {})
    eng = GpuObliviousEngine(store, torch.from_numpy(y), None, torch.zeros(n), obj, depth=args.depth, iterations=8,
                             learning_rate=0.1, l2_leaf_reg=3.0, leaf_iterations=1, use_graph=False)
    eng.step(2)
    torch.cuda.synchronize()

    if want("quantize"):
        xd = torch.from_numpy(X).to(dev)
        q = plan.quant
        borders = torch.from_numpy(np.concatenate(q.borders).astype(np.float32)).to(dev)
        boff = torch.from_numpy(np.concatenate([[0], np.cumsum([len(b) for b in q.borders])]).astype(np.int32)).to(dev)
        nanm = torch.from_numpy(q.nan_is_max).to(dev)
        tmp = torch.zeros_like(store.bins)
        ms = _time(lambda: lib.cb_quantize(P(xd), n, F, xd.stride(0), P(borders), P(boff), P(nanm), P(tmp), store.npad, 0,
                                           st()), args.reps, flush)
        report("cb_quantize_kernel", ms, n * F * 4 + n * ((F + 3) // 4) * 4, "float32 rows -> packed bins")
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        plain = tmp.clone()
        tmp.zero_()
        rc = lib.cb_quantize_tma(P(xd), n, F, xd.stride(0), P(borders), P(boff), P(nanm), P(tmp), store.npad, 0, P(status),
                                 st())
        if rc == 0:
            ms = _time(lambda: lib.cb_quantize_tma(P(xd), n, F, xd.stride(0), P(borders), P(boff), P(nanm), P(tmp),
                                                   store.npad, 0, P(status), st()), args.reps, flush)
            report("cb_quantize_tma_kernel", ms, n * F * 4 + n * ((F + 3) // 4) * 4,
                   f"tiled bulk copies into shared memory; status {int(status.item())}; equal to plain kernel: "
                   f"{bool(torch.equal(tmp, plain))}")
        del xd, tmp
    if want("grad"):
        ms = _time(lambda: eng._grad(), args.reps, flush)
        report("cb_grad_kernel", ms, n * (4 + 4 + 2 + 4 + 2 + 8), "approx rw, target, leaf rw, stats w")
    if want("leaf_pass"):
        def leaf_pass():
            lib.cb_leaf_pass(eng.loss_id, eng.p0, eng.p1, P(eng.approx), P(eng.target), None, P(eng.leaf), None, None, n,
                             eng.L, P(eng.delta), P(eng.sums), P(eng.counter), 1, 0, 1, 3.0, 0.1, P(eng.cur_vals), None,
                             None, eng.L, P(eng.iter_ptr), P(eng.leaf_w), None, sm * 2, st())
        ms = _time(leaf_pass, args.reps, flush)
        report("cb_leaf_pass_kernel", ms, n * (4 + 4 + 2), "first pass of a tree (fp32 cells): approx, target, leaf")
        vmax = torch.tensor([1.0, 0.25], dtype=torch.float32, device=dev)

        def leaf_pass_q():
            lib.cb_leaf_pass_q(eng.loss_id, eng.p0, eng.p1, P(eng.approx), P(eng.target), None, P(eng.leaf), None, None, n,
                               eng.L, P(eng.delta), P(eng.sums), P(eng.counter), 0, 0, 1, 3.0, 0.1, P(eng.cur_vals), None,
                               None, eng.L, P(eng.iter_ptr), P(eng.leaf_w), None, P(vmax), sm * 2, st())
        ms = _time(leaf_pass_q, args.reps, flush)
        report("cb_leaf_pass_kernel[newton step]", ms, n * (4 + 4 + 2), "later pass (fixed-point cells): approx, target, leaf")
    if want("update_leaf"):
        ms = _time(lambda: lib.cb_update_leaf(ctypes.c_void_p(store.handle), P(eng.leaf), P(eng.splits), P(eng.iter_ptr),
                                              eng.depth, 0, sm * 8, st()), args.reps, flush)
        report("cb_update_leaf_kernel", ms, n * (4 + 2 + 2), "one group word, leaf rw")
    if want("apply_tree"):
        ap_ = torch.zeros(store.npad, device=dev)
        zero = torch.zeros(1, dtype=torch.int32, device=dev)
        ms = _time(lambda: lib.cb_apply_tree_bins(ctypes.c_void_p(store.handle), P(ap_), store.npad, P(eng.splits), P(zero),
                                                  eng.depth, P(eng.cur_vals), 1, sm * 8, st()), args.reps, flush)
        report("cb_apply_tree_bins_kernel", ms, n * (4 * args.depth + 8), "depth group words (upper bound), approx rw")
    if want("hist"):
        leaf = torch.zeros(store.npad, dtype=torch.int16, device=dev)
        table = torch.zeros(1, dtype=torch.int16, device=dev)
        ms = _time(lambda: ops.hist(store, leaf, eng.stats, table, 1), args.reps, flush)
        report("cb_hist_kernel", ms, n * ((F + 3) // 4) * (4 + 2 + 8), "stand-alone fp32-atomic histogram, one slot")
    if want("fused"):
        for level in range(args.depth):
            ms = _time(lambda: eng._level_fused(level), args.reps, flush)
            report(f"cb_level_fused_kernel[level={level}]", ms, n * (((F + 3) // 4) * 4 + 2 + 8),
                   "whole level (leaf update, histogram, reduce, score, select); bytes = one pass over bins, leaf, stats")
    if want("predict"):
        model_eng = eng
        sp, vals, wts = model_eng.finish()
        from ..train.boosting import assemble_model

        class _Codec:
            class_names = [0, 1]
        trees = [dict(kind="oblivious", splits=sp[t % len(sp)], values=vals[t % len(sp)], weights=wts[t % len(sp)])
                 for t in range(args.trees)]
        m = assemble_model(o, plan, pool, store, trees, 1, np.zeros(1), _Codec())
        pred = GpuPredictor(m, dev)
        xd = torch.from_numpy(X).to(dev)
        res = torch.empty((1, n), dtype=torch.float32, device=dev)
        ms = _time(lambda: pred.predict_device(xd, res), args.reps, flush)
        report("cb_predict_kernel", ms, n * F * 4 + n * 4, f"{args.trees} trees depth {args.depth}; "
               f"{n / (ms * 1e-3):.3g} rows/s, {n * args.trees / (ms * 1e-3):.3g} tree-rows/s")
    if want("ctr"):
        # one categorical projection of Zipf-distributed values: the three CTR kernels after the (library) sort
        g = torch.Generator().manual_seed(1)
        card = 100_000
        h = (torch.rand(n, generator=g) ** 3 * card).long().to(dev) * 2654435761 - (1 << 40)
        order = torch.randperm(n, generator=g).to(dev)
        cls = torch.from_numpy((y > 0.5).astype(np.uint8)).to(dev)
        sorted_h, srt = torch.sort(h[order], stable=True)
        rows = order[srt]
        ms = _time(lambda: ops.ctr_scan(sorted_h, rows, cls, [0]), args.reps, flush)
        # reads: hash 8 + row id 8 + class 1 (gathered); writes: two prefix columns 8 + group number 4 + flag 1, read again
        # and rewritten by the fix-up pass
        report("cb_ctr_scan (3 launches)", ms, n * (8 + 8 + 1 + 13 + 8 + 13 + 12), "segmented scans of count + one indicator")
        excl, seg_id, uniq, totals = ops.ctr_scan(sorted_h, rows, cls, [0])
        descs = [(0, 1, 0.0, 1.0, 1.0), (0, 1, 0.5, 1.0, 1.0), (0, 1, 1.0, 1.0, 1.0),
                 (1, 0, 0.0, 1.0, float(totals[0].max().item()) + 1.0)]
        ms = _time(lambda: ops.ctr_minmax(descs[:3], excl, totals, seg_id), args.reps, flush)
        report("cb_ctr_minmax_kernel", ms, n * 8, "range of three target-statistic CTRs")
        borders = [np.linspace(0.02, 0.98, 15).astype(np.float32) for _ in descs]
        ms = _time(lambda: ops.ctr_binarize(descs, borders, excl, totals, seg_id, rows, 0, n), args.reps, flush)
        report("cb_ctr_binarize_kernel", ms, n * (8 + 4 + 8 + 4 * 1), "four CTRs -> bytes in document order (scattered)")
    if want("sort"):
        g = torch.Generator().manual_seed(2)
        keys = (torch.rand(n, generator=g) ** 3 * 1_000_000).long().to(dev) * 2654435761 - (1 << 40)
        ms = _time(lambda: ops.sort_pairs(keys), args.reps, flush)
        # 8 passes, each reads keys + values twice (count, scatter) and writes them once
        report("cb_sort_pairs_i64 (8 passes x 4 launches)", ms, n * 8 * (8 + 8 + 4 + 8 + 4), "stable radix sort of (int64 key, int32 position)")
        ms = _time(lambda: torch.sort(keys, stable=True), args.reps, flush)
        report("torch.sort(stable) for comparison", ms, n * 8 * (8 + 8 + 4 + 8 + 4), "library sort of the same keys")
    if want("mvs"):
        stats = eng.stats.clone()
        smax = torch.zeros(2, device=dev)
        ms = _time(lambda: lib.cb_mvs_sample(P(stats), store.npad, n, 0.5, -1.0, 7, P(eng.iter_ptr), P(smax), None, st()),
                   args.reps, flush)
        report("cb_mvs_kernel", ms, n * (4 + 4) * 2, "derivative + weight rows read and written; 40 bisection steps per block of 8192")
    if want("leaf_newton"):
        eng10 = GpuObliviousEngine(store, torch.from_numpy(y), None, torch.zeros(n), obj, depth=args.depth, iterations=4,
                                   learning_rate=0.1, l2_leaf_reg=3.0, leaf_iterations=10, use_graph=False)
        eng10.step(1)
        ms = _time(lambda: eng10._leaves(), args.reps, flush)
        report("cb_leaf_newton_kernel (10 steps, one launch)", ms, 10 * n * (4 + 4 + 2), "approx, target, leaf per step")
        eng10.close()
    if want("multiclass"):
        K = 5
        yk = rng.integers(0, K, n).astype(np.float32)
        for cells, label in ((True, "single int32 cells"), ("wide", "hi/lo cells")):
            engk = GpuObliviousEngine(store, torch.from_numpy(yk), None, torch.zeros((K, n)),
                                      make_objective("MultiClass", {}, n_classes=K), depth=args.depth, iterations=4,
                                      learning_rate=0.1, l2_leaf_reg=3.0, leaf_iterations=1, use_graph=False, dims=K,
                                      quantized_hist=cells)
            engk.step(1)
            if cells is True:
                ms = _time(lambda: engk._grad(), args.reps, flush)
                report("cb_mc_grad_kernel (K=5)", ms, n * (K * 4 * 2 + 4 + 2 + (K + 1) * 4), "approx rw, target, leaf, K + 1 statistic rows")
                ms = _time(lambda: engk._leaves(), args.reps, flush)
                report("cb_mc_leaf_kernel (K=5: sums + K x K Cholesky per leaf)", ms, n * (K * 4 + 4 + 2), "approx, target, leaf")
            for level in (0, args.depth - 1):
                ms = _time(lambda: engk._level_fused(level), args.reps, flush)
                report(f"cb_level_fused_kernel[K=5, level={level}, {label}]", ms, n * (((F + 3) // 4) * 4 + 2 + (K + 1) * 4),
                       "S = 6 statistics")
            engk.close()
    if want("yetirank"):
        from ..train.ranking import YetiRank, _GroupLayout
        g = torch.Generator().manual_seed(6)
        sizes = torch.randint(5, 201, (max(1, n // 100),), generator=g)
        off = torch.cat([torch.zeros(1, dtype=torch.long), torch.cumsum(sizes, 0)])
        off = off[off <= n]
        nq = int(off[-1])
        lay = _GroupLayout(off.to(dev))
        ya = YetiRank({})
        a_ = torch.randn(nq, generator=g).to(dev)
        t_ = torch.randint(0, 5, (nq,), generator=g).float().to(dev)
        ms = _time(lambda: ya._der_hess_device(a_, t_, None, lay), args.reps, flush)
        report("cb_yetirank_kernel (queries of 5..200 documents, 10 permutations)", ms, nq * (4 + 4 + 8),
               f"{lay.Q} queries, {nq} documents")
    if want("predict_wide"):
        Fw, Tw = 700, 200
        nw = min(n, 1_000_000)
        Xw = torch.rand((nw, Fw), generator=torch.Generator().manual_seed(3)).to(dev)
        S = Tw * 6
        gcol = torch.Generator().manual_seed(4)
        col = torch.randint(0, Fw, (S,), generator=gcol, dtype=torch.int32).to(dev)
        bor = torch.rand(S, generator=gcol).to(dev)
        depth_t = torch.full((Tw,), 6, dtype=torch.int32, device=dev)
        soff = (torch.arange(Tw, dtype=torch.int32) * 6).to(dev)
        loff = (torch.arange(Tw, dtype=torch.int64) * 64).to(dev)
        vals = torch.randn(Tw * 64, generator=gcol).to(dev)
        bias = torch.zeros(1, device=dev)
        res = torch.empty((1, nw), device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        os.environ["CB200_PREDICT_WIDE_TMA"] = "1"
        ms = _time(lambda: lib.cb_predict_oblivious_wide(P(Xw), nw, Fw, Fw, None, P(depth_t), P(soff), P(col), P(bor), P(loff),
                                                         P(vals), Tw, S, 1, Tw * 64, 1.0, P(bias), P(res), P(status), st()),
                   args.reps, flush)
        report("cb_predict_wide_tma_kernel (1M x 700, 200 trees)", ms, nw * Fw * 4 + nw * 4,
               f"{nw / (ms * 1e-3):.3g} rows/s; rows by bulk copies; status {int(status.item())}")
        ref = res.clone()
        os.environ["CB200_PREDICT_WIDE_TMA"] = "0"
        ms = _time(lambda: lib.cb_predict_oblivious_wide(P(Xw), nw, Fw, Fw, None, P(depth_t), P(soff), P(col), P(bor), P(loff),
                                                         P(vals), Tw, S, 1, Tw * 64, 1.0, P(bias), P(res), None, st()),
                   args.reps, flush)
        report("cb_predict_wide_kernel (1M x 700, 200 trees)", ms, nw * Fw * 4 + nw * 4,
               f"{nw / (ms * 1e-3):.3g} rows/s; rows by register-staged loads; largest difference to the bulk-copy variant "
               f"{float((res - ref).abs().max()):.3g}")
    if want("knn"):
        # distance GEMM + top-k on the tensor cores against the library route (bf16 matmul, then topk over the matrix)
        nq, ne, d = args.knn_queries, args.knn_cloud, args.knn_dim
        tf_peak, tf_src = (args.peak_tflops, "given") if args.peak_tflops > 0 else (1590.0, "default")
        gk = torch.Generator().manual_seed(5)
        dpad = (d + 63) // 64 * 64
        qb = torch.zeros((nq, dpad), dtype=torch.bfloat16, device=dev)
        eb = torch.zeros((ne, dpad), dtype=torch.bfloat16, device=dev)
        qb[:, :d] = torch.randn((nq, d), generator=gk).to(dev)
        eb[:, :d] = torch.randn((ne, d), generator=gk).to(dev)
        e2 = (eb.float() ** 2).sum(1).contiguous()
        C = args.knn_candidates
        splits = int(lib.cb_knn_splits(nq, ne))
        oi = torch.empty((nq, 2 * splits, C), dtype=torch.int32, device=dev)
        ov = torch.empty((nq, 2 * splits, C), dtype=torch.float32, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        flops = 2.0 * nq * ne * dpad
        ms = _time(lambda: lib.cb_knn_tc(P(qb), nq, P(eb), ne, dpad, P(e2), splits, C, P(oi), P(ov), P(status), st()),
                   args.reps, flush)
        tf = flops / (ms * 1e-3) / 1e12
        rec = {"kernel": f"cb_knn_tc_kernel ({nq} x {ne} x {dpad}, {splits} cloud ranges)", "ms": round(ms, 4),
               "TFLOPs": round(tf, 1), "frac_of_bf16_peak": round(tf / tf_peak, 3), "peak_source": f"{tf_src} {tf_peak} TFLOP/s",
               "note": f"tcgen05.mma + top-{C} epilogue, no distance matrix in memory; status {int(status.item())}"}
        out.append(rec)
        print(json.dumps(rec))

        def library():
            step = max(1, (1 << 30) // (ne * 2))
            for s0 in range(0, nq, step):
                sc = e2.unsqueeze(0) - 2.0 * (qb[s0:s0 + step] @ eb.t()).float()
                torch.topk(sc, C, dim=1, largest=False, sorted=True)

        ms2 = _time(library, max(1, args.reps // 2), flush)
        rec = {"kernel": "library route: bf16 matmul + topk in chunks of 1 GiB of scores", "ms": round(ms2, 4),
               "TFLOPs": round(flops / (ms2 * 1e-3) / 1e12, 1), "note": f"{ms2 / ms:.1f} x the fused kernel's time"}
        out.append(rec)
        print(json.dumps(rec))
    return 0


if __name__ == "__main__":
    sys.exit(main())
