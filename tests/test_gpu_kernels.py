"""Numerics of the CUDA kernels against plain PyTorch fp32 restatements of the same operation."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _store(n=5000, F=7, border_count=32, seed=0, device="cuda"):
    from catboost_b200.data.pool import Pool
    from catboost_b200.params import resolve_options
    from catboost_b200.parallel.runtime import DistContext
    from catboost_b200.train.boosting import build_store, plan_features
    rng = np.random.default_rng(seed)
    X = rng.standard_normal((n, F), dtype=np.float32)
    X[rng.random((n, F)) < 0.02] = np.nan
    y = (X[:, 0] + 0.5 * np.nan_to_num(X[:, 1]) > 0).astype(np.float32)
    pool = Pool(X, y)
    o = resolve_options(dict(border_count=border_count, task_type="GPU" if device == "cuda" else "CPU"), "Logloss", n)
    plan = plan_features(o, pool, DistContext(0, 1, torch.device(device)), None)
    store, _ = build_store(plan, pool, torch.device(device))
    return X, y, plan, store


def test_quantize_matches_searchsorted():
    X, y, plan, store = _store()
    torch.cuda.synchronize()
    for f in range(store.F):
        b = torch.from_numpy(plan.quant.borders[f])
        col = torch.from_numpy(X[:, f])
        ref = torch.searchsorted(b, col.contiguous(), right=False)      # number of borders < x
        ref = torch.where(torch.isnan(col), torch.zeros_like(ref), ref)
        got = store.column(f).cpu().long()
        assert torch.equal(got, ref), f"feature {f}"


@pytest.mark.parametrize("n,F", [(5000, 8), (70001, 28), (3001, 72)])
def test_quantize_tma_matches_searchsorted(n, F):
    """Row pitch a multiple of 16 bytes: the tiled-bulk-copy kernel is used; several feature boxes, ragged last tile."""
    from catboost_b200.data import quantization as Q
    X, y, plan, store = _store(n=n, F=F, border_count=64)
    assert Q.LAST_QUANTIZE["kernel"] == "tma"
    bins = store.bins.cpu().numpy()
    q = plan.quant
    for f in range(F):
        col = X[:, f]
        ref = np.searchsorted(q.borders[f], col, side="left")
        ref[np.isnan(col)] = len(q.borders[f]) if q.nan_is_max[f] else 0
        got = (bins[f // 4, :n].view(np.uint32) >> (8 * (f % 4))) & 255
        assert np.array_equal(got, ref.astype(np.uint32)), f


@pytest.mark.parametrize("nslots,S", [(1, 2), (8, 2), (5, 3), (64, 2)])
def test_hist_matches_reference(nslots, S):
    from catboost_b200.ops import api as ops
    X, y, plan, store = _store(n=20011, F=9, border_count=64, seed=1)
    g = torch.Generator().manual_seed(3)
    n, npad = store.n, store.npad
    leaf = torch.zeros(npad, dtype=torch.int16)
    leaf[:n] = torch.randint(0, nslots + 2, (n,), generator=g).short()
    table = torch.full((nslots + 2,), -1, dtype=torch.int16)
    table[:nslots] = torch.arange(nslots, dtype=torch.int16)
    stats = torch.zeros((S, npad))
    stats[:, :n] = torch.randn((S, n), generator=g)
    got = ops.hist(store, leaf.cuda(), stats.cuda(), table.cuda(), nslots)
    ref = ops.hist_reference(store, leaf.cuda(), stats.cuda(), table.cuda(), nslots)
    torch.cuda.synchronize()
    assert torch.allclose(got, ref, rtol=1e-4, atol=2e-3), float((got - ref).abs().max())


def test_leaf_index_and_update_match_reference():
    from catboost_b200.ops import api as ops
    X, y, plan, store = _store(n=7001, F=6, border_count=16, seed=2)
    splits = torch.tensor([[0, 3, 0, 0], [2, 7, 0, 0], [-1, 0, 0, 0], [5, 1, 0, 0]], dtype=torch.int32)
    got = ops.leaf_index(store, splits.cuda())[: store.n].long().cpu()
    ref = ops.leaf_index_reference(store, splits.numpy()).cpu()
    assert torch.equal(got, ref)
    leaf = torch.zeros(store.npad, dtype=torch.int16, device="cuda")
    for k, (f, b, _, fl) in enumerate(splits.tolist()):
        if f >= 0:
            ops.update_leaf(store, leaf, f, b, bool(fl & 1), k)
    assert torch.equal(leaf[: store.n].long().cpu(), ref)


def _engine_vs_generic(depth, n, F, loss="Logloss", score="Cosine", leaf_iters=3):
    """One tree of the fused device trainer against the generic (tensor-op) learner on identical statistics."""
    from catboost_b200.params import resolve_options
    from catboost_b200.train.generic import GenericLearner, estimate_leaves
    from catboost_b200.train.gpu_engine import GpuObliviousEngine
    from catboost_b200.train.objectives import make_objective
    X, y, plan, store = _store(n=n, F=F, border_count=32, seed=5)
    if loss == "RMSE":
        y = (np.nan_to_num(X[:, 0]) * 2 + np.nan_to_num(X[:, 1]) ** 2).astype(np.float32)
    obj = make_objective(loss, {})
    o = resolve_options(dict(loss_function=loss, depth=depth, task_type="GPU", bootstrap_type="No", random_strength=0,
                             score_function=score, leaf_estimation_iterations=leaf_iters, learning_rate=0.5,
                             l2_leaf_reg=3.0, border_count=32), loss, n)
    eng = GpuObliviousEngine(store, torch.from_numpy(y), None, torch.zeros(n), obj, depth=depth, iterations=3,
                             learning_rate=0.5, l2_leaf_reg=3.0, score_function=score, random_strength=0.0,
                             bootstrap_type="No", leaf_method="Newton", leaf_iterations=leaf_iters, seed=0)
    eng.step(1)
    sp, vals, wts = eng.finish()
    # generic learner
    approx = torch.zeros((1, store.npad), device="cuda")
    target = torch.from_numpy(y).cuda()
    der, hess = obj.der_hess(approx[:, :n], target, None)
    dp = torch.zeros((1, store.npad), device="cuda"); hp = torch.zeros((1, store.npad), device="cuda")
    dp[:, :n], hp[:, :n] = der, hess
    gl = GenericLearner(store, o, 1)
    tr = gl.build_tree(dp, hp, None, 0)
    gv, gw = estimate_leaves(obj, approx, target, None, tr.leaf, tr.n_leaves, n, o)
    assert np.array_equal(sp[0][:, :2], tr.splits[:, :2]), (sp[0], tr.splits)
    assert np.allclose(wts[0], gw, rtol=1e-5, atol=1e-3)
    assert np.allclose(vals[0], gv[:, 0], rtol=2e-3, atol=2e-4), float(np.abs(vals[0] - gv[:, 0]).max())
    eng.close()


@pytest.mark.parametrize("depth", [1, 2, 4, 6])
def test_fused_level_kernel_matches_generic_learner(depth):
    _engine_vs_generic(depth, 30011, 10)


def test_fused_level_kernel_rmse_l2():
    _engine_vs_generic(5, 20000, 6, loss="RMSE", score="L2", leaf_iters=1)


def test_graph_replay_equals_eager():
    from catboost_b200.train.gpu_engine import GpuObliviousEngine
    from catboost_b200.train.objectives import make_objective
    X, y, plan, store = _store(n=40000, F=8, border_count=64, seed=7)
    obj = make_objective("Logloss", {})
    outs = []
    for use_graph in (False, True):
        eng = GpuObliviousEngine(store, torch.from_numpy(y), None, torch.zeros(len(y)), obj, depth=5, iterations=6,
                                 learning_rate=0.3, l2_leaf_reg=3.0, random_strength=1.0, bootstrap_type="Bayesian",
                                 leaf_iterations=2, seed=3, use_graph=use_graph)
        eng.step(6)
        sp, vals, wts = eng.finish()
        outs.append((sp, vals, eng.learn_loss_history()))
        eng.close()
    assert np.array_equal(outs[0][0][:, :, :2], outs[1][0][:, :, :2])
    assert np.allclose(outs[0][1], outs[1][1], rtol=1e-3, atol=1e-4)
    assert outs[1][2][-1] < outs[1][2][0]


def test_unfused_path_matches_fused():
    from catboost_b200.train.gpu_engine import GpuObliviousEngine
    from catboost_b200.train.objectives import make_objective
    X, y, plan, store = _store(n=25000, F=8, border_count=32, seed=9)
    obj = make_objective("Logloss", {})
    res = []
    for fused in (True, False):
        eng = GpuObliviousEngine(store, torch.from_numpy(y), None, torch.zeros(len(y)), obj, depth=4, iterations=3,
                                 learning_rate=0.3, l2_leaf_reg=3.0, random_strength=0.0, bootstrap_type="No",
                                 leaf_iterations=1, seed=3, use_graph=False)
        if not fused:
            eng.reduce = "nccl"          # stand-alone kernels (hist, score, select) without the cooperative launch
            eng.partial = torch.zeros((eng.slots_max * eng.S, eng.TB), device="cuda")
        eng.step(3)
        res.append(eng.finish())
        eng.close()
    assert np.array_equal(res[0][0][:, :, :2], res[1][0][:, :, :2])
    assert np.allclose(res[0][1], res[1][1], rtol=1e-3, atol=1e-4)


def test_gpu_fit_predict_and_gpu_apply():
    import catboost_b200 as cb
    rng = np.random.default_rng(0)
    n, F = 60000, 16
    X = rng.standard_normal((n, F), dtype=np.float32)
    w = rng.standard_normal(F).astype(np.float32)
    y = (X @ w + 0.5 * rng.standard_normal(n, dtype=np.float32) > 0).astype(int)
    m = cb.CatBoostClassifier(iterations=40, depth=6, learning_rate=0.2, task_type="GPU", devices="0", verbose=False,
                              allow_writing_files=False)
    m.fit(X[:50000], y[:50000], eval_set=(X[50000:], y[50000:]))
    ev = m.get_evals_result()
    assert ev["validation"]["Logloss"][-1] < 0.45
    p_cpu = m.predict(X[50000:], prediction_type="RawFormulaVal")
    p_gpu = m.predict(X[50000:], prediction_type="RawFormulaVal", task_type="GPU")
    assert np.allclose(p_cpu, p_gpu, rtol=1e-4, atol=1e-4)
    acc = float((m.predict(X[50000:]) == y[50000:]).mean())
    assert acc > 0.88, acc
    # deeper than 8 levels: the apply kernel takes its per-row path instead of the four-rows-per-word compare
    deep = cb.CatBoostClassifier(iterations=6, depth=10, learning_rate=0.2, task_type="GPU", devices="0", verbose=False,
                                 allow_writing_files=False).fit(X[:50000], y[:50000])
    assert np.allclose(deep.predict(X[50000:], prediction_type="RawFormulaVal"),
                       deep.predict(X[50000:], prediction_type="RawFormulaVal", task_type="GPU"), rtol=1e-4, atol=1e-4)


def test_gpu_regression_rmse():
    import catboost_b200 as cb
    rng = np.random.default_rng(1)
    X = rng.standard_normal((30000, 8), dtype=np.float32)
    y = X[:, 0] * 2 + np.sin(X[:, 1] * 2) + 0.1 * rng.standard_normal(30000, dtype=np.float32)
    m = cb.CatBoostRegressor(iterations=60, depth=5, learning_rate=0.2, task_type="GPU", verbose=False,
                             allow_writing_files=False)
    m.fit(X, y)
    rmse = float(np.sqrt(np.mean((m.predict(X) - y) ** 2)))
    assert rmse < 0.45, rmse


def test_gpu_ranking_objectives_use_fused_engine():
    """Query-wise losses have no device formula: their derivatives come from the objective's tensor code, the tree
    structure and the leaves from the fused level kernels and the leaf pass."""
    import catboost_b200 as cb
    rng = np.random.default_rng(0)
    sizes = rng.integers(5, 40, 400)
    gid = np.repeat(np.arange(400), sizes)
    n = len(gid)
    X = rng.standard_normal((n, 10)).astype(np.float32)
    score = X @ rng.standard_normal(10) + 0.5 * rng.standard_normal(n)
    rel = np.digitize(score, np.quantile(score, [0.5, 0.8, 0.95])).astype(np.float32)
    for loss in ("YetiRank", "QueryRMSE", "PairLogit"):
        m = cb.CatBoostRanker(loss_function=loss, iterations=30, depth=4, learning_rate=0.3, verbose=False,
                              allow_writing_files=False, eval_metric="NDCG", task_type="GPU", devices="0",
                              leaf_estimation_iterations=1)
        m.fit(X, rel, group_id=gid)
        assert m._train_info.get("launches_per_iter", 0) > 0, loss
        ev = m.eval_metrics(cb.Pool(X, rel, group_id=gid), ["NDCG"], eval_period=29)["NDCG"]
        assert ev[-1] > 0.9, (loss, ev)


def test_yetirank_kernel_matches_tensor_reference():
    """cb_yetirank_kernel with given uniforms against the same computation written with tensor ops."""
    from catboost_b200.train.ranking import YetiRank, _GroupLayout
    rng = np.random.default_rng(5)
    sizes = rng.integers(1, 70, 300)
    # longer queries: 4 and 8 keys per lane in the warp-per-permutation kernel, and two that the block-wide kernel takes
    sizes[3], sizes[10], sizes[20], sizes[30], sizes[40] = 130, 250, 256, 300, 600
    off = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
    n = int(off[-1])
    dev = torch.device("cuda")
    a = torch.from_numpy(rng.standard_normal(n).astype(np.float32)).to(dev)
    t = torch.from_numpy(rng.integers(0, 4, n).astype(np.float32)).to(dev)
    w = torch.from_numpy(rng.uniform(0.5, 2.0, n).astype(np.float32)).to(dev)
    obj = YetiRank({"permutations": 6, "decay": 0.85})
    lay = _GroupLayout(torch.from_numpy(off).to(dev))
    P = obj.permutations
    noise = torch.from_numpy(rng.uniform(0.01, 0.99, (P, n)).astype(np.float32)).to(dev)
    der, hess = obj._der_hess_device(a, t, w, lay, noise=noise)
    # reference
    A, T = lay.gather(a, -1e30), lay.gather(t)
    Q, L = lay.Q, lay.Lmax
    rd = torch.zeros((Q, L), device=dev, dtype=torch.float64)
    rh = torch.zeros((Q, L), device=dev, dtype=torch.float64)
    decay_pow = 0.85 ** torch.arange(L - 1, device=dev, dtype=torch.float64)
    for p_ in range(P):
        u = lay.gather(noise[p_], 0.5).clamp(1e-6, 1 - 1e-6)
        noisy = torch.where(lay.mask, A + torch.log(u / (1.000001 - u)), torch.full_like(A, -1e30))
        order = torch.argsort(noisy, dim=1, descending=True, stable=True)
        first, second = order[:, :-1], order[:, 1:]
        valid = lay.mask.gather(1, first) & lay.mask.gather(1, second)
        t1, t2 = T.gather(1, first), T.gather(1, second)
        wgt = 0.15 * decay_pow.unsqueeze(0) * (t1 - t2).abs().double() * valid
        win = torch.where(t1 > t2, first, second)
        los = torch.where(t1 > t2, second, first)
        pr = torch.sigmoid((A.gather(1, los) - A.gather(1, win)).double())
        rd.scatter_add_(1, win, wgt * pr); rd.scatter_add_(1, los, -wgt * pr)
        rh.scatter_add_(1, win, wgt * pr * (1 - pr)); rh.scatter_add_(1, los, wgt * pr * (1 - pr))
    W = lay.gather(w).double()
    ref_d = lay.scatter(rd / P * W, n).float()
    ref_h = lay.scatter(rh / P * W, n).float().clamp_min(1e-16)
    assert torch.allclose(der[0], ref_d, rtol=2e-4, atol=2e-6), float((der[0] - ref_d).abs().max())
    assert torch.allclose(hess[0], ref_h, rtol=2e-4, atol=2e-6)


def test_training_is_repeatable():
    """Two runs with the same seed choose the same splits (the tile reduction has a fixed order; only the last bits of
    the double-precision leaf sums may differ between runs)."""
    import catboost_b200 as cb
    rng = np.random.default_rng(2)
    X = rng.standard_normal((150000, 12), dtype=np.float32)
    y = (X[:, 0] * X[:, 1] + X[:, 2] + 0.3 * rng.standard_normal(150000) > 0).astype(int)
    runs = []
    for _ in range(2):
        m = cb.CatBoostClassifier(iterations=25, depth=6, learning_rate=0.2, task_type="GPU", devices="0", verbose=False,
                                  allow_writing_files=False, random_seed=7)
        m.fit(X, y)
        runs.append(m)
    s0 = [(s.feature, s.border) for s in runs[0]._model.splits]
    s1 = [(s.feature, s.border) for s in runs[1]._model.splits]
    assert s0 == s1
    p0 = runs[0].predict(X[:5000], prediction_type="RawFormulaVal")
    p1 = runs[1].predict(X[:5000], prediction_type="RawFormulaVal")
    assert np.allclose(p0, p1, rtol=1e-5, atol=1e-6)


def test_logged_learn_curve_matches_model():
    """Per-iteration logging reads the learn loss from the device history behind the launches: the logged curve must be
    the loss of the model after each tree."""
    import io
    import catboost_b200 as cb
    rng = np.random.default_rng(3)
    X = rng.standard_normal((40000, 8), dtype=np.float32)
    y = (X[:, 0] + X[:, 1] * X[:, 2] > 0).astype(int)
    for T in (1, 2, 9):
        m = cb.CatBoostClassifier(iterations=T, depth=4, learning_rate=0.3, task_type="GPU", devices="0", verbose=True,
                                  allow_writing_files=False)
        m.fit(X, y, log_cout=io.StringIO())
        logged = m.get_evals_result()["learn"]["Logloss"]
        assert len(logged) == T
        ref = m.eval_metrics(cb.Pool(X, y), ["Logloss"])["Logloss"]
        assert np.allclose(logged, ref, rtol=1e-4, atol=1e-5), (T, logged, ref)


def test_generic_gpu_path_metrics_match_host():
    """MultiClass trains through the general learner on the GPU; its per-iteration metrics are evaluated on the device
    and must agree with the host metric code."""
    import catboost_b200 as cb
    rng = np.random.default_rng(4)
    X = rng.standard_normal((20000, 8), dtype=np.float32)
    y = np.argmax(X[:, :3] + 0.3 * rng.standard_normal((20000, 3)), 1)
    m = cb.CatBoostClassifier(loss_function="MultiClass", iterations=8, depth=4, learning_rate=0.3, task_type="GPU",
                              devices="0", verbose=False, allow_writing_files=False, custom_metric=["Accuracy"])
    m.fit(X, y)
    ev = m.get_evals_result()["learn"]
    ref = m.eval_metrics(cb.Pool(X, y), ["MultiClass", "Accuracy"])
    assert np.allclose(ev["MultiClass"], ref["MultiClass"], rtol=1e-4, atol=1e-5)
    assert np.allclose(ev["Accuracy"], ref["Accuracy"], atol=1e-6)
    assert ev["Accuracy"][-1] > 0.8


def test_gpu_categorical_features_with_ctrs():
    """Categorical columns: hashing, grouping and ordered target statistics on the device, trees by the fused engine; the
    CPU evaluator applies the stored CTR tables to the same rows."""
    import catboost_b200 as cb
    import pandas as pd
    rng = np.random.default_rng(6)
    n = 60000
    c1, c2 = rng.integers(0, 500, n), rng.integers(0, 30, n)
    num = rng.standard_normal((n, 3)).astype(np.float32)
    eff = rng.standard_normal(500)[c1] + 0.5 * rng.standard_normal(30)[c2]
    y = (0.5 * num[:, 0] + eff + 0.3 * rng.standard_normal(n) > 0).astype(int)
    df = pd.DataFrame({"a": num[:, 0], "b": num[:, 1], "c": num[:, 2], "k1": c1, "k2": c2})
    tr, te = slice(0, 50000), slice(50000, n)
    m = cb.CatBoostClassifier(iterations=60, depth=6, learning_rate=0.2, task_type="GPU", devices="0", verbose=False,
                              allow_writing_files=False, one_hot_max_size=2, max_ctr_complexity=1)
    m.fit(df.iloc[tr], y[tr], cat_features=["k1", "k2"])
    assert m._train_info.get("launches_per_iter", 0) > 0            # the fused engine trained it
    acc = float((m.predict(df.iloc[te]) == y[te]).mean())
    assert acc > 0.85, acc
    base = cb.CatBoostClassifier(iterations=60, depth=6, learning_rate=0.2, task_type="GPU", devices="0", verbose=False,
                                 allow_writing_files=False).fit(num[tr], y[tr])
    assert acc > float((base.predict(num[te]) == y[te]).mean()) + 0.1      # the categorical signal is used


def test_device_wait_times_out_without_hanging():
    """A wait on a tag nobody writes returns with the status word set (bounded spin, no trap)."""
    from catboost_b200.ops import native
    from catboost_b200.parallel.runtime import ArenaLayout, DistContext, PeerArena
    dev = torch.device("cuda", 0)
    ctx = DistContext(0, 1, dev)
    arena = PeerArena(ctx, ArenaLayout(1, 256, 64), timeout_s=0.05)
    lib = native.cuda_lib()
    # pretend to be rank 0 of 2 whose peer never writes: build a 2-rank comm over the same local buffer
    L = ArenaLayout(2, 256, 64)
    buf = torch.zeros(L.total_bytes, dtype=torch.uint8, device=dev)
    arr = ctypes.c_void_p * 2
    base = buf.data_ptr()
    h = lib.cb_comm_create(0, 2, int(0.05e9), ctypes.c_void_p(arena.status.data_ptr()),
                           ctypes.c_void_p(arena.epoch.data_ptr()), arr(base + L.off_mbox, base + L.off_mbox),
                           arr(base + L.off_mbox_flag, base + L.off_mbox_flag),
                           256, arr(base + L.off_slots, base + L.off_slots),
                           arr(base + L.off_slot_flag, base + L.off_slot_flag), 64)
    vals = torch.ones(4, dtype=torch.float64, device=dev)
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.cb_allreduce_sum(ctypes.c_void_p(h), ctypes.c_void_p(vals.data_ptr()), 4, st) == 0
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="timed out"):
        arena.check_status()
    lib.cb_comm_destroy(ctypes.c_void_p(h))


@pytest.mark.gpu
@pytest.mark.parametrize("n,card,nb", [(50_000, 37, 1), (300_001, 5, 2), (20_000, 15_000, 0), (4097, 1, 1), (9000, 3, 4)])
def test_ctr_kernels_match_tensor_implementation(n, card, nb):
    """Segmented scans, totals, value ranges and buckets of the CTR kernels against the tensor code."""
    from catboost_b200.train.ctr import _KernelGroup, _TensorGroup
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(n + card)
    # long and short groups, negative hashes included; several tiles
    h = (torch.randint(0, card, (n,), generator=g) * 7919 - 3 * card * 1000).to(dev)
    order = torch.randperm(n, generator=g).to(dev)
    cls = torch.randint(0, nb + 2, (n,), generator=g).to(dev)
    need_tb = list(range(nb))
    kg = _KernelGroup(h, order, cls.to(torch.uint8), need_tb, True)
    tg = _TensorGroup(h, order, cls, need_tb, True)
    assert torch.equal(kg.uniq_t, tg.uniq_t)
    assert torch.equal(kg.totals, tg.totals)
    # exclusive prefixes: kernel output is in sorted order, the tensor code's in document order
    back = torch.empty_like(tg.prefix)
    back[:, kg.rows_t] = kg.excl.float()
    assert torch.equal(back, tg.prefix)
    keys = torch.empty(n, dtype=torch.int64, device=dev)
    keys[kg.rows_t] = kg.seg_id.long()
    assert torch.equal(keys, tg.keys_t)
    descs = [(0, 1 + k, 0.5 * (k + 1), 1.0, 1.0) for k in range(nb)] + [(1, 0, 0.0, 1.0, float(tg.totals[0].max()) + 1.0),
                                                                       (1, 0, 1.0, 1.0, float(n) + 1.0)]
    target = [d for d in descs if d[0] == 0]
    assert kg.value_ranges(target) == tg.value_ranges(target)
    rng = np.random.default_rng(0)
    borders = [np.sort(rng.uniform(0.0, 1.0, 15)).astype(np.float32) for _ in descs]
    lo, cnt = n // 5, n // 2
    a = kg.binarize(descs, borders, lo, cnt)
    b = tg.binarize(descs, borders, lo, cnt)
    for x, y in zip(a, b):
        assert torch.equal(x, y)
    sample = torch.arange(0, n, 7, device=dev)
    assert torch.equal(kg.sample_values(descs[-1], sample), tg.sample_values(descs[-1], sample))


@pytest.mark.gpu
def test_gpu_apply_streams_chunks_through_two_buffers():
    """Host rows in several chunks (the last one short), three output dimensions."""
    import catboost_b200 as cb
    from catboost_b200.models.gpu_apply import GpuPredictor
    rng = np.random.default_rng(4)
    X = rng.standard_normal((4500, 9)).astype(np.float32)
    y = np.digitize(X[:, 0] + 0.4 * X[:, 3], [-0.4, 0.5])
    m = cb.CatBoostClassifier(iterations=25, depth=5, loss_function="MultiClass", verbose=False, allow_writing_files=False,
                              task_type="CPU").fit(X, y)
    want = m.predict(X, prediction_type="RawFormulaVal")
    pred = GpuPredictor(m._model, "cuda:0")
    for chunk in (1000, 4500, 7000):
        got = pred.predict(X, chunk_rows=chunk)
        np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-5)


def test_gpu_snapshot_resume_equals_uninterrupted(tmp_path):
    """The device trainer stops after 7 of 20 iterations, a second fit picks the snapshot up and ends with exactly the
    model of an uninterrupted run (random bootstrap weights and score noise included: they are functions of the
    iteration counter, which the snapshot restores)."""
    import catboost_b200 as cb
    rng = np.random.default_rng(4)
    X = rng.standard_normal((30_000, 9)).astype(np.float32)
    y = (X[:, 0] * X[:, 1] + 0.5 * X[:, 2] > 0).astype(int)
    Xe, ye = X[:5000], y[:5000]
    common = dict(depth=5, learning_rate=0.3, verbose=False, random_seed=3, task_type="GPU", train_dir=str(tmp_path),
                  allow_writing_files=True, leaf_estimation_iterations=3)
    full = cb.CatBoostClassifier(iterations=20, **common).fit(X, y, eval_set=(Xe, ye))
    part = cb.CatBoostClassifier(iterations=7, save_snapshot=True, snapshot_file="g.snap", **common).fit(X, y, eval_set=(Xe, ye))
    assert part.tree_count_ == 7 and (tmp_path / "g.snap").exists()
    import shutil
    shutil.copy(tmp_path / "g.snap", tmp_path / "g2.snap")
    resumed = cb.CatBoostClassifier(iterations=20, save_snapshot=True, snapshot_file="g.snap", **common).fit(X, y, eval_set=(Xe, ye))
    assert resumed.tree_count_ == 20
    a = resumed.predict(X, prediction_type="RawFormulaVal")
    b = full.predict(X, prediction_type="RawFormulaVal")
    # same structure; the values agree to float rounding (the per-leaf sums are added with floating-point atomics, whose
    # order is not fixed, so not even two identical runs agree to the last bit)
    assert [(s.feature, s.border) for s in resumed._model.splits] == [(s.feature, s.border) for s in full._model.splits]
    assert np.allclose(a, b, rtol=1e-5, atol=1e-5), float(np.abs(a - b).max())
    ev_full = full.get_evals_result()["validation"]["Logloss"]
    ev_res = resumed.get_evals_result()["validation"]["Logloss"]
    assert len(ev_res) == len(ev_full) and np.allclose(ev_res, ev_full, rtol=1e-6)
    # the general learner (taken here because of rsm < 1) continues a snapshot written by the device trainer: same
    # container, same state
    cont = cb.CatBoostClassifier(iterations=9, save_snapshot=True, snapshot_file="g2.snap", rsm=0.9, **common).fit(X, y)
    assert cont.tree_count_ == 9
    first = lambda m, k: [(s.feature, s.border) for t in m._model.trees[:k] for s in (m._model.splits[i] for i in t.splits)]
    assert first(cont, 7) == first(part, 7)


def test_gpu_apply_from_pinned_memory_and_several_devices():
    """predict(task_type='GPU'): rows taken straight from pinned memory (no staging copy) and, with more than one GPU,
    sharded over the devices, against the CPU evaluator."""
    import catboost_b200 as cb
    rng = np.random.default_rng(6)
    X = rng.standard_normal((60_000, 12)).astype(np.float32)
    y = (X[:, 0] + X[:, 1] * X[:, 2] > 0).astype(int)
    m = cb.CatBoostClassifier(iterations=25, depth=5, learning_rate=0.3, task_type="GPU", verbose=False,
                              allow_writing_files=False).fit(X, y)
    ref = m.predict(X, prediction_type="RawFormulaVal")
    Xp = torch.from_numpy(X).pin_memory().numpy()
    assert torch.from_numpy(Xp).is_pinned()
    got = m.predict(Xp, prediction_type="RawFormulaVal", task_type="GPU", devices="0")
    assert np.allclose(got, ref, rtol=1e-5, atol=1e-5)
    from catboost_b200.models.gpu_apply import GpuPredictor
    small = GpuPredictor(m._model, "cuda:0").predict(Xp, chunk_rows=7000)          # several chunks, short last one
    assert np.allclose(small[:, 0], ref, rtol=1e-5, atol=1e-5)
    if torch.cuda.device_count() >= 2:
        both = m.predict(Xp, prediction_type="RawFormulaVal", task_type="GPU", devices="0-1")
        assert np.allclose(both, ref, rtol=1e-5, atol=1e-5)
        # the same model on the second device after the first (function attributes are per device)
        second = m.predict(X, prediction_type="RawFormulaVal", task_type="GPU", devices="1")
        assert np.allclose(second, ref, rtol=1e-5, atol=1e-5)


def test_device_side_metrics_match_host_metrics():
    """AUC / F1 / Precision / Recall logged during a GPU fit are evaluated where the cursor lives; they agree with the
    host implementations applied to the finished model."""
    import catboost_b200 as cb
    rng = np.random.default_rng(12)
    X = rng.standard_normal((15_000, 6)).astype(np.float32)
    y = (X[:, 0] + 0.5 * X[:, 1] + 0.7 * rng.standard_normal(15_000) > 0.2).astype(int)
    w = (rng.random(15_000) + 0.5).astype(np.float32)
    names = ["AUC", "F1", "Precision", "Recall"]
    m = cb.CatBoostClassifier(iterations=10, depth=4, learning_rate=0.3, task_type="GPU", verbose=False,
                              allow_writing_files=False, custom_metric=names)
    m.fit(X, y, sample_weight=w)
    ev = m.get_evals_result()["learn"]
    ref = m.eval_metrics(cb.Pool(X, y, weight=w), names)
    for nm in names:
        assert len(ev[nm]) == 10
        assert np.allclose(ev[nm], ref[nm], rtol=1e-4, atol=1e-5), (nm, ev[nm][-1], ref[nm][-1])


@pytest.mark.parametrize("n", [1, 31, 2048, 2049, 1_000_003])
def test_radix_sort_is_stable_and_matches_framework_sort(n):
    from catboost_b200.ops import api as ops
    g = torch.Generator().manual_seed(n)
    # few distinct keys (long runs of equal keys test stability), negative keys, and full-range 64-bit keys
    for keys in (torch.randint(-5, 5, (n,), generator=g, dtype=torch.int64),
                 torch.randint(-2 ** 62, 2 ** 62, (n,), generator=g, dtype=torch.int64) * 2 + 1):
        k = keys.cuda()
        sk, order = ops.sort_pairs(k)
        ref_k, ref_o = torch.sort(k, stable=True)
        assert torch.equal(sk, ref_k)
        assert torch.equal(order, ref_o)


@pytest.mark.parametrize("n,rate,lam", [(8192 * 3 + 517, 0.3, 0.01), (5000, 0.7, -1.0)])
def test_mvs_sampling_kernel(n, rate, lam):
    """Minimal-variance sampling: per block of 8192 documents the threshold mu solves sum min(1, c / mu) = rate * m
    with c = sqrt(der^2 + lambda); a kept document's statistics are scaled by max(1, mu / c), a dropped one's are zero."""
    import ctypes
    from catboost_b200.ops import native
    lib = native.cuda_lib()
    g = torch.Generator().manual_seed(5)
    npad = (n + 255) // 256 * 256
    stats = torch.zeros((2, npad))
    stats[0, :n] = torch.randn(n, generator=g) * torch.rand(n, generator=g)
    stats[1, :n] = torch.rand(n, generator=g) + 0.1
    before = stats.clone()
    st = stats.cuda()
    blk = lib.cb_mvs_block_docs()
    nblk = (n + blk - 1) // blk
    mu = torch.zeros(nblk, device="cuda")
    it = torch.zeros(1, dtype=torch.int32, device="cuda")
    smax = torch.zeros(2, device="cuda")
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    native.cuda_check(lib.cb_mvs_sample(p(st), npad, n, rate, lam, 12345, p(it), p(smax), p(mu),
                                        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "cb_mvs_sample")
    torch.cuda.synchronize()
    after, mu = st.cpu(), mu.cpu()
    kept_total = 0
    for b in range(nblk):
        lo, hi = b * blk, min(n, (b + 1) * blk)
        d = before[0, lo:hi].double()
        lam_b = lam if lam >= 0 else float(d.abs().mean()) ** 2
        c = torch.sqrt(d * d + lam_b)
        m = hi - lo
        f = torch.clamp(c / float(mu[b]), max=1.0).sum().item()
        assert abs(f - rate * m) <= 2e-3 * m, (b, f, rate * m)
        w_full = torch.clamp(float(mu[b]) / c, min=1.0)
        ratio1 = after[1, lo:hi].double() / before[1, lo:hi].double()
        kept = ratio1 > 0
        assert torch.allclose(ratio1[kept], w_full[kept], rtol=1e-4)
        assert torch.allclose(after[0, lo:hi].double()[kept], (d * w_full)[kept], rtol=1e-4, atol=1e-7)
        assert (after[0, lo:hi][~kept] == 0).all()
        assert bool(kept[c >= float(mu[b])].all())               # large gradients are always kept
        kept_total += int(kept.sum())
    assert abs(kept_total / n - rate) < 0.03
    assert float(smax[0]) >= float(after[0].abs().max()) - 1e-6 and float(smax[1]) >= float(after[1].abs().max()) - 1e-6


def test_fit_with_mvs_bootstrap_runs_on_the_device_trainer():
    import catboost_b200 as cb
    rng = np.random.default_rng(3)
    n = 60_000
    X = rng.standard_normal((n, 12)).astype(np.float32)
    y = (X[:, 0] - 0.8 * X[:, 3] + 0.5 * X[:, 5] * X[:, 6] + 0.4 * rng.standard_normal(n) > 0).astype(np.float32)
    accs = {}
    for bt, extra in (("MVS", dict(subsample=0.4)), ("No", {})):
        m = cb.CatBoostClassifier(iterations=80, depth=6, learning_rate=0.2, task_type="GPU", bootstrap_type=bt,
                                  verbose=False, allow_writing_files=False, **extra)
        m.fit(X[:50_000], y[:50_000])
        assert m._train_info["launches_per_iter"] > 0              # the device engine, not the general learner
        accs[bt] = float((m.predict(X[50_000:]) == y[50_000:]).mean())
    assert accs["MVS"] > accs["No"] - 0.02 and accs["MVS"] > 0.85, accs


def test_gpu_apply_geometries_match_cpu_apply(monkeypatch):
    """The batch-apply kernel in its three shapes -- 1024 threads x 4 rows (many rows, narrow model), 256 x 4 and
    256 x 1 (wide model) -- with the leaf values of a chunk of trees staged in shared memory, and with them left in
    global memory: all equal to the CPU evaluator."""
    import catboost_b200 as cb
    from catboost_b200.models.gpu_apply import GpuPredictor
    rng = np.random.default_rng(21)
    # narrow model, enough rows for the 1024-thread shape; depth 9 takes the per-row (not four-rows-per-word) walk
    X = rng.standard_normal((700_000, 10)).astype(np.float32)
    X[rng.random(X.shape) < 0.01] = np.nan
    y = (np.nan_to_num(X[:, 0]) + 0.5 * np.nan_to_num(X[:, 3]) * np.nan_to_num(X[:, 4]) + 0.3 * rng.standard_normal(len(X))).astype(np.float32)
    for depth, iters in ((6, 70), (9, 12)):
        m = cb.CatBoostRegressor(iterations=iters, depth=depth, learning_rate=0.2, border_count=64, task_type="GPU",
                                 verbose=False, allow_writing_files=False).fit(X[:60_000], y[:60_000])
        want = m.predict(X, prediction_type="RawFormulaVal")
        xd = torch.from_numpy(X).cuda()
        for lv in ("1", "0"):
            monkeypatch.setenv("CB200_PREDICT_LV", lv)
            got = GpuPredictor(m._model, "cuda:0").predict_device(xd)[0].double().cpu().numpy()
            assert np.allclose(got, want, rtol=1e-5, atol=1e-5), (depth, lv, float(np.abs(got - want).max()))
            small = GpuPredictor(m._model, "cuda:0").predict_device(xd[:5001])[0].double().cpu().numpy()
            assert np.allclose(small, want[:5001], rtol=1e-5, atol=1e-5)
    # wide model: more used features than four rows per thread allow
    Xw = rng.standard_normal((30_000, 400)).astype(np.float32)
    yw = (Xw @ rng.choice([-1.0, 1.0], 400).astype(np.float32) + rng.standard_normal(len(Xw))).astype(np.float32)
    mw = cb.CatBoostRegressor(iterations=200, depth=6, learning_rate=0.2, border_count=32, task_type="GPU", verbose=False,
                              allow_writing_files=False).fit(Xw, yw)
    assert len({s.feature for s in mw._model.splits}) > 210          # beyond what four rows per thread can stage
    want = mw.predict(Xw, prediction_type="RawFormulaVal")
    monkeypatch.setenv("CB200_PREDICT_WIDE", "0")
    for lv in ("1", "0"):
        monkeypatch.setenv("CB200_PREDICT_LV", lv)
        got = GpuPredictor(mw._model, "cuda:0").predict_device(torch.from_numpy(Xw).cuda())[0].double().cpu().numpy()
        assert np.allclose(got, want, rtol=1e-5, atol=1e-4), float(np.abs(got - want).max())
    # the same models through the kernel that compares raw values with borders (no quantisation): chosen by itself for
    # the wide model, forced for the narrow one; NaNs take the side their column's NaN mode gives them
    monkeypatch.setenv("CB200_PREDICT_WIDE", "auto")
    pw = GpuPredictor(mw._model, "cuda:0")
    assert pw.wide is not None
    for tma in ("0", "1"):                 # rows staged through registers / brought in by bulk copies against mbarriers
        monkeypatch.setenv("CB200_PREDICT_WIDE_TMA", tma)
        got = pw.predict_device(torch.from_numpy(Xw).cuda())[0].double().cpu().numpy()
        assert np.allclose(got, want, rtol=1e-5, atol=1e-4), (tma, float(np.abs(got - want).max()))
        part = pw.predict_device(torch.from_numpy(Xw).cuda()[:1237])[0].double().cpu().numpy()
        assert np.allclose(part, want[:1237], rtol=1e-5, atol=1e-4)
        pw.check_status()
    monkeypatch.setenv("CB200_PREDICT_WIDE_TMA", "0")
    monkeypatch.setenv("CB200_PREDICT_WIDE", "1")
    pn = GpuPredictor(m._model, "cuda:0")
    assert pn.wide is not None
    got = pn.predict_device(xd[:100_003])[0].double().cpu().numpy()
    assert np.allclose(got, m.predict(X[:100_003], prediction_type="RawFormulaVal"), rtol=1e-5, atol=1e-5)
    mm = cb.CatBoostClassifier(iterations=30, depth=5, learning_rate=0.3, task_type="GPU", verbose=False,
                               allow_writing_files=False, nan_mode="Max").fit(X[:40_000], (y[:40_000] > 0).astype(int) + (y[:40_000] > 1))
    pm = GpuPredictor(mm._model, "cuda:0")
    assert pm.wide is not None and pm.dims == 3
    got = pm.predict_device(xd[:50_000]).t().double().cpu().numpy()
    assert np.allclose(got, mm.predict(X[:50_000], prediction_type="RawFormulaVal"), rtol=1e-5, atol=1e-5)


def test_querywise_derivative_kernels_match_the_tensor_formulations():
    """QueryRMSE / QuerySoftMax / PairLogit (pairs from labels and explicit pairs) on the device against the tensor code
    of train/ranking.py on the same inputs."""
    from catboost_b200.train import ranking as R
    from catboost_b200.train.ranking import make_ranking_objective
    g = torch.Generator().manual_seed(11)
    sizes = torch.randint(1, 70, (400,), generator=g)
    sizes[7] = 300                                        # a query longer than a warp several times over
    off = torch.cat([torch.zeros(1, dtype=torch.long), torch.cumsum(sizes, 0)])
    n = int(off[-1])
    approx = torch.randn(1, n, generator=g).cuda()
    target = torch.randint(0, 5, (n,), generator=g).float().cuda()
    weight = (torch.rand(n, generator=g) + 0.5).cuda()

    class Ctx:
        pass
    ctx = Ctx()
    ctx.group_offsets, ctx.pairs, ctx.pairs_weight, ctx.device = off.cuda(), None, None, torch.device("cuda")
    for loss, w in (("QueryRMSE", weight), ("QueryRMSE", None), ("QuerySoftMax", weight), ("PairLogit", None)):
        obj = make_ranking_objective(loss, {})
        R.USE_KERNELS = True
        d1, h1 = obj.der_hess(approx, target, w, ctx)
        R.USE_KERNELS = False
        try:
            d0, h0 = obj.der_hess(approx, target, w, ctx)
        finally:
            R.USE_KERNELS = True
        assert torch.allclose(d1, d0, rtol=2e-4, atol=2e-5), (loss, float((d1 - d0).abs().max()))
        assert torch.allclose(h1, h0, rtol=2e-4, atol=2e-5), (loss, float((h1 - h0).abs().max()))
    # explicit pairs
    P = 5000
    q = torch.randint(0, 400, (P,), generator=g)
    lo, sz = off[q], sizes[q]
    wi = lo + (torch.rand(P, generator=g) * sz).long().clamp(max=sz - 1)
    li = lo + (torch.rand(P, generator=g) * sz).long().clamp(max=sz - 1)
    keep = wi != li
    ctx.pairs = torch.stack([wi[keep], li[keep]], 1).cuda()
    ctx.pairs_weight = (torch.rand(int(keep.sum()), generator=g) + 0.5).cuda()
    obj = make_ranking_objective("PairLogit", {})
    d1, h1 = obj.der_hess(approx, target, None, ctx)
    R.USE_KERNELS = False
    try:
        d0, h0 = obj.der_hess(approx, target, None, ctx)
    finally:
        R.USE_KERNELS = True
    assert torch.allclose(d1, d0, rtol=1e-4, atol=1e-5) and torch.allclose(h1, h0, rtol=1e-4, atol=1e-5)


def test_device_side_ndcg_matches_the_host_metric():
    """NDCG / DCG (top, Exp gains, position denominator) evaluated on the device with the stable radix sort against the
    host metric, including queries whose approximations tie."""
    from catboost_b200.data.pool import Pool
    from catboost_b200.metrics import make_metric
    from catboost_b200.train.loop import _device_metric
    rng = np.random.default_rng(5)
    sizes = rng.integers(1, 40, 700)
    gid = np.repeat(np.arange(len(sizes)), sizes)
    n = len(gid)
    X = rng.standard_normal((n, 3)).astype(np.float32)
    y = rng.integers(0, 5, n).astype(np.float32)
    approx = np.round(rng.standard_normal(n), 1).astype(np.float32)         # one decimal: plenty of ties
    pool = Pool(X, y, group_id=gid)
    a_dev = torch.from_numpy(approx).cuda().unsqueeze(0)
    for desc in ("PairLogit", "PairAccuracy"):          # pairs from labels, then the pool's explicit pairs
        metric = make_metric(desc)
        got = _device_metric(metric, a_dev, y, None, pool)
        want = metric.eval(approx.reshape(-1, 1).astype(np.float64), y, None, group_offsets=pool.group_offsets())
        assert got is not None and abs(got - want) < 1e-5 * max(1.0, abs(want)), (desc, got, want)
        offs = pool.group_offsets()
        qs = rng.integers(0, len(sizes), 3000)
        pairs = np.stack([offs[qs] + rng.integers(0, 1 << 30, 3000) % sizes[qs], offs[qs] + rng.integers(0, 1 << 30, 3000) % sizes[qs]], 1)
        pairs = pairs[pairs[:, 0] != pairs[:, 1]]
        pw = (rng.random(len(pairs)) + 0.5).astype(np.float32)
        pool_p = Pool(X, y, group_id=gid, pairs=pairs, pairs_weight=pw)
        got = _device_metric(metric, a_dev, y, None, pool_p)
        want = metric.eval(approx.reshape(-1, 1).astype(np.float64), y, None, pairs=pairs, pairs_weight=pw)
        assert got is not None and abs(got - want) < 1e-5 * max(1.0, abs(want)), (desc, got, want)
    yp = (y / 4.0).astype(np.float32)                                       # PFound takes relevances in [0, 1]
    for desc in ("PFound", "PFound:top=4;decay=0.7"):
        metric = make_metric(desc)
        poolp = Pool(X, yp, group_id=gid)
        got = _device_metric(metric, a_dev, yp, None, poolp)
        want = metric.eval(approx.reshape(-1, 1).astype(np.float64), yp, None, group_offsets=poolp.group_offsets())
        assert got is not None and abs(got - want) < 1e-6 * max(1.0, abs(want)), (desc, got, want)
    for desc in ("NDCG", "NDCG:top=5", "NDCG:type=Exp", "NDCG:top=3;type=Exp;denominator=Position", "DCG:top=10"):
        metric = make_metric(desc)
        got = _device_metric(metric, a_dev, y, None, pool)
        want = metric.eval(approx.reshape(-1, 1).astype(np.float64), y, None, group_offsets=pool.group_offsets())
        assert got is not None and abs(got - want) < 1e-6 * max(1.0, abs(want)), (desc, got, want)


def test_engine_invariant_checks(monkeypatch):
    """CB200_CHECK=1: the trainer verifies its device state after every iteration (split ranges, leaf indices, finite
    values, leaf weights against the data); a state that breaks an invariant is reported."""
    import catboost_b200 as cb
    rng = np.random.default_rng(9)
    X = rng.standard_normal((30_000, 8)).astype(np.float32)
    y = (X[:, 0] + X[:, 1] * X[:, 2] > 0).astype(int)
    w = (rng.random(30_000) + 0.5).astype(np.float32)
    monkeypatch.setenv("CB200_CHECK", "1")
    m = cb.CatBoostClassifier(iterations=12, depth=5, learning_rate=0.3, task_type="GPU", verbose=False,
                              allow_writing_files=False)
    m.fit(X, y, sample_weight=w)
    assert m._train_info["launches_per_iter"] > 0
    # a corrupted state is caught
    store = __import__("tests.test_gpu_precision", fromlist=["_store_of"])._store_of(X, y.astype(np.float32), 32)
    eng = __import__("tests.test_gpu_precision", fromlist=["_engine"])._engine(store, y.astype(np.float32), "narrow", 4, 3)
    eng.step(2)
    eng.check_invariants()
    eng.model_wts[1, 0] += 100.0
    with pytest.raises(RuntimeError, match="leaf weights"):
        eng.check_invariants()
    eng.model_wts[1, 0] -= 100.0
    eng.approx[5] = float("nan")
    with pytest.raises(RuntimeError, match="non-finite"):
        eng.check_invariants()
    eng.close()


def test_exact_quantile_leaves_on_the_device_match_the_cpu_trainer():
    """MAE / Quantile with leaf_estimation_method='Exact': the per-leaf weighted quantiles come from one radix sort by
    (leaf, residual) on the device; the model equals the CPU trainer's on the same borders."""
    import catboost_b200 as cb
    rng = np.random.default_rng(14)
    X = rng.standard_normal((20_000, 6)).astype(np.float32)
    y = (X[:, 0] + 0.5 * X[:, 1] ** 2 + rng.standard_t(3, 20_000) * 0.3).astype(np.float32)
    for loss in ("MAE", "Quantile:alpha=0.8"):
        preds = {}
        for task in ("GPU", "CPU"):
            m = cb.CatBoostRegressor(loss_function=loss, iterations=15, depth=4, learning_rate=0.3, task_type=task,
                                     leaf_estimation_method="Exact", bootstrap_type="No", random_strength=0, border_count=32,
                                     verbose=False, allow_writing_files=False, boost_from_average=True)
            m.fit(X, y)
            preds[task] = m.predict(X)
        assert np.allclose(preds["GPU"], preds["CPU"], rtol=1e-3, atol=1e-3), (loss, float(np.abs(preds["GPU"] - preds["CPU"]).max()))


@pytest.mark.parametrize("policy,loss", [("Depthwise", "Logloss"), ("Lossguide", "RMSE"), ("Depthwise", "Poisson")])
def test_leaf_kernel_in_the_general_learner_matches_tensor_code(policy, loss):
    """Depthwise / Lossguide trees estimate their leaves with the device trainer's cooperative kernel (all steps in one
    launch, backtracking included); the models agree with the tensor formulation of the same steps."""
    import catboost_b200 as cb
    from catboost_b200.train import generic as G
    rng = np.random.default_rng(31)
    X = rng.standard_normal((40_000, 8)).astype(np.float32)
    f = X[:, 0] * X[:, 1] + X[:, 2]
    y = {"Logloss": (f + 0.4 * rng.standard_normal(len(X)) > 0).astype(np.float32),
         "RMSE": (f + 0.2 * rng.standard_normal(len(X))).astype(np.float32),
         "Poisson": rng.poisson(np.exp(0.4 * f)).astype(np.float32)}[loss]
    w = (rng.random(len(X)) + 0.5).astype(np.float32)
    cls = cb.CatBoostClassifier if loss == "Logloss" else cb.CatBoostRegressor
    preds = {}
    for use in (True, False):
        G.USE_LEAF_KERNEL = use
        try:
            m = cls(loss_function=loss, iterations=12, depth=4, learning_rate=0.3, task_type="GPU", grow_policy=policy,
                    max_leaves=12, bootstrap_type="No", random_strength=0, verbose=False, allow_writing_files=False)
            m.fit(X, y, sample_weight=w)
        finally:
            G.USE_LEAF_KERNEL = True
        preds[use] = m.predict(X, prediction_type="RawFormulaVal")
    assert np.allclose(preds[True], preds[False], rtol=2e-3, atol=2e-3), float(np.abs(preds[True] - preds[False]).max())


@pytest.mark.parametrize("nq,ne,d", [(300, 1000, 96), (130, 129, 200), (256, 40000, 64), (1000, 5000, 384),
                                      (200, 3000, 500), (150, 2000, 768)])
def test_knn_tensor_core_candidates_match_fp32_reference(nq, ne, d):
    """tcgen05 distance GEMM + top-k epilogue against a plain fp32 computation on the same bf16-rounded inputs."""
    from catboost_b200.ops import api as ops
    g = torch.Generator(device="cpu").manual_seed(nq + ne + d)
    Q = torch.randn((nq, d), generator=g).cuda()
    E = torch.randn((ne, d), generator=g).cuda()
    out = ops.knn_candidates(Q, E)
    assert out is not None
    idx, val = out
    assert idx.shape[1] == 32                # two lists of 16 per cloud tile half, merged: the first 16 are the exact top 16
    C = 16
    qb, eb = Q.bfloat16().float(), E.bfloat16().float()
    ref = (eb * eb).sum(1).unsqueeze(0) - 2.0 * qb @ eb.t()
    rv, ri = torch.topk(ref, min(C, ne), dim=1, largest=False, sorted=True)
    m = min(C, ne)
    assert bool((idx[:, :m] >= 0).all())
    assert torch.allclose(val[:, :m], rv, atol=2e-3 * d ** 0.5, rtol=1e-4)
    # the same rows are selected; rows whose scores tie within rounding may swap places
    same = (idx[:, :m] == ri).float().mean().item()
    assert same > 0.99, same
    # the score reported for a candidate is the score of that candidate
    assert torch.allclose(val[:, :m], ref.gather(1, idx[:, :m]), atol=2e-3 * d ** 0.5, rtol=1e-4)
    # end to end: candidates re-ranked in fp32 against the exact neighbours (k = 5: lists of 8; k = 8: lists of 16)
    d2 = torch.cdist(Q, E)
    for k in (5, 8):
        got = ops.knn_search(Q, E, k)
        want = torch.topk(d2, k, dim=1, largest=False, sorted=True).indices
        recall = np.mean([len(set(a.tolist()) & set(b.tolist())) / k for a, b in zip(got.cpu(), want.cpu())])
        assert recall > 0.995, (k, recall)


def test_knn_search_falls_back_for_many_neighbours():
    from catboost_b200.ops import api as ops
    g = torch.Generator(device="cpu").manual_seed(3)
    Q = torch.randn((50, 40), generator=g).cuda()
    E = torch.randn((400, 40), generator=g).cuda()
    got = ops.knn_search(Q, E, 12)                                # more than half the kernel's candidate list: library GEMM
    want = torch.topk(torch.cdist(Q, E), 12, dim=1, largest=False).indices
    assert (got.sort(1).values == want.sort(1).values).float().mean().item() > 0.99


def test_embedding_knn_features_from_the_device_match_the_host():
    """The KNN class votes of an embedding column computed through the tensor-core search against the host search."""
    import catboost_b200 as cb
    from catboost_b200.data.estimated import _EmbeddingCalcers
    rng = np.random.default_rng(4)
    n, d = 6000, 48
    cls = rng.integers(0, 3, n)
    centers = rng.standard_normal((3, d))
    E = (centers[cls] * 0.5 + rng.standard_normal((n, d))).astype(np.float32)
    host = _EmbeddingCalcers(5, ("KNN",)).fit(E[:4000], cls[:4000], 3)
    dev = _EmbeddingCalcers(5, ("KNN",), device=torch.device("cuda", 0)).fit(E[:4000], cls[:4000], 3)
    a, b = host.transform(E[4000:]), dev.transform(E[4000:])
    assert a.shape == b.shape == (2000, 3)
    assert np.mean(np.abs(a - b) < 1e-6) > 0.995                 # votes are multiples of 1/5: equal unless a neighbour differs
    # the ordered learn features too: every block searched in the documents before it
    blocks = np.array_split(rng.permutation(4000), 4)
    la, lb = host.transform_learn(E[:4000], blocks), dev.transform_learn(E[:4000], blocks)
    assert np.mean(np.abs(la - lb) < 1e-6) > 0.995
    # end to end on the GPU trainer
    X = np.empty((n, 2), dtype=object)
    X[:, 0] = rng.standard_normal(n).astype(np.float32)
    for i in range(n):
        X[i, 1] = E[i]
    m = cb.CatBoostClassifier(iterations=30, depth=4, learning_rate=0.2, verbose=False, allow_writing_files=False,
                              task_type="GPU", devices="0")
    m.fit(X[:5000], cls[:5000], embedding_features=[1])
    acc = float((m.predict(X[5000:]).reshape(-1).astype(int) == cls[5000:]).mean())
    assert acc > 0.8, acc


def test_objectives_without_device_formula_train_on_gpu():
    """Survival, focal, multi-quantile and filter objectives on task_type='GPU' (general learner or external derivatives)."""
    import catboost_b200 as cb
    rng = np.random.default_rng(2)
    n = 3000
    X = rng.normal(size=(n, 5)).astype(np.float32)
    t = np.exp(1.0 + 0.8 * X[:, 0] + 0.2 * rng.normal(size=n))
    lo, up = t.copy(), t.copy()
    up[: n // 3] = -1
    lo[: n // 3] *= 0.7
    kw = dict(iterations=40, depth=3, learning_rate=0.2, verbose=0, task_type="GPU", devices="0", allow_writing_files=False)
    m = cb.CatBoostRegressor(loss_function="SurvivalAft:dist=Normal;scale=0.5", **kw).fit(X, np.stack([lo, up], 1).astype(np.float32))
    assert np.corrcoef(m.predict(X), np.log(t))[0, 1] > 0.9
    risk = X[:, 0] - 0.5 * X[:, 1]
    time = rng.exponential(np.exp(-risk)) + 0.01
    yc = np.where(rng.random(n) < 0.25, -time, time).astype(np.float32)
    m = cb.CatBoostRegressor(loss_function="Cox", **kw).fit(X, yc)
    assert np.corrcoef(m.predict(X), risk)[0, 1] > 0.7
    yb = (risk + 0.3 * rng.normal(size=n) > 0).astype(np.float32)
    m = cb.CatBoostClassifier(loss_function="Focal:focal_alpha=0.5;focal_gamma=2", **kw).fit(X, yb)
    assert (m.predict(X).astype(np.float32).reshape(-1) == yb).mean() > 0.85
    yq = (X[:, 0] + rng.normal(size=n)).astype(np.float32)
    m = cb.CatBoostRegressor(loss_function="MultiQuantile:alpha=0.1,0.9", **kw).fit(X, yq)
    pr = m.predict(X)
    assert abs((yq <= pr[:, 0]).mean() - 0.1) < 0.06 and abs((yq <= pr[:, 1]).mean() - 0.9) < 0.06
    m = cb.CatBoostRegressor(first_feature_use_penalties={0: 1e9}, **kw).fit(X, yq)
    assert m.get_feature_importance()[0] == 0


def test_gpu_apply_of_model_with_more_used_features_than_one_launch_holds():
    """2000 columns and about a thousand used features: neither apply kernel takes the model in one launch, so it is
    evaluated as a sum of tree ranges."""
    import catboost_b200 as cb
    from catboost_b200.models.gpu_apply import GpuPredictor
    rng = np.random.default_rng(9)
    n, F = 3000, 2000
    X = rng.standard_normal((n, F)).astype(np.float32)
    y = (X[:, :50].sum(1) + rng.standard_normal(n) * 3 > 0).astype(np.float32)
    m = cb.CatBoostClassifier(iterations=300, depth=6, learning_rate=0.1, verbose=False, allow_writing_files=False,
                              task_type="GPU", devices="0", random_strength=5.0)
    m.fit(X, y)
    pred = GpuPredictor(m._model, torch.device("cuda", 0))
    assert pred.U > GpuPredictor.MAX_USED and pred.parts is not None and len(pred.parts) >= 2
    assert all(p.U <= GpuPredictor.MAX_USED for p in pred.parts)
    host = m.predict(X, prediction_type="RawFormulaVal")
    dev = m.predict(X, prediction_type="RawFormulaVal", task_type="GPU")
    assert np.max(np.abs(host - dev)) < 1e-4
