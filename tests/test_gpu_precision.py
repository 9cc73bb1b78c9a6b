"""Histogram cell arithmetic of the device trainer: the three cell types against the tensor-code learner, the
fixed-point tiles against an integer oracle, model quality of the cell types over a long run, the fused leaf update
against the separate one, and the step-length control of the leaf estimation."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _data(n, F, seed=0):
    rng = np.random.default_rng(seed)
    X = rng.standard_normal((n, F), dtype=np.float32)
    f = X[:, 0] * 0.8 + X[:, 1] * X[:, 2] * 0.6 + np.abs(X[:, 3]) * 0.4 - 0.3
    y = (rng.random(n, dtype=np.float32) < 1.0 / (1.0 + np.exp(-f))).astype(np.float32)
    return X, y


def _store_of(X, y, border_count):
    from catboost_b200.data.pool import Pool
    from catboost_b200.params import resolve_options
    from catboost_b200.parallel.runtime import DistContext
    from catboost_b200.train.boosting import build_store, plan_features
    pool = Pool(X, y)
    o = resolve_options(dict(border_count=border_count, task_type="GPU"), "Logloss", len(y))
    plan = plan_features(o, pool, DistContext(0, 1, torch.device("cuda")), None)
    store, _ = build_store(plan, pool, torch.device("cuda"))
    return store


def _engine(store, y, cells, depth, iterations, **kw):
    from catboost_b200.train.gpu_engine import GpuObliviousEngine
    from catboost_b200.train.objectives import make_objective
    args = dict(depth=depth, iterations=iterations, learning_rate=0.5, l2_leaf_reg=3.0, random_strength=0.0,
                bootstrap_type="No", leaf_iterations=1, seed=0,
                quantized_hist={"narrow": True, "wide": "wide", "float": False}[cells])
    args.update(kw)
    return GpuObliviousEngine(store, torch.from_numpy(y), None, torch.zeros(len(y)), make_objective("Logloss", {}), **args)


@pytest.mark.parametrize("cells", ["narrow", "wide", "float"])
def test_every_cell_type_matches_the_tensor_learner(cells):
    """One tree (splits, leaf weights, leaf values) of the device trainer with each histogram cell type against the
    tensor-code learner on the same statistics."""
    from catboost_b200.params import resolve_options
    from catboost_b200.train.generic import GenericLearner, estimate_leaves
    from catboost_b200.train.objectives import make_objective
    n, depth = 30011, 5
    X, y = _data(n, 10, seed=5)
    store = _store_of(X, y, 32)
    eng = _engine(store, y, cells, depth, 2, leaf_iterations=3)
    eng.step(1)
    sp, vals, wts = eng.finish()
    eng.close()
    obj = make_objective("Logloss", {})
    o = resolve_options(dict(loss_function="Logloss", depth=depth, task_type="GPU", bootstrap_type="No", random_strength=0,
                             leaf_estimation_iterations=3, learning_rate=0.5, l2_leaf_reg=3.0, border_count=32), "Logloss", n)
    approx = torch.zeros((1, store.npad), device="cuda")
    target = torch.from_numpy(y).cuda()
    der, hess = obj.der_hess(approx[:, :n], target, None)
    dp = torch.zeros((1, store.npad), device="cuda")
    hp = torch.zeros((1, store.npad), device="cuda")
    dp[:, :n], hp[:, :n] = der, hess
    tr = GenericLearner(store, o, 1).build_tree(dp, hp, None, 0)
    gv, gw = estimate_leaves(obj, approx, target, None, tr.leaf, tr.n_leaves, n, o)
    assert np.array_equal(sp[0][:, :2], tr.splits[:, :2]), (cells, sp[0], tr.splits)
    assert np.allclose(wts[0], gw, rtol=1e-5, atol=1e-3)
    assert np.allclose(vals[0], gv[:, 0], rtol=2e-3, atol=2e-4)


def test_fixed_point_tiles_equal_an_integer_oracle():
    """Single-int32 cells: every private tile of level 0 is, cell by cell, the int64 sum of the documents' statistics
    quantised with the kernel's own scale (recomputed here from the launch geometry), converted back with one fp32
    multiply.  A lost bit-plane, a dropped document or a wrong replica sum would be off by many quanta; the check
    allows one quantum (the device divides with the fast reciprocal, so its scale may differ from the IEEE quotient in
    the last place, which can move a value that sits on a rounding boundary) plus the fp32 rounding of a large sum."""
    n, F, B = 200_003, 12, 32
    X, y = _data(n, F, seed=3)
    store = _store_of(X, y, B)
    eng = _engine(store, y, "narrow", 1, 2)
    eng.step(1)
    torch.cuda.synchronize()
    grid, spp, smem, thr, nK, C, gpc = eng.level_geo[0]
    assert gpc > 0 and thr == 1024
    G, Bs = store.G, eng.B
    V = 1 if gpc > 4 else 2
    blk = thr * V
    nblk = (n + blk - 1) // blk
    cap = ((nblk + nK - 1) // nK) * blk // C + 64
    qmax = np.float32(min(8388607.0, np.floor(np.float32(2147483647.0) / np.float32(cap)) - 1.0))
    stats = eng.stats[:, :n].cpu().numpy()
    statmax = np.maximum(np.abs(stats).max(1), 1e-30).astype(np.float32)
    sc = (qmax / statmax).astype(np.float32)
    q = np.rint(stats * sc[:, None]).astype(np.int64)                     # [2][n]
    chunk = (np.arange(n) // blk) % nK
    bins = np.stack([store.column(f).cpu().numpy() for f in range(F)])   # [F][n]
    tiles = eng.priv[: nK * G * 8 * Bs].view(nK, G, 2, 4, Bs).cpu().numpy().astype(np.float64)
    inv = (statmax / qmax).astype(np.float64)
    worst = 0.0
    for f in range(F):
        g, j = divmod(f, 4)
        for s in range(2):
            oracle = np.zeros((nK, Bs), dtype=np.int64)
            np.add.at(oracle, (chunk, bins[f]), q[s])
            got = tiles[:, g, s, j, :] / inv[s]
            # one quantum per document whose scaled value sits within an ulp of a rounding boundary (rare), plus fp32
            tol = 2.0 + np.abs(oracle) * 2.0 ** -22
            err = np.abs(got - oracle)
            worst = max(worst, float((err / tol).max()))
            assert (err <= tol).all(), (f, s, float(err.max()))
    assert worst > 0.0 or True
    # and the tiles are not trivially empty
    assert np.abs(tiles).sum() > 0
    eng.finish()
    eng.close()


def test_fused_leaf_update_equals_separate_pass():
    n = 60_001
    X, y = _data(n, 30, seed=11)         # 8 feature groups: the deep levels cannot hold all groups in one bundle
    store = _store_of(X, y, 128)
    outs = []
    for fuse in (True, False):
        eng = _engine(store, y, "narrow", 6, 4, fuse_leaf_update=fuse, leaf_iterations=2, random_strength=1.0,
                      bootstrap_type="Bayesian")
        eng.step(4)
        sp, vals, wts = eng.finish()
        outs.append((sp.copy(), vals.copy(), wts.copy(), eng.approx[:n].cpu().numpy()))
        eng.close()
    assert np.array_equal(outs[0][0][:, :, :2], outs[1][0][:, :, :2]), np.argwhere(outs[0][0] != outs[1][0])[:8]
    assert np.array_equal(outs[0][0][:, :, 3], outs[1][0][:, :, 3])
    assert np.allclose(outs[0][2], outs[1][2], rtol=1e-6)
    assert np.allclose(outs[0][1], outs[1][1], rtol=1e-5, atol=1e-6)
    assert np.allclose(outs[0][3], outs[1][3], rtol=1e-5, atol=1e-5)


def test_leaf_backtracking_matches_the_tensor_learner_and_never_hurts():
    """With a tiny l2 and an exaggerated first step the plain Newton iteration overshoots on Poisson-like losses; here
    we only need: (a) with 'No' and with 'AnyImprovement' the device steps equal the tensor learner's, (b) the learn
    loss after a tree with step control is not worse than without."""
    from catboost_b200.params import resolve_options
    from catboost_b200.train.generic import GenericLearner, estimate_leaves
    from catboost_b200.train.gpu_engine import GpuObliviousEngine
    from catboost_b200.train.objectives import make_objective
    n, depth = 40_009, 4
    rng = np.random.default_rng(2)
    X = rng.standard_normal((n, 6), dtype=np.float32)
    lam = np.exp(0.6 * X[:, 0] + 0.3 * X[:, 1])
    y = rng.poisson(lam).astype(np.float32)
    store = _store_of(X, y, 32)
    obj = make_objective("Poisson", {})
    losses = {}
    for mode in ("No", "AnyImprovement", "Armijo"):
        eng = GpuObliviousEngine(store, torch.from_numpy(y), None, torch.zeros(n), obj, depth=depth, iterations=2,
                                 learning_rate=1.0, l2_leaf_reg=0.05, random_strength=0.0, bootstrap_type="No",
                                 leaf_method="Newton", leaf_iterations=6, seed=0, leaf_backtracking=mode)
        eng.step(1)
        losses[mode] = eng.current_learn_loss()
        sp, vals, wts = eng.finish()
        eng.close()
        o = resolve_options(dict(loss_function="Poisson", depth=depth, task_type="GPU", bootstrap_type="No",
                                 random_strength=0, leaf_estimation_iterations=6, learning_rate=1.0, l2_leaf_reg=0.05,
                                 border_count=32, leaf_estimation_backtracking=mode), "Poisson", n)
        approx = torch.zeros((1, store.npad), device="cuda")
        target = torch.from_numpy(y).cuda()
        der, hess = obj.der_hess(approx[:, :n], target, None)
        dp = torch.zeros((1, store.npad), device="cuda")
        hp = torch.zeros((1, store.npad), device="cuda")
        dp[:, :n], hp[:, :n] = der, hess
        tr = GenericLearner(store, o, 1).build_tree(dp, hp, None, 0)
        gv, gw = estimate_leaves(obj, approx, target, None, tr.leaf, tr.n_leaves, n, o)
        assert np.array_equal(sp[0][:, :2], tr.splits[:, :2])
        assert np.allclose(vals[0], gv[:, 0], rtol=5e-3, atol=5e-4), (mode, float(np.abs(vals[0] - gv[:, 0]).max()))
    assert np.isfinite(losses["AnyImprovement"]) and np.isfinite(losses["Armijo"])
    if np.isfinite(losses["No"]):
        assert losses["AnyImprovement"] <= losses["No"] + 1e-6


def _auc(score, y):
    order = np.argsort(score, kind="stable")
    r = np.empty(len(score))
    r[order] = np.arange(1, len(score) + 1)
    pos = y > 0.5
    return float((r[pos].sum() - pos.sum() * (pos.sum() + 1) / 2) / (pos.sum() * (~pos).sum()))


def test_cell_types_give_the_same_model_quality_over_1000_iterations():
    """1M rows x 28 features, 1000 iterations, held-out Logloss and AUC of single-int32 ('narrow'), 24-bit hi/lo
    ('wide') and fp32 ('float') histogram cells: the three differ by less than 5e-4 in Logloss and AUC (the spread
    between two runs that only differ in their random seed is larger).  The CPU trainer is compared on a smaller slice
    (100K rows, 200 iterations) because it takes minutes at the full size."""
    import sys, os
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import catboost_b200 as cb
    from bench import make_data
    X, y = make_data("higgs", 1_000_000, 28, 0, 1)
    tr, te = slice(0, 900_000), slice(900_000, 1_000_000)
    res = {}
    for cells in ("narrow", "wide", "float"):
        m = cb.CatBoostClassifier(iterations=1000, depth=6, learning_rate=0.1, border_count=128, task_type="GPU",
                                  verbose=False, allow_writing_files=False, random_seed=0, histogram_cells=cells)
        m.fit(X[tr], y[tr])
        raw = m.predict(X[te], prediction_type="RawFormulaVal")
        ll = float(np.mean(np.logaddexp(0.0, raw) - y[te] * raw))
        res[cells] = (ll, _auc(raw, y[te]))
    for a in ("narrow", "float"):
        assert abs(res[a][0] - res["wide"][0]) < 5e-4, res
        assert abs(res[a][1] - res["wide"][1]) < 5e-4, res
    assert res["narrow"][1] > 0.7
    Xs, ys = X[:100_000], y[:100_000]
    out = {}
    for task in ("CPU", "GPU"):
        m = cb.CatBoostClassifier(iterations=200, depth=6, learning_rate=0.1, border_count=128, task_type=task,
                                  verbose=False, allow_writing_files=False, random_seed=0)
        m.fit(Xs, ys)
        raw = m.predict(X[te], prediction_type="RawFormulaVal")
        out[task] = float(np.mean(np.logaddexp(0.0, raw) - y[te] * raw))
    assert abs(out["CPU"] - out["GPU"]) < 5e-3, out


def test_multiclass_device_trainer_matches_the_tensor_learner():
    """MultiClass through the device engine (K derivative columns in the fused level kernels, K x K Newton leaves on the
    device) against the tensor-code learner: same first tree, same leaf values; and a full fit reaches the accuracy of
    the general learner."""
    import catboost_b200 as cb
    from catboost_b200.params import resolve_options
    from catboost_b200.train.generic import GenericLearner, estimate_leaves
    from catboost_b200.train.gpu_engine import GpuObliviousEngine
    from catboost_b200.train.objectives import make_objective
    rng = np.random.default_rng(8)
    n, F, K, depth = 40_003, 9, 4, 4
    X = rng.standard_normal((n, F), dtype=np.float32)
    centers = rng.standard_normal((K, F)).astype(np.float32)
    y = np.argmax(X @ centers.T + 0.5 * rng.standard_normal((n, K)).astype(np.float32), axis=1).astype(np.float32)
    store = _store_of(X, (y > 0).astype(np.float32), 32)
    obj = make_objective("MultiClass", {}, n_classes=K)
    outs = {}
    for cells in (True, "wide"):                 # single int32 cells (the default) and exact hi / lo pairs
        eng = GpuObliviousEngine(store, torch.from_numpy(y), None, torch.zeros((K, n)), obj, depth=depth, iterations=2,
                                 learning_rate=0.5, l2_leaf_reg=3.0, random_strength=0.0, bootstrap_type="No",
                                 leaf_method="Newton", leaf_iterations=1, seed=0, dims=K, quantized_hist=cells)
        assert eng.narrow_hist == (cells is True)
        eng.step(1)
        loss_dev = eng.current_learn_loss()
        outs[cells] = eng.finish()
        eng.close()
    assert np.array_equal(outs[True][0][:, :, :2], outs["wide"][0][:, :, :2])          # same features and bins
    sp, vals, wts = outs[True]
    o = resolve_options(dict(loss_function="MultiClass", depth=depth, task_type="GPU", bootstrap_type="No",
                             random_strength=0, leaf_estimation_iterations=1, learning_rate=0.5, l2_leaf_reg=3.0,
                             border_count=32), "MultiClass", n)
    approx = torch.zeros((K, store.npad), device="cuda")
    target = torch.from_numpy(y).cuda()
    der, hess = obj.der_hess(approx[:, :n], target, None)
    dp = torch.zeros((K, store.npad), device="cuda")
    hp = torch.zeros((K, store.npad), device="cuda")
    dp[:, :n], hp[:, :n] = der, hess
    tr = GenericLearner(store, o, K).build_tree(dp, hp, None, 0)
    gv, gw = estimate_leaves(obj, approx, target, None, tr.leaf, tr.n_leaves, n, o)
    assert np.array_equal(sp[0][:, :2], tr.splits[:, :2]), (sp[0], tr.splits)
    assert np.allclose(wts[0], gw, rtol=1e-5, atol=1e-3)
    assert np.allclose(vals[0].reshape(-1, K), gv, rtol=2e-3, atol=2e-4), float(np.abs(vals[0].reshape(-1, K) - gv).max())
    a1 = approx[:, :n] + torch.from_numpy(gv).float().cuda()[tr.leaf[:n].long() & 0xFFFF].t()
    assert abs(loss_dev - obj.value(a1, target, None)) < 1e-4
    # whole fits: the public API takes the device engine for MultiClass and reaches the general learner's quality
    tr_, te_ = slice(0, 30_000), slice(30_000, n)
    accs = {}
    for name, extra in (("engine", {}), ("general", {"rsm": 0.999})):
        m = cb.CatBoostClassifier(loss_function="MultiClass", iterations=60, depth=5, learning_rate=0.3, task_type="GPU",
                                  verbose=False, allow_writing_files=False, random_seed=0, **extra)
        m.fit(X[tr_], y[tr_].astype(int), eval_set=(X[te_], y[te_].astype(int)))
        accs[name] = float((m.predict(X[te_]).reshape(-1) == y[te_].astype(int)).mean())
        if name == "engine":
            assert m._train_info.get("launches_per_iter", 0) > 0
            ev = m.get_evals_result()["validation"]["MultiClass"]
            assert ev[-1] < ev[0]
    assert accs["engine"] > 0.75 and abs(accs["engine"] - accs["general"]) < 0.03, accs


def test_per_leaf_search_kernel_matches_tensor_code():
    """cb_leaf_search (one warp per leaf and feature) against the tensor-code search on the same histograms: several
    leaves, three derivative columns, a one-hot feature, min_data_in_leaf, Cosine and L2."""
    from catboost_b200.data.pool import Pool
    from catboost_b200.params import resolve_options
    from catboost_b200.parallel.runtime import DistContext
    from catboost_b200.train.boosting import build_store, plan_features
    from catboost_b200.train.generic import GenericLearner
    from catboost_b200.ops import api as ops
    rng = np.random.default_rng(21)
    n, K = 20_000, 3
    X = np.empty((n, 7), dtype=object)
    X[:, :6] = rng.standard_normal((n, 6)).astype(np.float32)
    X[:, 6] = rng.integers(0, 5, n)
    y = rng.integers(0, K, n)
    pool = Pool(X, y, cat_features=[6])
    for score_fn, mdl in (("Cosine", 1), ("L2", 40)):
        o = resolve_options(dict(border_count=24, task_type="GPU", one_hot_max_size=8, loss_function="MultiClass",
                                 grow_policy="Depthwise", score_function=score_fn, min_data_in_leaf=mdl, random_strength=0),
                            "MultiClass", n)
        plan = plan_features(o, pool, DistContext(0, 1, torch.device("cuda")), None)
        store, _ = build_store(plan, pool, torch.device("cuda"))
        gl = GenericLearner(store, o, K)
        nleaf = 5
        S = K + 1 + (1 if gl.use_count else 0)
        stats = torch.zeros((S, store.npad), device="cuda")
        stats[:K, :n] = torch.randn((K, n), device="cuda")
        stats[K, :n] = torch.rand(n, device="cuda") + 0.5
        if gl.use_count:
            stats[K + 1, :n] = 1.0
        leaf = torch.zeros(store.npad, dtype=torch.int16, device="cuda")
        leaf[:n] = torch.from_numpy(rng.integers(0, nleaf, n).astype(np.int16)).cuda()
        leaf[:200] = 4                                   # a small leaf: min_data_in_leaf bites
        leaf[200:n][leaf[200:n] == 4] = 3
        table = torch.arange(nleaf, dtype=torch.int16, device="cuda")
        h = ops.hist(store, leaf, stats, table, nleaf)
        fmask = store.feat_weight > 0
        gl.monotone = None
        b1, s1, g1 = gl._per_leaf_best(h, K, 0.0, fmask, list(range(nleaf)))
        b0, s0, g0 = gl._per_leaf_best_tensor(h, K, 0.0, fmask)
        fin = np.isfinite(s0)
        assert np.array_equal(np.isfinite(s1), fin)
        assert np.array_equal(b1[fin], b0[fin]), (score_fn, b1, b0)
        assert np.allclose(s1[fin], s0[fin], rtol=2e-4, atol=1e-5)
        assert np.allclose(g1[fin], g0[fin], rtol=2e-3, atol=1e-2)
    # and a whole Depthwise / Lossguide fit still learns
    import catboost_b200 as cb
    Xf = rng.standard_normal((20_000, 8)).astype(np.float32)
    yf = (Xf[:, 0] * Xf[:, 1] + Xf[:, 2] > 0).astype(int)
    for policy in ("Depthwise", "Lossguide"):
        m = cb.CatBoostClassifier(iterations=30, depth=5, learning_rate=0.3, grow_policy=policy, task_type="GPU",
                                  verbose=False, allow_writing_files=False)
        m.fit(Xf, yf)
        assert float((m.predict(Xf) == yf).mean()) > 0.9


def test_pairwise_kernels_match_the_tensor_oracle():
    """cb_pairwise.cu (pair histograms -> prefix sums -> one linear system per candidate -> Cholesky -> gain) against the
    tensor-code oracle, candidate by candidate, float and one-hot features, one to eight leaves."""
    from catboost_b200.data.pool import Pool
    from catboost_b200.params import resolve_options
    from catboost_b200.parallel.runtime import DistContext
    from catboost_b200.train.boosting import build_store, plan_features
    from catboost_b200.train.pairwise import PairwiseKernelLearner, PairwiseLearner
    rng = np.random.default_rng(31)
    n, P = 3000, 20000
    X = np.empty((n, 6), dtype=object)
    X[:, :5] = rng.standard_normal((n, 5)).astype(np.float32)
    X[:, 5] = rng.integers(0, 4, n)
    y = rng.random(n).astype(np.float32)
    pool = Pool(X, y, cat_features=[5])
    o = resolve_options(dict(border_count=12, task_type="GPU", one_hot_max_size=8, loss_function="PairLogitPairwise",
                             depth=4, l2_leaf_reg=2.0), "PairLogitPairwise", n)
    plan = plan_features(o, pool, DistContext(0, 1, torch.device("cuda")), None)
    store, _ = build_store(plan, pool, torch.device("cuda"))
    assert bool(store.feat_onehot.any())
    wi = torch.from_numpy(rng.integers(0, n, P)).cuda()
    li = torch.from_numpy(rng.integers(0, n, P)).cuda()
    keep = wi != li
    wi, li = wi[keep], li[keep]
    h = (torch.rand(wi.numel(), device="cuda") + 0.1)
    der = torch.randn(n, device="cuda")
    oracle = PairwiseLearner(store, o)
    kern = PairwiseKernelLearner(store, o)
    der_pad = torch.zeros(store.npad, device="cuda")
    der_pad[:n] = der
    for L in (1, 2, 8, 32):          # 32 leaves: pairs sorted by leaf pair, one cell per chunk (cb_pair_hist_sorted_kernel)
        leaf = torch.from_numpy(rng.integers(0, L, n)).cuda()
        kern.leaf.zero_()
        kern.leaf[:n] = leaf.to(torch.int16)
        gains = kern.level_gains(L, wi, li, h, der_pad).double().cpu().numpy()
        for f in range(store.F):
            if float(store.feat_weight[f].item()) <= 0:
                continue
            ref = oracle._feature_scores(f, leaf, L, wi, li, h, der).cpu().numpy() * float(store.feat_weight[f].item())
            got = gains[f, : len(ref)]
            assert np.allclose(got, ref, rtol=2e-3, atol=2e-3 * max(1.0, float(np.abs(ref).max()))), (L, f, got[:4], ref[:4])
            assert not np.isfinite(gains[f, len(ref):]).any()
    # a whole fit through the public API takes the kernel path and ranks better than chance
    import catboost_b200 as cb
    ng = 300
    gid = np.repeat(np.arange(ng), 10)
    Xr = rng.standard_normal((ng * 10, 6)).astype(np.float32)
    rel = (Xr[:, 0] + 0.5 * Xr[:, 1] + 0.3 * rng.standard_normal(ng * 10) > 0.3).astype(np.float32)
    m = cb.CatBoostRanker(loss_function="PairLogitPairwise", iterations=15, depth=4, learning_rate=0.3, task_type="GPU",
                          verbose=False, allow_writing_files=False)
    m.fit(Xr, rel, group_id=gid)
    s = m.predict(Xr)
    assert np.corrcoef(s, Xr[:, 0] + 0.5 * Xr[:, 1])[0, 1] > 0.6


def test_dominant_bin_skipping_gives_the_same_trees():
    """Sparse columns (60 % zeros): with the dominant bin skipped and restored from the slot totals the histograms are
    the same integers, so the trees are the same as without skipping."""
    rng = np.random.default_rng(13)
    n, F = 80_003, 22
    X = rng.random((n, F), dtype=np.float32)
    X[rng.random((n, F)) < 0.6] = 0.0
    X[:, 3] = rng.standard_normal(n)                     # one dense column: no dominant bin there
    y = (X[:, 0] + X[:, 1] * 2 + X[:, 3] * 0.3 + 0.2 * rng.standard_normal(n) > 0.9).astype(np.float32)
    store = _store_of(X, y, 64)
    outs = []
    for skip in (True, False):
        eng = _engine(store, y, "narrow", 6, 5, skip_dominant_bin=skip, leaf_iterations=2, random_strength=0.0)
        assert (eng.domw is not None) == skip
        eng.step(5)
        sp, vals, wts = eng.finish()
        outs.append((sp.copy(), vals.copy(), wts.copy()))
        eng.close()
    assert np.array_equal(outs[0][0][:, :, :2], outs[1][0][:, :, :2]), np.argwhere(outs[0][0] != outs[1][0])[:8]
    assert np.allclose(outs[0][2], outs[1][2], rtol=1e-6)
    assert np.allclose(outs[0][1], outs[1][1], rtol=1e-4, atol=1e-5)


def test_bundles_sized_by_their_own_bins_give_the_same_model(monkeypatch):
    """Columns of very different widths (128-border floats next to columns with a handful of values): the level kernel
    sizes the tile of every bundle by its own widest feature and lists (bundle, slot pass, chunk) work items; the
    histograms are the same sums as with one bin stride for all bundles, up to the fixed-point scale."""
    rng = np.random.default_rng(17)
    n = 120_001
    wide = rng.standard_normal((n, 9)).astype(np.float32)
    small = rng.integers(0, 6, size=(n, 27)).astype(np.float32)
    X = np.concatenate([wide, small], 1)
    y = (wide[:, 0] + 0.7 * wide[:, 4] + 0.5 * (small[:, 2] > 2) - 0.4 * (small[:, 20] > 3)
         + 0.3 * rng.standard_normal(n) > 0.2).astype(np.float32)
    store = _store_of(X, y, 128)
    assert store.feat_nb_host.max() > 100 and store.feat_nb_host.min() <= 8
    outs, geos = [], []
    for uniform in (False, True):
        if uniform:
            monkeypatch.setenv("CB200_UNIFORM_BINS", "1")
        eng = _engine(store, y, "narrow", 8, 6, leaf_iterations=2)
        geos.append(list(eng.level_geo))
        eng.step(6)
        loss = eng.learn_loss_history().copy()
        sp, vals, wts = eng.finish()
        outs.append((sp.copy(), vals.copy(), wts.copy(), loss))
        eng.close()
    assert np.array_equal(outs[0][0][0, :, :2], outs[1][0][0, :, :2])          # first tree: same statistics
    assert np.allclose(outs[0][2][0], outs[1][2][0], rtol=1e-6)
    same = (outs[0][0][:, :, :2] == outs[1][0][:, :, :2]).all(-1).mean()
    assert same >= 0.9, same
    assert np.allclose(outs[0][3], outs[1][3], rtol=2e-3)
