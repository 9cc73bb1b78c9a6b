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
    assert np.array_equal(outs[0][0], outs[1][0])
    assert np.array_equal(outs[0][2], outs[1][2])
    assert np.allclose(outs[0][1], outs[1][1], rtol=1e-6, atol=1e-7)
    assert np.allclose(outs[0][3], outs[1][3], rtol=1e-6, atol=1e-6)


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
