"""CPU trainer, API surface and model behaviour (runs without a GPU)."""
import numpy as np
import pytest

import catboost_b200 as cb


def _binary(n=4000, F=8, seed=0):
    rng = np.random.default_rng(seed)
    X = rng.standard_normal((n, F), dtype=np.float32)
    w = rng.standard_normal(F).astype(np.float32)
    y = (X @ w + 0.3 * rng.standard_normal(n, dtype=np.float32) > 0).astype(int)
    return X, y


def test_classifier_learns_and_predicts():
    X, y = _binary()
    m = cb.CatBoostClassifier(iterations=40, depth=4, learning_rate=0.3, verbose=False, allow_writing_files=False)
    m.fit(X[:3000], y[:3000], eval_set=(X[3000:], y[3000:]))
    assert m.tree_count_ == 40 or m.tree_count_ == m.best_iteration_ + 1
    acc = (m.predict(X[3000:]) == y[3000:]).mean()
    assert acc > 0.85
    proba = m.predict_proba(X[:10])
    assert proba.shape == (10, 2) and np.allclose(proba.sum(1), 1)
    ev = m.get_evals_result()
    assert ev["learn"]["Logloss"][-1] < ev["learn"]["Logloss"][0]
    raw = m.predict(X[:50], prediction_type="RawFormulaVal")
    staged = list(m.staged_predict(X[:50], prediction_type="RawFormulaVal"))
    assert np.allclose(staged[-1], raw, atol=1e-9)


@pytest.mark.parametrize("policy", ["SymmetricTree", "Depthwise", "Lossguide"])
def test_grow_policies(policy):
    X, y = _binary(3000, 6, 1)
    m = cb.CatBoostClassifier(iterations=25, depth=4, grow_policy=policy, max_leaves=12, learning_rate=0.3,
                              verbose=False, allow_writing_files=False)
    m.fit(X, y)
    assert (m.predict(X) == y).mean() > 0.85


def test_regressor_losses():
    rng = np.random.default_rng(2)
    X = rng.standard_normal((3000, 5), dtype=np.float32)
    y = X[:, 0] * 2 + X[:, 1] ** 2 + 0.1 * rng.standard_normal(3000)
    for loss in ["RMSE", "MAE", "Quantile:alpha=0.7", "Huber:delta=1.0", "LogCosh", "Poisson"]:
        yy = np.abs(y) if loss == "Poisson" else y
        m = cb.CatBoostRegressor(iterations=40, depth=4, learning_rate=0.3, loss_function=loss, verbose=False,
                                 allow_writing_files=False)
        m.fit(X, yy)
        ev = m.get_evals_result()["learn"]
        k = list(ev.keys())[0]
        assert ev[k][-1] < ev[k][0], loss


def test_multiclass():
    rng = np.random.default_rng(3)
    X = rng.standard_normal((3000, 6), dtype=np.float32)
    y = np.argmax(X[:, :3] + 0.3 * rng.standard_normal((3000, 3)), axis=1)
    labels = np.array(["a", "b", "c"])[y]
    m = cb.CatBoostClassifier(iterations=30, depth=4, learning_rate=0.3, verbose=False, allow_writing_files=False)
    m.fit(X, labels)
    assert m._model.loss_name == "MultiClass"
    assert (m.predict(X) == labels).mean() > 0.85
    assert m.predict_proba(X).shape == (3000, 3)


def test_one_hot_categorical():
    rng = np.random.default_rng(4)
    n = 3000
    c = rng.integers(0, 3, n)
    x = rng.standard_normal(n).astype(np.float32)
    y = ((c == 1) * 2.0 + x > 0.5).astype(int)
    data = np.empty((n, 2), dtype=object)
    data[:, 0] = x
    data[:, 1] = np.array(["u", "v", "w"])[c]
    m = cb.CatBoostClassifier(iterations=30, depth=3, learning_rate=0.3, one_hot_max_size=10, verbose=False,
                              allow_writing_files=False)
    m.fit(data, y, cat_features=[1])
    assert (m.predict(data) == y).mean() > 0.95


def test_params_validation_and_synonyms():
    with pytest.raises(cb.CatBoostError):
        cb.CatBoostClassifier(no_such_param=1)
    m = cb.CatBoostRegressor(n_estimators=5, eta=0.5, max_depth=3, verbose=False, allow_writing_files=False)
    X, y = _binary(500, 4)
    m.fit(X, y.astype(float))
    assert m.tree_count_ == 5
    assert m.get_all_params()["learning_rate"] == 0.5
    from catboost_b200.params import parse_devices
    assert parse_devices("0-3") == [0, 1, 2, 3] and parse_devices("0:2:5") == [0, 2, 5]
    assert parse_devices("-1", 4) == [0, 1, 2, 3]


def test_overfitting_detector_and_best_model():
    X, y = _binary(2000, 5, 5)
    yn = y.copy()
    flip = np.random.default_rng(0).random(2000) < 0.35
    yn[flip] = 1 - yn[flip]
    m = cb.CatBoostClassifier(iterations=300, depth=6, learning_rate=0.5, early_stopping_rounds=10, verbose=False,
                              allow_writing_files=False)
    m.fit(X[:1000], yn[:1000], eval_set=(X[1000:], yn[1000:]))
    assert m.tree_count_ < 300
    assert m.best_iteration_ is not None and m.tree_count_ == m.best_iteration_ + 1


def test_border_selection_native():
    from catboost_b200.data.quantization import select_borders
    rng = np.random.default_rng(0)
    X = rng.standard_normal((5000, 3)).astype(np.float32)
    X[:, 2] = np.round(X[:, 2])      # few distinct values
    for bt in ["GreedyLogSum", "Median", "Uniform", "UniformAndQuantiles", "MinEntropy"]:
        borders, _ = select_borders(X, 16, bt)
        for f, b in enumerate(borders):
            assert len(b) <= 16 and np.all(np.diff(b) > 0)
        assert len(borders[0]) == 16
    # greedy borders of a near-uniform sample are close to quantiles
    b, _ = select_borders(X[:, :1], 15, "GreedyLogSum")
    q = np.searchsorted(np.sort(X[:, 0]), b[0]) / 5000
    assert np.all(np.abs(np.diff(q) - 1 / 16) < 0.02)


def test_overfitting_detectors_follow_the_reference_statistics():
    from catboost_b200.utils.overfit import OverfittingDetector, wilcoxon_signed_rank_pvalue
    # Iter: stops od_wait iterations after the best value
    od = OverfittingDetector("Iter", wait=3, max_optimal=False)
    stops = [od.add(v) for v in [1.0, 0.9, 0.8, 0.85, 0.86, 0.87, 0.88]]
    assert stops == [False, False, False, False, False, True, True] and od.best_iter == 2
    # IncToDec: a metric that rose by 1.0 and then loses 0.5 over a long stretch has ratio about 2 * 0.99^k ...
    od = OverfittingDetector("IncToDec", wait=5, pval=0.9, max_optimal=True)
    seq = [0.0, 0.5, 1.0] + [1.0 - 0.02 * k for k in range(1, 40)]
    fired = [od.add(v) for v in seq]
    assert not any(fired[:8]) and any(fired)
    k = fired.index(True)
    assert od.best_iter == 2 and k >= 8
    od = OverfittingDetector("IncToDec", wait=5, pval=0.9, max_optimal=True)
    for v in seq[: k + 1]:
        od.add(v)
    assert od.stopped and od.cur_pval < 0.9
    # hand check of the statistic at the first stop: p = exp(-0.5 / (expected_inc / drop))
    import math
    drop = 1.0 - seq[k]
    assert abs(od.cur_pval - math.exp(-0.5 / (od.expected_inc / drop))) < 1e-12
    # Wilcoxon: all deteriorations positive -> small p; mixed signs -> large p
    assert wilcoxon_signed_rank_pvalue([0.1] * 12) < 0.01
    assert wilcoxon_signed_rank_pvalue([0.1, -0.1] * 6) > 0.5
    od = OverfittingDetector("Wilcoxon", wait=6, pval=0.05, max_optimal=False)
    vals = [1.0, 0.5] + [0.5 + 0.01 * k for k in range(1, 15)]
    fired = [od.add(v) for v in vals]
    assert any(fired) and not any(fired[:7])


def test_option_handling_eval_fraction_output_borders_and_refusals(tmp_path):
    import catboost_b200 as cb
    rng = np.random.default_rng(1)
    X = rng.standard_normal((1200, 4)).astype(np.float32)
    y = (X[:, 0] > 0).astype(int)
    borders = tmp_path / "borders.tsv"
    m = cb.CatBoostClassifier(iterations=8, depth=3, verbose=False, allow_writing_files=False, eval_fraction=0.25,
                              output_borders=str(borders), border_count=16)
    m.fit(X, y)
    ev = m.get_evals_result()
    assert "validation" in ev and len(ev["validation"]["Logloss"]) == 8
    lines = borders.read_text().strip().split("\n")
    assert len(lines) == 4 * 16 and lines[0].split("\t")[0] == "0"
    # borders written by one run can be fed to the next one
    m2 = cb.CatBoostClassifier(iterations=8, depth=3, verbose=False, allow_writing_files=False, eval_fraction=0.25,
                               input_borders=str(borders), border_count=16).fit(X, y)
    assert np.allclose(m2.predict(X, prediction_type="RawFormulaVal"), m.predict(X, prediction_type="RawFormulaVal"))
    # options without an implementation are refused when set to something else than their default, hints are accepted
    with pytest.raises(cb.CatBoostError, match="not implemented"):
        cb.CatBoostClassifier(iterations=2, fixed_binary_splits=[0], verbose=False, allow_writing_files=False).fit(X, y)
    cb.CatBoostClassifier(iterations=2, used_ram_limit="4gb", sampling_unit="Object", verbose=False,
                          allow_writing_files=False).fit(X, y)


def test_posterior_sampling_group_sampling_and_per_feature_ctr():
    import catboost_b200 as cb
    from catboost_b200.params import resolve_options
    o = resolve_options(dict(posterior_sampling=True), "RMSE", 500)
    assert o.langevin and o.diffusion_temperature == 500.0 and abs(o.model_shrink_rate - 1e-3) < 1e-12
    with pytest.raises(cb.CatBoostError):
        resolve_options(dict(posterior_sampling=True, diffusion_temperature=5.0), "RMSE", 500)
    rng = np.random.default_rng(2)
    n = 1200
    X = rng.standard_normal((n, 4)).astype(np.float32)
    y = (X[:, 0] + 0.1 * rng.standard_normal(n)).astype(np.float32)
    m = cb.CatBoostRegressor(iterations=30, depth=3, posterior_sampling=True, verbose=False, allow_writing_files=False)
    m.fit(X, y)
    assert np.corrcoef(m.predict(X), y)[0, 1] > 0.9
    # one bootstrap draw per query
    gid = np.repeat(np.arange(n // 10), 10)
    r = cb.CatBoostRanker(iterations=10, depth=3, loss_function="QueryRMSE", sampling_unit="Group", bootstrap_type="Bernoulli",
                          subsample=0.5, verbose=False, allow_writing_files=False)
    r.fit(X, y, group_id=gid)
    assert np.corrcoef(r.predict(X), y)[0, 1] > 0.5
    with pytest.raises(cb.CatBoostError):
        cb.CatBoostRegressor(iterations=2, sampling_unit="Group", verbose=False, allow_writing_files=False).fit(X, y)
    # per-feature CTR descriptions override simple_ctr for that feature only
    c = rng.integers(0, 30, n)
    c2 = rng.integers(0, 25, n)
    Xo = np.empty((n, 3), dtype=object)
    Xo[:, 0], Xo[:, 1], Xo[:, 2] = X[:, 0], c, c2
    yc = (rng.standard_normal(30)[c] + 0.3 * rng.standard_normal(n) > 0).astype(np.float32)
    m = cb.CatBoostClassifier(iterations=20, depth=3, per_feature_ctr=["1:Counter"], max_ctr_complexity=1, one_hot_max_size=2,
                              verbose=False, allow_writing_files=False)
    m.fit(Xo, yc, cat_features=[1, 2])
    kinds = {}
    for cf in m._model.ctrs:
        kinds.setdefault(tuple(cf.cat_features), set()).add(cf.ctr_type)
    assert kinds[(0,)] == {"Counter"} and "Borders" in kinds[(1,)]
    with pytest.raises(cb.CatBoostError):
        cb.CatBoostClassifier(iterations=2, per_feature_ctr=["0:Counter"], verbose=False, allow_writing_files=False).fit(
            Xo, yc, cat_features=[1, 2])


def test_native_cpu_leaf_estimation_matches_tensor_path():
    """cbc_leaf_newton (all steps of a tree's leaf estimation in one native call, with step-length control) against the
    tensor formulation of the general learner."""
    import catboost_b200 as cb
    from catboost_b200.train import generic
    rng = np.random.default_rng(0)
    n, F = 20000, 10
    X = rng.standard_normal((n, F), dtype=np.float32)
    y = (X[:, 0] + X[:, 1] * X[:, 2] + 0.5 * rng.standard_normal(n) > 0).astype(np.float32)
    w = rng.random(n).astype(np.float32)
    out = {}
    try:
        for native in (True, False):
            generic.USE_NATIVE_CPU_LEAVES = native
            for loss, target, bt in (("Logloss", y, "AnyImprovement"), ("Logloss", y, "Armijo"), ("Logloss", y, "No"),
                                     ("RMSE", X[:, 0] + 0.1 * y, "AnyImprovement")):
                kw = dict(loss_function=loss, iterations=15, depth=5, learning_rate=0.5, verbose=False, allow_writing_files=False,
                          bootstrap_type="No", random_strength=0, leaf_estimation_backtracking=bt, leaf_estimation_iterations=8)
                m = (cb.CatBoostClassifier if loss == "Logloss" else cb.CatBoostRegressor)(**kw).fit(X, target, sample_weight=w)
                out[(native, loss, bt)] = m.predict(X[:3000], prediction_type="RawFormulaVal")
    finally:
        generic.USE_NATIVE_CPU_LEAVES = True
    for key in [k[1:] for k in out if k[0]]:
        assert np.max(np.abs(out[(True,) + key] - out[(False,) + key])) < 2e-5, key


def test_native_cpu_level_scores_match_tensor_scorer():
    """cbc_symmetric_scores against SplitScorer's tensor code: same trees for Cosine and L2, float and one-hot splits."""
    import catboost_b200 as cb
    from catboost_b200.train import generic
    rng = np.random.default_rng(1)
    n = 15000
    X = rng.standard_normal((n, 8), dtype=np.float32)
    y = (X[:, 0] + X[:, 1] * X[:, 2] + 0.5 * rng.standard_normal(n) > 0).astype(np.float32)
    Xc = np.c_[X[:, :5], rng.integers(0, 4, n)].astype(object)
    out = {}
    try:
        for native in (True, False):
            generic.USE_NATIVE_CPU_SCORES = native
            for sf in ("Cosine", "L2", "NewtonL2"):
                m = cb.CatBoostClassifier(iterations=12, depth=5, verbose=False, allow_writing_files=False, bootstrap_type="No",
                                          random_strength=0, score_function=sf).fit(X, y)
                out[(native, sf)] = m.predict(X[:2000], prediction_type="RawFormulaVal")
            m = cb.CatBoostClassifier(iterations=12, depth=4, verbose=False, allow_writing_files=False, bootstrap_type="No",
                                      random_strength=0, one_hot_max_size=8).fit(Xc, y, cat_features=[5])
            out[(native, "onehot")] = m.predict(Xc[:2000], prediction_type="RawFormulaVal")
    finally:
        generic.USE_NATIVE_CPU_SCORES = True
    for key in [k[1] for k in out if k[0]]:
        assert np.max(np.abs(out[(True, key)] - out[(False, key)])) < 1e-6, key
