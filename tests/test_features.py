"""Categorical / CTR features, ranking, model IO, importances, CV, CLI, snapshots (CPU)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import catboost_b200 as cb

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("CATBOOST_REFERENCE", os.path.join(os.path.dirname(ROOT), "reference"))


def _cat_data(n=6000, seed=0):
    rng = np.random.default_rng(seed)
    c1, c2 = rng.integers(0, 40, n), rng.integers(0, 150, n)
    x = rng.standard_normal(n).astype(np.float32)
    e1, e2 = rng.standard_normal(40), rng.standard_normal(150)
    y = (e1[c1] + 0.7 * e2[c2] + 0.5 * x + 0.5 * rng.standard_normal(n) > 0).astype(int)
    data = np.empty((n, 3), dtype=object)
    data[:, 0], data[:, 1], data[:, 2] = x, c1, np.array([f"v{k}" for k in c2])
    return data, y


def test_ctr_training_and_model_roundtrip(tmp_path):
    data, y = _cat_data()
    m = cb.CatBoostClassifier(iterations=40, depth=4, learning_rate=0.3, verbose=False, allow_writing_files=False,
                              max_ctr_complexity=2)
    m.fit(data[:4500], y[:4500], cat_features=[1, 2], eval_set=(data[4500:], y[4500:]))
    assert (m.predict(data[4500:]) == y[4500:]).mean() > 0.8
    assert len(m._model.ctrs) > 0
    raw = m.predict(data[4500:], prediction_type="RawFormulaVal")
    for fmt in ("cbm", "json"):
        f = str(tmp_path / f"m.{fmt}")
        m.save_model(f, format=fmt)
        m2 = cb.CatBoostClassifier().load_model(f, format=fmt)
        assert np.allclose(m2.predict(data[4500:], prediction_type="RawFormulaVal"), raw, atol=1e-9)
        assert list(m2.classes_) == [0, 1]


def test_ordered_ctr_matches_plain_python_oracle():
    """Ordered target statistic of one categorical column against a sequential re-implementation."""
    import torch
    from catboost_b200.train.ctr import _group_rows, _segment_stats
    rng = np.random.default_rng(1)
    n = 500
    keys = rng.integers(-6, 7, n)
    order = rng.permutation(n)
    good = (rng.random(n) < 0.3).astype(np.int32)
    rows, seg_id, first_idx, uniq = _group_rows(torch.from_numpy(keys), torch.from_numpy(order))
    assert uniq.tolist() == sorted(set(keys.tolist()))
    totals, got = _segment_stats([torch.ones(n, dtype=torch.int32), torch.from_numpy(good)], rows, seg_id, first_idx, True)
    cnt, pos = {}, {}
    exp = np.zeros((2, n))
    for i in order:
        k = keys[i]
        exp[0, i], exp[1, i] = cnt.get(k, 0), pos.get(k, 0)
        cnt[k] = cnt.get(k, 0) + 1
        pos[k] = pos.get(k, 0) + good[i]
    assert np.allclose(got.numpy(), exp)
    assert totals[0].tolist() == [cnt[k] for k in uniq.tolist()] and totals[1].tolist() == [pos[k] for k in uniq.tolist()]


def test_cat_hash_known_values():
    """Hashes stored in the CTR tables of a model produced by the reference must be reproduced from the raw strings."""
    path = os.path.join(REF, "catboost/pytest/data/models/features_num_cat__dataset_adult.cbm")
    adult = os.path.join(REF, "catboost/pytest/data/adult")
    if not os.path.exists(path):
        pytest.skip("reference model files are not available")
    from catboost_b200.models.ctr import projection_hash
    m = cb.CatBoost().load_model(path)
    pool = cb.Pool(os.path.join(adult, "train_small"), column_description=os.path.join(adult, "train.cd"))
    fd, ch = m._model.pool_arrays(pool)
    checked = 0
    for ctr in m._model.ctrs:
        if len(ctr.cat_features) != 1 or len(ctr.hashes) == 0:
            continue
        ours = set(np.unique(projection_hash([ch[ctr.cat_features[0]]])).tolist())
        stored = set(int(h) for h in ctr.hashes)
        assert len(ours & stored) >= 0.9 * len(ours), (ctr.cat_features, len(ours & stored), len(ours))
        checked += 1
    assert checked >= 5


def test_reference_models_load_and_predict():
    iris = os.path.join(REF, "catboost/dotnet/CatBoostNetTests/testbed/iris")
    if not os.path.exists(iris):
        pytest.skip("reference model files are not available")
    rows = [l.strip().split(",") for l in open(os.path.join(iris, "iris.data")) if l.strip()]
    X = np.array([[float(v) for v in r[:4]] for r in rows], dtype=np.float32)
    names = sorted({r[4] for r in rows})
    yi = np.array([names.index(r[4]) for r in rows])
    m = cb.CatBoostClassifier().load_model(os.path.join(iris, "iris_model.cbm"))
    assert (np.asarray(m.predict(X)).astype(int) == yi).mean() > 0.97
    adult = os.path.join(REF, "catboost/pytest/data/adult")
    m = cb.CatBoostRegressor().load_model(os.path.join(REF, "catboost/pytest/data/models/features_num_cat__dataset_adult.cbm"))
    pool = cb.Pool(os.path.join(adult, "train_small"), column_description=os.path.join(adult, "train.cd"))
    pred = m.predict(pool)
    lab = np.asarray(pool.label, dtype=float)
    assert np.sqrt(np.mean((pred - lab) ** 2)) < 0.2          # the model was fitted on these rows (CTR tables included)


def test_ranking_losses():
    rng = np.random.default_rng(0)
    sizes = rng.integers(5, 30, 150)
    gid = np.repeat(np.arange(150), sizes)
    n = len(gid)
    X = rng.standard_normal((n, 8)).astype(np.float32)
    score = X @ rng.standard_normal(8) + 0.5 * rng.standard_normal(n)
    rel = np.digitize(score, np.quantile(score, [0.5, 0.8, 0.95])).astype(np.float32)
    for loss in ("YetiRank", "QueryRMSE", "PairLogit", "LambdaMart"):
        m = cb.CatBoostRanker(loss_function=loss, iterations=25, depth=4, learning_rate=0.3, verbose=False,
                              allow_writing_files=False, eval_metric="NDCG")
        m.fit(X, rel, group_id=gid)
        ev = m.get_evals_result()["learn"]["NDCG"]
        assert ev[-1] > ev[0] and ev[-1] > 0.9, (loss, ev[0], ev[-1])
    with pytest.raises(cb.CatBoostError):
        cb.CatBoostRanker(loss_function="YetiRank", iterations=2, verbose=False, allow_writing_files=False).fit(X, rel)


def test_importances_and_shap_sum_to_prediction():
    rng = np.random.default_rng(0)
    X = rng.standard_normal((1500, 5)).astype(np.float32)
    y = 3 * X[:, 0] + X[:, 1] * X[:, 2] + 0.1 * rng.standard_normal(1500)
    m = cb.CatBoostRegressor(iterations=30, depth=4, learning_rate=0.3, verbose=False, allow_writing_files=False)
    m.fit(X, y)
    imp = m.get_feature_importance()
    assert abs(imp.sum() - 100) < 1e-6 and imp.argmax() == 0 and imp[4] < 5
    pool = cb.Pool(X[:40], y[:40])
    sv = m.get_feature_importance(pool, type="ShapValues")
    assert sv.shape == (40, 6)
    assert np.allclose(sv.sum(1), m.predict(X[:40]), atol=1e-6)
    lfc = m.get_feature_importance(cb.Pool(X[:300], y[:300]), type="LossFunctionChange")
    assert lfc.argmax() == 0
    inter = m.get_feature_importance(type="Interaction")
    assert len(inter) > 0


def test_cv_and_grid_search():
    rng = np.random.default_rng(0)
    X = rng.standard_normal((1200, 5)).astype(np.float32)
    y = (X[:, 0] + X[:, 1] > 0).astype(int)
    res = cb.cv(cb.Pool(X, y), dict(loss_function="Logloss", iterations=15, depth=3, learning_rate=0.3), fold_count=3,
                as_pandas=False)
    assert len(res["test-Logloss-mean"]) == 15 and res["test-Logloss-mean"][-1] < res["test-Logloss-mean"][0]
    m = cb.CatBoostClassifier(iterations=10, verbose=False, allow_writing_files=False)
    out = m.grid_search({"depth": [2, 4], "learning_rate": [0.1, 0.5]}, X, y, verbose=False)
    assert set(out["params"]) == {"depth", "learning_rate"} and m.is_fitted()


def test_snapshot_resume_equals_uninterrupted(tmp_path):
    rng = np.random.default_rng(0)
    X = rng.standard_normal((1500, 6)).astype(np.float32)
    y = (X[:, 0] * X[:, 1] > 0).astype(int)
    common = dict(depth=4, learning_rate=0.3, verbose=False, random_seed=3, bootstrap_type="No", random_strength=0,
                  train_dir=str(tmp_path), allow_writing_files=True)
    full = cb.CatBoostClassifier(iterations=20, **common).fit(X, y)
    part = cb.CatBoostClassifier(iterations=8, save_snapshot=True, snapshot_file="s.snap", **common).fit(X, y)
    assert part.tree_count_ == 8
    resumed = cb.CatBoostClassifier(iterations=20, save_snapshot=True, snapshot_file="s.snap", **common).fit(X, y)
    assert resumed.tree_count_ == 20
    assert np.allclose(resumed.predict(X, prediction_type="RawFormulaVal"),
                       full.predict(X, prediction_type="RawFormulaVal"), atol=1e-9)
    # a corrupted snapshot is detected
    p = tmp_path / "s.snap"
    blob = bytearray(p.read_bytes())
    blob[-5] ^= 0xFF
    p.write_bytes(bytes(blob))
    with pytest.raises(cb.CatBoostError):
        cb.CatBoostClassifier(iterations=22, save_snapshot=True, snapshot_file="s.snap", **common).fit(X, y)


def test_cli_fit_calc(tmp_path):
    rng = np.random.default_rng(0)
    X = rng.standard_normal((400, 4))
    y = (X[:, 0] > 0).astype(int)
    train = tmp_path / "train.tsv"
    with open(train, "w") as fh:
        for i in range(400):
            fh.write("\t".join([str(y[i])] + [f"{v:.6f}" for v in X[i]]) + "\n")
    cd = tmp_path / "train.cd"
    cd.write_text("0\tLabel\n")
    model = tmp_path / "model.bin"
    env = dict(os.environ, PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-m", "catboost_b200", "fit", "-f", str(train), "--cd", str(cd), "-m", str(model),
                        "--loss-function", "Logloss", "-i", "10", "--verbose", "0", "--train-dir", str(tmp_path / "info")],
                       capture_output=True, text=True, env=env, cwd=str(tmp_path))
    assert r.returncode == 0, r.stderr
    out = tmp_path / "pred.tsv"
    r = subprocess.run([sys.executable, "-m", "catboost_b200", "calc", "-m", str(model), "--input-path", str(train),
                        "--cd", str(cd), "-o", str(out), "--prediction-type", "Probability"],
                       capture_output=True, text=True, env=env, cwd=str(tmp_path))
    assert r.returncode == 0, r.stderr
    lines = out.read_text().strip().split("\n")
    assert len(lines) == 401


def test_sum_models_and_metrics():
    rng = np.random.default_rng(0)
    X = rng.standard_normal((800, 4)).astype(np.float32)
    y = X[:, 0] + 0.1 * rng.standard_normal(800)
    a = cb.CatBoostRegressor(iterations=5, depth=3, verbose=False, allow_writing_files=False, random_seed=1).fit(X, y)
    b = cb.CatBoostRegressor(iterations=7, depth=3, verbose=False, allow_writing_files=False, random_seed=2).fit(X, y)
    s = cb.sum_models([a, b], weights=[0.5, 0.5])
    assert np.allclose(s.predict(X), 0.5 * a.predict(X) + 0.5 * b.predict(X), atol=1e-9)
    ev = a.eval_metrics(cb.Pool(X, y), ["RMSE", "R2", "MAE"])
    assert len(ev["RMSE"]) == 5 and ev["RMSE"][-1] <= ev["RMSE"][0]
    from catboost_b200.metrics import make_metric
    yb = (y > 0).astype(float)
    assert abs(make_metric("AUC").eval(y.reshape(-1, 1), yb) - 1.0) < 1e-12
    assert make_metric("NDCG:top=3").eval(np.array([[3.0], [2.0], [1.0]]), np.array([2.0, 1.0, 0.0]),
                                          group_offsets=np.array([0, 3])) == pytest.approx(1.0)


def test_ordered_boosting_regularises():
    rng = np.random.default_rng(0)
    X = rng.standard_normal((2400, 6)).astype(np.float32)
    y = (X[:, 0] + X[:, 1] * X[:, 2] + 0.8 * rng.standard_normal(2400) > 0).astype(int)
    res = {}
    for bt in ("Plain", "Ordered"):
        m = cb.CatBoostClassifier(iterations=60, depth=5, learning_rate=0.2, boosting_type=bt, verbose=False,
                                  allow_writing_files=False)
        m.fit(X[:1200], y[:1200], eval_set=(X[1200:], y[1200:]), use_best_model=False)
        ev = m.get_evals_result()
        res[bt] = (ev["learn"]["Logloss"][-1], min(ev["validation"]["Logloss"]))
    assert res["Ordered"][0] > res["Plain"][0]            # fits the training rows less tightly
    assert res["Ordered"][1] < res["Plain"][1] + 0.02     # and generalises at least as well


def test_pairwise_histograms_match_bruteforce_and_train():
    """The range-update construction of the per-candidate pair systems against a direct loop over pairs and borders,
    then end-to-end training with the pairwise losses."""
    import torch
    from catboost_b200.data.pool import Pool
    from catboost_b200.params import resolve_options
    from catboost_b200.parallel.runtime import DistContext
    from catboost_b200.train.boosting import build_store, plan_features
    from catboost_b200.train.pairwise import PairwiseLearner, _solve_pairwise
    rng = np.random.default_rng(3)
    n, F = 80, 4
    X = rng.standard_normal((n, F)).astype(np.float32)
    pool = Pool(X, rng.random(n).astype(np.float32))
    o = resolve_options(dict(border_count=8, depth=3, l2_leaf_reg=1.0), "PairLogitPairwise", n)
    plan = plan_features(o, pool, DistContext(0, 1, torch.device("cpu")), None)
    store, _ = build_store(plan, pool, torch.device("cpu"))
    pl = PairwiseLearner(store, o)
    P = 300
    wi = torch.from_numpy(rng.integers(0, n, P))
    li = torch.from_numpy(rng.integers(0, n, P))
    keep = wi != li
    wi, li = wi[keep], li[keep]
    h = torch.from_numpy(rng.random(len(wi)).astype(np.float32))
    der = torch.from_numpy(rng.standard_normal(n).astype(np.float32))
    L = 2
    leaf = torch.from_numpy(rng.integers(0, L, n))
    for f in range(F):
        got = pl._feature_scores(f, leaf, L, wi, li, h, der).numpy()
        nb = int(store.feat_nb_host[f])
        b = pl.bins[f]
        ref = []
        for t in range(nb - 1):
            child = leaf + (b > t).long() * L
            S = 2 * L
            M = torch.zeros((S, S), dtype=torch.float64)
            for p in range(len(wi)):
                a_, b_ = int(child[wi[p]]), int(child[li[p]])
                w = float(h[p])
                M[a_, a_] += w; M[b_, b_] += w; M[a_, b_] -= w; M[b_, a_] -= w
            d = torch.zeros(S, dtype=torch.float64).index_add_(0, child, der.double())
            ref.append(float(_solve_pairwise(M, d, pl.l2, pl.prior)[1]))
        assert np.allclose(got, np.array(ref), rtol=1e-8, atol=1e-10), f
    # training
    sizes = rng.integers(5, 25, 80)
    gid = np.repeat(np.arange(80), sizes)
    m_ = len(gid)
    Xr = rng.standard_normal((m_, 6)).astype(np.float32)
    sc = Xr @ rng.standard_normal(6) + 0.3 * rng.standard_normal(m_)
    rel = np.digitize(sc, np.quantile(sc, [0.5, 0.8])).astype(np.float32)
    for loss in ("PairLogitPairwise", "YetiRankPairwise"):
        m = cb.CatBoostRanker(loss_function=loss, iterations=12, depth=3, learning_rate=0.3, verbose=False,
                              allow_writing_files=False, eval_metric="NDCG", border_count=16)
        m.fit(Xr, rel, group_id=gid)
        ev = m.get_evals_result()["learn"]["NDCG"]
        assert ev[-1] > ev[0] and ev[-1] > 0.95, (loss, ev[0], ev[-1])


def test_monotone_constraints():
    rng = np.random.default_rng(0)
    n = 3000
    X = rng.uniform(-2, 2, (n, 3)).astype(np.float32)
    y = (np.sin(3 * X[:, 0]) + 0.5 * X[:, 0] + X[:, 1] ** 2 + 0.1 * rng.standard_normal(n)).astype(np.float32)
    grid = np.linspace(-2, 2, 150).astype(np.float32)

    def worst_decrease(m, sign):
        w = 0.0
        for x1 in (-1.0, 0.0, 1.5):
            Z = np.stack([grid, np.full(150, x1, np.float32), np.zeros(150, np.float32)], 1)
            w = max(w, float(np.max(-sign * np.diff(m.predict(Z)))))
        return w

    free = cb.CatBoostRegressor(iterations=60, depth=4, learning_rate=0.2, verbose=False, allow_writing_files=False).fit(X, y)
    assert worst_decrease(free, 1) > 0.05
    for spec, sign in (([1, 0, 0], 1), ("0:-1", -1), ({"0": 1}, 1)):
        m = cb.CatBoostRegressor(iterations=60, depth=4, learning_rate=0.2, verbose=False, allow_writing_files=False,
                                 monotone_constraints=spec).fit(X, y)
        assert worst_decrease(m, sign) <= 1e-9, spec


def test_shap_interaction_values():
    rng = np.random.default_rng(0)
    X = rng.standard_normal((600, 4)).astype(np.float32)
    y = (2 * X[:, 0] + X[:, 1] * X[:, 2] + 0.05 * rng.standard_normal(600)).astype(np.float32)
    m = cb.CatBoostRegressor(iterations=15, depth=3, learning_rate=0.3, verbose=False, allow_writing_files=False).fit(X, y)
    P = cb.Pool(X[:5], y[:5])
    sv = m.get_feature_importance(P, type="ShapValues")
    iv = m.get_feature_importance(P, type="ShapInteractionValues")
    assert iv.shape == (5, 5, 5)
    assert np.allclose(iv[:, :4, :4].sum(2), sv[:, :4], atol=1e-10)            # rows add up to the SHAP values
    assert np.allclose(iv[:, :4, :4], iv[:, :4, :4].transpose(0, 2, 1), atol=1e-10)
    assert np.allclose(iv.sum((1, 2)), m.predict(X[:5]), atol=1e-8)
    mean_abs = np.abs(iv[:, :4, :4]).mean(0)
    assert mean_abs[1, 2] > 5 * mean_abs[0, 3]                                  # the x1 * x2 term is the interaction


def test_text_and_embedding_features(tmp_path):
    rng = np.random.default_rng(0)
    n = 900
    pos, neg = ["great", "excellent", "love", "good"], ["bad", "awful", "hate", "poor"]
    neutral = ["the", "a", "movie", "was", "it", "very", "film"]
    y = rng.integers(0, 2, n)
    data = np.empty((n, 4), dtype=object)
    data[:, :2] = rng.standard_normal((n, 2)).astype(np.float32)
    centers = rng.standard_normal((2, 6))
    for i in range(n):
        w = list(rng.choice(neutral, 4)) + list(rng.choice(pos if y[i] else neg, 2))
        rng.shuffle(w)
        data[i, 2] = " ".join(w)
        data[i, 3] = (centers[y[i]] * 0.6 + rng.standard_normal(6)).astype(np.float32)
    tr, te = slice(0, 700), slice(700, n)
    m = cb.CatBoostClassifier(iterations=30, depth=4, learning_rate=0.2, verbose=False, allow_writing_files=False)
    m.fit(data[tr], y[tr], text_features=[2], embedding_features=[3], eval_set=(data[te], y[te]))
    acc = float((m.predict(data[te]) == y[te]).mean())
    assert acc > 0.9, acc
    assert any(nm.startswith("text2_bow_") for nm in m._model.feature_names)
    assert any(nm.startswith("emb3_knn_") for nm in m._model.feature_names)
    path = str(tmp_path / "text.cbm")
    m.save_model(path)
    m2 = cb.CatBoostClassifier().load_model(path)
    assert np.allclose(m2.predict(data[te], prediction_type="RawFormulaVal"),
                       m.predict(data[te], prediction_type="RawFormulaVal"))
    # text only, regression: bag of words without target statistics
    yr = np.array([t.count("great") + t.count("love") - t.count("bad") for t in data[:, 2]], dtype=np.float32)
    r = cb.CatBoostRegressor(iterations=40, depth=4, learning_rate=0.3, verbose=False, allow_writing_files=False)
    r.fit(data[tr][:, [2]], yr[tr], text_features=[0])
    assert float(np.sqrt(np.mean((r.predict(data[te][:, [2]]) - yr[te]) ** 2))) < 0.5


def test_training_logs_and_tensorboard_events(tmp_path):
    import struct
    from catboost_b200.utils.logging import _masked_crc32c
    rng = np.random.default_rng(0)
    X = rng.standard_normal((400, 4)).astype(np.float32)
    y = (X[:, 0] > 0).astype(int)
    d = str(tmp_path / "info")
    cb.CatBoostClassifier(iterations=5, depth=3, verbose=False, train_dir=d).fit(X[:300], y[:300], eval_set=(X[300:], y[300:]))
    assert os.path.exists(os.path.join(d, "learn_error.tsv")) and os.path.exists(os.path.join(d, "catboost_training.json"))
    for part in ("learn", "test"):
        raw = open(os.path.join(d, part, "events.out.tfevents"), "rb").read()
        pos, records = 0, 0
        while pos < len(raw):
            (ln,) = struct.unpack("<Q", raw[pos:pos + 8])
            assert struct.unpack("<I", raw[pos + 8:pos + 12])[0] == _masked_crc32c(raw[pos:pos + 8])
            payload = raw[pos + 12:pos + 12 + ln]
            assert struct.unpack("<I", raw[pos + 12 + ln:pos + 16 + ln])[0] == _masked_crc32c(payload)
            pos += 16 + ln
            records += 1
        assert records == 1 + 5            # the version record + one scalar per iteration
        assert b"Logloss" in raw
    assert _masked_crc32c(b"123456789") == ((((0xE3069283 >> 15) | (0xE3069283 << 17)) & 0xFFFFFFFF) + 0xA282EAD8) & 0xFFFFFFFF


def _pb_fields(buf):
    """Generic protobuf reader: list of (field, wire type, value) of one message."""
    out, pos = [], 0
    while pos < len(buf):
        key, shift = 0, 0
        while True:
            b = buf[pos]; pos += 1
            key |= (b & 0x7F) << shift; shift += 7
            if not b & 0x80:
                break
        field, wire = key >> 3, key & 7
        if wire == 0:
            v, shift = 0, 0
            while True:
                b = buf[pos]; pos += 1
                v |= (b & 0x7F) << shift; shift += 7
                if not b & 0x80:
                    break
        elif wire == 2:
            ln, shift = 0, 0
            while True:
                b = buf[pos]; pos += 1
                ln |= (b & 0x7F) << shift; shift += 7
                if not b & 0x80:
                    break
            v = buf[pos:pos + ln]; pos += ln
        elif wire == 5:
            v = buf[pos:pos + 4]; pos += 4
        else:
            v = buf[pos:pos + 8]; pos += 8
        out.append((field, wire, v))
    return out


def test_onnx_and_pmml_export(tmp_path):
    """The ONNX file is decoded with a generic protobuf reader and its tree ensemble is evaluated by hand; the PMML file is
    parsed as XML and evaluated by hand.  Both must reproduce the model's predictions."""
    import struct
    import xml.etree.ElementTree as ET
    rng = np.random.default_rng(0)
    X = rng.standard_normal((400, 5)).astype(np.float32)
    y = (2 * X[:, 0] - X[:, 3] + 0.1 * rng.standard_normal(400)).astype(np.float32)
    m = cb.CatBoostRegressor(iterations=12, depth=3, learning_rate=0.3, verbose=False, allow_writing_files=False).fit(X, y)
    ref = m.predict(X[:30])
    # ---- ONNX
    p = str(tmp_path / "m.onnx")
    m.save_model(p, format="onnx")
    model = _pb_fields(open(p, "rb").read())
    graph = _pb_fields([v for f, w, v in model if f == 7][0])
    node = _pb_fields([v for f, w, v in graph if f == 1][0])
    assert [v for f, w, v in node if f == 4][0] == b"TreeEnsembleRegressor"
    attrs = {}
    for f, w, v in node:
        if f == 5:
            a = _pb_fields(v)
            name = [x for ff, ww, x in a if ff == 1][0].decode()
            if any(ff == 8 for ff, _, _ in a):
                packed = [x for ff, ww, x in a if ff == 8][0]
                vals, pos = [], 0
                while pos < len(packed):
                    val, shift = 0, 0
                    while True:
                        b = packed[pos]; pos += 1
                        val |= (b & 0x7F) << shift; shift += 7
                        if not b & 0x80:
                            break
                    vals.append(val)
                attrs[name] = vals
            elif any(ff == 7 for ff, _, _ in a):
                packed = [x for ff, ww, x in a if ff == 7][0]
                attrs[name] = list(struct.unpack(f"<{len(packed) // 4}f", packed))
            elif any(ff == 9 for ff, _, _ in a):
                attrs[name] = [x.decode() for ff, ww, x in a if ff == 9]
    nodes = {(t, n): k for k, (t, n) in enumerate(zip(attrs["nodes_treeids"], attrs["nodes_nodeids"]))}
    leaf_w = {(t, n): w for t, n, w in zip(attrs["target_treeids"], attrs["target_nodeids"], attrs["target_weights"])}
    pred = np.full(30, attrs["base_values"][0], dtype=np.float64)
    for r in range(30):
        for t in sorted(set(attrs["nodes_treeids"])):
            n = 0
            while True:
                k = nodes[(t, n)]
                if attrs["nodes_modes"][k] == "LEAF":
                    pred[r] += leaf_w[(t, n)]
                    break
                go = X[r, attrs["nodes_featureids"][k]] > attrs["nodes_values"][k]
                n = attrs["nodes_truenodeids"][k] if go else attrs["nodes_falsenodeids"][k]
    assert np.allclose(pred, ref, atol=1e-4)
    # ---- PMML
    p2 = str(tmp_path / "m.pmml")
    m.save_model(p2, format="pmml")
    ns = {"p": "http://www.dmg.org/PMML-4_3"}
    root = ET.parse(p2).getroot()
    names = [f"{i}" for i in range(5)]
    const = float(root.find(".//p:Target", ns).get("rescaleConstant"))

    def walk(node, row):
        for child in node.findall("p:Node", ns):
            sp = child.find("p:SimplePredicate", ns)
            ok = True if sp is None else row[names.index(sp.get("field"))] > float(sp.get("value"))
            if ok:
                return float(child.get("score")) if child.get("score") is not None else walk(child, row)
        raise AssertionError("no branch taken")

    pred2 = np.full(30, const)
    for r in range(30):
        for tm in root.iterfind(".//p:TreeModel", ns):
            top = tm.find("p:Node", ns)
            pred2[r] += float(top.get("score")) if top.get("score") is not None else walk(top, X[r])
    assert np.allclose(pred2, ref, atol=1e-4)


def test_partial_dependence():
    rng = np.random.default_rng(0)
    X = rng.uniform(-2, 2, (2000, 3)).astype(np.float32)
    y = (3 * X[:, 0] + np.sin(X[:, 1]) + 0.05 * rng.standard_normal(2000)).astype(np.float32)
    m = cb.CatBoostRegressor(iterations=40, depth=4, learning_rate=0.3, verbose=False, allow_writing_files=False,
                             border_count=16).fit(X, y)
    pd0, fig = m.plot_partial_dependence(X[:300], 0)
    assert fig is None and pd0.ndim == 1 and len(pd0) == len(m._model.float_features[0].borders) + 1
    assert np.all(np.diff(pd0) > -0.05) and pd0[-1] - pd0[0] > 6          # increasing like 3 * x0 over [-2, 2]
    pd2, _ = m.plot_partial_dependence(X[:100], [0, 2])
    assert pd2.shape == (len(m._model.float_features[0].borders) + 1, len(m._model.float_features[2].borders) + 1)
    assert np.abs(pd2[:, 0] - pd2[:, -1]).max() < 0.5                      # x2 carries no signal


def _refit_leaves(model, leaf_tr, leaf_te, y, w, lr, l2, loss):
    """Leaf values of fixed tree structures re-estimated with document weights ``w`` (one Newton step per tree)."""
    T = leaf_tr.shape[1]
    bias = float(np.ravel(model.bias)[0])
    a = np.full(len(y), bias)
    at = np.full(leaf_te.shape[0], bias)
    for t in range(T):
        if loss == "RMSE":
            der, hess = y - a, np.ones_like(a)
        else:
            p = 1.0 / (1.0 + np.exp(-a))
            der, hess = y - p, p * (1 - p)
        L = model.trees[t].leaf_values.shape[0]
        D = np.bincount(leaf_tr[:, t], weights=w * der, minlength=L)
        H = np.bincount(leaf_tr[:, t], weights=w * hess, minlength=L) + l2
        val = lr * D / H
        a = a + val[leaf_tr[:, t]]
        at = at + val[leaf_te[:, t]]
    return at


@pytest.mark.parametrize("loss", ["RMSE", "Logloss"])
def test_object_importance_against_reweighted_refit(loss):
    rng = np.random.default_rng(5)
    n, m = 120, 15
    X = rng.standard_normal((n + m, 4)).astype(np.float32)
    f = X[:, 0] + 0.5 * X[:, 1] * X[:, 2]
    y = (f + 0.3 * rng.standard_normal(n + m)).astype(np.float32) if loss == "RMSE" else (f > 0).astype(np.float32)
    cls = cb.CatBoostRegressor if loss == "RMSE" else cb.CatBoostClassifier
    lr, l2 = 0.3, 2.0
    mdl = cls(iterations=8, depth=3, learning_rate=lr, l2_leaf_reg=l2, bootstrap_type="No", leaf_estimation_iterations=1,
              leaf_estimation_method="Newton", boost_from_average=False, random_strength=0, verbose=False,
              allow_writing_files=False, loss_function=loss).fit(X[:n], y[:n])
    train, test = cb.Pool(X[:n], y[:n]), cb.Pool(X[n:], y[n:])
    M = mdl._model
    leaf_tr, leaf_te = M.leaf_indices(X[:n]), M.leaf_indices(X[n:])
    base = _refit_leaves(M, leaf_tr, leaf_te, y[:n].astype(np.float64), np.ones(n), lr, l2, loss)
    np.testing.assert_allclose(base, mdl.predict(X[n:], prediction_type="RawFormulaVal"), rtol=1e-4, atol=1e-4)
    from catboost_b200.ostr import object_importance
    from catboost_b200.train.objectives import make_objective
    scores = object_importance(M, make_objective(loss, {}), M.params, train, test, y[:n], y[n:], update_method="AllPoints",
                               device="cpu")
    if loss == "RMSE":
        der_te = y[n:] - base
    else:
        der_te = y[n:] - 1.0 / (1.0 + np.exp(-base))
    eps = 1e-4
    for i in (0, 7, 33, 90):
        w = np.ones(n)
        w[i] = 1 + eps
        up = _refit_leaves(M, leaf_tr, leaf_te, y[:n].astype(np.float64), w, lr, l2, loss)
        w[i] = 1 - eps
        dn = _refit_leaves(M, leaf_tr, leaf_te, y[:n].astype(np.float64), w, lr, l2, loss)
        np.testing.assert_allclose(scores[i], der_te * (up - dn) / (2 * eps), rtol=2e-3, atol=1e-7)
    # the public call: ordering, signs, sizes
    idx, val = mdl.get_object_importance(test, train, top_size=10, update_method="AllPoints")
    assert len(idx) == 10 and np.all(np.diff(np.abs(val)) <= 1e-15)
    np.testing.assert_allclose(val, scores.mean(axis=1)[idx], rtol=1e-9, atol=1e-12)
    idx_p, val_p = mdl.get_object_importance(test, train, importance_values_sign="Positive", update_method="SinglePoint")
    assert np.all(val_p > 0) and len(idx_p) <= n
    per_idx, per_val = mdl.get_object_importance(test, train, type="PerObject", top_size=3, update_method="AllPoints")
    assert len(per_idx) == m and all(len(v) == 3 for v in per_val)


def test_eval_features_finds_the_useful_feature(tmp_path):
    rng = np.random.default_rng(3)
    n = 900
    X = rng.standard_normal((n, 4)).astype(np.float32)
    y = (2.0 * X[:, 1] + 0.1 * rng.standard_normal(n)).astype(np.float32)      # only feature 1 matters
    res = cb.eval_features(cb.Pool(X, y), {"loss_function": "RMSE", "iterations": 30, "depth": 3, "learning_rate": 0.3},
                           [1, 3], eval_type="SeqAddAndAll", fold_count=6)
    cases = res["RMSE"]["cases"]
    assert set(cases) == {"all features", "with 1", "with 3"} and len(res["RMSE"]["baseline"]) == 6
    assert cases["with 1"]["delta_mean"] > 0.5 and cases["with 1"]["decision"] == "GOOD"
    assert abs(cases["with 3"]["delta_mean"]) < 0.1 and cases["with 3"]["decision"] != "GOOD"
    assert cases["all features"]["decision"] == "GOOD"
    # command line: the same evaluation from a file, and object importance of a saved model
    from catboost_b200 import cli
    data = tmp_path / "d.tsv"
    np.savetxt(data, np.column_stack([y, X]), delimiter="\t", fmt="%.6g")
    out = tmp_path / "fe.json"
    assert cli.main(["eval-feature", "-f", str(data), "--features-to-evaluate", "1", "--fold-count", "3", "-i", "15",
                     "-o", str(out)]) == 0
    import json
    assert json.loads(out.read_text())["RMSE"]["cases"]["all features"]["delta_mean"] > 0.3
    m = cb.CatBoostRegressor(iterations=10, depth=3, verbose=False, allow_writing_files=False).fit(X, y)
    m.save_model(str(tmp_path / "m.cbm"))
    ostr = tmp_path / "ostr.tsv"
    assert cli.main(["ostr", "-m", str(tmp_path / "m.cbm"), "-f", str(data), "-t", str(data), "--top-size", "5",
                     "-o", str(ostr)]) == 0
    assert len(ostr.read_text().strip().splitlines()) == 5


def test_utils_module(tmp_path):
    from catboost_b200 import utils
    cd = tmp_path / "train.cd"
    utils.create_cd(label=0, cat_features=[2, 4], weight=5, auxiliary_columns=[6], feature_names={1: "age", 2: "city"},
                    output_path=str(cd))
    assert cd.read_text().splitlines() == ["0\tLabel\t", "1\tNum\tage", "2\tCateg\tcity", "4\tCateg\t", "5\tWeight\t",
                                           "6\tAuxiliary\t"]
    with pytest.raises(cb.CatBoostError):
        utils.create_cd(label=0, cat_features=[0], output_path=str(cd))
    info = utils.read_cd(str(cd), column_count=8)
    assert info["cat_feature_indices"] == [1, 3] and info["non_feature_column_indices"] == [0, 5, 6]
    assert info["column_type_to_indices"]["Categ"] == [2, 4] and info["column_names"][1] == "age"
    rng = np.random.default_rng(0)
    X = rng.standard_normal((800, 4)).astype(np.float32)
    y = (X[:, 0] + 0.3 * rng.standard_normal(800) > 0).astype(int)
    m = cb.CatBoostClassifier(iterations=20, depth=3, verbose=False, allow_writing_files=False).fit(X, y)
    pool = cb.Pool(X, y)
    raw = m.predict(X, prediction_type="RawFormulaVal")
    from catboost_b200.metrics import make_metric
    assert utils.eval_metric(y, raw, "Logloss") == [make_metric("Logloss").eval(raw, y.astype(float))]
    assert utils.eval_metric(y, raw, "AUC")[0] > 0.9
    fpr, tpr, thr = utils.get_roc_curve(m, pool)
    assert fpr[0] == 0 and tpr[-1] == 1 and np.all(np.diff(fpr) >= 0) and np.all(np.diff(thr) <= 0)
    t_fpr, f = utils.get_fpr_curve(curve=(fpr, tpr, thr))
    t_fnr, g = utils.get_fnr_curve(m, pool)
    assert np.allclose(f, fpr) and np.allclose(g, 1 - tpr)
    b = utils.select_threshold(m, pool, FPR=0.05)
    p = m.predict_proba(X)[:, 1]
    assert np.mean(p[y == 0] >= b) <= 0.05 + 1e-9
    assert 0 < utils.select_threshold(curve=(fpr, tpr, thr)) < 1
    cm = utils.get_confusion_matrix(m, pool)
    pred = np.asarray(m.predict(X)).astype(int).reshape(-1)
    assert cm.sum() == 800 and cm[1, 1] == np.sum((y == 1) & (pred == 1)) and cm[0, 1] == np.sum((y == 0) & (pred == 1))
    grid = utils.calculate_quantization_grid(X[:, 0], 7, "Median")
    assert len(grid) == 7 and np.all(np.diff(grid) > 0)
    data = tmp_path / "d.tsv"
    np.savetxt(data, np.column_stack([y, X]), delimiter="\t", fmt="%.6g")
    qp = utils.quantize(str(data), border_count=16)
    assert qp.is_quantized() and qp.num_row() == 800
    assert isinstance(utils.get_gpu_device_count(), int)
    onx = utils.convert_to_onnx_object(m)
    assert onx is not None


def test_remaining_public_methods(tmp_path):
    rng = np.random.default_rng(8)
    X = rng.standard_normal((900, 4)).astype(np.float32)
    y = (X[:, 0] - 0.5 * X[:, 2] + 0.2 * rng.standard_normal(900)).astype(np.float32)
    m = cb.CatBoostRegressor(iterations=40, depth=3, learning_rate=0.2, verbose=False, allow_writing_files=False,
                             border_count=12).fit(X[:700], y[:700], eval_set=(X[700:], y[700:]))
    # virtual ensembles: the last one is the whole model; uncertainty columns
    ve = m.virtual_ensembles_predict(X[:50], virtual_ensembles_count=5)
    assert ve.shape == (50, 5, 1)
    np.testing.assert_allclose(ve[:, -1, 0], m.predict(X[:50]), rtol=1e-6, atol=1e-8)
    T = m.tree_count_
    np.testing.assert_allclose(ve[:, 0, 0], m.predict(X[:50], ntree_end=T - 4 * (T // 10)), rtol=1e-6, atol=1e-8)
    tu = m.virtual_ensembles_predict(X[:50], prediction_type="TotalUncertainty", virtual_ensembles_count=5)
    assert tu.shape == (50, 2) and np.all(tu[:, 1] >= 0)
    with pytest.raises(cb.CatBoostError):
        m.virtual_ensembles_predict(X[:5], virtual_ensembles_count=40)
    clf = cb.CatBoostClassifier(iterations=20, depth=3, verbose=False, allow_writing_files=False).fit(X, (y > 0).astype(int))
    cu = clf.virtual_ensembles_predict(X[:30], prediction_type="TotalUncertainty", virtual_ensembles_count=4)
    assert cu.shape == (30, 2) and np.all(cu[:, 1] + 1e-12 >= cu[:, 0])          # total >= data uncertainty
    # evaluation-set predictions, leaf iteration, metadata, names, borders
    np.testing.assert_allclose(m.get_test_eval()[:, 0], m.predict(X[700:]), rtol=1e-6)
    rows = list(m.iterate_leaf_indexes(X[:3]))
    assert len(rows) == 3 and len(rows[0]) == T
    assert m.get_n_features_in() == 4 and m.get_text_feature_indices() == [] and isinstance(m.get_metadata(), dict)
    m.set_feature_names(["a", "b", "c", "d"])
    assert m.feature_names_ == ["a", "b", "c", "d"]
    m.save_borders(str(tmp_path / "borders.tsv"))
    assert len((tmp_path / "borders.tsv").read_text().splitlines()) == sum(len(f.borders) for f in m._model.float_features)
    # leaf values can be replaced as a flat vector
    before = m.predict(X[:20])
    flat = np.concatenate([t.leaf_values.reshape(-1) for t in m._model.trees])
    m.set_leaf_values(flat * 2.0)
    bias = float(np.ravel(m._model.bias)[0])
    np.testing.assert_allclose(m.predict(X[:20]) - bias, 2.0 * (before - bias), rtol=1e-6, atol=1e-8)
    m.set_leaf_values(flat)
    # feature statistics, prediction curves, model comparison, batched metrics
    st = m.calc_feature_statistics(X, y, feature=0)
    nb = len(st["borders"]) + 1
    assert len(st["mean_target"]) == nb and st["objects_per_bin"].sum() == 900
    assert st["predictions_on_varying_feature"][-1] > st["predictions_on_varying_feature"][0]
    pp, fig = m.plot_predictions(X[:10], [0])
    assert fig is None and pp[0].shape == (10, nb)
    m2 = cb.CatBoostRegressor(iterations=T, depth=2, verbose=False, allow_writing_files=False).fit(X[:700], y[:700])
    cmp_ = m.compare(m2, cb.Pool(X[700:], y[700:]), ["RMSE"], eval_period=10)
    assert len(cmp_["RMSE"][0]) == len(cmp_["RMSE"][1]) == len(sorted(set(list(range(0, T, 10)) + [T - 1])))
    calc = m.create_metric_calcer(["RMSE"], eval_period=20)
    calc.add(cb.Pool(X[:400], y[:400]))
    calc.add(cb.Pool(X[400:], y[400:]))
    whole = m.eval_metrics(cb.Pool(X, y), ["RMSE"], eval_period=20)["RMSE"]
    np.testing.assert_allclose(calc.eval_metrics()["RMSE"], whole, rtol=1e-9)
    # pool helpers
    pool = cb.Pool(X, (y > 0).astype(int))
    tr, ev = pool.train_eval_split(is_classification=True, eval_fraction=0.25)
    assert tr.num_row() + ev.num_row() == 900 and abs(ev.num_row() - 225) <= 2
    pool.set_timestamp(np.arange(900)[::-1])
    tr, ev = pool.train_eval_split(has_time=True, eval_fraction=0.1)
    assert ev.num_row() == 90 and np.array_equal(np.asarray(ev.timestamp), np.arange(810, 900)[::-1])


def test_features_data_shrinkage_and_gp_sampling():
    rng = np.random.default_rng(2)
    n = 400
    num = rng.standard_normal((n, 3)).astype(np.float32)
    cat = np.array([[f"c{v}".encode()] for v in rng.integers(0, 4, n)], dtype=object)
    y = (num[:, 0] + (cat[:, 0] == b"c1") * 2.0).astype(np.float32)
    fdata = cb.FeaturesData(num, cat, num_feature_names=["a", "b", "c"], cat_feature_names=["k"])
    assert fdata.get_feature_count() == 4 and fdata.get_feature_names() == ["a", "b", "c", "k"]
    pool = cb.Pool(fdata, y)
    assert pool.get_cat_feature_indices() == [3] and pool.get_feature_names() == ["a", "b", "c", "k"]
    m = cb.CatBoostRegressor(iterations=30, depth=3, learning_rate=0.3, verbose=False, allow_writing_files=False).fit(pool)
    assert np.sqrt(np.mean((m.predict(pool) - y) ** 2)) < 0.5
    assert cb.CatboostError is cb.CatBoostError and cb.EShapCalcType.Exact == "Exact"
    # shrinkage pulls the model towards zero: smaller predictions, and the stored trees reproduce the training cursor
    X = num
    t = (2.0 * X[:, 0]).astype(np.float32)
    kw = dict(iterations=40, depth=3, learning_rate=0.2, verbose=False, allow_writing_files=False, boost_from_average=False,
              bootstrap_type="No", random_strength=0)
    plain = cb.CatBoostRegressor(**kw).fit(X, t)
    shr = cb.CatBoostRegressor(model_shrink_rate=1.0, **kw).fit(X, t)
    assert np.abs(shr.predict(X)).mean() < 0.9 * np.abs(plain.predict(X)).mean()
    res = np.sqrt(np.mean((shr.predict(X) - t) ** 2))
    assert abs(shr.evals_result_["learn"]["RMSE"][-1] - res) < 1e-4
    # posterior samples: close to the data where there is data, different from each other
    models = cb.sample_gaussian_process(X, t, samples=3, posterior_iterations=60, prior_iterations=10, depth=3, sigma=0.5,
                                        random_seed=1)
    assert len(models) == 3
    preds = np.stack([mm.predict(X) for mm in models])
    assert np.sqrt(np.mean((preds.mean(0) - t) ** 2)) < 0.8
    assert np.abs(preds[0] - preds[1]).max() > 1e-3


def test_probability_threshold_is_stored_with_the_model(tmp_path):
    rng = np.random.default_rng(0)
    X = rng.standard_normal((500, 3)).astype(np.float32)
    y = (X[:, 0] > 0).astype(int)
    m = cb.CatBoostClassifier(iterations=20, depth=3, verbose=False, allow_writing_files=False).fit(X, y)
    p = m.predict_proba(X)[:, 1]
    m.set_probability_threshold(0.8)
    assert np.array_equal(np.asarray(m.predict(X)).astype(int).reshape(-1), (p > 0.8).astype(int))
    m.save_model(str(tmp_path / "m.cbm"))
    assert cb.CatBoostClassifier().load_model(str(tmp_path / "m.cbm")).get_probability_threshold() == 0.8
    m.set_probability_threshold(None)
    assert np.array_equal(np.asarray(m.predict(X)).astype(int).reshape(-1), (p > 0.5).astype(int))
    assert len(list(m.staged_predict_log_proba(X[:5], eval_period=10))) == 2


def test_metric_objects():
    from catboost_b200 import metrics
    assert str(metrics.Quantile(alpha=0.3)) == "Quantile:alpha=0.3" and str(metrics.RMSE()) == "RMSE"
    assert metrics.AUC().is_max_optimal() and not metrics.Logloss().is_max_optimal()
    y, a = np.array([0, 1, 1, 0, 1.0]), np.array([-1, 2, 0.5, -0.2, 0.1])
    assert metrics.AUC().eval(y, a) == 1.0
    rng = np.random.default_rng(0)
    X = rng.standard_normal((300, 3)).astype(np.float32)
    t = (X[:, 0] + 0.5 * rng.standard_normal(300) > 0).astype(int)
    m = cb.CatBoostClassifier(iterations=10, depth=2, verbose=False, allow_writing_files=False, eval_metric=metrics.AUC(),
                              custom_metric=[metrics.Accuracy()], use_best_model=False).fit(X, t, eval_set=(X, t))
    assert list(m.evals_result_["validation"]) == ["AUC", "Accuracy", "Logloss"]
    assert len(m.eval_metrics(cb.Pool(X, t), [metrics.F1()], eval_period=5)["F1"]) == 3        # iterations 0, 5, 9


def test_public_tokenizer_and_dictionary(tmp_path):
    from catboost_b200.text_processing import Dictionary, Tokenizer
    tk = Tokenizer(lowercasing=True, separator_type="BySense", token_types=["Word", "Number"])
    assert tk.tokenize("The cat, the CAT and 42 dogs!") == ["the", "cat", "the", "cat", "and", "42", "dogs"]
    toks, kinds = tk.tokenize("a 7", types=True)
    assert kinds == ["Word", "Number"]
    assert Tokenizer(number_process_policy="Replace", number_token="#").tokenize("buy 3 apples") == ["buy", "#", "apples"]
    assert Tokenizer(delimiter=",;", split_by_set=True).tokenize("a,b;;c") == ["a", "b", "c"]
    assert Tokenizer(delimiter=",", skip_empty=False).tokenize("a,,b") == ["a", "", "b"]
    docs = ["the cat sat", "the cat ran", "a dog ran", "the end"]
    d = Dictionary(occurence_lower_bound=2).fit(docs, tk)
    assert d.size == 3 and d.get_top_tokens() == ["the", "cat", "ran"] and d.get_token(0) == "the"
    assert d.apply(docs, tk) == [[0, 1], [0, 1, 2], [2], [0]]
    assert d.apply("the unknown cat", tk, unknown_token_policy="Insert") == [0, d.unknown_token_id, 1]
    assert d.min_unused_token_id == d.unknown_token_id + 2
    bi = Dictionary(gram_order=2, occurence_lower_bound=2).fit(docs, tk)
    assert bi.get_top_tokens() == ["the cat"]
    letters = Dictionary(token_level_type="Letter", occurence_lower_bound=4, end_of_word_policy="Skip").fit(docs, tk)
    assert set(letters.get_top_tokens()) == {"a", "t", "e"}
    d.save(str(tmp_path / "dict.tsv"))
    d2 = Dictionary().load(str(tmp_path / "dict.tsv"))
    assert d2.get_top_tokens() == d.get_top_tokens() and d2.apply(docs, tk) == d.apply(docs, tk)
    with pytest.raises(cb.CatBoostError):
        Dictionary().size


def test_polynomial_view_reproduces_the_model():
    from catboost_b200 import monoforest
    rng = np.random.default_rng(6)
    X = rng.standard_normal((600, 4)).astype(np.float32)
    y = (X[:, 0] * X[:, 1] + X[:, 2]).astype(np.float32)
    m = cb.CatBoostRegressor(iterations=25, depth=3, learning_rate=0.3, verbose=False, allow_writing_files=False,
                             border_count=8).fit(X, y)
    poly = monoforest.to_polynom(m)
    assert poly[0].splits == [] and all(len(mn.splits) <= 3 for mn in poly)
    np.testing.assert_allclose(monoforest.eval_polynom(poly, X)[:, 0], m.predict(X), rtol=1e-6, atol=1e-6)
    # merged monomials: at most one condition per feature, no duplicates
    keys = [tuple((s.feature_idx, s.border) for s in mn.splits) for mn in poly]
    assert len(set(keys)) == len(keys) and all(len({f for f, _ in k}) == len(k) for k in keys)
    assert monoforest.to_polynom_string(m).count(" + ") == len(poly) - 1
    expl = monoforest.explain_features(m)
    assert {e.feature for e in expl} <= {0, 1, 2, 3}
    strength = monoforest.calc_features_strength(m)
    assert strength[3] < min(strength[0], strength[2])             # the noise feature matters least
    xs, ys = expl[0].calc_pdp()
    assert len(ys) == len(xs) + 1
    mc = cb.CatBoostClassifier(iterations=8, depth=2, loss_function="MultiClass", verbose=False,
                               allow_writing_files=False).fit(X, np.digitize(X[:, 0], [-0.5, 0.5]))
    pm = monoforest.to_polynom(mc)
    np.testing.assert_allclose(monoforest.eval_polynom(pm, X), mc.predict(X, prediction_type="RawFormulaVal"), rtol=1e-6,
                               atol=1e-6)
    dw = cb.CatBoostRegressor(iterations=3, depth=2, grow_policy="Depthwise", verbose=False, allow_writing_files=False).fit(X, y)
    with pytest.raises(cb.CatBoostError):
        monoforest.to_polynom(dw)


def _pb_fields(buf):
    """Generic protobuf wire decoding: list of (field number, wire type, value)."""
    import struct
    out, pos = [], 0
    while pos < len(buf):
        key, shift = 0, 0
        while True:
            b = buf[pos]; pos += 1
            key |= (b & 0x7F) << shift; shift += 7
            if not b & 0x80:
                break
        field, wire = key >> 3, key & 7
        if wire == 0:
            v, shift = 0, 0
            while True:
                b = buf[pos]; pos += 1
                v |= (b & 0x7F) << shift; shift += 7
                if not b & 0x80:
                    break
        elif wire == 1:
            v = struct.unpack_from("<d", buf, pos)[0]; pos += 8
        elif wire == 2:
            ln, shift = 0, 0
            while True:
                b = buf[pos]; pos += 1
                ln |= (b & 0x7F) << shift; shift += 7
                if not b & 0x80:
                    break
            v = buf[pos:pos + ln]; pos += ln
        elif wire == 5:
            v = struct.unpack_from("<f", buf, pos)[0]; pos += 4
        else:
            raise AssertionError("unexpected wire type")
        out.append((field, wire, v))
    return out


def test_coreml_export_decodes_to_the_same_trees(tmp_path):
    rng = np.random.default_rng(9)
    X = rng.standard_normal((500, 4)).astype(np.float32)
    y = (X[:, 0] - X[:, 3] > 0).astype(int)
    m = cb.CatBoostClassifier(iterations=12, depth=3, verbose=False, allow_writing_files=False).fit(X, y)
    path = tmp_path / "m.mlmodel"
    m.save_model(str(path), format="coreml", export_parameters={"prediction_type": "probability"})
    top = _pb_fields(path.read_bytes())
    assert [f for f, _, _ in top] == [1, 2, 302] and top[0][2] == 1
    desc = _pb_fields(top[1][2])
    names = [_pb_fields(v)[0][2].decode() for f, _, v in desc if f == 1]
    assert names == ["0", "1", "2", "3"]
    assert [v for f, _, v in desc if f == 11][0] == b"prediction"
    reg = _pb_fields(top[2][2])
    assert [v for f, _, v in reg if f == 2] == [2]                       # logistic transform
    ens = _pb_fields([v for f, _, v in reg if f == 1][0])
    import struct
    base = struct.unpack("<d", [v for f, _, v in ens if f == 3][0])[0]
    nodes = {}
    for f, _, v in ens:
        if f == 1:
            d = {}
            for ff, _, vv in _pb_fields(v):
                d.setdefault(ff, []).append(vv)
            nodes[(d.get(1, [0])[0], d.get(2, [0])[0])] = d
    # evaluate the decoded ensemble on a few rows
    for row in X[:25]:
        total = base
        for t in range(12):
            node = 0
            while True:
                d = nodes[(t, node)]
                if d[3][0] == 6:
                    total += _pb_fields(d[20][0])[-1][2]
                    break
                assert d[3][0] == 3
                go = row[d.get(10, [0])[0]] > d[11][0]
                node = d.get(12, [0])[0] if go else d.get(13, [0])[0]
        want = m.predict(row.reshape(1, -1), prediction_type="RawFormulaVal")[0]
        assert abs(total - want) < 1e-6
    with pytest.raises(cb.CatBoostError):
        cb.CatBoostRegressor(iterations=2, depth=2, verbose=False, allow_writing_files=False).fit(X, y.astype(float)) \
            .save_model(str(path), format="coreml", export_parameters={"prediction_type": "probability"})


def test_model_file_cannot_run_code_on_load(tmp_path):
    """A .cbm whose text/embedding block was replaced by a pickle (or names a foreign class) is rejected and nothing
    from it is executed; the plain-data container round-trips the values it is meant for."""
    import base64
    import pickle
    from catboost_b200.data.pool import CatBoostError
    from catboost_b200.models import io as mio
    from catboost_b200.utils import plainser

    state = {"a": [1, 2.5, "x", None, True], "t": (np.arange(6, dtype=np.int32).reshape(2, 3), b"raw"),
             ("k", 1): np.float32(3.5)}
    back = plainser.loads(plainser.dumps(state))
    assert back["a"] == state["a"] and back["t"][1] == b"raw" and back[("k", 1)] == 3.5
    assert back["t"][0].dtype == np.int32 and np.array_equal(back["t"][0], state["t"][0])
    with pytest.raises(plainser.PlainDataError):
        plainser.loads(plainser.dumps(state)[:-3])

    rng = np.random.default_rng(0)
    X = rng.standard_normal((300, 3)).astype(np.float32)
    y = (X[:, 0] > 0).astype(int)
    m = cb.CatBoostClassifier(iterations=3, depth=2, verbose=False, allow_writing_files=False).fit(X, y)
    marker = tmp_path / "executed"

    class Evil:
        def __reduce__(self):
            return (open, (str(marker), "w"))

    for payload in (pickle.dumps(Evil()), plainser.dumps([1]).replace(b"\x07", b"\x0b", 1) + b"\x04\x00\x00\x00Evil"):
        m._model.info["catboost_b200_estimators"] = base64.b64encode(payload).decode("ascii")
        blob = mio.model_to_cbm_bytes(m._model)
        with pytest.raises(CatBoostError):
            mio.model_from_cbm_bytes(blob)
        assert not marker.exists()


def test_cli_run_worker_and_model_based_eval(tmp_path):
    """Two `run-worker` processes train one model over a gloo group (the multi-host CPU path on one machine), and
    `model-based-eval` compares continuations of a baseline with and without a feature set."""
    import json
    import socket
    rng = np.random.default_rng(0)
    n = 3000
    X = rng.standard_normal((n, 5))
    y = (X[:, 0] + 0.5 * X[:, 1] > 0).astype(int)
    train = tmp_path / "train.tsv"
    with open(train, "w") as fh:
        for i in range(n):
            fh.write("\t".join([str(y[i])] + [f"{v:.6f}" for v in X[i]]) + "\n")
    cd = tmp_path / "train.cd"
    cd.write_text("0\tLabel\n")
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, PYTHONPATH=ROOT)
    model = tmp_path / "dist.bin"
    procs = []
    for r in range(2):
        cmd = [sys.executable, "-m", "catboost_b200", "run-worker", "--rank", str(r), "--world-size", "2", "--master-addr",
               "127.0.0.1", "--master-port", str(port), "--", "-f", str(train), "--cd", str(cd), "-m", str(model),
               "--loss-function", "Logloss", "-i", "15", "--verbose", "0", "--train-dir", str(tmp_path / f"info{r}")]
        procs.append(subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env, cwd=str(tmp_path)))
    for p in procs:
        out, err = p.communicate(timeout=300)
        assert p.returncode == 0, err[-2000:]
    m = cb.CatBoostClassifier().load_model(str(model))
    assert m.tree_count_ == 15
    assert float((m.predict(X.astype(np.float32)) == y).mean()) > 0.9
    out_json = tmp_path / "mbe.json"
    r = subprocess.run([sys.executable, "-m", "catboost_b200", "model-based-eval", "-f", str(train), "--cd", str(cd),
                        "--baseline-model", str(model), "--offset", "5", "--experiment-size", "10",
                        "--features-to-evaluate", "0;3,4", "-o", str(out_json)],
                       capture_output=True, text=True, env=env, cwd=str(tmp_path))
    assert r.returncode == 0, r.stderr[-2000:]
    rep = json.loads(out_json.read_text())
    assert len(rep) == 2 and rep[0]["features"] == [0]
    # the informative feature matters (lower Logloss with it), the noise features hardly do
    assert rep[0]["delta"] < -0.01 and abs(rep[1]["delta"]) < abs(rep[0]["delta"])


def test_diff_tools_and_model_comparator(tmp_path):
    """Tolerant comparison of delimiter-separated files, JSON, numpy files and models, and the apply-speed tool."""
    import json
    from catboost_b200 import difftools as dt
    a, b = tmp_path / "a.tsv", tmp_path / "b.tsv"
    a.write_text("id\tv\nx\t1.000000\ny\t2.5\n")
    b.write_text("id\tv\nx\t1.000001\ny\t2.5\n")
    assert dt.dsv_diff(str(a), str(b), diff_limit=0.0, have_header=True)
    assert not dt.dsv_diff(str(a), str(b), diff_limit=1e-5, have_header=True)
    assert not dt.json_diff({"a": [1.0, {"b": 2}], "t": "x"}, {"a": [1.0 + 1e-9, {"b": 2}], "t": "x"}, 1e-6)
    assert dt.json_diff({"a": 1}, {"a": 1, "c": 2}, 1e-6) and not dt.json_diff({"a": 1}, {"a": 1, "c": 2}, 0, ignore_keys=("c",))
    np.save(tmp_path / "x.npy", np.arange(6.0).reshape(2, 3))
    np.save(tmp_path / "y.npy", np.arange(6.0).reshape(2, 3) + 1e-9)
    assert not dt.numpy_diff(str(tmp_path / "x.npy"), str(tmp_path / "y.npy"), 1e-6)
    assert dt.numpy_diff(str(tmp_path / "x.npy"), str(tmp_path / "y.npy"), 0.0)
    rng = np.random.default_rng(0)
    X = rng.standard_normal((600, 4)).astype(np.float32)
    y = (X[:, 0] > 0).astype(int)
    m1 = cb.CatBoostClassifier(iterations=6, depth=3, verbose=False, allow_writing_files=False, random_seed=1).fit(X, y)
    m2 = cb.CatBoostClassifier(iterations=6, depth=3, verbose=False, allow_writing_files=False, random_seed=1).fit(X, y)
    m3 = cb.CatBoostClassifier(iterations=6, depth=3, verbose=False, allow_writing_files=False, random_seed=2,
                               learning_rate=0.5).fit(X, y)
    assert not dt.compare_models(m1._model, m2._model, 1e-9)
    assert dt.compare_models(m1._model, m3._model, 1e-9)
    p1, p3 = tmp_path / "m1.cbm", tmp_path / "m3.cbm"
    m1.save_model(str(p1)); m3.save_model(str(p3))
    env = dict(os.environ, PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-m", "catboost_b200", "compare-models", str(p1), str(p1)], capture_output=True, text=True, env=env)
    assert r.returncode == 0 and "EQUAL" in r.stdout
    r = subprocess.run([sys.executable, "-m", "catboost_b200", "compare-models", str(p1), str(p3)], capture_output=True, text=True, env=env)
    assert r.returncode == 1 and "DIFFER" in r.stdout
    perf = dt.model_perftest(m1, rows=2000, repeats=1)
    assert perf["rows_per_second"] > 0 and perf["trees"] == 6


def test_additional_metrics_against_independent_implementations():
    from sklearn.metrics import average_precision_score, cohen_kappa_score, fbeta_score
    from catboost_b200.metrics import make_metric
    rng = np.random.default_rng(0)
    n = 800
    a = rng.standard_normal(n)
    y = (a + rng.standard_normal(n) > 0).astype(float)
    pred = (a > 0).astype(int)
    assert abs(make_metric("F:beta=2").eval(a, y) - fbeta_score(y, pred, beta=2)) < 1e-12
    assert abs(make_metric("WKappa").eval(a, y) - cohen_kappa_score(y.astype(int), pred, weights="quadratic")) < 1e-12
    assert abs(make_metric("PRAUC").eval(a, y) - average_precision_score(y, a)) < 0.01
    yy = np.abs(rng.standard_normal(n)) + 0.5
    assert abs(make_metric("RMSPE").eval(a, yy) - np.sqrt(np.mean(((yy - a) / yy) ** 2))) < 1e-12
    p = 1 / (1 + np.exp(-a))
    pt = np.where(y > 0.5, p, 1 - p)
    at = np.where(y > 0.5, 0.25, 0.75)
    assert abs(make_metric("Focal").eval(a, y) - np.mean(-at * (1 - pt) ** 2 * np.log(pt))) < 1e-12
    off = np.arange(0, n + 1, 8)
    assert 0.0 <= make_metric("ERR").eval(a, np.clip(y, 0, 1), group_offsets=off) <= 1.0
    assert make_metric("QueryAverage:top=2").eval(a, y, group_offsets=off) >= make_metric("QueryAverage:top=8").eval(a, y, group_offsets=off) - 1e-9
    # Cox: shifting all scores by a constant leaves the partial likelihood unchanged
    t = np.where(rng.random(n) < 0.7, 1, -1) * (rng.random(n) + 0.1)
    assert abs(make_metric("Cox").eval(a, t) - make_metric("Cox").eval(a + 3.0, t)) < 1e-6


def test_quantized_pool_file_round_trip(tmp_path):
    """A quantized pool written to disk (one byte per value + the border grids) trains the same model as the original."""
    rng = np.random.default_rng(5)
    X = rng.standard_normal((3000, 24)).astype(np.float32)
    X[rng.random(X.shape) < 0.03] = np.nan
    y = (np.nan_to_num(X[:, 0]) + np.nan_to_num(X[:, 1]) ** 2 > 0.5).astype(int)
    pool = cb.Pool(X, y)
    pool.quantize(border_count=32)
    path = str(tmp_path / "pool.bin")
    pool.save(path)
    assert os.path.getsize(path) < X.nbytes // 2                # a byte per value, not a float
    back = cb.Pool("quantized://" + path)
    assert back.is_quantized() and back.num_row() == 3000
    kw = dict(iterations=15, depth=4, learning_rate=0.3, verbose=False, allow_writing_files=False, border_count=32)
    a = cb.CatBoostClassifier(**kw).fit(pool)
    b = cb.CatBoostClassifier(**kw).fit(back)
    assert [(s.feature, s.border) for s in a._model.splits] == [(s.feature, s.border) for s in b._model.splits]
    assert np.allclose(a.predict(X, prediction_type="RawFormulaVal"), b.predict(X, prediction_type="RawFormulaVal"))


def test_carry_model_fixes_features():
    from catboost_b200.models.ops import carry_model
    rng = np.random.default_rng(2)
    X = rng.standard_normal((1500, 5)).astype(np.float32)
    y = X[:, 0] + X[:, 1] * X[:, 2] + 0.1 * rng.standard_normal(1500)
    m = cb.CatBoostRegressor(iterations=20, depth=4, learning_rate=0.3, verbose=False, allow_writing_files=False).fit(X, y)
    carried = carry_model(m._model, {1: 0.7, 4: -0.2})
    Xf = X.copy()
    Xf[:, 1], Xf[:, 4] = 0.7, -0.2
    ref = m._model.predict_raw(Xf)
    Xg = X.copy()
    Xg[:, 1], Xg[:, 4] = rng.standard_normal(1500), 99.0          # the carried model ignores these columns
    assert np.allclose(carried.predict_raw(Xg), ref)
    assert sum(len(t.splits) for t in carried.trees) < sum(len(t.splits) for t in m._model.trees)


def test_sage_values_rank_the_informative_features():
    """SAGE: the loss rises most when the features the target depends on are replaced by marginal draws; a noise column
    gets a value near zero (catboost/libs/fstr/sage_values.cpp)."""
    import catboost_b200 as cb
    rng = np.random.default_rng(4)
    n = 3000
    X = rng.standard_normal((n, 5)).astype(np.float32)
    y = (2.0 * X[:, 1] + 0.7 * X[:, 3] + 0.2 * rng.standard_normal(n)).astype(np.float32)
    m = cb.CatBoostRegressor(iterations=60, depth=4, learning_rate=0.3, verbose=False, allow_writing_files=False)
    m.fit(X, y)
    sage = m.get_feature_importance(cb.Pool(X, y), type="SageValues")
    assert sage.shape == (5,)
    assert int(np.argmax(sage)) == 1 and sage[1] > sage[3] > max(sage[0], sage[2], sage[4])
    assert abs(sage[0]) < 0.1 * sage[1]


def test_bpe_dictionary(tmp_path):
    """Byte-pair encoding over letters: the most frequent neighbouring pair becomes a unit, repeatedly; applying the
    dictionary replays the merges in the order they were learned; two files round-trip."""
    from catboost_b200.text_processing import Dictionary, Tokenizer
    corpus = ["low low low low low", "lower lower", "newest newest newest newest newest newest", "widest widest widest"]
    d = Dictionary(token_level_type="Letter", occurence_lower_bound=1, dictionary_type="Bpe", num_bpe_units=6)
    d.fit(corpus, Tokenizer(lowercasing=True))
    base = d.size - 6
    assert base == len(set("".join(corpus).replace(" ", ""))) + 1          # letters + the end-of-word mark
    new_units = d.get_top_tokens()[base:]
    assert new_units[0] in ("es", "st", "we", "lo", "ow", "w ")               # a frequent pair first
    assert any(len(u) >= 3 for u in new_units)                                  # merges build on merges
    ids = d.apply(["newest lowest"], Tokenizer(lowercasing=True))[0]
    plain = Dictionary(token_level_type="Letter", occurence_lower_bound=1).fit(corpus, Tokenizer(lowercasing=True))
    assert len(ids) < len(plain.apply(["newest lowest"], Tokenizer(lowercasing=True))[0])
    assert "".join(d.get_tokens(ids)) == "newest lowest "
    f1, f2 = str(tmp_path / "dict.tsv"), str(tmp_path / "bpe.tsv")
    d.save(f1, f2)
    d2 = Dictionary().load(f1, f2)
    assert d2.apply(["newest lowest"], Tokenizer(lowercasing=True))[0] == ids
    # a run of equal letters: pairs are replaced left to right without overlap
    r = Dictionary(token_level_type="Letter", occurence_lower_bound=1, dictionary_type="Bpe", num_bpe_units=1,
                   end_of_word_policy="Skip").fit(["aaaaa aaaa"], Tokenizer())
    assert [r.get_token(i) for i in r.apply(["aaaaa"], Tokenizer())[0]] == ["aa", "aa", "a"]


def test_text_features_with_dictionaries_and_tokenizers(tmp_path):
    """`dictionaries` (word + bi-gram), `tokenizers` and `feature_calcers`: every dictionary yields its own block of
    features; a signal that only a word pair carries is found through the bi-gram dictionary; the model file round-trips."""
    import catboost_b200 as cb
    rng = np.random.default_rng(8)
    words = ["red", "green", "blue", "cat", "dog", "bird", "big", "small"]
    n = 1500
    docs, y = [], []
    for _ in range(n):
        w = list(rng.choice(words, size=6))
        lab = int(rng.random() < 0.5)
        if lab:                                  # the label is carried by the ordered pair "big dog" only
            k = int(rng.integers(0, 5))
            w[k], w[k + 1] = "big", "dog"
        else:
            w = [t for t in w if t != "dog"] + ["dog", "big"]
        docs.append(" ".join(w))
        y.append(lab)
    X = np.empty((n, 2), dtype=object)
    X[:, 0] = rng.standard_normal(n)
    X[:, 1] = docs
    y = np.asarray(y, dtype=np.float32)
    kw = dict(iterations=40, depth=4, learning_rate=0.3, verbose=False, allow_writing_files=False)
    uni = cb.CatBoostClassifier(dictionaries=["Word:gram_order=1,occurrence_lower_bound=1"], feature_calcers=["BoW"], **kw)
    uni.fit(X[:1200], y[:1200], text_features=[1])
    both = cb.CatBoostClassifier(
        tokenizers=[{"tokenizer_id": "Space", "separator_type": "ByDelimiter", "delimiter": " ", "lowercasing": "true"}],
        dictionaries=["Word:gram_order=1,occurrence_lower_bound=1", {"dictionary_id": "BiGram", "gram_order": "2",
                                                                      "occurrence_lower_bound": "1"}],
        feature_calcers=["BoW:top_tokens_count=200"], **kw)
    both.fit(X[:1200], y[:1200], text_features=[1])
    acc_uni = float((uni.predict(X[1200:]) == y[1200:]).mean())
    acc_both = float((both.predict(X[1200:]) == y[1200:]).mean())
    assert acc_both > 0.95 and acc_both > acc_uni + 0.1, (acc_uni, acc_both)
    path = str(tmp_path / "text.cbm")
    both.save_model(path)
    again = cb.CatBoostClassifier().load_model(path)
    assert np.allclose(again.predict(X[1200:], prediction_type="RawFormulaVal"),
                       both.predict(X[1200:], prediction_type="RawFormulaVal"))


def test_reference_boston_and_mushroom_models():
    """The reference's own acceptance criteria for two of its model files
    (catboost/dotnet/CatBoostNetTests/CatBoostModelEvaluatorTest.cs:46-131): the boston model (numerical features)
    predicts log(target) within 0.4 on all but at most 7 rows; the mushroom model (categorical features only, so every
    prediction goes through the CTR tables stored in the file: hashes, priors, shifts, scales, target borders) puts
    every one of the 8124 rows in its class."""
    bed = os.path.join(REF, "catboost/dotnet/CatBoostNetTests/testbed")
    if not os.path.exists(bed):
        pytest.skip("reference model files are not available")
    rows = [l.split() for l in open(os.path.join(bed, "boston", "housing.data")) if l.strip()]
    X = np.array([[float(v) for v in r[:-1]] for r in rows], dtype=np.float32)
    target = np.array([float(r[-1]) for r in rows])
    m = cb.CatBoostRegressor().load_model(os.path.join(bed, "boston", "boston_housing_model.cbm"))
    pred = np.asarray(m.predict(X), dtype=float)
    assert int((np.abs(pred - np.log(target)) >= 0.4).sum()) <= 7
    rows = [l.strip().split(",") for l in open(os.path.join(bed, "mushrooms", "mushrooms.csv")) if l.strip()]
    labels = np.array([r[0] for r in rows])
    data = np.array([r[1:] for r in rows], dtype=object)
    m = cb.CatBoostClassifier().load_model(os.path.join(bed, "mushrooms", "mushroom_model.cbm"))
    raw = np.asarray(m.predict(cb.Pool(data, cat_features=list(range(data.shape[1]))), prediction_type="RawFormulaVal"), dtype=float)
    got = np.where(raw > 0, "p", "e")
    assert (got == labels).all(), int((got != labels).sum())


def test_carry_and_uplift():
    """catboost.carry: a model with float features fixed reads them no more; lists of values give one output dimension
    each; uplift is the difference between two fixings.  By flat index and by name."""
    from catboost_b200.carry import carry, uplift
    rng = np.random.default_rng(0)
    X = rng.standard_normal((2500, 5)).astype(np.float32)
    y = (2 * X[:, 1] + X[:, 3] * X[:, 1] + 0.1 * rng.standard_normal(2500)).astype(np.float32)
    m = cb.CatBoostRegressor(iterations=40, depth=4, learning_rate=0.3, verbose=False, allow_writing_files=False)
    m.fit(cb.Pool(X, y, feature_names=["a", "b", "c", "d", "e"]))
    fixed = X.copy()
    fixed[:, 1] = 0.5
    assert np.allclose(carry(m, {1: 0.5}).predict(X), m.predict(fixed))
    assert np.allclose(carry(m, {"b": 0.5}).predict(X), m.predict(fixed))
    p = carry(m, {1: [0.5, -1.0], 3: [0.0, 2.0]}).predict(X, prediction_type="RawFormulaVal")
    assert p.shape == (2500, 2)
    for j, (v1, v3) in enumerate([(0.5, 0.0), (-1.0, 2.0)]):
        fixed[:, 1], fixed[:, 3] = v1, v3
        assert np.allclose(p[:, j], m.predict(fixed))
    lo, hi = X.copy(), X.copy()
    lo[:, 1], hi[:, 1] = 0.0, 1.0
    assert np.allclose(uplift(m, {"b": (0.0, 1.0)}).predict(X), m.predict(hi) - m.predict(lo), atol=1e-9)
    with pytest.raises(cb.CatBoostError):
        carry(m, {1: [1.0, 2.0], 3: [1.0]})


# ---- survival, focal, multi-quantile and group-quantile objectives -----------------------------------------------
def _autograd_check(obj, approx, target, neg_loglik, tol=2e-4):
    """der of the objective = -d(loss)/d(approx), hess = d2(loss)/d(approx)^2 on the diagonal."""
    import torch
    a = approx.clone().double().requires_grad_(True)
    loss = neg_loglik(a)
    g, = torch.autograd.grad(loss, a, create_graph=True)
    der, hess = obj.der_hess(approx.float().unsqueeze(0), target, None)
    assert torch.allclose(der[0].double(), -g.detach(), atol=tol, rtol=1e-3)
    h = torch.stack([torch.autograd.grad(g[i], a, retain_graph=True)[0][i] for i in range(len(a))])
    assert torch.allclose(hess[0].double(), h.clamp_min(1e-16), atol=tol, rtol=1e-3)


def test_focal_derivatives_match_autograd():
    import torch
    from catboost_b200.train.objectives import make_objective
    torch.manual_seed(0)
    a = torch.randn(40)
    y = (torch.rand(40) > 0.5).float()
    obj = make_objective("Focal", {"focal_alpha": 0.3, "focal_gamma": 1.5})

    def loss(x):
        p = torch.sigmoid(x)
        pt = torch.where(y > 0.5, p, 1 - p)
        at = torch.where(y > 0.5, torch.tensor(0.3, dtype=x.dtype), torch.tensor(0.7, dtype=x.dtype))
        return (-at * (1 - pt) ** 1.5 * torch.log(pt)).sum()

    x = a.clone().double().requires_grad_(True)
    gr, = torch.autograd.grad(loss(x), x)
    der, _ = obj.der_hess(a.unsqueeze(0), y, None)
    assert torch.allclose(der[0].double(), -gr, atol=1e-5)


def test_cox_derivatives_match_autograd():
    import torch
    from catboost_b200.train.objectives import make_objective
    torch.manual_seed(1)
    n = 30
    a = torch.randn(n)
    t = (torch.rand(n) * 10 + 0.1) * torch.where(torch.rand(n) < 0.3, -1.0, 1.0)
    obj = make_objective("Cox", {})

    def nll(x):
        order = torch.sort(t.abs(), stable=True).indices
        xs = x[order]
        lse = torch.flip(torch.logcumsumexp(torch.flip(xs, [0]), 0), [0])
        return -((xs - lse) * (t[order] > 0).double()).sum()

    _autograd_check(obj, a, t, nll)
    # the value reported by the objective is the same negative log-likelihood
    assert abs(obj.value(a.unsqueeze(0), t, None) - float(nll(a.double()))) < 1e-6


@pytest.mark.parametrize("dist", ["Normal", "Logistic", "Extreme"])
def test_survival_aft_derivatives_match_autograd(dist):
    import torch
    from catboost_b200.train.objectives import make_objective
    torch.manual_seed(2)
    n = 24
    a = torch.randn(n) * 0.5
    lo = torch.rand(n) * 3 + 0.2
    up = lo + torch.rand(n) * 2 + 0.1
    up[:8] = lo[:8]                      # observed
    up[8:12] = -1.0                      # right-censored
    lo[12:16] = -1.0                     # left-censored
    target = torch.stack([lo, up])
    s = 0.8
    obj = make_objective("SurvivalAft", {"dist": dist, "scale": s})

    def cdf(z):
        if dist == "Normal":
            return 0.5 + 0.5 * torch.erf(z / 2 ** 0.5)
        if dist == "Logistic":
            return torch.sigmoid(z)
        return 1 - torch.exp(-torch.exp(z))

    def logpdf(z):
        if dist == "Normal":
            return -0.5 * z * z
        if dist == "Logistic":
            return z - 2 * torch.log1p(torch.exp(z))
        return z - torch.exp(z)

    def nll(x):
        lod, upd = lo.double(), up.double()
        zl = (torch.log(lod.clamp_min(1e-30)) - x) / s
        zu = (torch.log(upd.clamp_min(1e-30)) - x) / s
        cu = torch.where(upd == -1, torch.ones_like(x), cdf(zu))
        cl = torch.where(lod == -1, torch.zeros_like(x), cdf(zl))
        ll = torch.where(lod == upd, logpdf(zl), torch.log((cu - cl).clamp_min(1e-300)))
        return -ll.sum()

    _autograd_check(obj, a, target, nll, tol=5e-4)


def test_survival_and_quantile_objectives_learn():
    rng = np.random.default_rng(5)
    n = 600
    X = rng.normal(size=(n, 5)).astype(np.float32)
    risk = X[:, 0] - 0.5 * X[:, 1]
    # Cox: larger risk -> earlier event; 25 % censored
    time = rng.exponential(np.exp(-risk)) + 0.01
    y = np.where(rng.random(n) < 0.25, -time, time).astype(np.float32)
    m = cb.CatBoostRegressor(iterations=40, depth=3, learning_rate=0.2, loss_function="Cox", verbose=0).fit(X, y)
    ll = m.evals_result_["learn"]["Cox"]
    assert ll[-1] > ll[0]                                  # the partial log-likelihood grows
    assert np.corrcoef(m.predict(X), risk)[0, 1] > 0.7
    # SurvivalAft: log time = signal + noise, a third right-censored, a third interval-censored
    t = np.exp(1.0 + 0.8 * X[:, 0] + 0.2 * rng.normal(size=n))
    lo, up = t.copy(), t.copy()
    up[: n // 3] = -1
    lo[: n // 3] *= 0.7
    lo[n // 3: 2 * n // 3] *= 0.8
    up[n // 3: 2 * n // 3] *= 1.2
    ya = np.stack([lo, up], 1).astype(np.float32)
    m = cb.CatBoostRegressor(iterations=60, depth=3, learning_rate=0.2, loss_function="SurvivalAft:dist=Normal;scale=0.5",
                             verbose=0).fit(X, ya)
    v = list(m.evals_result_["learn"].values())[0]
    assert v[-1] < 0.5 * v[0]
    assert np.corrcoef(m.predict(X), np.log(t))[0, 1] > 0.9
    assert np.allclose(m.predict(X, prediction_type="Exponent"), np.exp(m.predict(X)))
    # MultiQuantile: one column per level, ordered on average, each close to its own coverage
    yq = (X[:, 0] + rng.normal(size=n)).astype(np.float32)
    m = cb.CatBoostRegressor(iterations=80, depth=3, learning_rate=0.2, loss_function="MultiQuantile:alpha=0.1,0.5,0.9",
                             verbose=0).fit(X, yq)
    pr = m.predict(X)
    assert pr.shape == (n, 3)
    cover = [(yq <= pr[:, k]).mean() for k in range(3)]
    assert abs(cover[0] - 0.1) < 0.06 and abs(cover[1] - 0.5) < 0.08 and abs(cover[2] - 0.9) < 0.06
    # Focal and GroupQuantile
    yb = (risk + 0.3 * rng.normal(size=n) > 0).astype(np.float32)
    m = cb.CatBoostClassifier(iterations=40, depth=3, loss_function="Focal:focal_alpha=0.5;focal_gamma=2", verbose=0).fit(X, yb)
    assert (m.predict(X).astype(np.float32) == yb).mean() > 0.85
    assert m.predict_proba(X).shape == (n, 2)
    gid = np.repeat(np.arange(n // 10), 10)
    m = cb.CatBoostRanker(iterations=30, depth=3, loss_function="GroupQuantile:alpha=0.5", verbose=0).fit(X, yq, group_id=gid)
    v = list(m.evals_result_["learn"].values())[0]
    assert v[-1] < v[0]
    # StochasticFilter: relevant documents are worth 1, keeping an irrelevant one costs 0.5
    rel = (X[:, 0] + 0.3 * rng.normal(size=n) > 0.3)
    yf = np.where(rel, 1.0, -0.5).astype(np.float32)
    m = cb.CatBoostRanker(iterations=40, depth=3, learning_rate=0.3, verbose=0,
                          loss_function="StochasticFilter:sigma=1;num_estimations=5").fit(X, yf, group_id=gid)
    p = m.predict(X)
    assert (p[rel] > 0).mean() > 0.7 and (p[~rel] > 0).mean() < 0.2


def test_feature_penalties_and_per_level_sampling():
    rng = np.random.default_rng(11)
    n = 1500
    X = rng.normal(size=(n, 5)).astype(np.float32)
    X[:, 1] = X[:, 0] + 0.05 * rng.normal(size=n).astype(np.float32)         # a near copy of feature 0
    y = (X[:, 0] + 0.5 * X[:, 2] + 0.1 * rng.normal(size=n)).astype(np.float32)

    def used(model):
        imp = model.get_feature_importance()
        return set(int(i) for i in np.nonzero(np.asarray(imp) > 0)[0])

    kw = dict(iterations=15, depth=3, learning_rate=0.3, verbose=0, bootstrap_type="No", random_strength=0)
    base = cb.CatBoostRegressor(**kw).fit(X, y)
    assert 0 in used(base)
    # a large first-use penalty on feature 0 sends the trees to its near copy instead
    pen = cb.CatBoostRegressor(first_feature_use_penalties={0: 1e9}, **kw).fit(X, y)
    assert 0 not in used(pen) and 1 in used(pen)
    # the coefficient scales the penalty: zero switches it off again
    off = cb.CatBoostRegressor(first_feature_use_penalties="0:1e9", penalties_coefficient=0.0, **kw).fit(X, y)
    assert np.allclose(off.predict(X), base.predict(X))
    # per-object penalties, symmetric and non-symmetric trees
    for gp in ("SymmetricTree", "Depthwise", "Lossguide"):
        m = cb.CatBoostRegressor(per_object_feature_penalties=[1e6, 0, 0, 0, 0], grow_policy=gp, **kw).fit(X, y)
        assert 0 not in used(m), gp
    # a small penalty is paid once: after its first use the feature competes without it
    small = cb.CatBoostRegressor(first_feature_use_penalties={0: 1e-6}, **kw).fit(X, y)
    assert 0 in used(small)
    # bootstrap weights redrawn at every level: a different model than one draw per tree, same quality
    kw2 = dict(iterations=30, depth=4, learning_rate=0.2, verbose=0, bootstrap_type="Bernoulli", subsample=0.5, random_seed=3)
    a = cb.CatBoostRegressor(**kw2).fit(X, y)
    for gp in ("SymmetricTree", "Depthwise", "Lossguide"):
        b = cb.CatBoostRegressor(sampling_frequency="PerTreeLevel", grow_policy=gp, **kw2).fit(X, y)
        rm = float(np.sqrt(np.mean((b.predict(X) - y) ** 2)))
        assert rm < 0.35, (gp, rm)
    b = cb.CatBoostRegressor(sampling_frequency="PerTreeLevel", **kw2).fit(X, y)
    assert not np.allclose(a.predict(X), b.predict(X))


def test_eval_package_and_dataset_cache(tmp_path):
    from catboost_b200 import datasets
    from catboost_b200.eval import (CatboostEvaluation, EvalType, ExecutionCase, ScoreType, calc_bootstrap_ci_for_mean,
                                    calc_wilcoxon_test)
    rng = np.random.default_rng(0)
    n = 2400
    X = rng.normal(size=(n, 5)).astype(np.float32)
    y = (X[:, 0] + 0.7 * X[:, 1] + 0.3 * rng.normal(size=n) > 0).astype(int)
    # the same data as a file with a column description
    path, cd = tmp_path / "data.tsv", tmp_path / "cd.tsv"
    with open(path, "w") as fh:
        for i in range(n):
            fh.write(str(y[i]) + "\t" + "\t".join(f"{v:.6g}" for v in X[i]) + "\n")
    cd.write_text("0\tLabel\n")
    ev = CatboostEvaluation(str(path), fold_size=400, fold_count=6, column_description=str(cd))
    params = {"iterations": 20, "depth": 3, "loss_function": "Logloss", "learning_rate": 0.3}
    res = ev.eval_features(params, [0, 4], eval_type=EvalType.SeqAddAndAll, eval_metrics=["AUC"], eval_step=5)
    assert set(res.get_metrics()) == {"AUC", "Logloss"}
    mr = res.get_metric_results("Logloss")
    assert len(mr.get_fold_ids()) == 6 and len(mr.get_cases()) == 4
    table = mr.get_baseline_comparison(ScoreType.Rel)
    # bringing the informative feature back helps by far more than the noise feature
    assert table.loc["Features: 0", "Score"] > 20 and abs(table.loc["Features: 4", "Score"]) < 5
    assert table.loc["Features: 0", "PValue"] < 0.05
    assert res.get_metric_results("AUC").get_baseline_comparison(ScoreType.Abs).loc["Features: 0", "Score"] > 0.05
    curve = mr.get_case_result(mr.get_baseline_case()).get_fold_curve(0)
    assert len(curve) == 5                                            # iterations 0, 5, 10, 15 and the last one
    # two configurations compared directly
    short = ExecutionCase(dict(params, iterations=5), label="short")
    long_ = ExecutionCase(dict(params, iterations=40), label="long")
    cmp_ = ev.eval_cases(short, [long_], ["Logloss"]).get_metric_results("Logloss").get_baseline_comparison()
    assert cmp_.loc["long", "Score"] > 0
    with pytest.raises(cb.CatBoostError):
        ev.eval_cases(short, [short], ["Logloss"])
    assert calc_wilcoxon_test([1, 2, 3], [1, 2, 3]) == 1.0
    lo, hi = calc_bootstrap_ci_for_mean(np.array([1.0, 2.0, 3.0, 4.0]))
    assert 1.0 <= lo <= hi <= 4.0
    # datasets: read from a local cache, never downloaded
    datasets.set_cache_path(tmp_path / "cache")
    with pytest.raises(cb.CatBoostError, match="does not download"):
        datasets.higgs()
    d = tmp_path / "cache" / "higgs"
    d.mkdir(parents=True)
    block = datasets.synthetic("higgs", rows=50, seed=1)
    assert block.shape == (50, 29) and set(np.unique(block[:, 0])) <= {0.0, 1.0}
    for name, part in (("train.tsv", block[:40]), ("test.tsv", block[40:])):
        with open(d / name, "w") as fh:
            for row in part:
                fh.write("\t".join(f"{v:.9g}" for v in row) + "\n")
    tr, te = datasets.higgs()
    assert tr.shape == (40, 29) and te.shape == (10, 29) and np.allclose(tr, block[:40], rtol=1e-6)
    d = tmp_path / "cache" / "titanic"
    d.mkdir()
    (d / "train.csv").write_text("PassengerId,Survived,Sex\n1,0,male\n2,1,female\n")
    (d / "test.csv").write_text("PassengerId,Sex\n3,male\n")
    tr, te = datasets.titanic()
    assert list(tr.columns) == ["PassengerId", "Survived", "Sex"] and len(te) == 1
    m = cb.CatBoostRegressor(iterations=3, depth=2)
    assert m.get_init_params() == {"iterations": 3, "depth": 2}


def test_code_export_with_categorical_features(tmp_path):
    """Stand-alone Python and C++ apply code of a model with float, one-hot and CTR splits against predict()."""
    import pandas as pd
    from catboost_b200.data.cat_hash import hash_strings
    rng = np.random.default_rng(0)
    n = 1500
    Xn = rng.normal(size=(n, 3)).astype(np.float32)
    Xn[rng.random((n, 3)) < 0.05] = np.nan
    cat1 = rng.integers(0, 40, n)
    cat2 = rng.choice(["red", "green", "blue"], n)
    y = ((np.nan_to_num(Xn[:, 0]) + (cat1 % 3 == 0) * 1.0 + (cat2 == "red") * 0.7 + 0.3 * rng.normal(size=n)) > 0.5).astype(int)
    df = pd.DataFrame({"a": Xn[:, 0], "k1": cat1.astype(str), "b": Xn[:, 1], "k2": cat2, "c": Xn[:, 2]})
    m = cb.CatBoostClassifier(iterations=30, depth=4, verbose=0, allow_writing_files=False, one_hot_max_size=4)
    m.fit(df, y, cat_features=["k1", "k2"])
    assert {s.kind for s in m._model.splits} == {"float", "onehot", "ctr"}
    raw = m.predict(df, prediction_type="RawFormulaVal")
    py = tmp_path / "model.py"
    m.save_model(str(py), format="python")
    ns = {}
    exec(py.read_text(), ns)
    # the pure-Python CityHash of the generated code against the native one, over every length class of the algorithm
    strs = ["", "a", "abcd", "abcdefgh", "x" * 15, "y" * 17, "z" * 33, "w" * 64, "q" * 65, "long " * 50, "ünï"] + [str(i) for i in range(50)]
    assert [int(h) for h in hash_strings(strs)] == [ns["calc_cat_feature_hash"](s) for s in strs]
    got = [ns["apply_catboost_model"]([float(r.a), float(r.b), float(r.c)], [r.k1, r.k2]) for r in df.iloc[:150].itertuples()]
    assert np.max(np.abs(np.array(got) - raw[:150])) < 1e-9
    import shutil
    if shutil.which("g++") is None:
        return
    m.save_model(str(tmp_path / "model.cpp"), format="cpp")
    (tmp_path / "main.cpp").write_text(r'''
#include <cstdio>
#include <cstdlib>
#include "model.cpp"
int main() {
    char k1[64], k2[64], fa[64], fb[64], fc[64];
    while (scanf("%63s %63s %63s %63s %63s", fa, k1, fb, k2, fc) == 5) {
        std::vector<float> f = {(float)atof(fa), (float)atof(fb), (float)atof(fc)};
        std::vector<std::string> c = {k1, k2};
        printf("%.12g\n", ApplyCatboostModel(f, c)[0]);
    }
}
''')
    subprocess.check_call(["g++", "-O1", "-std=c++17", "-o", str(tmp_path / "app"), str(tmp_path / "main.cpp")], cwd=tmp_path)
    inp = "\n".join(f"{r.a:.9g} {r.k1} {r.b:.9g} {r.k2} {r.c:.9g}" for r in df.iloc[:150].itertuples())
    out = subprocess.run([str(tmp_path / "app")], input=inp.encode(), capture_output=True, check=True).stdout.decode().split()
    assert np.max(np.abs(np.array([float(v) for v in out]) - raw[:150])) < 1e-7


def test_libsvm_files_and_sparse_matrices(tmp_path):
    import scipy.sparse as sp
    X = sp.random(400, 12, density=0.3, format="csr", random_state=0, dtype=np.float32)
    Xd = X.toarray()
    y = (Xd[:, 0] + Xd[:, 1] > 0.4).astype(int)
    path = tmp_path / "data.svm"
    with open(path, "w") as fh:
        for i in range(400):
            fh.write(f"{y[i]} qid:{i // 20} " + " ".join(f"{j + 1}:{Xd[i, j]:.7g}" for j in range(12) if Xd[i, j] != 0) + "\n")
    pool = cb.Pool("libsvm://" + str(path))
    assert pool.shape[1] <= 12 and pool.num_row() == 400                 # indices in the file start from 1
    assert np.allclose(pool.get_features()[:, :pool.shape[1]], Xd[:, :pool.shape[1]], atol=1e-6)
    assert np.array_equal(np.asarray(pool.group_id) if pool.group_id.dtype.kind in "iu" else pool.group_id, pool.group_id)
    assert len(np.unique(pool.group_id)) == 20
    (tmp_path / "bad.svm").write_text("1 0:3.5\n")
    with pytest.raises(cb.CatBoostError, match="start from 1"):
        cb.Pool("libsvm://" + str(tmp_path / "bad.svm"))
    # scipy matrices train like their dense form
    kw = dict(iterations=15, depth=3, verbose=False, allow_writing_files=False)
    a = cb.CatBoostClassifier(**kw).fit(X, y).predict(X, prediction_type="RawFormulaVal")
    b = cb.CatBoostClassifier(**kw).fit(Xd, y).predict(Xd, prediction_type="RawFormulaVal")
    assert np.allclose(a, b)
    assert np.allclose(cb.CatBoostClassifier(**kw).fit(sp.csc_matrix(X), y).predict(sp.coo_matrix(X), prediction_type="RawFormulaVal"), b)


def test_functional_train_and_single_object_predict():
    rng = np.random.default_rng(0)
    X = rng.normal(size=(300, 4)).astype(np.float32)
    y = (X[:, 0] > 0).astype(int)
    import catboost_b200.train.boosting  # noqa: F401  (the sub-package import must not shadow the function)
    m = cb.train(cb.Pool(X, y), {"loss_function": "Logloss", "iterations": 5, "verbose": 0})
    assert isinstance(m, cb.CatBoost) and m.tree_count_ == 5
    r = cb.CatBoostRegressor(iterations=5, verbose=0, allow_writing_files=False).fit(X, X[:, 0])
    one = r.predict(X[0])
    assert np.ndim(one) == 0 and one == r.predict(X[:1])[0] == r.predict([float(v) for v in X[0]])
    c = cb.CatBoostClassifier(iterations=5, verbose=0, allow_writing_files=False).fit(X, y)
    assert c.predict_proba(X[0]).shape == (2,) and c.predict(X[0]) in (0, 1)


def test_metric_visualizer_reads_training_logs(tmp_path):
    from catboost_b200.widget import MetricVisualizer, MetricsPlotter
    rng = np.random.default_rng(0)
    X = rng.normal(size=(400, 4)).astype(np.float32)
    y = (X[:, 0] > 0).astype(int)
    cb.CatBoostClassifier(iterations=12, verbose=0, train_dir=str(tmp_path / "run")).fit(X[:300], y[:300], eval_set=(X[300:], y[300:]))
    viz = MetricVisualizer(str(tmp_path), subdirs=True)
    curves = viz.curves()
    (run, parts), = curves.items()
    assert set(parts) == {"learn", "test"} and len(parts["learn"]["Logloss"]) == 12 and len(parts["test"]["Logloss"]) == 12
    assert parts["learn"]["Logloss"][-1] < parts["learn"]["Logloss"][0]
    assert "learn Logloss" in viz.to_text()
    p = MetricsPlotter(["loss"])
    for i in range(5):
        p.log(i, True, {"loss": 1.0 / (i + 1)})
    assert p.curves()["run"]["learn"]["loss"] == [1.0, 0.5, 1 / 3, 0.25, 0.2]
    with pytest.raises(cb.CatBoostError):
        p.log(0, True, {"other": 1.0})


def test_combination_loss():
    rng = np.random.default_rng(0)
    n = 2000
    X = rng.normal(size=(n, 5)).astype(np.float32)
    y = (X[:, 0] + 0.3 * rng.normal(size=n) > 0).astype(np.float32)
    pool = cb.Pool(X, y, group_id=np.repeat(np.arange(n // 10), 10))
    kw = dict(iterations=20, depth=4, learning_rate=0.2, verbose=0, allow_writing_files=False, bootstrap_type="No",
              random_strength=0, leaf_estimation_iterations=1, boost_from_average=False)
    only = "Combination:loss0=Logloss;weight0=1.0;loss1=QueryRMSE;weight1=0.0"
    a = cb.CatBoost(dict(loss_function=only, **kw)).fit(pool)
    b = cb.CatBoost(dict(loss_function="Logloss", **kw)).fit(pool)
    assert np.max(np.abs(a.predict(X) - b.predict(X))) < 1e-5            # a part with weight 0 is left out
    # reported by the metric of the first weighted part
    assert np.allclose(a.evals_result_["learn"][only], b.evals_result_["learn"]["Logloss"], atol=1e-6)
    mixed = "Combination:loss0=Logloss;weight0=1.0;loss1=QueryRMSE;weight1=0.5"
    c = cb.CatBoost(dict(loss_function=mixed, **kw)).fit(pool)
    curve = c.evals_result_["learn"][mixed]
    assert curve[-1] < curve[0] and np.max(np.abs(c.predict(X) - b.predict(X))) > 1e-3
    for bad in ("Combination:loss0=Logloss;weight0=-1;loss1=RMSE;weight1=1", "Combination:loss0=Logloss;weight0=1",
                "Combination:loss0=MultiClass;weight0=1;loss1=RMSE;weight1=1"):
        with pytest.raises(cb.CatBoostError):
            cb.CatBoost(dict(loss_function=bad, **kw)).fit(pool)


def test_custom_multi_dimensional_objectives():
    rng = np.random.default_rng(0)
    n = 500
    X = rng.normal(size=(n, 4)).astype(np.float32)
    Y = np.stack([X[:, 0] * 2 + 0.1 * rng.normal(size=n), X[:, 1] - X[:, 2]], 1).astype(np.float32)

    class SquaredError(cb.MultiTargetCustomObjective):
        def calc_ders_multi(self, approx, target, weight):
            return (np.asarray(target) - np.asarray(approx)) * weight, -np.eye(len(approx)) * weight

    kw = dict(iterations=25, depth=3, learning_rate=0.3, verbose=0, allow_writing_files=False)
    m = cb.CatBoostRegressor(loss_function=SquaredError(), eval_metric="MultiRMSE", **kw).fit(X, Y)
    ref = cb.CatBoostRegressor(loss_function="MultiRMSE", boost_from_average=False, **kw).fit(X, Y)
    assert m.predict(X).shape == (n, 2) and np.allclose(m.predict(X), ref.predict(X), atol=1e-5)

    class Softmax:
        def calc_ders_multi(self, approx, target, weight):
            e = np.exp(approx - approx.max())
            p = e / e.sum()
            d = -p.copy()
            d[int(target)] += 1
            return d * weight, -(np.diag(p) - np.outer(p, p)) * weight

    y = np.digitize(X[:, 0], [-0.5, 0.5])
    mc = cb.CatBoostClassifier(loss_function=Softmax(), classes_count=3, **kw).fit(X, y)
    raw = mc.predict(X, prediction_type="RawFormulaVal")
    assert raw.shape == (n, 3) and (raw.argmax(1) == y).mean() > 0.95
    assert list(mc.evals_result_["learn"]) == ["MultiClass"]


def test_default_prediction_types_follow_the_loss():
    rng = np.random.default_rng(0)
    X = rng.normal(size=(400, 4)).astype(np.float32)
    kw = dict(iterations=20, depth=3, verbose=0, allow_writing_files=False)
    y = rng.poisson(np.exp(0.5 * X[:, 0])).astype(np.float32)
    r = cb.CatBoostRegressor(loss_function="Poisson", **kw).fit(X, y)
    assert np.allclose(r.predict(X), np.exp(r.predict(X, prediction_type="RawFormulaVal")))       # log link: Exponent
    assert r.score(X, y) > 0.1
    u = cb.CatBoostRegressor(loss_function="RMSEWithUncertainty", **kw).fit(X, X[:, 0])
    assert u.predict(X).shape == (400, 2) and (u.predict(X)[:, 1] > 0).all()                       # mean and variance
    Y = np.stack([X[:, 0] > 0, X[:, 1] > 0], 1).astype(np.float32)
    m = cb.CatBoostClassifier(loss_function="MultiLogloss", **kw).fit(X, Y)
    p = m.predict(X, prediction_type="MultiProbability")
    assert p.shape == (400, 2) and ((p > 0.5) == (Y > 0.5)).mean() > 0.9
    with pytest.raises(cb.CatBoostError):
        r.predict(X, prediction_type="MultiProbability")


def test_estimator_classes_refuse_losses_of_another_task():
    rng = np.random.default_rng(0)
    X = rng.normal(size=(100, 3)).astype(np.float32)
    y = (X[:, 0] > 0).astype(int)
    with pytest.raises(cb.CatBoostError, match="for classifier use"):
        cb.CatBoostClassifier(loss_function="RMSE", iterations=2, verbose=0).fit(X, y)
    with pytest.raises(cb.CatBoostError, match="for regressor use"):
        cb.CatBoostRegressor(loss_function="Logloss", iterations=2, verbose=0).fit(X, y)
    cb.CatBoost(dict(loss_function="Logloss", iterations=2, verbose=0, allow_writing_files=False)).fit(X, y)   # the base class takes any


def test_adult_reader_and_grouped_evaluation_folds(tmp_path):
    from catboost_b200 import datasets
    from catboost_b200.eval import CatboostEvaluation, ExecutionCase
    d = tmp_path / "cache" / "adult"
    d.mkdir(parents=True)
    (d / "adult.data").write_text("39, State-gov, 77516, Bachelors, 13, Never-married, Adm-clerical, Not-in-family, White, Male, 2174, 0, 40, United-States, <=50K\n"
                                  "50, ?, 83311, Bachelors, 13, Married-civ-spouse, Exec-managerial, Husband, White, Male, 0, 0, 13, United-States, >50K\n")
    (d / "adult.test").write_text("|1x3 Cross validator\n"
                                  "25, Private, 226802, 11th, 7, Never-married, Machine-op-inspct, Own-child, Black, Male, 0, 0, 40, United-States, <=50K.\n")
    datasets.set_cache_path(tmp_path / "cache")
    tr, te = datasets.adult()
    assert list(tr.columns)[:3] == ["age", "workclass", "fnlwgt"] and tr["age"].dtype == float
    assert tr["workclass"].isna().sum() == 1 and te["income"].iloc[0] == "<=50K"        # '?' is missing; the dot is cut
    # folds of a grouped pool keep whole groups together
    rng = np.random.default_rng(0)
    n = 1200
    X = rng.normal(size=(n, 4)).astype(np.float32)
    y = (X[:, 0] + 0.3 * rng.normal(size=n)).astype(np.float32)
    gid = np.repeat(np.arange(n // 12), 12)
    pool = cb.Pool(X, y, group_id=gid)
    ev = CatboostEvaluation(pool, fold_size=240, fold_count=4)
    folds = ev._folds(pool)
    assert len(folds) >= 4 and sum(len(f) for f in folds) == n
    for f in folds:
        g = gid[f]
        assert all((gid == v).sum() == (g == v).sum() for v in np.unique(g))
    base = ExecutionCase({"loss_function": "QueryRMSE", "iterations": 10, "depth": 3}, label="ten")
    more = ExecutionCase({"loss_function": "QueryRMSE", "iterations": 30, "depth": 3}, label="thirty")
    table = ev.eval_cases(base, [more], ["QueryRMSE"]).get_metric_results("QueryRMSE").get_baseline_comparison()
    assert table.loc["thirty", "Score"] > 0


def test_plot_tree_dot_text():
    import pandas as pd
    rng = np.random.default_rng(0)
    X = rng.normal(size=(400, 3)).astype(np.float32)
    c = rng.choice(["a", "b", "c"], 400)
    y = ((X[:, 0] + (c == "a")) > 0.3).astype(int)
    df = pd.DataFrame({"x0": X[:, 0], "x1": X[:, 1], "k": c})
    m = cb.CatBoostClassifier(iterations=3, depth=2, verbose=0, allow_writing_files=False, one_hot_max_size=4).fit(df, y, cat_features=["k"])
    dot = m.plot_tree(0).source
    assert dot.startswith("digraph {") and dot.count("[shape=ellipse") == 4 and dot.count("->") == 6 and "value >" in dot
    texts = [m.plot_tree(i).source for i in range(3)]
    assert any("k, value = " in t for t in texts) or all("x" in t for t in texts)
    ns = cb.CatBoostClassifier(iterations=2, depth=3, verbose=0, allow_writing_files=False, grow_policy="Lossguide", max_leaves=5).fit(X, y)
    dot = ns.plot_tree(1).source
    assert dot.count("[shape=ellipse") == 5 and dot.count("->") == 8
    with pytest.raises(cb.CatBoostError):
        m.plot_tree(99)


def test_knn_search_on_the_host_is_exact():
    """Off the GPU ops.knn_search takes the chunked fp32 distance matrix: exact neighbours."""
    import torch
    from catboost_b200.ops import api as ops
    g = torch.Generator().manual_seed(0)
    Q, E = torch.randn((70, 24), generator=g), torch.randn((900, 24), generator=g)
    got = ops.knn_search(Q, E, 6)
    want = torch.topk(torch.cdist(Q, E), 6, dim=1, largest=False).indices
    assert torch.equal(got.sort(1).values, want.sort(1).values)
    assert ops.knn_search(Q, E[:3], 6).shape == (70, 3)                  # fewer cloud rows than k
