"""The stand-alone evaluator library behind the C interface, checked against the Python evaluator on the same model
files (the reference tests its library the same way: catboost/libs/model_interface/ut/c_api_ut.cpp)."""
import numpy as np
import pandas as pd
import pytest

import catboost_b200 as cb
from catboost_b200.models.capi import NativeModelCalcer, NativeModelError, integer_cat_hash, string_cat_hash


def _data(n=1500, seed=0):
    rng = np.random.default_rng(seed)
    X = rng.standard_normal((n, 6)).astype(np.float32)
    y = (X[:, 0] + 0.5 * X[:, 1] * X[:, 2] + 0.1 * rng.standard_normal(n) > 0).astype(np.float32)
    return X, y


def test_numeric_binary_model(tmp_path):
    X, y = _data()
    X[::17, 3] = np.nan
    m = cb.CatBoostClassifier(iterations=30, depth=5, verbose=False, allow_writing_files=False).fit(X, y)
    path = tmp_path / "m.cbm"
    m.save_model(str(path))
    nm = NativeModelCalcer(str(path))
    assert nm.tree_count == 30 and nm.dimensions == 1 and nm.float_features_count == 6 and nm.cat_features_count == 0
    assert nm.float_feature_indices() == list(range(6))
    raw = m.predict(X, prediction_type="RawFormulaVal")
    np.testing.assert_allclose(nm.predict_flat(X)[:, 0], raw, rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(nm.predict_flat(X, transposed=True)[:, 0], raw, rtol=1e-6, atol=1e-6)
    # staged evaluation: the two halves add up to the whole (the bias is part of the first half only)
    a = nm.predict_flat(X, 0, 10)[:, 0]
    b = nm.predict_flat(X, 10, 30)[:, 0]
    np.testing.assert_allclose(a + b, raw, rtol=1e-6, atol=1e-6)
    nm.set_prediction_type("Probability")
    np.testing.assert_allclose(nm.predict_flat(X)[:, 0], m.predict_proba(X)[:, 1], rtol=1e-6, atol=1e-7)
    nm.set_prediction_type("Class")
    assert nm.prediction_dimensions == 1
    np.testing.assert_array_equal(nm.predict_flat(X)[:, 0].astype(int), np.asarray(m.predict(X)).astype(int).reshape(-1))
    assert nm.metadata("params") is not None and nm.metadata("no such key") is None
    assert set(nm.used_feature_names()) <= {str(i) for i in range(6)} and "0" in nm.used_feature_names()
    # loading from memory gives the same model
    nm2 = NativeModelCalcer(blob=path.read_bytes())
    np.testing.assert_allclose(nm2.predict_flat(X)[:, 0], raw, rtol=1e-6, atol=1e-6)


def test_multiclass_and_nonsymmetric(tmp_path):
    rng = np.random.default_rng(1)
    X = rng.standard_normal((1200, 5)).astype(np.float32)
    y = np.digitize(X[:, 0] + 0.3 * X[:, 1], [-0.5, 0.5])
    for policy in ("SymmetricTree", "Depthwise", "Lossguide"):
        m = cb.CatBoostClassifier(iterations=15, depth=4, grow_policy=policy, loss_function="MultiClass", verbose=False,
                                  allow_writing_files=False).fit(X, y)
        path = tmp_path / f"{policy}.cbm"
        m.save_model(str(path))
        nm = NativeModelCalcer(str(path))
        assert nm.dimensions == 3
        np.testing.assert_allclose(nm.predict_flat(X), m.predict(X, prediction_type="RawFormulaVal"), rtol=1e-6, atol=1e-6)
        np.testing.assert_allclose(nm.predict_class_flat(X, 2), m.predict(X, prediction_type="RawFormulaVal")[:, 2],
                                   rtol=1e-6, atol=1e-6)
        nm.set_prediction_type("Probability")
        np.testing.assert_allclose(nm.predict_flat(X), m.predict_proba(X), rtol=1e-6, atol=1e-7)
        nm.set_prediction_type("Class")
        np.testing.assert_array_equal(nm.predict_flat(X)[:, 0].astype(int), np.asarray(m.predict(X)).reshape(-1).astype(int))


def test_categorical_model_with_ctrs_and_one_hot(tmp_path):
    rng = np.random.default_rng(2)
    n = 3000
    c1 = rng.integers(0, 40, n)
    c2 = rng.integers(0, 3, n)                      # low cardinality: one-hot
    x = rng.standard_normal((n, 2)).astype(np.float32)
    eff = rng.standard_normal(40)
    y = (eff[c1] + (c2 == 1) + 0.5 * x[:, 0] + 0.2 * rng.standard_normal(n) > 0).astype(np.float32)
    df = pd.DataFrame({"a": x[:, 0], "c1": [f"v{v}" for v in c1], "b": x[:, 1], "c2": [f"k{v}" for v in c2]})
    m = cb.CatBoostClassifier(iterations=40, depth=4, verbose=False, allow_writing_files=False, one_hot_max_size=4,
                              cat_features=["c1", "c2"]).fit(df, y)
    assert m._model.ctrs and m._model.one_hot
    path = tmp_path / "cat.cbm"
    m.save_model(str(path))
    nm = NativeModelCalcer(str(path))
    assert nm.cat_features_count == 2 and nm.float_features_count == 2
    assert nm.cat_feature_indices() == [1, 3] and nm.float_feature_indices() == [0, 2]
    raw = m.predict(df, prediction_type="RawFormulaVal")
    floats = df[["a", "b"]].to_numpy(np.float32)
    cats = df[["c1", "c2"]].to_numpy().tolist()
    np.testing.assert_allclose(nm.predict(floats, cats)[:, 0], raw, rtol=1e-5, atol=1e-5)
    hashes = np.array([[string_cat_hash(v) for v in row] for row in cats], dtype=np.uint32)
    np.testing.assert_allclose(nm.predict_hashed(floats, hashes)[:, 0], raw, rtol=1e-5, atol=1e-5)
    flat = np.zeros((n, 4), dtype=np.float32)
    flat[:, 0], flat[:, 2] = floats[:, 0], floats[:, 1]
    flat[:, 1], flat[:, 3] = hashes[:, 0].view(np.float32), hashes[:, 1].view(np.float32)
    np.testing.assert_allclose(nm.predict_flat(flat)[:, 0], raw, rtol=1e-5, atol=1e-5)
    assert set(nm.used_feature_names()) <= {"a", "b", "c1", "c2"}


def test_hashes_and_errors(tmp_path):
    from catboost_b200.data.cat_hash import hash_strings
    assert string_cat_hash("hello") == int(hash_strings(["hello"])[0])
    assert integer_cat_hash(-17) == int(hash_strings(["-17"])[0])
    with pytest.raises(NativeModelError, match="cannot open"):
        NativeModelCalcer(str(tmp_path / "missing.cbm"))
    with pytest.raises(NativeModelError, match="bad magic"):
        NativeModelCalcer(blob=b"not a model at all")
    X, y = _data(400)
    m = cb.CatBoostRegressor(iterations=5, depth=3, verbose=False, allow_writing_files=False).fit(X, y)
    path = tmp_path / "r.cbm"
    m.save_model(str(path))
    blob = path.read_bytes()
    with pytest.raises(NativeModelError, match="truncated"):
        NativeModelCalcer(blob=blob[: len(blob) // 2])
    nm = NativeModelCalcer(blob=blob)
    with pytest.raises(NativeModelError, match="feature values per document"):
        nm.predict_flat(X[:, :2])
    with pytest.raises(NativeModelError, match="unknown prediction type"):
        nm.set_prediction_type("Nonsense")
    assert not nm._lib.EnableGPUEvaluation(nm._h, 0)
    nm.set_prediction_type("Exponent")
    np.testing.assert_allclose(nm.predict_flat(X)[:, 0], np.exp(m.predict(X)), rtol=1e-6)


_C_PROGRAM = r"""
#include <stdio.h>
#include <stdlib.h>
#include "cb_model_capi.h"

int main(int argc, char** argv) {
    ModelCalcerHandle* h = ModelCalcerCreate();
    if (!LoadFullModelFromFile(h, argv[1])) { fprintf(stderr, "%s\n", GetErrorString()); return 1; }
    float row[6];
    for (int k = 0; k < 6; ++k) row[k] = (float)atof(argv[2 + k]);
    const float* rows[1] = {row};
    double out = 0.0;
    if (!CalcModelPredictionFlat(h, 1, rows, 6, &out, 1)) { fprintf(stderr, "%s\n", GetErrorString()); return 2; }
    printf("%zu %.12g\n", GetTreeCount(h), out);
    ModelCalcerDelete(h);
    return 0;
}
"""


def test_header_is_plain_c_and_links(tmp_path):
    """A C99 program compiled against the header and linked to the library gives the Python evaluator's value."""
    import shutil
    import subprocess
    from pathlib import Path
    from catboost_b200.ops import native
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        pytest.skip("no C compiler")
    lib = native.build_model_lib()
    X, y = _data(500)
    m = cb.CatBoostRegressor(iterations=12, depth=4, verbose=False, allow_writing_files=False).fit(X, y)
    path = tmp_path / "m.cbm"
    m.save_model(str(path))
    src = tmp_path / "prog.c"
    src.write_text(_C_PROGRAM)
    exe = tmp_path / "prog"
    inc = Path(native.MODEL_SRC[1]).parent
    subprocess.run([cc, "-std=c99", "-Wall", "-Werror", "-I", str(inc), str(src), str(lib), "-o", str(exe),
                    f"-Wl,-rpath,{Path(lib).parent}"], check=True, capture_output=True)
    res = subprocess.run([str(exe), str(path)] + [repr(float(v)) for v in X[7]], check=True, capture_output=True, text=True)
    trees, value = res.stdout.split()
    assert int(trees) == 12
    assert abs(float(value) - float(m.predict(X[7:8])[0])) < 1e-6


def test_model_files_written_by_the_reference():
    """Models saved by the reference itself (numerical + categorical with 26 CTR features; text models are refused)."""
    import os
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ref = os.environ.get("CATBOOST_REFERENCE", os.path.join(os.path.dirname(here), "reference")) + "/catboost/pytest/data"
    path = ref + "/models/features_num_cat__dataset_adult.cbm"
    if not os.path.exists(path):
        pytest.skip("reference model files are not available")
    m = cb.CatBoost().load_model(path)
    pool = cb.Pool(ref + "/adult/test_small", column_description=ref + "/adult/train.cd")
    nm = NativeModelCalcer(path)
    assert nm.tree_count == m.tree_count_ and nm.cat_features_count == 11
    fd, ch = m._model.pool_arrays(pool)
    np.testing.assert_allclose(nm.predict_hashed(fd, ch.T)[:, 0], m.predict(pool, prediction_type="RawFormulaVal"),
                               rtol=1e-6, atol=1e-6)
    with pytest.raises(NativeModelError, match="text or embedding"):
        NativeModelCalcer(ref + "/models/features_num_cat_text__dataset_rotten_tomatoes__binclass.cbm")
