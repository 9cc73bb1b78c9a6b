"""Doc-parallel training over several ranks: gloo ranks on the CPU (always), NCCL ranks on GPUs (when >= 2)."""
import os
import pickle
import subprocess
import sys
import tempfile

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import os, sys, pickle
import numpy as np
import torch
import torch.distributed as dist
sys.path.insert(0, {root!r})
backend, out_path, mode = sys.argv[1], sys.argv[2], sys.argv[3]
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
if backend == "nccl":
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
else:
    dist.init_process_group("gloo", rank=rank, world_size=world)
import catboost_b200 as cb
rng = np.random.default_rng(0)
n, F = 24000, 10
X = rng.standard_normal((n, F), dtype=np.float32)
w = rng.standard_normal(F).astype(np.float32)
y = (X @ w + 0.3 * rng.standard_normal(n, dtype=np.float32) > 0).astype(np.float32)
lo, hi = n * rank // world, n * (rank + 1) // world
params = dict(iterations=12, depth=5, learning_rate=0.3, verbose=False, allow_writing_files=False, random_strength=0,
              bootstrap_type="No", task_type="GPU" if backend == "nccl" else "CPU", border_count=32)
fit_kw = {{}}
if mode == "cat":
    # two categorical columns with many values: their target statistics must come from the rows of all ranks
    c1 = rng.integers(0, 300, n)
    c2 = rng.integers(0, 40, n)
    eff = rng.standard_normal(300)[c1] + 0.5 * rng.standard_normal(40)[c2]
    y = (0.3 * (X @ w) + eff + 0.3 * rng.standard_normal(n) > 0).astype(np.float32)
    Xo = np.empty((n, F + 2), dtype=object)
    Xo[:, :F] = X
    Xo[:, F] = c1
    Xo[:, F + 1] = c2
    X = Xo
    fit_kw["cat_features"] = [F, F + 1]
    params.update(one_hot_max_size=2, max_ctr_complexity=1)
elif mode == "ordered":
    params["boosting_type"] = "Ordered"
elif mode.startswith("onefeature"):
    # fewer features than ranks: some rank owns no histogram column at all
    X = X[:, :1].copy()
    y = (X[:, 0] + 0.3 * rng.standard_normal(n, dtype=np.float32) > 0).astype(np.float32)
    params["histogram_reduce"] = mode.split(":")[1]
elif mode != "default":
    params["histogram_reduce"] = mode
m = cb.CatBoostClassifier(**params)
m.fit(X[lo:hi], y[lo:hi], **fit_kw)
pred = m.predict(X[:2000], prediction_type="RawFormulaVal")
if rank == 0:
    with open(out_path, "wb") as fh:
        pickle.dump(dict(pred=pred, splits=[(s.feature, s.border) for s in m._model.splits],
                         acc=float(((pred > 0) == (y[:2000] > 0.5)).mean())), fh)
dist.barrier()
dist.destroy_process_group()
'''


def _run(world, backend, mode="default", port=29611):
    d = tempfile.mkdtemp()
    script = os.path.join(d, "worker.py")
    with open(script, "w") as fh:
        fh.write(WORKER.format(root=ROOT))
    out = os.path.join(d, "out.pkl")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), script, backend, out, mode]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    with open(out, "rb") as fh:
        return pickle.load(fh)


def _single(task_type):
    import catboost_b200 as cb
    rng = np.random.default_rng(0)
    n, F = 24000, 10
    X = rng.standard_normal((n, F), dtype=np.float32)
    w = rng.standard_normal(F).astype(np.float32)
    y = (X @ w + 0.3 * rng.standard_normal(n, dtype=np.float32) > 0).astype(np.float32)
    m = cb.CatBoostClassifier(iterations=12, depth=5, learning_rate=0.3, verbose=False, allow_writing_files=False,
                              random_strength=0, bootstrap_type="No", task_type=task_type, border_count=32)
    m.fit(X, y)
    return m.predict(X[:2000], prediction_type="RawFormulaVal"), [(sp.feature, sp.border) for sp in m._model.splits]


def test_gloo_two_ranks_match_single_process():
    res = _run(2, "gloo", port=29613)
    ref, ref_splits = _single("CPU")
    assert res["acc"] > 0.9
    # the border grid is built from the rows of all ranks, so the two runs see the same candidates, choose the same
    # splits and differ only by the summation order of the histograms
    assert res["splits"] == ref_splits
    assert np.allclose(res["pred"], ref, rtol=1e-3, atol=1e-3)


def test_gloo_two_ranks_ordered_boosting():
    """boosting_type='Ordered' on two ranks: the blocks of the global permutation are spread over the ranks and their
    per-leaf statistics are summed, so the run learns as well as a single process does."""
    res = _run(2, "gloo", "ordered", port=29619)
    assert res["acc"] > 0.9


def test_split_columns_with_fewer_features_than_ranks():
    from catboost_b200.parallel.runtime import split_columns
    off = np.array([0, 128, 256, 384])                       # 3 features, 8 ranks: some ranks own nothing
    fb, cb = split_columns(off, 8)
    assert len(fb) == 9 and fb[0] == 0 and fb[-1] == 3 and all(b >= a for a, b in zip(fb, fb[1:]))
    assert cb == [int(off[f]) for f in fb]
    assert sum(1 for a, b in zip(fb, fb[1:]) if b > a) == 3
    fb1, cb1 = split_columns(np.array([0, 64]), 2)
    assert fb1 == [0, 0, 1] or fb1 == [0, 1, 1]


@pytest.mark.gpu
def test_two_gpus_fused_matches_nccl_baseline():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    fused = _run(2, "nccl", "fused", port=29615)
    base = _run(2, "nccl", "nccl", port=29617)
    assert fused["acc"] > 0.9 and base["acc"] > 0.9
    assert fused["splits"] == base["splits"]
    assert np.allclose(fused["pred"], base["pred"], rtol=1e-3, atol=1e-3)
    # one feature on two ranks: rank 1 owns no column, scores nothing and still takes part in every exchange
    f1 = _run(2, "nccl", "onefeature:fused", port=29621)
    b1 = _run(2, "nccl", "onefeature:nccl", port=29623)
    assert f1["acc"] > 0.85 and f1["splits"] == b1["splits"]
    assert np.allclose(f1["pred"], b1["pred"], rtol=1e-3, atol=1e-3)


@pytest.mark.gpu
def test_two_gpus_training_is_repeatable():
    """Two runs of the fused two-GPU trainer on the same data: the histograms are integer sums added in rank order, so the
    splits are the same and the predictions agree to rounding of the first (fp32) leaf step."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    a = _run(2, "nccl", "fused", port=29631)
    b = _run(2, "nccl", "fused", port=29633)
    assert a["splits"] == b["splits"]
    assert np.allclose(a["pred"], b["pred"], rtol=1e-4, atol=1e-5)


@pytest.mark.gpu
def test_two_gpus_categorical_features_sharded_by_hash(monkeypatch):
    """The CTR engine on two GPUs: categories dealt to the ranks by hash (device sort, scan and bucketing kernels on the
    owner, two all-to-alls) against every rank computing every table from all-gathered columns."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    res = _run(2, "nccl", mode="cat", port=29625)
    assert res["acc"] > 0.85, res["acc"]
    monkeypatch.setenv("CB200_CTR_GATHER", "1")
    ref = _run(2, "nccl", mode="cat", port=29627)
    assert res["splits"] == ref["splits"]
    assert np.allclose(res["pred"], ref["pred"], rtol=1e-3, atol=1e-3)


@pytest.mark.gpu
def test_four_gpus_fused_matches_nccl_baseline():
    import torch
    if torch.cuda.device_count() < 4:
        pytest.skip("needs four GPUs")
    fused = _run(4, "nccl", "fused", port=29625)
    base = _run(4, "nccl", "nccl", port=29627)
    assert fused["acc"] > 0.9 and fused["splits"] == base["splits"]
    assert np.allclose(fused["pred"], base["pred"], rtol=1e-3, atol=1e-3)
    again = _run(4, "nccl", "fused", port=29629)
    assert again["splits"] == fused["splits"] and np.allclose(again["pred"], fused["pred"], rtol=1e-5, atol=1e-5)


FAIL_WORKER = r'''
import os, sys, time, datetime
import numpy as np
import torch
import torch.distributed as dist
sys.path.insert(0, {root!r})
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
import catboost_b200 as cb
rng = np.random.default_rng(rank)
X = rng.standard_normal((3000, 6), dtype=np.float32)
y = (X[:, 0] > 0).astype(np.float32)
if rank == 1:
    # the failure is made on the host: this rank never joins the training collectives
    time.sleep(1.0)
    os._exit(17)
t0 = time.time()
try:
    cb.CatBoostClassifier(iterations=5, depth=3, verbose=False, allow_writing_files=False, task_type="CPU").fit(X, y)
    print("RESULT finished-without-error", flush=True)
except BaseException as e:
    print("RESULT error-after %.1f s: %s" % (time.time() - t0, type(e).__name__), flush=True)
os._exit(0)
'''


def test_gloo_two_ranks_with_categorical_features(monkeypatch):
    """CTR statistics are computed from the rows of all ranks: the two-rank model must be as good as a model trained on
    one rank with all rows (shard-local statistics would lose most of the signal of a 300-value feature).  The
    categories are dealt to the ranks by hash; mirroring the categorical columns on every rank instead (the older
    scheme) must give the same model."""
    res = _run(2, "gloo", mode="cat", port=29619)
    assert res["acc"] > 0.85, res["acc"]
    monkeypatch.setenv("CB200_CTR_GATHER", "1")
    ref = _run(2, "gloo", mode="cat", port=29621)
    assert res["splits"] == ref["splits"]
    assert np.allclose(res["pred"], ref["pred"], atol=1e-6)


def test_lost_rank_is_detected_by_the_survivor():
    """A rank that exits before the first collective: the other rank's next collective ends with an error inside the
    process-group timeout instead of waiting forever (host-side failure, CPU ranks)."""
    d = tempfile.mkdtemp()
    script = os.path.join(d, "fail_worker.py")
    with open(script, "w") as fh:
        fh.write(FAIL_WORKER.format(root=ROOT))
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT="29617")
        procs.append(subprocess.Popen([sys.executable, script], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                                      env=env))
    out0, _ = procs[0].communicate(timeout=180)
    procs[1].wait(timeout=60)
    assert procs[1].returncode == 17
    line = [l for l in out0.splitlines() if l.startswith("RESULT")]
    assert line and line[0].startswith("RESULT error-after"), out0[-2000:]


def test_corrupted_snapshot_is_rejected(tmp_path):
    import catboost_b200 as cb
    rng = np.random.default_rng(0)
    X = rng.standard_normal((500, 4)).astype(np.float32)
    y = (X[:, 0] > 0).astype(int)
    snap = str(tmp_path / "snap.bin")
    kw = dict(iterations=6, depth=3, verbose=False, allow_writing_files=True, train_dir=str(tmp_path / "info"),
              save_snapshot=True, snapshot_file=snap, task_type="CPU")
    cb.CatBoostClassifier(**kw).fit(X, y)
    blob = bytearray(open(snap, "rb").read())
    blob[-20] ^= 0xFF                                   # flip a byte of the payload: the stored md5 no longer matches
    open(snap, "wb").write(bytes(blob))
    with pytest.raises(cb.CatBoostError, match="corrupted"):
        cb.CatBoostClassifier(**kw).fit(X, y)


def test_launcher_hands_the_pool_over_in_shared_memory():
    """fit() from one process on several devices: the workers map the parent's arrays from shared memory and train on
    views of their own rows (gloo ranks on the CPU here); the model equals the single-process one."""
    import catboost_b200 as cb
    from catboost_b200.parallel.launcher import attach_pool, share_pool, spawn_training
    rng = np.random.default_rng(0)
    n, F = 24000, 10
    X = rng.standard_normal((n, F), dtype=np.float32)
    w = rng.standard_normal(F).astype(np.float32)
    y = (X @ w + 0.3 * rng.standard_normal(n, dtype=np.float32) > 0).astype(np.float32)
    pool = cb.Pool(X, y)
    desc, segs = share_pool(pool)
    try:
        assert "float_data" in desc["arrays"] and len(desc["small"]) < 100_000
        back, handles = attach_pool(desc)
        assert np.array_equal(back.float_data, pool.float_data) and np.array_equal(back.label, pool.label)
        view = back.slice_range(100, 200)
        assert view.float_data.base is not None and np.array_equal(view.float_data, pool.float_data[100:200])
        del back, view
        for h in handles:
            h.close()
    finally:
        for s in segs:
            s.close()
            s.unlink()
    params = dict(iterations=12, depth=5, learning_rate=0.3, verbose=False, allow_writing_files=False, random_strength=0,
                  bootstrap_type="No", task_type="CPU", border_count=32, loss_function="Logloss")
    res = spawn_training(params, pool, [], [0, 1], default_loss="Logloss", backend="gloo")
    ref, ref_splits = _single("CPU")
    got_splits = [(s.feature, s.border) for s in res.model.splits]
    assert got_splits == ref_splits


def test_gloo_two_ranks_feature_penalties_match_single_process():
    """Per-object feature penalties count documents over all ranks: two CPU ranks build the trees of one process."""
    import catboost_b200 as cb
    from catboost_b200.parallel.launcher import spawn_training
    rng = np.random.default_rng(5)
    n = 3000
    X = rng.standard_normal((n, 5)).astype(np.float32)
    X[:, 1] = X[:, 0] + 0.05 * rng.standard_normal(n).astype(np.float32)
    y = (X[:, 0] + 0.5 * X[:, 2] + 0.1 * rng.standard_normal(n)).astype(np.float32)
    pool = cb.Pool(X, y)
    for policy in ("SymmetricTree", "Depthwise"):
        params = dict(iterations=8, depth=3, learning_rate=0.3, verbose=False, allow_writing_files=False, random_strength=0,
                      bootstrap_type="No", task_type="CPU", border_count=32, loss_function="RMSE", grow_policy=policy,
                      per_object_feature_penalties={0: 1e-4}, first_feature_use_penalties={2: 1e-3})
        res = spawn_training(params, pool, [], [0, 1], default_loss="RMSE", backend="gloo")
        ref = cb.CatBoostRegressor(**params).fit(pool)
        got = [(s.feature, round(float(s.border), 5)) for s in res.model.splits]
        want = [(s.feature, round(float(s.border), 5)) for s in ref._model.splits]
        assert got == want, policy


def test_gloo_two_ranks_survival_and_multi_quantile_match_single_process():
    import catboost_b200 as cb
    from catboost_b200.parallel.launcher import spawn_training
    rng = np.random.default_rng(6)
    n = 2400
    X = rng.standard_normal((n, 4)).astype(np.float32)
    t = np.exp(1.0 + 0.8 * X[:, 0] + 0.2 * rng.standard_normal(n))
    lo, up = t.copy(), t.copy()
    up[::3] = -1
    lo[::3] *= 0.7
    cases = [("SurvivalAft:dist=Logistic;scale=0.7", np.stack([lo, up], 1).astype(np.float32)),
             ("MultiQuantile:alpha=0.2,0.8", (X[:, 0] + rng.standard_normal(n)).astype(np.float32))]
    for loss, y in cases:
        pool = cb.Pool(X, y)
        params = dict(iterations=8, depth=3, learning_rate=0.3, verbose=False, allow_writing_files=False, random_strength=0,
                      bootstrap_type="No", task_type="CPU", border_count=32, loss_function=loss, boost_from_average=False)
        res = spawn_training(params, pool, [], [0, 1], default_loss="RMSE", backend="gloo")
        ref = cb.CatBoostRegressor(**params).fit(pool)
        got = [(s.feature, round(float(s.border), 5)) for s in res.model.splits]
        want = [(s.feature, round(float(s.border), 5)) for s in ref._model.splits]
        assert got == want, loss
