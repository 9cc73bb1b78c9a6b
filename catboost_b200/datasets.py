"""Named datasets (the ``catboost.datasets`` interface, catboost/python-package/catboost/datasets.py).

The reference downloads each archive on first use.  This module never opens a connection: it reads the unpacked files
from a cache directory (``set_cache_path``; default ``./catboost_cached_datasets``), laid out as the reference leaves its
own cache, ``<cache>/<name>/<train file>`` and ``<cache>/<name>/<test file>``, so a cache filled by the reference (or by
hand) is picked up as is.  A missing file raises an error that names the path it looked for.

``synthetic(name, rows)`` returns random data with the column layout of the numeric benchmark sets (higgs, epsilon),
which is what the benchmarks of this package run on.
"""
from __future__ import annotations

import os
from typing import Optional, Tuple

import numpy as np

from .data.pool import CatBoostError

_cache_path: Optional[str] = None

# name -> (train file, test file, reader, separator, header row, (train rows, test rows, columns) for numeric readers)
_REGISTRY = {
    "titanic": ("train.csv", "test.csv", "frame", ",", "infer", None),
    "amazon": ("train.csv", "test.csv", "frame", ",", "infer", None),
    "msrank": ("train.tsv", "test.tsv", "frame", "\t", None, None),
    "msrank_10k": ("train.csv", "test.csv", "frame", ",", None, None),
    "rotten_tomatoes": ("learn.tsv", "test.tsv", "frame", "\t", "infer", None),
    "imdb": ("learn.tsv", "test.tsv", "frame", "\t", "infer", None),
    "monotonic1": ("train.tsv", "test.tsv", "frame", "\t", "infer", None),
    "monotonic2": ("train.tsv", "test.tsv", "frame", "\t", "infer", None),
    "epsilon": ("train.tsv", "test.tsv", "numeric", "\t", None, (400000, 100000, 2001)),
    "higgs": ("train.tsv", "test.tsv", "numeric", "\t", None, (10500000, 500000, 29)),
    "adult": ("adult.data", "adult.test", "adult", ",", None, None),
}

_ADULT_NAMES = ("age", "workclass", "fnlwgt", "education", "education-num", "marital-status", "occupation", "relationship",
                "race", "sex", "capital-gain", "capital-loss", "hours-per-week", "native-country", "income")
_ADULT_FLOAT = ("age", "fnlwgt", "education-num", "capital-gain", "capital-loss", "hours-per-week")


def _get_cache_path() -> str:
    return _cache_path if _cache_path is not None else os.path.join(os.getcwd(), "catboost_cached_datasets")


def set_cache_path(path) -> None:
    global _cache_path
    _cache_path = os.fspath(path)


def _paths(name: str) -> Tuple[str, str]:
    train_file, test_file = _REGISTRY[name][:2]
    d = os.path.join(_get_cache_path(), name)
    tr, te = os.path.join(d, train_file), os.path.join(d, test_file)
    for p in (tr, te):
        if not os.path.exists(p):
            raise CatBoostError(f"dataset {name!r}: {p} does not exist. This package does not download datasets; unpack "
                                f"the archive into {d} or point set_cache_path() at a filled cache.")
    return tr, te


def _read_numeric(path: str, columns: int, sep: str) -> np.ndarray:
    """Float32 matrix in column-major order, parsed in blocks of lines (a numeric-only file has one shape of row, so
    one ``fromstring`` per block replaces a parser call per row)."""
    blocks = []
    with open(path, "rb") as fh:
        while True:
            lines = fh.readlines(64 << 20)
            if not lines:
                break
            flat = np.fromstring(b"".join(lines).replace(b"\n", sep.encode()), dtype=np.float32, sep=sep)
            if flat.size % columns:
                raise CatBoostError(f"{path}: expected rows of {columns} columns")
            blocks.append(flat.reshape(-1, columns))
    data = np.concatenate(blocks) if blocks else np.zeros((0, columns), dtype=np.float32)
    return np.asfortranarray(data)


def _load(name: str):
    import pandas as pd
    train_file, test_file, reader, sep, header, shape = _REGISTRY[name]
    tr, te = _paths(name)
    if reader == "frame":
        return pd.read_csv(tr, header=header, sep=sep), pd.read_csv(te, header=header, sep=sep)
    if reader == "numeric":
        return _read_numeric(tr, shape[2], sep), _read_numeric(te, shape[2], sep)
    # adult: comma + blanks, '?' = missing, the test part has a banner line and a dot after the class
    kw = dict(names=_ADULT_NAMES, header=None, sep=r",\s*", na_values=["?"], engine="python")
    train = pd.read_csv(tr, **kw)
    test = pd.read_csv(te, skiprows=1, converters={"income": lambda x: x[:-1]}, **kw)
    dtype = {c: (float if c in _ADULT_FLOAT else object) for c in _ADULT_NAMES}
    return train.astype(dtype), test.astype(dtype)


def titanic():
    return _load("titanic")


def amazon():
    return _load("amazon")


def msrank():
    return _load("msrank")


def msrank_10k():
    return _load("msrank_10k")


def rotten_tomatoes():
    return _load("rotten_tomatoes")


def imdb():
    return _load("imdb")


def epsilon():
    """(train, test) float32 matrices, class in the first column, 2000 features."""
    return _load("epsilon")


def monotonic1():
    return _load("monotonic1")


def monotonic2():
    return _load("monotonic2")


def adult():
    return _load("adult")


def higgs():
    """(train, test) float32 matrices, class in the first column, 28 features."""
    return _load("higgs")


def synthetic(name: str, rows: Optional[int] = None, seed: int = 0) -> np.ndarray:
    """Random stand-in with the layout of a numeric benchmark set: column 0 is a binary class that depends on a few of
    the features, the rest are standard normal features."""
    if name not in _REGISTRY or _REGISTRY[name][2] != "numeric":
        raise CatBoostError(f"synthetic data exists for the numeric sets only: "
                            f"{sorted(k for k, v in _REGISTRY.items() if v[2] == 'numeric')}")
    full_rows, _, columns = _REGISTRY[name][5]
    n = int(rows) if rows is not None else full_rows
    rng = np.random.default_rng(seed)
    out = np.empty((n, columns), dtype=np.float32, order="F")
    for c in range(1, columns):
        out[:, c] = rng.standard_normal(n, dtype=np.float32)
    k = min(8, columns - 1)
    w = rng.standard_normal(k).astype(np.float32)
    score = out[:, 1:1 + k] @ w + 0.5 * rng.standard_normal(n, dtype=np.float32)
    out[:, 0] = (score > 0).astype(np.float32)
    return out
