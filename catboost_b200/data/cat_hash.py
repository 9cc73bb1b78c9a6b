"""Hashing of categorical feature values.

A categorical value is identified by the low 32 bits of the 64-bit CityHash (2011 version) of its string
form, exactly as catboost/libs/cat_feature/cat_feature.cpp:4-6 does, so that hashes stored in model files
stay interchangeable.  Integer values are stringified first; floats are rejected like the reference does.
"""
from __future__ import annotations

import ctypes

import numpy as np

from ..ops import native


def hash_strings(strings) -> np.ndarray:
    """uint32 hash of every string in ``strings`` (str or bytes)."""
    lib = native.cpu_lib()
    enc = [s if isinstance(s, bytes) else str(s).encode("utf-8") for s in strings]
    off = np.zeros(len(enc) + 1, dtype=np.int64)
    if enc:
        off[1:] = np.cumsum([len(e) for e in enc])
    buf = b"".join(enc)
    out = np.empty(len(enc), dtype=np.uint32)
    lib.cbc_cat_hash_batch(ctypes.c_char_p(buf), off.ctypes.data_as(ctypes.c_void_p), ctypes.c_longlong(len(enc)),
                           out.ctypes.data_as(ctypes.c_void_p))
    return out


def hash_cat_values(col):
    """Hash one categorical column.  Returns (uint32 hashes per row, {string: hash} for the distinct values, sorted
    distinct hashes)."""
    col = np.asarray(col)
    lib = native.cpu_lib()
    if col.dtype.kind in "iu":
        c64 = np.ascontiguousarray(col, dtype=np.int64).reshape(-1)
        mn, mx = (int(c64.min()), int(c64.max())) if c64.size else (0, 0)
        if c64.size and mx - mn <= max(50_000_000, 4 * c64.size):
            # dense integer codes: a direct table indexed by value, filled by the rows themselves
            rng_ = mx - mn + 1
            table = np.zeros(rng_, dtype=np.uint32)
            seen = np.zeros(rng_, dtype=np.uint8)
            out = np.empty(c64.size, dtype=np.uint32)
            lib.cbc_cat_hash_dense_ints(c64.ctypes.data_as(ctypes.c_void_p), ctypes.c_longlong(c64.size),
                                        ctypes.c_longlong(mn), ctypes.c_longlong(rng_),
                                        out.ctypes.data_as(ctypes.c_void_p), table.ctypes.data_as(ctypes.c_void_p),
                                        seen.ctypes.data_as(ctypes.c_void_p))
            present = np.flatnonzero(seen)
            hs = table[present]
            strs = {} if len(present) > 100000 else {str(int(u) + mn): int(h) for u, h in zip(present, hs)}
            return out, strs, np.unique(hs)
        uniq, inv = np.unique(c64, return_inverse=True)
        out = np.empty(len(uniq), dtype=np.uint32)
        lib.cbc_cat_hash_ints(uniq.ctypes.data_as(ctypes.c_void_p), ctypes.c_longlong(len(uniq)),
                              out.ctypes.data_as(ctypes.c_void_p))
        strs = {} if len(uniq) > 100000 else {str(int(u)): int(h) for u, h in zip(uniq, out)}
        return out[inv.reshape(-1)], strs, np.unique(out)
    if col.dtype.kind == "f":
        if np.all(np.isfinite(col)) and np.all(col == np.floor(col)):
            return hash_cat_values(col.astype(np.int64))
        raise ValueError("categorical features must be integers or strings, got fractional floats")
    vals = [v.decode("utf-8") if isinstance(v, bytes) else ("nan" if v is None else str(v)) for v in col.tolist()]
    uniq = sorted(set(vals))
    hashes = hash_strings(uniq)
    table = dict(zip(uniq, (int(h) for h in hashes)))
    return np.fromiter((table[v] for v in vals), dtype=np.uint32, count=len(vals)), table, np.unique(hashes)
