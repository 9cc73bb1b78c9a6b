"""Stand-alone apply code for models with categorical features (``save_model(format='python' | 'cpp')``).

The reference writes such code with the string hash, the CTR tables and the trees inlined
(catboost/libs/model/model_export/python_exporter.cpp, cpp_exporter.cpp).  The code generated here evaluates the same
three kinds of binary features as ``Model._split_outcomes_block``: a float feature above a border (NaN goes the way of
the feature's nan mode), a categorical value equal to a one-hot value, and a CTR -- (good + prior) / (total + prior) of
the projection's table entry -- above a border.  A categorical value enters as its string; its hash is the low 32 bits
of the 64-bit CityHash (2011) of the UTF-8 bytes, and a projection of several features combines the sign-extended
hashes with ``MAGIC * (acc + MAGIC * h)``.

Entry points of the generated code follow the reference: ``apply_catboost_model(float_features, cat_features)`` in
Python, ``ApplyCatboostModel(floatFeatures, catFeatures)`` in C++; both lists are in the model's float / categorical
feature order.  Oblivious trees only.
"""
from __future__ import annotations

from pathlib import Path

import numpy as np

from ..data.pool import CatBoostError
from .model import Model, ObliviousTree

_MAGIC = 0x4906BA494954CB65

_PY_HASH = '''
_M64 = (1 << 64) - 1
_K0, _K1, _K2, _K3, _KMUL = 0xc3a5c85c97cb3127, 0xb492b66fbe98f273, 0x9ae16a3b2f90404f, 0xc949d7c7509e6557, 0x9ddfea08eb382d69


def _ld64(s, i):
    return int.from_bytes(s[i:i + 8], "little")


def _ld32(s, i):
    return int.from_bytes(s[i:i + 4], "little")


def _ror(v, k):
    k &= 63
    return v if k == 0 else ((v >> k) | (v << (64 - k))) & _M64


def _smix(v):
    return v ^ (v >> 47)


def _h16(u, v):
    a = ((u ^ v) * _KMUL) & _M64
    a ^= a >> 47
    b = ((v ^ a) * _KMUL) & _M64
    b ^= b >> 47
    return (b * _KMUL) & _M64


def _weak32(w, x, y, z, a, b):
    a = (a + w) & _M64
    b = _ror((b + a + z) & _M64, 21)
    c = a
    a = (a + x + y) & _M64
    b = (b + _ror(a, 44)) & _M64
    return (a + z) & _M64, (b + c) & _M64


def _weak32s(s, i, a, b):
    return _weak32(_ld64(s, i), _ld64(s, i + 8), _ld64(s, i + 16), _ld64(s, i + 24), a, b)


def city_hash_64(s):
    n = len(s)
    if n <= 16:
        if n > 8:
            a, b = _ld64(s, 0), _ld64(s, n - 8)
            return _h16(a, _ror((b + n) & _M64, n)) ^ b
        if n >= 4:
            return _h16((n + (_ld32(s, 0) << 3)) & _M64, _ld32(s, n - 4))
        if n > 0:
            y = (s[0] + (s[n >> 1] << 8)) & 0xffffffff
            z = (n + (s[n - 1] << 2)) & 0xffffffff
            return (_smix(((y * _K2) & _M64) ^ ((z * _K3) & _M64)) * _K2) & _M64
        return _K2
    if n <= 32:
        a, b = (_ld64(s, 0) * _K1) & _M64, _ld64(s, 8)
        c, d = (_ld64(s, n - 8) * _K2) & _M64, (_ld64(s, n - 16) * _K0) & _M64
        return _h16((_ror((a - b) & _M64, 43) + _ror(c, 30) + d) & _M64, (a + _ror(b ^ _K3, 20) - c + n) & _M64)
    if n <= 64:
        z = _ld64(s, 24)
        a = (_ld64(s, 0) + (n + _ld64(s, n - 16)) * _K0) & _M64
        b, c = _ror((a + z) & _M64, 52), _ror(a, 37)
        a = (a + _ld64(s, 8)) & _M64
        c = (c + _ror(a, 7)) & _M64
        a = (a + _ld64(s, 16)) & _M64
        vf, vs = (a + z) & _M64, (b + _ror(a, 31) + c) & _M64
        a = (_ld64(s, 16) + _ld64(s, n - 32)) & _M64
        z = _ld64(s, n - 8)
        b, c = _ror((a + z) & _M64, 52), _ror(a, 37)
        a = (a + _ld64(s, n - 24)) & _M64
        c = (c + _ror(a, 7)) & _M64
        a = (a + _ld64(s, n - 16)) & _M64
        wf, ws = (a + z) & _M64, (b + _ror(a, 31) + c) & _M64
        r = _smix(((vf + ws) * _K2 + (wf + vs) * _K0) & _M64)
        return (_smix((r * _K0 + vs) & _M64) * _K2) & _M64
    x, y, z = _ld64(s, 0), _ld64(s, n - 16) ^ _K1, _ld64(s, n - 56) ^ _K0
    v = _weak32s(s, n - 64, n, y)
    w = _weak32s(s, n - 32, (n * _K1) & _M64, _K0)
    z = (z + _smix(v[1]) * _K1) & _M64
    x = (_ror((z + x) & _M64, 39) * _K1) & _M64
    y = (_ror(y, 33) * _K1) & _M64
    left, i = (n - 1) & ~63, 0
    while left:
        x = (_ror((x + y + v[0] + _ld64(s, i + 16)) & _M64, 37) * _K1) & _M64
        y = (_ror((y + v[1] + _ld64(s, i + 48)) & _M64, 42) * _K1) & _M64
        x ^= w[1]
        y ^= v[0]
        z = _ror(z ^ w[0], 33)
        v = _weak32s(s, i, (v[1] * _K1) & _M64, (x + w[0]) & _M64)
        w = _weak32s(s, i + 32, (z + w[1]) & _M64, y)
        z, x = x, z
        i += 64
        left -= 64
    return _h16((_h16(v[0], w[0]) + _smix(y) * _K1 + z) & _M64, (_h16(v[1], w[1]) + x) & _M64)


def calc_cat_feature_hash(value):
    """uint32 identifier of a categorical value given as a string (integers: their decimal form)."""
    b = value if isinstance(value, bytes) else str(value).encode("utf-8")
    return city_hash_64(b) & 0xffffffff
'''

_PY_APPLY = '''

def _projection_hash(hashes):
    acc = 0
    for h in hashes:
        b = (h - (1 << 32) if h >= (1 << 31) else h) & _M64          # the 32-bit hash as a sign-extended integer
        acc = (MAGIC * ((acc + MAGIC * b) & _M64)) & _M64
    return acc


def _ctr_value(ctr, cat_hashes):
    cats, counter, prior_num, prior_denom, denominator, shift, scale, table = ctr
    good, total = table.get(_projection_hash([cat_hashes[c] for c in cats]), (0.0, 0.0))
    v = (good + prior_num) / ((denominator if counter else total) + prior_denom)
    return (v + shift) * scale


def apply_catboost_model(float_features, cat_features=None):
    """float_features / cat_features: the model's float and categorical features, each in the model's own order;
    categorical values as strings (or integers, hashed through their decimal form)."""
    cat_hashes = [calc_cat_feature_hash(v) for v in (cat_features or [])]
    ctr_values = [_ctr_value(c, cat_hashes) for c in CTRS]
    outcome = []
    for kind, feature, border, value, nan_right in SPLITS:
        if kind == 0:
            x = float_features[feature]
            outcome.append(nan_right if x != x else x > border)
        elif kind == 1:
            outcome.append(cat_hashes[feature] == value)
        else:
            outcome.append(FLOAT32(ctr_values[feature]) > border)
    result = [0.0] * DIMS
    v = 0
    for splits in TREE_SPLITS:
        leaf = 0
        for k, s in enumerate(splits):
            leaf |= int(outcome[s]) << k
        for d in range(DIMS):
            result[d] += LEAF_VALUES[(v + leaf) * DIMS + d]
        v += 1 << len(splits)
    result = [SCALE * r + b for r, b in zip(result, BIAS)]
    return result[0] if DIMS == 1 else result
'''


def _check(m: Model):
    if not m.trees or not all(isinstance(t, ObliviousTree) for t in m.trees):
        raise CatBoostError("code export supports oblivious trees only")
    if getattr(m, "estimators", None) is not None:
        raise CatBoostError("code export does not cover text and embedding features")


def _split_rows(m: Model):
    nan_right = {f.feature_index: f.nan_mode == "Max" for f in m.float_features}
    rows = []
    for sp in m.splits:
        if sp.kind == "float":
            rows.append((0, int(sp.feature), float(np.float32(sp.border)), 0, bool(nan_right.get(sp.feature, False))))
        elif sp.kind == "onehot":
            rows.append((1, int(sp.feature), 0.0, int(np.uint32(sp.value)), False))
        else:
            rows.append((2, int(sp.feature), float(np.float32(sp.border)), 0, False))
    return rows


def model_to_python_general(m: Model) -> str:
    _check(m)
    ctrs = []
    for c in m.ctrs or []:
        counter = c.ctr_type in ("Counter", "FeatureFreq")
        table = {int(h): (float(g), float(t)) for h, g, t in zip(c.hashes, c.good, c.total)}
        ctrs.append((list(map(int, c.cat_features)), counter, float(c.prior_num), float(c.prior_denom), float(c.denominator),
                     float(c.shift), float(c.scale), table))
    vals = np.concatenate([t.leaf_values.reshape(-1, m.dims) for t in m.trees]).reshape(-1)
    head = ["# Stand-alone apply code generated by catboost_b200", "import struct", "", f"MAGIC = {_MAGIC:#x}", "", "",
            "def FLOAT32(x):", '    return struct.unpack("f", struct.pack("f", x))[0]', ""]
    data = ["", f"SPLITS = {_split_rows(m)!r}", f"CTRS = {ctrs!r}",
            f"TREE_SPLITS = {[list(map(int, t.splits)) for t in m.trees]!r}",
            f"LEAF_VALUES = {[float(x) for x in vals]!r}", f"DIMS = {int(m.dims)}", f"SCALE = {float(m.scale)!r}",
            f"BIAS = {[float(x) for x in np.broadcast_to(m.bias, (m.dims,))]!r}"]
    return "\n".join(head) + _PY_HASH + "\n".join(data) + "\n" + _PY_APPLY


def model_to_cpp_general(m: Model) -> str:
    _check(m)
    city = (Path(__file__).resolve().parent.parent / "ops" / "cpu" / "cb_cityhash.h").read_text()
    city = "\n".join(ln for ln in city.splitlines() if not ln.startswith("#pragma once"))
    rows = _split_rows(m)

    def arr(name, ctype, vals):
        return f"static const {ctype} {name}[] = {{{', '.join(vals) if vals else '0'}}};"

    ctr_cat_off, ctr_cats, tab_off, tab_hash, tab_good, tab_total, ctr_meta = [0], [], [0], [], [], [], []
    for c in m.ctrs or []:
        ctr_cats += [str(int(x)) for x in c.cat_features]
        ctr_cat_off.append(len(ctr_cats))
        tab_hash += [f"{int(h)}ULL" for h in c.hashes]
        tab_good += [repr(float(g)) for g in c.good]
        tab_total += [repr(float(t)) for t in c.total]
        tab_off.append(len(tab_hash))
        counter = 1 if c.ctr_type in ("Counter", "FeatureFreq") else 0
        ctr_meta.append("{%d, %r, %r, %r, %r, %r}" % (counter, float(c.prior_num), float(c.prior_denom), float(c.denominator),
                                                     float(c.shift), float(c.scale)))
    depth = [len(t.splits) for t in m.trees]
    tsplits = [str(int(s)) for t in m.trees for s in t.splits]
    vals = np.concatenate([t.leaf_values.reshape(-1, m.dims) for t in m.trees]).reshape(-1)
    body = [
        "// Stand-alone apply code generated by catboost_b200", "#include <algorithm>", "#include <cmath>", "#include <string>",
        "#include <vector>", city, "",
        "struct CbSplit { int kind; int feature; float border; unsigned int value; int nanRight; };",
        "struct CbCtr { int counter; double priorNum, priorDenom, denominator, shift, scale; };",
        arr("kSplits", "CbSplit", ["{%d, %d, %rf, %dU, %d}" % (k, f, b, v, int(nr)) for k, f, b, v, nr in rows]),
        arr("kCtrs", "CbCtr", ctr_meta), arr("kCtrCatOff", "int", [str(x) for x in ctr_cat_off]), arr("kCtrCats", "int", ctr_cats),
        arr("kTabOff", "int", [str(x) for x in tab_off]), arr("kTabHash", "unsigned long long", tab_hash),
        arr("kTabGood", "double", tab_good), arr("kTabTotal", "double", tab_total),
        arr("kDepth", "int", [str(d) for d in depth]), arr("kTreeSplits", "int", tsplits),
        arr("kLeaf", "double", [repr(float(x)) for x in vals]),
        arr("kBias", "double", [repr(float(x)) for x in np.broadcast_to(m.bias, (m.dims,))]), "",
        f"static const int kDims = {int(m.dims)}, kTrees = {len(m.trees)}, kSplitCount = {len(rows)}, kCtrCount = {len(m.ctrs or [])};",
        f"static const double kScale = {float(m.scale)!r};", "",
        "inline unsigned int CalcCatFeatureHash(const std::string& s) { return (unsigned int)(city1::hash(s.data(), s.size()) & 0xffffffffULL); }",
        "",
        "std::vector<double> ApplyCatboostModel(const std::vector<float>& floatFeatures, const std::vector<std::string>& catFeatures) {",
        "    const unsigned long long kMagic = 0x4906BA494954CB65ULL;",
        "    std::vector<unsigned int> catHash(catFeatures.size());",
        "    for (size_t i = 0; i < catFeatures.size(); ++i) catHash[i] = CalcCatFeatureHash(catFeatures[i]);",
        "    std::vector<float> ctr(kCtrCount > 0 ? kCtrCount : 1);",
        "    for (int c = 0; c < kCtrCount; ++c) {",
        "        unsigned long long acc = 0;",
        "        for (int k = kCtrCatOff[c]; k < kCtrCatOff[c + 1]; ++k)",
        "            acc = kMagic * (acc + kMagic * (unsigned long long)(long long)(int)catHash[kCtrCats[k]]);",
        "        const unsigned long long* lo = kTabHash + kTabOff[c];",
        "        const unsigned long long* hi = kTabHash + kTabOff[c + 1];",
        "        const unsigned long long* it = std::lower_bound(lo, hi, acc);",
        "        double good = 0.0, total = 0.0;",
        "        if (it != hi && *it == acc) { good = kTabGood[it - kTabHash]; total = kTabTotal[it - kTabHash]; }",
        "        const CbCtr& m = kCtrs[c];",
        "        const double v = (good + m.priorNum) / ((m.counter ? m.denominator : total) + m.priorDenom);",
        "        ctr[c] = (float)((v + m.shift) * m.scale);",
        "    }",
        "    std::vector<char> outcome(kSplitCount);",
        "    for (int s = 0; s < kSplitCount; ++s) {",
        "        const CbSplit& sp = kSplits[s];",
        "        if (sp.kind == 0) { const float x = floatFeatures[sp.feature]; outcome[s] = std::isnan(x) ? (char)sp.nanRight : (char)(x > sp.border); }",
        "        else if (sp.kind == 1) outcome[s] = (char)(catHash[sp.feature] == sp.value);",
        "        else outcome[s] = (char)(ctr[sp.feature] > sp.border);",
        "    }",
        "    std::vector<double> res(kDims, 0.0);", "    int s = 0; long long v = 0;",
        "    for (int t = 0; t < kTrees; ++t) {", "        int leaf = 0;",
        "        for (int k = 0; k < kDepth[t]; ++k) leaf |= int(outcome[kTreeSplits[s + k]]) << k;",
        "        for (int d = 0; d < kDims; ++d) res[d] += kLeaf[(v + leaf) * kDims + d];",
        "        s += kDepth[t]; v += 1LL << kDepth[t];", "    }",
        "    for (int d = 0; d < kDims; ++d) res[d] = res[d] * kScale + kBias[d];", "    return res;", "}", ""]
    return "\n".join(body)
