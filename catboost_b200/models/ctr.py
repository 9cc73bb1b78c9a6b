"""CTR features of a trained model: value tables, apply, and (de)serialisation in the reference's layout.

A table maps the 64-bit hash of a projection (combination of categorical feature hashes, combined with
``MAGIC_MULT * (a + MAGIC_MULT * b)``, catboost/libs/model/hash.h:11-14; each 32-bit category hash enters as a
sign-extended int, catboost/libs/model/static_ctr_provider.cpp) to learn-set statistics.  At apply time
``value = (good + prior_num) / (total + prior_denom)``.

Binary layout (``.cbm`` model part ``static_provider_v1``, catboost/libs/model/ctr_data.cpp, ctr_value_table.cpp,
catboost/libs/helpers/dense_hash_view.h): ``count``, then per table a size-prefixed FlatBuffers ``TCtrValueTable``
whose ``IndexHashRaw`` is an open-addressing array of 12-byte buckets ``{u64 hash, u32 index}`` (2^k buckets, linear
probing, empty = all ones) and whose ``CTRBlob`` holds per-bucket ``int`` class counts (Borders / Buckets),
``{float sum, int count}`` pairs (mean-value types) or ``int`` counts (Counter / FeatureFreq).
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field
from typing import Dict, List, Sequence

import numpy as np

from ..utils.flatbuf import Builder, Table

MAGIC_MULT = np.uint64(0x4906BA494954CB65)
CTR_TYPES = ["Borders", "Buckets", "BinarizedTargetMeanValue", "FloatTargetMeanValue", "Counter", "FeatureFreq"]


def projection_hash(cat_hash_columns: Sequence[np.ndarray]) -> np.ndarray:
    """uint64 hash per row of a combination of categorical columns (uint32 hashes)."""
    n = len(cat_hash_columns[0])
    res = np.zeros(n, dtype=np.uint64)
    with np.errstate(over="ignore"):
        for col in cat_hash_columns:
            b = np.asarray(col, dtype=np.uint32).view(np.int32).astype(np.int64).view(np.uint64)
            res = MAGIC_MULT * (res + MAGIC_MULT * b)
    return res


@dataclass
class CtrFeature:
    cat_features: List[int]              # categorical feature indices of the projection (sorted)
    ctr_type: str
    prior_num: float
    prior_denom: float
    target_border_idx: int
    hashes: np.ndarray                   # uint64, sorted
    good: np.ndarray                     # float64 per hash: rows of the counted class (or the count for counter types)
    total: np.ndarray                    # float64 per hash: rows in the category
    denominator: float = 0.0             # Counter: max category count; FeatureFreq: learn rows
    shift: float = 0.0
    scale: float = 1.0
    class_counts: np.ndarray = field(default=None)   # optional int [n_hashes, classes] (tables loaded from a cbm)

    def apply(self, cat_hashes: np.ndarray) -> np.ndarray:
        """CTR value per row; cat_hashes: uint32 [n_model_cat_features, n]."""
        h = projection_hash([cat_hashes[c] for c in self.cat_features])
        U = len(self.hashes)
        if U == 0:
            good = total = np.zeros(len(h))
        else:
            pos = np.clip(np.searchsorted(self.hashes, h), 0, U - 1)
            ok = self.hashes[pos] == h
            good = np.where(ok, self.good[pos], 0.0)
            total = np.where(ok, self.total[pos], 0.0)
        if self.ctr_type in ("Counter", "FeatureFreq"):
            v = (good + self.prior_num) / (self.denominator + self.prior_denom)
        else:
            v = (good + self.prior_num) / (total + self.prior_denom)
        return ((v + self.shift) * self.scale).astype(np.float32)

    def base_key(self):
        return (tuple(self.cat_features), self.ctr_type)


# ---- json -------------------------------------------------------------------------------------------------
def ctr_to_json(c: CtrFeature) -> dict:
    return {"cat_features": list(c.cat_features), "ctr_type": c.ctr_type, "prior_numerator": c.prior_num,
            "prior_denomerator": c.prior_denom, "target_border_idx": c.target_border_idx, "shift": c.shift,
            "scale": c.scale, "denominator": c.denominator, "hashes": [str(int(h)) for h in c.hashes],
            "good": c.good.tolist(), "total": c.total.tolist()}


def ctr_from_json(d: dict) -> CtrFeature:
    return CtrFeature(list(d["cat_features"]), d["ctr_type"], d["prior_numerator"], d["prior_denomerator"],
                      d.get("target_border_idx", 0), np.array([int(h) for h in d["hashes"]], dtype=np.uint64),
                      np.array(d["good"], dtype=np.float64), np.array(d["total"], dtype=np.float64),
                      d.get("denominator", 0.0), d.get("shift", 0.0), d.get("scale", 1.0))


# ---- flatbuffers --------------------------------------------------------------------------------------------
def _ctr_base(b: Builder, c: CtrFeature) -> int:
    comb = b.table(3, [(0, "o", b.vector(c.cat_features, np.int32))])
    fields = [(0, "o", comb)]
    t = CTR_TYPES.index(c.ctr_type)
    if t:
        fields.append((1, "b", t))
    return b.table(3, fields)


def serialize_ctr_feature(b: Builder, c: CtrFeature, borders) -> int:
    """TCtrFeature { Ctr: TModelCtr, Borders: [float] }."""
    base = _ctr_base(b, c)
    fields = [(0, "o", base)]
    if c.target_border_idx:
        fields.append((1, "i", int(c.target_border_idx)))
    if c.prior_num != 0.0:
        fields.append((2, "f", float(c.prior_num)))
    if c.prior_denom != 1.0:
        fields.append((3, "f", float(c.prior_denom)))
    if c.shift != 0.0:
        fields.append((4, "f", float(c.shift)))
    if c.scale != 1.0:
        fields.append((5, "f", float(c.scale)))
    ctr = b.table(6, fields)
    return b.table(2, [(0, "o", ctr), (1, "o", b.vector(borders, np.float32))])


def _build_buckets(hashes: np.ndarray):
    """Open-addressing index (load factor <= 0.5) -> (bytes of 12-byte buckets, index of every hash)."""
    n = len(hashes)
    size = 2
    while size < max(2, int(n / 0.5)):
        size <<= 1
    hb = np.full(size, 0xFFFFFFFFFFFFFFFF, dtype=np.uint64)
    ib = np.zeros(size, dtype=np.uint32)
    mask = size - 1
    for k, h in enumerate(hashes.tolist()):
        z = h & mask
        while hb[z] != 0xFFFFFFFFFFFFFFFF:
            z = (z + 1) & mask
        hb[z] = h
        ib[z] = k
    rec = np.zeros(size, dtype=np.dtype([("h", "<u8"), ("i", "<u4")]))
    rec["h"], rec["i"] = hb, ib
    return rec.tobytes()


def serialize_static_provider(ctrs: List[CtrFeature]) -> bytes:
    """Model part with one value table per (projection, type)."""
    groups: Dict[tuple, List[CtrFeature]] = {}
    for c in ctrs:
        groups.setdefault(c.base_key(), []).append(c)
    out = [struct.pack("<I", len(groups))]
    for key in sorted(groups, key=lambda k: (len(k[0]), k[0], CTR_TYPES.index(k[1]))):
        members = groups[key]
        c0 = members[0]
        b = Builder()
        base = _ctr_base(b, c0)
        buckets = _build_buckets(c0.hashes)
        n_classes = 0
        denom = 0
        if c0.ctr_type in ("Counter", "FeatureFreq"):
            blob = np.asarray(np.rint(c0.total), dtype=np.int32).tobytes()
            denom = int(round(c0.denominator))
        elif c0.ctr_type in ("Borders", "Buckets"):
            if c0.class_counts is not None:
                cc = np.asarray(c0.class_counts, dtype=np.int32)
            else:
                tb = sorted({m.target_border_idx for m in members})
                n_classes = max(tb) + 2
                by_tb = {m.target_border_idx: m for m in members}
                cc = np.zeros((len(c0.hashes), n_classes), dtype=np.int32)
                prev = np.rint(c0.total)
                for k in range(n_classes - 1):
                    g = np.rint(by_tb[k].good) if k in by_tb else np.zeros(len(c0.hashes))
                    cc[:, k] = (prev - g).astype(np.int32)        # rows with class == k
                    prev = g
                cc[:, n_classes - 1] = prev.astype(np.int32)
            n_classes = cc.shape[1]
            blob = np.ascontiguousarray(cc).tobytes()
        else:
            rec = np.zeros(len(c0.hashes), dtype=np.dtype([("s", "<f4"), ("c", "<i4")]))
            rec["s"], rec["c"] = c0.good.astype(np.float32), np.rint(c0.total).astype(np.int32)
            blob = rec.tobytes()
        fields = [(0, "o", base), (1, "o", b.vector(np.frombuffer(buckets, dtype=np.uint8), np.uint8)),
                  (2, "o", b.vector(np.frombuffer(blob, dtype=np.uint8), np.uint8))]
        if denom:
            fields.append((3, "i", denom))
        if n_classes:
            fields.append((4, "i", n_classes))
        fb = b.finish(b.table(5, fields))
        out.append(struct.pack("<I", len(fb)) + fb)
    return b"".join(out)


def _read_base(t: Table):
    comb = t.table(0)
    cats = comb.vector(0, np.int32).tolist() if comb is not None else []
    return tuple(cats), CTR_TYPES[t.scalar(1, "b", 0)]


def deserialize_static_provider(blob: bytes) -> Dict[tuple, dict]:
    pos = 0
    cnt = struct.unpack_from("<I", blob, pos)[0]
    pos += 4
    tables = {}
    for _ in range(cnt):
        size = struct.unpack_from("<I", blob, pos)[0]
        pos += 4
        buf = blob[pos:pos + size]
        pos += size
        t = Table.root(buf)
        key = _read_base(t.table(0))
        raw = t.bytes_vector(1)
        rec = np.frombuffer(raw, dtype=np.dtype([("h", "<u8"), ("i", "<u4")]))
        used = rec["h"] != np.uint64(0xFFFFFFFFFFFFFFFF)
        hashes, index = rec["h"][used], rec["i"][used]
        order = np.argsort(hashes)
        tables[key] = dict(hashes=hashes[order].astype(np.uint64), index=index[order].astype(np.int64),
                           blob=t.bytes_vector(2), denominator=t.scalar(3, "i", 0), n_classes=t.scalar(4, "i", 0))
    return tables


def deserialize_ctr_feature(t: Table, tables: Dict[tuple, dict]):
    """TCtrFeature table -> (CtrFeature, borders)."""
    ctr = t.table(0)
    key = _read_base(ctr.table(0))
    tb_idx = ctr.scalar(1, "i", 0)
    pn, pd = ctr.scalar(2, "f", 0.0), ctr.scalar(3, "f", 1.0)
    shift, scale = ctr.scalar(4, "f", 0.0), ctr.scalar(5, "f", 1.0)
    borders = t.vector(1, np.float32)
    cats, ctype = key
    tab = tables.get(key)
    if tab is None:
        return CtrFeature(list(cats), ctype, pn, pd, tb_idx, np.zeros(0, np.uint64), np.zeros(0), np.zeros(0), 0.0,
                          shift, scale), borders
    idx = tab["index"]
    cc = None
    if ctype in ("Counter", "FeatureFreq"):
        counts = np.frombuffer(tab["blob"], dtype=np.int32)[idx].astype(np.float64)
        good, total = counts, counts
    elif ctype in ("Borders", "Buckets"):
        k = max(tab["n_classes"], 1)
        cc = np.frombuffer(tab["blob"], dtype=np.int32).reshape(-1, k)[idx]
        total = cc.sum(1).astype(np.float64)
        good = (cc[:, tb_idx + 1:].sum(1) if ctype == "Borders" else cc[:, min(tb_idx, k - 1)]).astype(np.float64)
    else:
        rec = np.frombuffer(tab["blob"], dtype=np.dtype([("s", "<f4"), ("c", "<i4")]))[idx]
        good, total = rec["s"].astype(np.float64), rec["c"].astype(np.float64)
    return CtrFeature(list(cats), ctype, pn, pd, tb_idx, tab["hashes"], good, total, float(tab["denominator"]), shift,
                      scale, cc), borders
