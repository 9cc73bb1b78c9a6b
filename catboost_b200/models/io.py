"""Model persistence and export.

* ``cbm``  -- the reference's binary container: ``"CBM1"`` magic, ``ui32`` size of the FlatBuffers ``TModelCore``
  (catboost/libs/model/flatbuffers/model.fbs, features.fbs, ctr_data.fbs; catboost/libs/model/model.cpp:1113-1230),
  then the model parts (the static CTR provider when the model has CTR features).  Binary-feature numbering is the
  reference's: every border of every used float feature, then every one-hot value, then every CTR border
  (model.cpp:471-540).
* ``json`` -- the same content as a JSON document with the reference's key names (``oblivious_trees``,
  ``features_info``, ``scale_and_bias``).
* ``cpp`` / ``python`` -- stand-alone apply code for float-only oblivious models.
"""
from __future__ import annotations

import json
import struct
from typing import Dict, List

import numpy as np

from ..data.pool import CatBoostError
from ..utils.flatbuf import Builder, Table
from .model import (CatFeatureInfo, FloatFeatureInfo, Model, NonSymmetricTree, ObliviousTree, OneHotFeatureInfo, Split)


def _estimator_registry() -> Dict[str, type]:
    """The only classes a model file's text/embedding block may instantiate."""
    from ..data import estimated as est
    return {c.__name__: c for c in (est.EstimatedFeatures, est._Dictionary, est._TextCalcers, est._EmbeddingCalcers)}

MAGIC = b"CBM1"
CORE_FORMAT = "FlabuffersModel_v1"
STATIC_CTR_PART = "static_provider_v1"


# ---------------------------------------------------------------------------------------------------------
def _bin_feature_order(m: Model):
    """(kind, feature, border/value) of every binary feature in the reference's numbering + lookup by Split.key()."""
    used_f: Dict[int, set] = {}
    used_o: Dict[int, set] = {}
    used_c: Dict[int, set] = {}
    for t in m.trees:
        idxs = t.splits if isinstance(t, ObliviousTree) else [s for s in t.split_of_node if s >= 0]
        for si in idxs:
            sp = m.splits[si]
            if sp.kind == "float":
                used_f.setdefault(sp.feature, set()).add(float(np.float32(sp.border)))
            elif sp.kind == "onehot":
                used_o.setdefault(sp.feature, set()).add(int(sp.value))
            else:
                used_c.setdefault(sp.feature, set()).add(float(np.float32(sp.border)))
    order, lookup = [], {}
    float_borders = {f: sorted(v) for f, v in used_f.items()}
    for ff in m.float_features:
        for b in float_borders.get(ff.feature_index, []):
            lookup[("float", ff.feature_index, b, 0)] = len(order)
            order.append(("float", ff.feature_index, b))
    onehot_vals = {f: sorted(v) for f, v in used_o.items()}
    for f in sorted(onehot_vals):
        for v in onehot_vals[f]:
            lookup[("onehot", f, 0.0, v)] = len(order)
            order.append(("onehot", f, v))
    ctr_borders = {f: sorted(v) for f, v in used_c.items()}
    for f in sorted(ctr_borders):
        for b in ctr_borders[f]:
            lookup[("ctr", f, b, 0)] = len(order)
            order.append(("ctr", f, b))
    return order, lookup, float_borders, onehot_vals, ctr_borders


def _key(sp: Split):
    if sp.kind == "onehot":
        return ("onehot", sp.feature, 0.0, int(sp.value))
    return (sp.kind, sp.feature, float(np.float32(sp.border)), 0)


def model_to_cbm_bytes(m: Model) -> bytes:
    order, lookup, float_borders, onehot_vals, ctr_borders = _bin_feature_order(m)
    b = Builder()
    oblivious = m.is_oblivious()
    tree_splits: List[int] = []
    tree_sizes: List[int] = []
    tree_starts: List[int] = []
    leaf_values: List[np.ndarray] = []
    leaf_weights: List[np.ndarray] = []
    step_nodes: List[tuple] = []
    node_to_leaf: List[int] = []
    value_pos = 0
    for t in m.trees:
        tree_starts.append(len(tree_splits))
        if oblivious:
            tree_splits += [lookup[_key(m.splits[s])] for s in t.splits]
            tree_sizes.append(len(t.splits))
            leaf_values.append(np.asarray(t.leaf_values, dtype=np.float64).reshape(-1))
            leaf_weights.append(np.asarray(t.leaf_weights, dtype=np.float64).reshape(-1))
            continue
        if isinstance(t, ObliviousTree):
            t = oblivious_to_nonsymmetric(t)
        # pre-order emission so that children always follow their parent
        base = len(step_nodes)
        emitted = {}

        def emit(node):
            nid = len(step_nodes)
            emitted[node] = nid
            if t.split_of_node[node] < 0:
                step_nodes.append((0, 0))
                tree_splits.append(0)
                node_to_leaf.append(value_pos + int(t.leaf_of_node[node]) * m.dims)
                return nid
            step_nodes.append(None)
            tree_splits.append(lookup[_key(m.splits[int(t.split_of_node[node])])])
            node_to_leaf.append(0xFFFFFFFF)
            l = emit(int(t.left[node]))
            r = emit(int(t.right[node]))
            if l - nid > 65535 or r - nid > 65535:
                raise CatBoostError("tree too large for the cbm step-node encoding")
            step_nodes[nid] = (l - nid, r - nid)
            return nid

        import sys
        sys.setrecursionlimit(max(sys.getrecursionlimit(), 10000))
        emit(0)
        tree_sizes.append(len(step_nodes) - base)
        leaf_values.append(np.asarray(t.leaf_values, dtype=np.float64).reshape(-1))
        leaf_weights.append(np.asarray(t.leaf_weights, dtype=np.float64).reshape(-1))
        value_pos += t.leaf_values.shape[0] * m.dims

    # feature tables
    cat_offs = []
    used_cat = {f for f in onehot_vals} | {c for ctr in m.ctrs for c in ctr.cat_features}
    for c in m.cat_features:
        fid = b.string(c.name or str(c.flat_index))
        cat_offs.append(b.table(4, [(0, "i", c.feature_index), (1, "i", c.flat_index), (2, "o", fid)]
                                + ([] if c.feature_index in used_cat else [(3, "?", False)])))
    float_offs = []
    for f in m.float_features:
        borders = b.vector(float_borders.get(f.feature_index, []), np.float32)
        fid = b.string(f.name or str(f.flat_index))
        nan_t = 0 if not f.has_nans else (2 if f.nan_mode == "Max" else 1)
        fields = [(1, "i", f.feature_index), (2, "i", f.flat_index), (3, "o", borders), (4, "o", fid)]
        if f.has_nans:
            fields.append((0, "?", True))
        if nan_t:
            fields.append((5, "b", nan_t))
        float_offs.append(b.table(6, fields))
    onehot_offs = []
    for f in sorted(onehot_vals):
        vals = b.vector(np.array(onehot_vals[f], dtype=np.uint32).view(np.int32), np.int32)
        strs = b.offset_vector([b.string(m.cat_hash_to_string.get(int(v), "")) for v in onehot_vals[f]])
        onehot_offs.append(b.table(3, [(0, "i", f), (1, "o", vals), (2, "o", strs)]))
    ctr_offs = []
    parts = b""
    if ctr_borders:
        from .ctr import serialize_ctr_feature, serialize_static_provider
        for f in sorted(ctr_borders):
            ctr_offs.append(serialize_ctr_feature(b, m.ctrs[f], ctr_borders[f]))
        parts = serialize_static_provider([m.ctrs[f] for f in sorted(ctr_borders)])
    fields = [(0, "i", m.dims),
              (1, "o", b.vector(tree_splits, np.int32)), (2, "o", b.vector(tree_sizes, np.int32)),
              (3, "o", b.vector(tree_starts, np.int32)),
              (4, "o", b.offset_vector(cat_offs)), (5, "o", b.offset_vector(float_offs)),
              (6, "o", b.offset_vector(onehot_offs)), (7, "o", b.offset_vector(ctr_offs)),
              (8, "o", b.vector(np.concatenate(leaf_values) if leaf_values else [], np.float64)),
              (9, "o", b.vector(np.concatenate(leaf_weights) if leaf_weights else [], np.float64)),
              (14, "d", float(m.scale)),
              (16, "o", b.vector(np.broadcast_to(m.bias, (m.dims,)), np.float64))]
    if not oblivious:
        fields.append((10, "o", b.vector(np.array(step_nodes, dtype=np.uint16).reshape(-1, 2), np.uint16)))
        fields.append((11, "o", b.vector(node_to_leaf, np.uint32)))
    trees_off = b.table(19, fields)
    info = dict(m.info)
    if m.class_names is not None:
        info.setdefault("class_params", json.dumps({"class_names": [_jsonable(c) for c in m.class_names],
                                                    "class_to_label": list(range(len(m.class_names))),
                                                    "classes_count": 0}))
    info.setdefault("params", json.dumps({"loss_function": {"type": m.loss_name}}))
    info["catboost_b200_meta"] = json.dumps({"loss_name": m.loss_name, "n_features": m.n_features,
                                             "feature_names": m.feature_names})
    if getattr(m, "estimators", None) is not None:
        # text / embedding processing (dictionaries, class statistics, reference embeddings): this framework's own
        # extension of the container, ignored by other readers
        import base64
        from ..utils import plainser
        info["catboost_b200_estimators"] = base64.b64encode(
            plainser.dumps(m.estimators, _estimator_registry())).decode("ascii")
    kv = []
    for k in sorted(info):
        kv.append(b.table(2, [(0, "o", b.string(k)), (1, "o", b.string(info[k]))]))
    core_fields = [(0, "o", b.string(CORE_FORMAT)), (1, "o", trees_off), (2, "o", b.offset_vector(kv))]
    if parts:
        core_fields.append((3, "o", b.offset_vector([b.string(STATIC_CTR_PART)])))
    core = b.finish(b.table(4, core_fields))
    return MAGIC + struct.pack("<I", len(core)) + core + parts


def _jsonable(v):
    if isinstance(v, (np.integer,)):
        return int(v)
    if isinstance(v, (np.floating,)):
        return float(v)
    return v


def oblivious_to_nonsymmetric(t: ObliviousTree) -> NonSymmetricTree:
    depth = len(t.splits)
    n_nodes = (1 << (depth + 1)) - 1
    split_of_node = np.full(n_nodes, -1, dtype=np.int32)
    left = np.zeros(n_nodes, dtype=np.int32)
    right = np.zeros(n_nodes, dtype=np.int32)
    leaf_of_node = np.full(n_nodes, -1, dtype=np.int32)

    # heap layout; level d uses split d; path bits give the leaf index (bit d = outcome of split d)
    def fill(node, level, idx):
        if level == depth:
            leaf_of_node[node] = idx
            return
        split_of_node[node] = t.splits[level]
        left[node], right[node] = 2 * node + 1, 2 * node + 2
        fill(2 * node + 1, level + 1, idx)
        fill(2 * node + 2, level + 1, idx | (1 << level))

    fill(0, 0, 0)
    return NonSymmetricTree(split_of_node, left, right, leaf_of_node, t.leaf_values, t.leaf_weights)


# ---------------------------------------------------------------------------------------------------------
def model_from_cbm_bytes(blob: bytes) -> Model:
    if blob[:4] != MAGIC:
        raise CatBoostError("not a cbm file: bad magic")
    size = struct.unpack_from("<I", blob, 4)[0]
    pos = 8
    if size == 0xFFFFFFFF:
        size = struct.unpack_from("<Q", blob, 8)[0]
        pos = 16
    core_buf = blob[pos:pos + size]
    rest = blob[pos + size:]
    core = Table.root(core_buf)
    if core.string(0) != CORE_FORMAT:
        raise CatBoostError(f"unsupported model format {core.string(0)!r}")
    mt = core.table(1)
    m = Model()
    for kv in core.table_vector(2):
        m.info[kv.string(0)] = kv.string(1)
    m.dims = mt.scalar(0, "i", 1) or 1
    tree_splits = mt.vector(1, np.int32)
    tree_sizes = mt.vector(2, np.int32)
    tree_starts = mt.vector(3, np.int32)
    for ct in mt.table_vector(4):
        m.cat_features.append(CatFeatureInfo(ct.scalar(1, "i", -1), ct.scalar(0, "i", -1), ct.string(2) or ""))
    for ft in mt.table_vector(5):
        nan_t = ft.scalar(5, "b", 0)
        m.float_features.append(FloatFeatureInfo(ft.scalar(2, "i", -1), ft.scalar(1, "i", -1), ft.vector(3, np.float32),
                                                 "Max" if nan_t == 2 else "Min", bool(ft.scalar(0, "?", False)),
                                                 ft.string(4) or ""))
    m.float_features.sort(key=lambda f: f.feature_index)
    m.cat_features.sort(key=lambda c: c.feature_index)
    order = []
    for f in m.float_features:
        for bd in f.borders:
            order.append(Split("float", f.feature_index, border=float(bd)))
    for ot in mt.table_vector(6):
        idx = ot.scalar(0, "i", -1)
        vals = ot.vector(1, np.int32).view(np.uint32)
        strs = ot.string_vector(2)
        m.one_hot[idx] = OneHotFeatureInfo(idx, vals, strs)
        for v, s in zip(vals, strs + [""] * len(vals)):
            if s:
                m.cat_hash_to_string[int(v)] = s
        for v in vals:
            order.append(Split("onehot", idx, value=int(v)))
    ctr_tables = mt.table_vector(7)
    if ctr_tables:
        from .ctr import deserialize_ctr_feature, deserialize_static_provider
        parts = core.string_vector(3)
        tables = deserialize_static_provider(rest) if STATIC_CTR_PART in parts else {}
        for k, ctt in enumerate(ctr_tables):
            ctr, borders = deserialize_ctr_feature(ctt, tables)
            m.ctrs.append(ctr)
            for bd in borders:
                order.append(Split("ctr", k, border=float(bd)))
    m.splits = order
    leaf_values = mt.vector(8, np.float64)
    leaf_weights = mt.vector(9, np.float64)
    steps = mt.vector(10, np.dtype([('l', '<u2'), ('r', '<u2')]))
    steps = np.stack([steps['l'], steps['r']], axis=1) if len(steps) else np.zeros((0, 2), dtype=np.uint16)
    node_to_leaf = mt.vector(11, np.uint32)
    m.scale = mt.scalar(14, "d", 1.0)
    multi_bias = mt.vector(16, np.float64)
    m.bias = multi_bias if len(multi_bias) else np.full(m.dims, mt.scalar(15, "d", 0.0))
    if len(steps) == 0:
        vp = 0
        for k, d in enumerate(tree_sizes):
            s0 = tree_starts[k] if len(tree_starts) else int(np.sum(tree_sizes[:k]))
            nl = 1 << int(d)
            vals = leaf_values[vp * m.dims:(vp + nl) * m.dims].reshape(nl, m.dims)
            wts = leaf_weights[vp:vp + nl] if len(leaf_weights) >= vp + nl else np.zeros(nl)
            m.trees.append(ObliviousTree([int(x) for x in tree_splits[s0:s0 + d]], vals, wts))
            vp += nl
    else:
        for k, sz in enumerate(tree_sizes):
            s0 = int(tree_starts[k])
            m.trees.append(_read_nonsymmetric(tree_splits[s0:s0 + sz], steps[s0:s0 + sz], node_to_leaf[s0:s0 + sz],
                                              leaf_values, leaf_weights, m.dims))
    meta = json.loads(m.info.get("catboost_b200_meta", "{}")) if "catboost_b200_meta" in m.info else {}
    if "catboost_b200_estimators" in m.info:
        # plain data only: the stream can name the four estimator classes below and nothing else, and loading it
        # runs no code from the file (model files are routinely passed around)
        import base64
        import binascii
        from ..utils import plainser
        try:
            m.estimators = plainser.loads(base64.b64decode(m.info.pop("catboost_b200_estimators"), validate=True),
                                          _estimator_registry())
        except (plainser.PlainDataError, binascii.Error, UnicodeDecodeError, struct.error) as e:
            raise CatBoostError(f"the model file carries an unreadable text/embedding processing block: {e}") from e
    params = {}
    try:
        params = json.loads(m.info.get("params", "{}"))
    except ValueError:
        pass
    lf = params.get("loss_function")
    m.loss_name = meta.get("loss_name") or (lf.get("type") if isinstance(lf, dict) else (str(lf).split(":")[0] if lf else "RMSE"))
    m.params = params if "catboost_b200_meta" in m.info else {"loss_function": m.loss_name}
    if "class_params" in m.info:
        try:
            cp = json.loads(m.info["class_params"])
            if cp.get("class_names"):
                m.class_names = cp["class_names"]
        except ValueError:
            pass
    if m.class_names is None and m.loss_name in ("Logloss", "CrossEntropy", "Focal"):
        m.class_names = [0, 1]
    flat = [f.flat_index for f in m.float_features] + [c.flat_index for c in m.cat_features]
    m.n_features = meta.get("n_features") or (max(flat) + 1 if flat else 0)
    names = meta.get("feature_names")
    if names:
        m.feature_names = names
    else:
        m.feature_names = [str(i) for i in range(m.n_features)]
        for f in m.float_features:
            if f.name:
                m.feature_names[f.flat_index] = f.name
        for c in m.cat_features:
            if c.name:
                m.feature_names[c.flat_index] = c.name
    return m


def _read_nonsymmetric(splits, steps, node_to_leaf, leaf_values, leaf_weights, dims) -> NonSymmetricTree:
    n = len(splits)
    split_of_node, left, right, leaf_val_idx = [], [], [], []

    def new_leaf(value_index):
        split_of_node.append(-1); left.append(0); right.append(0); leaf_val_idx.append(int(value_index))
        return len(split_of_node) - 1

    # first pass: one node per stored node
    for i in range(n):
        l, r = int(steps[i][0]), int(steps[i][1])
        if l == 0 and r == 0:
            split_of_node.append(-1); left.append(0); right.append(0); leaf_val_idx.append(int(node_to_leaf[i]))
        else:
            split_of_node.append(int(splits[i])); left.append(i + l); right.append(i + r); leaf_val_idx.append(-1)
    # a zero step on one side only means "terminal here": give that side its own leaf node
    for i in range(n):
        l, r = int(steps[i][0]), int(steps[i][1])
        if (l == 0) != (r == 0):
            leaf = new_leaf(node_to_leaf[i])
            if l == 0:
                left[i] = leaf
            else:
                right[i] = leaf
    idxs = sorted({v for v in leaf_val_idx if v >= 0})
    remap = {v: k for k, v in enumerate(idxs)}
    leaf_of_node = np.array([remap[v] if v >= 0 else -1 for v in leaf_val_idx], dtype=np.int32)
    vals = np.stack([leaf_values[v:v + dims] for v in idxs]) if idxs else np.zeros((0, dims))
    wts = np.array([leaf_weights[v // dims] if v // dims < len(leaf_weights) else 0.0 for v in idxs])
    return NonSymmetricTree(np.array(split_of_node, dtype=np.int32), np.array(left, dtype=np.int32),
                            np.array(right, dtype=np.int32), leaf_of_node, vals, wts)


# ---------------------------------------------------------------------------------------------------------
def model_to_json(m: Model) -> dict:
    feats = {"float_features": [{"feature_index": f.feature_index, "flat_feature_index": f.flat_index,
                                 "borders": [float(x) for x in f.borders], "has_nans": bool(f.has_nans),
                                 "nan_value_treatment": ("AsIs" if not f.has_nans else ("AsTrue" if f.nan_mode == "Max" else "AsFalse")),
                                 "feature_id": f.name} for f in m.float_features]}
    if m.cat_features:
        feats["categorical_features"] = [{"feature_index": c.feature_index, "flat_feature_index": c.flat_index,
                                          "feature_id": c.name,
                                          **({"values": [int(v) for v in m.one_hot[c.feature_index].values]}
                                             if c.feature_index in m.one_hot else {})} for c in m.cat_features]
    if m.ctrs:
        from .ctr import ctr_to_json
        feats["ctrs"] = [ctr_to_json(c) for c in m.ctrs]

    def split_json(sp: Split):
        if sp.kind == "float":
            return {"split_type": "FloatFeature", "float_feature_index": sp.feature, "border": float(sp.border)}
        if sp.kind == "onehot":
            return {"split_type": "OneHotFeature", "cat_feature_index": sp.feature, "value": int(sp.value)}
        return {"split_type": "OnlineCtr", "ctr_index": sp.feature, "border": float(sp.border)}

    doc = {"features_info": feats, "scale_and_bias": [float(m.scale), [float(x) for x in np.broadcast_to(m.bias, (m.dims,))]],
           "model_info": {"params": m.params if _is_jsonable(m.params) else {}, "loss_name": m.loss_name,
                          "class_names": None if m.class_names is None else [_jsonable(c) for c in m.class_names],
                          "feature_names": m.feature_names, "n_features": m.n_features, "dims": m.dims,
                          "cat_hash_to_string": {str(k): v for k, v in m.cat_hash_to_string.items()}}}
    if m.is_oblivious():
        doc["oblivious_trees"] = [{"splits": [split_json(m.splits[s]) for s in t.splits],
                                   "leaf_values": np.asarray(t.leaf_values).reshape(-1).tolist(),
                                   "leaf_weights": np.asarray(t.leaf_weights).reshape(-1).tolist()} for t in m.trees]
    else:
        trees = []
        for t in m.trees:
            if isinstance(t, ObliviousTree):
                t = oblivious_to_nonsymmetric(t)
            trees.append({"nodes": [{"split": (split_json(m.splits[int(s)]) if s >= 0 else None), "left": int(l),
                                     "right": int(r), "leaf": int(lf)}
                                    for s, l, r, lf in zip(t.split_of_node, t.left, t.right, t.leaf_of_node)],
                          "leaf_values": np.asarray(t.leaf_values).reshape(-1).tolist(),
                          "leaf_weights": np.asarray(t.leaf_weights).reshape(-1).tolist()})
        doc["trees"] = trees
    return doc


def _is_jsonable(x):
    try:
        json.dumps(x)
        return True
    except (TypeError, ValueError):
        return False


def model_from_json(doc: dict) -> Model:
    m = Model()
    info = doc.get("model_info", {})
    m.dims = int(info.get("dims", 1))
    for f in doc["features_info"].get("float_features", []):
        m.float_features.append(FloatFeatureInfo(f["flat_feature_index"], f["feature_index"],
                                                 np.array(f["borders"], dtype=np.float32),
                                                 "Max" if f.get("nan_value_treatment") == "AsTrue" else "Min",
                                                 bool(f.get("has_nans")), f.get("feature_id", "")))
    for c in doc["features_info"].get("categorical_features", []):
        m.cat_features.append(CatFeatureInfo(c["flat_feature_index"], c["feature_index"], c.get("feature_id", "")))
        if "values" in c:
            m.one_hot[c["feature_index"]] = OneHotFeatureInfo(c["feature_index"], np.array(c["values"], dtype=np.uint32))
    if "ctrs" in doc["features_info"]:
        from .ctr import ctr_from_json
        m.ctrs = [ctr_from_json(c) for c in doc["features_info"]["ctrs"]]

    def split_from(js):
        t = js["split_type"]
        if t == "FloatFeature":
            return m.split_index(Split("float", js["float_feature_index"], border=js["border"]))
        if t == "OneHotFeature":
            return m.split_index(Split("onehot", js["cat_feature_index"], value=js["value"]))
        return m.split_index(Split("ctr", js["ctr_index"], border=js["border"]))

    for t in doc.get("oblivious_trees", []):
        sp = [split_from(s) for s in t["splits"]]
        nl = 1 << len(sp)
        m.trees.append(ObliviousTree(sp, np.array(t["leaf_values"], dtype=np.float64).reshape(nl, -1),
                                     np.array(t.get("leaf_weights", [0] * nl), dtype=np.float64)))
    for t in doc.get("trees", []):
        nodes = t["nodes"]
        so = np.array([split_from(nd["split"]) if nd["split"] else -1 for nd in nodes], dtype=np.int32)
        lv = np.array(t["leaf_values"], dtype=np.float64).reshape(-1, m.dims)
        m.trees.append(NonSymmetricTree(so, np.array([nd["left"] for nd in nodes], dtype=np.int32),
                                        np.array([nd["right"] for nd in nodes], dtype=np.int32),
                                        np.array([nd["leaf"] for nd in nodes], dtype=np.int32), lv,
                                        np.array(t.get("leaf_weights", [0] * len(lv)), dtype=np.float64)))
    sb = doc.get("scale_and_bias", [1.0, [0.0]])
    m.scale = float(sb[0])
    m.bias = np.array(sb[1] if isinstance(sb[1], list) else [sb[1]], dtype=np.float64)
    m.params = info.get("params", {})
    m.loss_name = info.get("loss_name", "RMSE")
    m.class_names = info.get("class_names")
    m.feature_names = info.get("feature_names", [])
    m.n_features = int(info.get("n_features", len(m.feature_names)))
    m.cat_hash_to_string = {int(k): v for k, v in info.get("cat_hash_to_string", {}).items()}
    return m


# ---------------------------------------------------------------------------------------------------------
def _export_arrays(m: Model):
    if not m._float_only_oblivious():
        raise CatBoostError("code export supports oblivious models over float features only")
    return m._packed_oblivious()


def model_to_python(m: Model) -> str:
    if not m._float_only_oblivious():
        from .codegen import model_to_python_general          # categorical features: hash, CTR tables and trees inlined
        return model_to_python_general(m)
    p = _export_arrays(m)
    lines = ["# Stand-alone apply code generated by catboost_b200", "import bisect", "",
             f"USED_FEATURES = {[int(m.float_features[int(f)].flat_index) for f in p['used']]}",
             f"BORDERS = {[p['borders'][p['boff'][i]:p['boff'][i + 1]].tolist() for i in range(len(p['used']))]}",
             f"TREE_DEPTH = {p['depth'].tolist()}", f"SPLIT_FEATURE = {p['sfeat'].tolist()}",
             f"SPLIT_BIN = {p['sbin'].tolist()}", f"LEAF_VALUES = {p['vals'].reshape(-1).tolist()}",
             f"DIMS = {m.dims}", f"SCALE = {float(m.scale)!r}",
             f"BIAS = {[float(x) for x in np.broadcast_to(m.bias, (m.dims,))]}", "", "",
             "def apply_catboost_model(float_features, cat_features=None):",
             "    bins = [bisect.bisect_left(BORDERS[u], float_features[f]) for u, f in enumerate(USED_FEATURES)]",
             "    result = [0.0] * DIMS", "    s = 0", "    v = 0", "    for depth in TREE_DEPTH:", "        leaf = 0",
             "        for k in range(depth):",
             "            leaf |= (bins[SPLIT_FEATURE[s + k]] > SPLIT_BIN[s + k]) << k",
             "        for d in range(DIMS):", "            result[d] += LEAF_VALUES[(v + leaf) * DIMS + d]",
             "        s += depth", "        v += 1 << depth",
             "    result = [SCALE * r + b for r, b in zip(result, BIAS)]",
             "    return result[0] if DIMS == 1 else result", ""]
    return "\n".join(lines)


def model_to_cpp(m: Model) -> str:
    if not m._float_only_oblivious():
        from .codegen import model_to_cpp_general
        return model_to_cpp_general(m)
    p = _export_arrays(m)
    def arr(name, ctype, vals):
        return f"static const {ctype} {name}[] = {{{', '.join(str(v) for v in vals)}}};"
    used = [int(m.float_features[int(f)].flat_index) for f in p["used"]]
    body = ["// Stand-alone apply code generated by catboost_b200", "#include <vector>", "#include <algorithm>", "",
            arr("kUsed", "int", used), arr("kBorders", "float", [repr(float(x)) + "f" for x in p["borders"]]),
            arr("kBorderOff", "int", p["boff"].tolist()), arr("kDepth", "int", p["depth"].tolist()),
            arr("kSplitFeature", "unsigned short", p["sfeat"].tolist()),
            arr("kSplitBin", "unsigned char", p["sbin"].tolist()),
            arr("kLeaf", "double", [repr(float(x)) for x in p["vals"].reshape(-1)]),
            arr("kBias", "double", [repr(float(x)) for x in np.broadcast_to(m.bias, (m.dims,))]), "",
            f"static const int kDims = {m.dims}, kTrees = {p['T']}, kUsedCount = {len(used)};",
            f"static const double kScale = {float(m.scale)!r};", "",
            "std::vector<double> ApplyCatboostModel(const std::vector<float>& features) {",
            "    std::vector<int> bins(kUsedCount);",
            "    for (int u = 0; u < kUsedCount; ++u)",
            "        bins[u] = int(std::lower_bound(kBorders + kBorderOff[u], kBorders + kBorderOff[u + 1], features[kUsed[u]]) - (kBorders + kBorderOff[u]));",
            "    std::vector<double> res(kDims, 0.0);", "    int s = 0; long long v = 0;",
            "    for (int t = 0; t < kTrees; ++t) {", "        int leaf = 0;",
            "        for (int k = 0; k < kDepth[t]; ++k) leaf |= int(bins[kSplitFeature[s + k]] > kSplitBin[s + k]) << k;",
            "        for (int d = 0; d < kDims; ++d) res[d] += kLeaf[(v + leaf) * kDims + d];",
            "        s += kDepth[t]; v += 1LL << kDepth[t];", "    }",
            "    for (int d = 0; d < kDims; ++d) res[d] = res[d] * kScale + kBias[d];", "    return res;", "}", ""]
    return "\n".join(body)


def save_model(m: Model, fname: str, format: str = "cbm", export_parameters=None, pool=None):
    fmt = format.lower()
    if fmt == "cbm":
        with open(fname, "wb") as fh:
            fh.write(model_to_cbm_bytes(m))
    elif fmt == "json":
        with open(fname, "w") as fh:
            json.dump(model_to_json(m), fh)
    elif fmt == "python":
        with open(fname, "w") as fh:
            fh.write(model_to_python(m))
    elif fmt == "cpp":
        with open(fname, "w") as fh:
            fh.write(model_to_cpp(m))
    elif fmt == "onnx":
        from .export import model_to_onnx_bytes
        with open(fname, "wb") as fh:
            fh.write(model_to_onnx_bytes(m))
    elif fmt == "pmml":
        from .export import model_to_pmml
        with open(fname, "w") as fh:
            fh.write(model_to_pmml(m))
    elif fmt == "coreml":
        from .export import model_to_coreml_bytes
        with open(fname, "wb") as fh:
            fh.write(model_to_coreml_bytes(m, export_parameters))
    else:
        raise CatBoostError(f"unknown model format {format!r}")


def load_model_blob(blob: bytes, format: str = "cbm") -> Model:
    fmt = format.lower()
    if fmt == "cbm":
        return model_from_cbm_bytes(bytes(blob))
    if fmt == "json":
        return model_from_json(json.loads(blob))
    raise CatBoostError(f"cannot load format {format!r}")


def load_model(fname: str, format: str = "cbm") -> Model:
    with open(fname, "rb") as fh:
        return load_model_blob(fh.read(), format)
