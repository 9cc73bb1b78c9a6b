"""Model export to ONNX (ai.onnx.ml TreeEnsemble operators), CoreML (TreeEnsembleRegressor) and PMML (MiningModel of
TreeModels).

The writers are self-contained: the ONNX and CoreML files are protobuf messages encoded by hand (field numbers of
onnx/onnx.proto and of the CoreML specification), the PMML file is plain XML.  As in the reference (catboost/libs/model/model_export/onnx_helpers.cpp,
pmml_helpers.cpp) only models over numerical features are exportable; a split "value > border" becomes the ONNX node
mode BRANCH_GT with the true branch on the right child.
"""
from __future__ import annotations

import struct
from typing import List
from xml.sax.saxutils import escape

import numpy as np

from ..data.pool import CatBoostError
from .model import Model, NonSymmetricTree


# ---- minimal protobuf encoder ------------------------------------------------------------------------------
def _varint(v: int) -> bytes:
    v &= (1 << 64) - 1
    out = bytearray()
    while True:
        b = v & 0x7F
        v >>= 7
        if v:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def _key(field: int, wire: int) -> bytes:
    return _varint((field << 3) | wire)


def _f_varint(field, v):
    return _key(field, 0) + _varint(int(v))


def _f_bytes(field, b: bytes):
    return _key(field, 2) + _varint(len(b)) + b


def _f_str(field, s: str):
    return _f_bytes(field, s.encode("utf-8"))


def _f_float(field, v):
    return _key(field, 5) + struct.pack("<f", float(v))


def _packed_floats(field, vals):
    return _f_bytes(field, struct.pack(f"<{len(vals)}f", *[float(v) for v in vals]))


def _packed_ints(field, vals):
    return _f_bytes(field, b"".join(_varint(int(v)) for v in vals))


# AttributeProto: name=1, f=2, i=3, s=4, floats=7, ints=8, strings=9, type=20 (FLOAT=1 INT=2 STRING=3 FLOATS=6 INTS=7 STRINGS=8)
def _attr_ints(name, vals):
    return _f_str(1, name) + _packed_ints(8, vals) + _f_varint(20, 7)


def _attr_floats(name, vals):
    return _f_str(1, name) + _packed_floats(7, vals) + _f_varint(20, 6)


def _attr_strings(name, vals):
    return _f_str(1, name) + b"".join(_f_bytes(9, v.encode()) for v in vals) + _f_varint(20, 8)


def _attr_int(name, v):
    return _f_str(1, name) + _f_varint(3, v) + _f_varint(20, 2)


def _attr_str(name, v):
    return _f_str(1, name) + _f_bytes(4, v.encode()) + _f_varint(20, 3)


def _value_info(name, elem_type, dims):
    # ValueInfoProto{name=1, type=2: TypeProto{tensor_type=1: {elem_type=1, shape=2: {dim=1: {dim_value=1 | dim_param=2}}}}}
    dim_b = b""
    for d in dims:
        dim_b += _f_bytes(1, _f_str(2, d) if isinstance(d, str) else _f_varint(1, d))
    tensor = _f_varint(1, elem_type) + _f_bytes(2, dim_b)
    return _f_str(1, name) + _f_bytes(2, _f_bytes(1, tensor))


def _flatten_trees(m: Model):
    """Per tree: node arrays in the order of the ONNX attributes."""
    from .io import oblivious_to_nonsymmetric
    if m.ctrs or m.cat_features or any(sp.kind != "float" for sp in m.splits):
        raise CatBoostError("only models over numerical features can be exported to this format")
    out = []
    for t in m.trees:
        ns = t if isinstance(t, NonSymmetricTree) else oblivious_to_nonsymmetric(t)
        out.append(ns)
    return out


def model_to_onnx_bytes(m: Model) -> bytes:
    trees = _flatten_trees(m)
    classifier = m.class_names is not None and m.loss_name in ("Logloss", "CrossEntropy", "Focal", "MultiClass", "MultiClassOneVsAll")
    dims = m.dims
    treeids, nodeids, featids, values, modes, trueids, falseids, missing = [], [], [], [], [], [], [], []
    t_tree, t_node, t_id, t_w = [], [], [], []
    for ti, ns in enumerate(trees):
        for node in range(len(ns.split_of_node)):
            si = int(ns.split_of_node[node])
            treeids.append(ti)
            nodeids.append(node)
            if si >= 0:
                sp = m.splits[si]
                ff = m.float_features[sp.feature]
                featids.append(ff.flat_index)
                values.append(sp.border)
                modes.append("BRANCH_GT")
                trueids.append(int(ns.right[node]))
                falseids.append(int(ns.left[node]))
                missing.append(1 if ff.nan_mode == "Max" else 0)
            else:
                featids.append(0)
                values.append(0.0)
                modes.append("LEAF")
                trueids.append(0)
                falseids.append(0)
                missing.append(0)
                lv = ns.leaf_values[int(ns.leaf_of_node[node])] * m.scale
                if classifier and dims == 1:
                    t_tree.append(ti); t_node.append(node); t_id.append(1); t_w.append(float(lv[0]))
                else:
                    for d in range(dims):
                        t_tree.append(ti); t_node.append(node); t_id.append(d); t_w.append(float(lv[d]))
    bias = [float(b) for b in np.broadcast_to(m.bias, (dims,))]
    attrs = [_attr_ints("nodes_treeids", treeids), _attr_ints("nodes_nodeids", nodeids),
             _attr_ints("nodes_featureids", featids), _attr_floats("nodes_values", values),
             _attr_strings("nodes_modes", modes), _attr_ints("nodes_truenodeids", trueids),
             _attr_ints("nodes_falsenodeids", falseids), _attr_ints("nodes_missing_value_tracks_true", missing)]
    if classifier:
        n_cls = 2 if dims == 1 else dims
        labels = list(range(n_cls))
        try:
            labels = [int(c) for c in m.class_names]
        except (TypeError, ValueError):
            pass
        attrs += [_attr_ints("class_treeids", t_tree), _attr_ints("class_nodeids", t_node), _attr_ints("class_ids", t_id),
                  _attr_floats("class_weights", t_w), _attr_ints("classlabels_int64s", labels),
                  _attr_str("post_transform", "LOGISTIC" if dims == 1 else "SOFTMAX"),
                  _attr_floats("base_values", [0.0, bias[0]] if dims == 1 else bias)]
        op, outputs = "TreeEnsembleClassifier", ["label", "probabilities"]
        out_infos = [_value_info("label", 7, ["N"]), _value_info("probabilities", 1, ["N", n_cls])]
    else:
        attrs += [_attr_ints("target_treeids", t_tree), _attr_ints("target_nodeids", t_node), _attr_ints("target_ids", t_id),
                  _attr_floats("target_weights", t_w), _attr_int("n_targets", dims), _attr_str("post_transform", "NONE"),
                  _attr_floats("base_values", bias)]
        op, outputs = "TreeEnsembleRegressor", ["predictions"]
        out_infos = [_value_info("predictions", 1, ["N", dims])]
    # NodeProto: input=1, output=2, name=3, op_type=4, attribute=5, domain=7
    node = _f_str(1, "features") + b"".join(_f_str(2, o) for o in outputs) + _f_str(3, "tree_ensemble") + _f_str(4, op) + \
        b"".join(_f_bytes(5, a) for a in attrs) + _f_str(7, "ai.onnx.ml")
    # GraphProto: node=1, name=2, input=11, output=12
    graph = _f_bytes(1, node) + _f_str(2, "catboost_b200") + _f_bytes(11, _value_info("features", 1, ["N", m.n_features])) + \
        b"".join(_f_bytes(12, o) for o in out_infos)
    # ModelProto: ir_version=1, producer_name=2, producer_version=3, graph=7, opset_import=8 {domain=1, version=2}
    return _f_varint(1, 7) + _f_str(2, "catboost_b200") + _f_str(3, "0.1") + _f_bytes(7, graph) + \
        _f_bytes(8, _f_str(1, "ai.onnx.ml") + _f_varint(2, 2)) + _f_bytes(8, _f_str(1, "") + _f_varint(2, 12))


# ---- PMML -------------------------------------------------------------------------------------------------
def model_to_pmml(m: Model) -> str:
    trees = _flatten_trees(m)
    if m.dims != 1:
        raise CatBoostError("PMML export supports one-dimensional models")
    names = [escape(str(n)) for n in m.feature_names]
    used = sorted({m.float_features[m.splits[int(s)].feature].flat_index for ns in trees for s in ns.split_of_node if s >= 0})
    out: List[str] = ['<?xml version="1.0" encoding="UTF-8"?>',
                      '<PMML xmlns="http://www.dmg.org/PMML-4_3" version="4.3">',
                      '  <Header description="catboost_b200 model"/>', '  <DataDictionary>']
    for c in used:
        out.append(f'    <DataField name="{names[c]}" optype="continuous" dataType="float"/>')
    out.append('    <DataField name="prediction" optype="continuous" dataType="double"/>')
    out += ['  </DataDictionary>', '  <MiningModel functionName="regression">', '    <MiningSchema>']
    for c in used:
        out.append(f'      <MiningField name="{names[c]}" usageType="active"/>')
    out += ['      <MiningField name="prediction" usageType="target"/>', '    </MiningSchema>']
    out.append(f'    <Targets><Target field="prediction" rescaleConstant="{float(np.ravel(m.bias)[0])!r}"/></Targets>')
    out.append('    <Segmentation multipleModelMethod="sum">')

    def emit(ns, node, pred, indent):
        pad = " " * indent
        si = int(ns.split_of_node[node])
        if si < 0:
            score = float(ns.leaf_values[int(ns.leaf_of_node[node])][0] * m.scale)
            out.append(f'{pad}<Node score="{score!r}">{pred}</Node>')
            return
        sp = m.splits[si]
        nm = names[m.float_features[sp.feature].flat_index]
        out.append(f'{pad}<Node>{pred}')
        emit(ns, int(ns.right[node]), f'<SimplePredicate field="{nm}" operator="greaterThan" value="{float(sp.border)!r}"/>', indent + 2)
        emit(ns, int(ns.left[node]), '<True/>', indent + 2)
        out.append(f'{pad}</Node>')

    for k, ns in enumerate(trees):
        out.append(f'      <Segment id="{k}"><True/>')
        out.append('        <TreeModel functionName="regression" missingValueStrategy="defaultChild" splitCharacteristic="binarySplit">')
        out.append('          <MiningSchema>' + "".join(f'<MiningField name="{names[c]}"/>' for c in used) + '</MiningSchema>')
        emit(ns, 0, '<True/>', 10)
        out.append('        </TreeModel>')
        out.append('      </Segment>')
    out += ['    </Segmentation>', '  </MiningModel>', '</PMML>']
    return "\n".join(out)


# ---- CoreML -------------------------------------------------------------------------------------------------
def _f_double(field, v):
    return _key(field, 1) + struct.pack("<d", float(v))


def model_to_coreml_bytes(m: Model, export_parameters=None) -> bytes:
    """CoreML ``Model`` with a TreeEnsembleRegressor (field numbers of Model.proto, TreeEnsemble.proto and
    FeatureTypes.proto of the CoreML specification; the reference writes the same structure in
    catboost/libs/model/model_export/coreml_helpers.cpp).  Every feature of the dataset is a double input named after
    the feature; the output ``prediction`` is the raw formula value, or the probability of the positive class with
    ``export_parameters={'prediction_type': 'probability'}`` on a binary classifier (logistic post-transform).  A split
    ``value > border`` is the node behaviour BranchOnValueGreaterThan."""
    trees = _flatten_trees(m)
    params = dict(export_parameters or {})
    want_proba = str(params.get("prediction_type", "raw")).lower() == "probability"
    if want_proba and not (m.dims == 1 and m.class_names is not None):
        raise CatBoostError("prediction_type 'probability' is exported for binary classifiers")
    dims = m.dims
    nodes = b""
    for ti, ns in enumerate(trees):
        for node in range(len(ns.split_of_node)):
            si = int(ns.split_of_node[node])
            body = _f_varint(1, ti) + _f_varint(2, node)
            if si >= 0:
                sp = m.splits[si]
                ff = m.float_features[sp.feature]
                body += _f_varint(3, 3) + _f_varint(10, ff.flat_index) + _f_double(11, sp.border) + \
                    _f_varint(12, int(ns.right[node])) + _f_varint(13, int(ns.left[node]))
                if ff.nan_mode == "Max":
                    body += _f_varint(14, 1)
            else:
                body += _f_varint(3, 6)
                lv = ns.leaf_values[int(ns.leaf_of_node[node])] * m.scale
                for d in range(dims):
                    body += _f_bytes(20, (_f_varint(1, d) if d else b"") + _f_double(2, lv[d]))
            nodes += _f_bytes(1, body)
    bias = [float(b) for b in np.broadcast_to(m.bias, (dims,))]
    ensemble = nodes + _f_varint(2, dims) + _f_bytes(3, b"".join(struct.pack("<d", b) for b in bias))
    regressor = _f_bytes(1, ensemble) + (_f_varint(2, 2) if want_proba else b"")
    double_type = _f_bytes(2, b"")                                   # FeatureType { doubleType {} }
    inputs = b"".join(_f_bytes(1, _f_str(1, str(nm)) + _f_bytes(3, double_type)) for nm in m.feature_names)
    if dims == 1:
        out_type = double_type
    else:
        out_type = _f_bytes(5, _packed_ints(1, [dims]) + _f_varint(2, 65600))     # multiArrayType { shape, DOUBLE }
    output = _f_bytes(10, _f_str(1, "prediction") + _f_bytes(3, out_type))
    meta = _f_str(1, "catboost_b200 model") + _f_str(2, "0.1")
    for k_, v_ in sorted(m.info.items()):
        if k_ in ("params", "model_guid", "catboost_version_info"):
            meta += _f_bytes(100, _f_str(1, k_) + _f_str(2, str(v_)))
    description = inputs + output + _f_str(11, "prediction") + _f_bytes(100, meta)
    return _f_varint(1, 1) + _f_bytes(2, description) + _f_bytes(302, regressor)
