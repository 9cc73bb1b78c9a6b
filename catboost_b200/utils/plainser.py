"""Plain-data binary container: nested dict / list / tuple / str / bytes / int / float / bool / None / numpy arrays
and instances of an explicit allow-list of classes, written as little-endian PODs with ``ui32`` size prefixes (the
style of the reference's ``ysaveload`` streams, catboost/libs/helpers/progress_helper.h:40-89, util/ysaveload.h).

Loading never executes code from the stream: a class is only ever looked up by name in the registry passed by the
caller, created with ``cls.__new__`` and filled field by field.  Anything else in the stream is rejected.  This is
what model files and snapshots use for state that the FlatBuffers model core has no table for.
"""
from __future__ import annotations

import struct
from typing import Dict, Optional

import numpy as np

_T_NONE, _T_FALSE, _T_TRUE, _T_INT, _T_FLOAT, _T_STR, _T_BYTES, _T_LIST, _T_TUPLE, _T_DICT, _T_ARRAY, _T_OBJ = range(12)
_MAX_DEPTH = 64
_DTYPES = ("bool", "int8", "int16", "int32", "int64", "uint8", "uint16", "uint32", "uint64", "float16", "float32",
           "float64")


class PlainDataError(ValueError):
    pass


def _u32(n: int) -> bytes:
    if n < 0 or n > 0xFFFFFFFF:
        raise PlainDataError("size does not fit the ui32 prefix")
    return struct.pack("<I", n)


def _dump(x, out: list, registry: Dict[str, type], depth: int):
    if depth > _MAX_DEPTH:
        raise PlainDataError("structure is nested too deeply")
    if x is None:
        out.append(bytes([_T_NONE]))
    elif isinstance(x, (bool, np.bool_)):
        out.append(bytes([_T_TRUE if bool(x) else _T_FALSE]))
    elif isinstance(x, (int, np.integer)):
        out.append(bytes([_T_INT]) + struct.pack("<q", int(x)))
    elif isinstance(x, (float, np.floating)):
        out.append(bytes([_T_FLOAT]) + struct.pack("<d", float(x)))
    elif isinstance(x, str):
        b = x.encode("utf-8")
        out.append(bytes([_T_STR]) + _u32(len(b)) + b)
    elif isinstance(x, (bytes, bytearray)):
        out.append(bytes([_T_BYTES]) + _u32(len(x)) + bytes(x))
    elif isinstance(x, (list, tuple)):
        out.append(bytes([_T_LIST if isinstance(x, list) else _T_TUPLE]) + _u32(len(x)))
        for v in x:
            _dump(v, out, registry, depth + 1)
    elif isinstance(x, dict):
        out.append(bytes([_T_DICT]) + _u32(len(x)))
        for k, v in x.items():
            _dump(k, out, registry, depth + 1)
            _dump(v, out, registry, depth + 1)
    elif isinstance(x, np.ndarray):
        if x.dtype.name not in _DTYPES:
            if x.dtype.kind in ("U", "O", "S"):
                _dump([v.item() if hasattr(v, "item") else v for v in x.reshape(-1)], out, registry, depth + 1)
                return
            raise PlainDataError(f"array dtype {x.dtype} is not storable")
        a = np.ascontiguousarray(x)
        if a.dtype.byteorder == ">":
            a = a.astype(a.dtype.newbyteorder("<"))
        raw = a.tobytes()
        out.append(bytes([_T_ARRAY, _DTYPES.index(a.dtype.name)]) + _u32(a.ndim) +
                   b"".join(struct.pack("<q", int(s)) for s in a.shape) + struct.pack("<Q", len(raw)) + raw)
    else:
        name = type(x).__name__
        if registry.get(name) is not type(x):
            raise PlainDataError(f"objects of type {type(x)!r} are not storable")
        fields = dict(vars(x))
        nb = name.encode("utf-8")
        out.append(bytes([_T_OBJ]) + _u32(len(nb)) + nb + _u32(len(fields)))
        for k, v in fields.items():
            _dump(str(k), out, registry, depth + 1)
            _dump(v, out, registry, depth + 1)


def dumps(x, registry: Optional[Dict[str, type]] = None) -> bytes:
    out: list = []
    _dump(x, out, registry or {}, 0)
    return b"".join(out)


class _Reader:
    def __init__(self, blob: bytes):
        self.b, self.p = memoryview(blob), 0

    def take(self, n: int) -> memoryview:
        if n < 0 or self.p + n > len(self.b):
            raise PlainDataError("truncated stream")
        v = self.b[self.p:self.p + n]
        self.p += n
        return v

    def u32(self) -> int:
        return struct.unpack("<I", self.take(4))[0]


def _load(r: _Reader, registry: Dict[str, type], depth: int):
    if depth > _MAX_DEPTH:
        raise PlainDataError("structure is nested too deeply")
    t = r.take(1)[0]
    if t == _T_NONE:
        return None
    if t == _T_FALSE:
        return False
    if t == _T_TRUE:
        return True
    if t == _T_INT:
        return struct.unpack("<q", r.take(8))[0]
    if t == _T_FLOAT:
        return struct.unpack("<d", r.take(8))[0]
    if t == _T_STR:
        return bytes(r.take(r.u32())).decode("utf-8")
    if t == _T_BYTES:
        return bytes(r.take(r.u32()))
    if t in (_T_LIST, _T_TUPLE):
        n = r.u32()
        if n > len(r.b) - r.p:
            raise PlainDataError("truncated stream")
        items = [_load(r, registry, depth + 1) for _ in range(n)]
        return items if t == _T_LIST else tuple(items)
    if t == _T_DICT:
        n = r.u32()
        if n > len(r.b) - r.p:
            raise PlainDataError("truncated stream")
        d = {}
        for _ in range(n):
            k = _load(r, registry, depth + 1)
            if isinstance(k, (list, dict)):
                raise PlainDataError("unhashable dictionary key")
            d[k] = _load(r, registry, depth + 1)
        return d
    if t == _T_ARRAY:
        code = r.take(1)[0]
        if code >= len(_DTYPES):
            raise PlainDataError("unknown array dtype")
        nd = r.u32()
        if nd > 32:
            raise PlainDataError("array rank too large")
        shape = tuple(struct.unpack("<q", r.take(8))[0] for _ in range(nd))
        nbytes = struct.unpack("<Q", r.take(8))[0]
        dt = np.dtype(_DTYPES[code]).newbyteorder("<")
        count = int(np.prod(shape, dtype=np.int64)) if nd else 1
        if any(s < 0 for s in shape) or count * dt.itemsize != nbytes:
            raise PlainDataError("array header does not match its payload")
        return np.frombuffer(bytes(r.take(nbytes)), dtype=dt).reshape(shape).astype(_DTYPES[code], copy=True)
    if t == _T_OBJ:
        name = bytes(r.take(r.u32())).decode("utf-8")
        cls = registry.get(name)
        if cls is None:
            raise PlainDataError(f"stream names a class that may not be loaded: {name!r}")
        obj = cls.__new__(cls)
        for _ in range(r.u32()):
            k = _load(r, registry, depth + 1)
            if not isinstance(k, str) or k.startswith("__"):
                raise PlainDataError("bad field name")
            setattr(obj, k, _load(r, registry, depth + 1))
        return obj
    raise PlainDataError(f"unknown tag {t}")


def loads(blob: bytes, registry: Optional[Dict[str, type]] = None):
    r = _Reader(blob)
    x = _load(r, registry or {}, 0)
    if r.p != len(r.b):
        raise PlainDataError("trailing bytes after the value")
    return x
