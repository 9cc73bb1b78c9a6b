"""A small FlatBuffers encoder / decoder (only what the ``.cbm`` model schema needs).

The ``flatbuffers`` Python package is not a dependency; the wire format is simple enough to emit directly:
little-endian scalars, tables with a vtable (``u16 vtable bytes, u16 table bytes, u16 field offsets...``) reached
through a signed 32-bit back-offset, vectors / strings as ``u32 length + payload``, and unsigned 32-bit forward
offsets between objects.  The builder works back to front (children before parents), tracking positions as
"bytes from the end" exactly like the official builders, so every forward offset is known when it is written.
"""
from __future__ import annotations

import struct
from typing import List, Optional, Sequence, Tuple

import numpy as np


class Builder:
    def __init__(self):
        self.chunks: List[bytes] = []
        self.size = 0
        self.minalign = 1

    # -- low level ------------------------------------------------------------------------------------
    def _push(self, b: bytes):
        self.chunks.append(b)
        self.size += len(b)

    def _prep(self, align: int, additional: int):
        self.minalign = max(self.minalign, align)
        pad = (-(self.size + additional)) % align
        if pad:
            self._push(b"\0" * pad)

    # -- leaves ---------------------------------------------------------------------------------------
    def string(self, s) -> int:
        b = s if isinstance(s, bytes) else str(s).encode("utf-8")
        self._prep(4, len(b) + 1)
        self._push(b + b"\0")
        self._push(struct.pack("<I", len(b)))
        return self.size

    def vector(self, arr, dtype) -> int:
        """Vector of scalars (or of fixed-size structs given as a structured / 2-D array of ``dtype``)."""
        a = np.ascontiguousarray(np.asarray(arr, dtype=dtype))
        raw = a.tobytes()
        count = a.shape[0] if a.ndim else 0
        elem = max(1, np.dtype(dtype).alignment if np.dtype(dtype).fields is None else
                   max(np.dtype(dtype).fields[f][0].alignment for f in np.dtype(dtype).names))
        self._prep(4, len(raw))
        self._prep(elem, len(raw))
        self._push(raw)
        self._push(struct.pack("<I", count))
        return self.size

    def offset_vector(self, offsets: Sequence[int]) -> int:
        self._prep(4, 4 * len(offsets))
        for off in reversed(list(offsets)):
            self._push(struct.pack("<I", self.size + 4 - off))
        self._push(struct.pack("<I", len(offsets)))
        return self.size

    # -- tables ---------------------------------------------------------------------------------------
    def table(self, n_fields: int, fields: Sequence[Tuple[int, str, object]]) -> int:
        """fields: (field id, kind, value); kind is a struct format char (``b B h H i I q Q f d ?``) for a scalar
        or ``'o'`` for an offset returned by another builder call.  Absent / default fields are simply left out."""
        start = self.size
        placed = {}
        order = sorted(fields, key=lambda f: -(4 if f[1] == "o" else struct.calcsize("<" + f[1])))
        for fid, kind, val in order:
            if kind == "o":
                self._prep(4, 0)
                self._push(struct.pack("<I", self.size + 4 - int(val)))
            else:
                sz = struct.calcsize("<" + kind)
                self._prep(sz, 0)
                self._push(struct.pack("<" + kind, val))
            placed[fid] = self.size
        self._prep(4, 0)
        vt_len = 4 + 2 * n_fields
        self._push(struct.pack("<i", vt_len))
        table_off = self.size
        vt = struct.pack("<HH", vt_len, table_off - start)
        for fid in range(n_fields):
            vt += struct.pack("<H", table_off - placed[fid] if fid in placed else 0)
        self._push(vt)     # chunks are emitted in reverse, so the vtable (pushed last) sits right before the table
        return table_off

    def finish(self, root: int) -> bytes:
        self._prep(self.minalign, 4)
        self._push(struct.pack("<I", self.size + 4 - root))
        return b"".join(reversed(self.chunks))


class Table:
    """Read-only view of a table inside a finished buffer."""

    def __init__(self, buf: bytes, pos: int):
        self.buf, self.pos = buf, pos
        self.vt = pos - struct.unpack_from("<i", buf, pos)[0]
        self.vt_len = struct.unpack_from("<H", buf, self.vt)[0]

    @staticmethod
    def root(buf: bytes, offset: int = 0) -> "Table":
        return Table(buf, offset + struct.unpack_from("<I", buf, offset)[0])

    def _field(self, fid: int) -> int:
        o = 4 + 2 * fid
        if o >= self.vt_len:
            return 0
        rel = struct.unpack_from("<H", self.buf, self.vt + o)[0]
        return self.pos + rel if rel else 0

    def scalar(self, fid: int, kind: str, default=0):
        p = self._field(fid)
        return struct.unpack_from("<" + kind, self.buf, p)[0] if p else default

    def _indirect(self, fid: int) -> int:
        p = self._field(fid)
        return p + struct.unpack_from("<I", self.buf, p)[0] if p else 0

    def string(self, fid: int) -> Optional[str]:
        p = self._indirect(fid)
        if not p:
            return None
        n = struct.unpack_from("<I", self.buf, p)[0]
        return self.buf[p + 4: p + 4 + n].decode("utf-8")

    def table(self, fid: int) -> Optional["Table"]:
        p = self._indirect(fid)
        return Table(self.buf, p) if p else None

    def vector(self, fid: int, dtype) -> np.ndarray:
        p = self._indirect(fid)
        if not p:
            return np.zeros(0, dtype=dtype)
        n = struct.unpack_from("<I", self.buf, p)[0]
        return np.frombuffer(self.buf, dtype=dtype, count=n, offset=p + 4).copy()

    def bytes_vector(self, fid: int) -> bytes:
        p = self._indirect(fid)
        if not p:
            return b""
        n = struct.unpack_from("<I", self.buf, p)[0]
        return bytes(self.buf[p + 4: p + 4 + n])

    def table_vector(self, fid: int) -> List["Table"]:
        p = self._indirect(fid)
        if not p:
            return []
        n = struct.unpack_from("<I", self.buf, p)[0]
        out = []
        for i in range(n):
            q = p + 4 + 4 * i
            out.append(Table(self.buf, q + struct.unpack_from("<I", self.buf, q)[0]))
        return out

    def string_vector(self, fid: int) -> List[str]:
        p = self._indirect(fid)
        if not p:
            return []
        n = struct.unpack_from("<I", self.buf, p)[0]
        out = []
        for i in range(n):
            q = p + 4 + 4 * i
            s = q + struct.unpack_from("<I", self.buf, q)[0]
            ln = struct.unpack_from("<I", self.buf, s)[0]
            out.append(self.buf[s + 4: s + 4 + ln].decode("utf-8"))
        return out
