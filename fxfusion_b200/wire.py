"""Graph file format: the FlatBuffers `Graph` the reference serializer emits.

Schema (reference schema/graph.fbs:1-68), field ids in declaration order:

    Tensor { id:uint(0) kind:byte(1) offset:long=-1(2) size_bytes:ulong(3) shape:[long](4)
             dtype:byte(5) alias_of:int=-1(6) data:[ubyte](7) }
    Node   { op_code:byte(0) input_ids:[uint](1) output_ids:[uint](2)
             int_params:[long](3) float_params:[float](4) }
    Graph  { name:string(0) arena_size:ulong(1) tensors:[Tensor](2) nodes:[Node](3) }

Neither `flatc` nor the `flatbuffers` package is needed: this module writes and reads the
FlatBuffers binary encoding directly (little-endian scalars, vtables, uoffset-relative
references).  The writer lays objects out front-to-back (parents before children), which the
encoding allows because every uoffset still points forward.  Scalars equal to their schema
default are omitted, as the official builders do, so readers must apply the defaults
`offset=-1` and `alias_of=-1` (reference serializer.py:279-296 only adds them when an
allocation record exists).
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np

# enums (reference schema/graph.fbs:3-40)
KIND_INPUT, KIND_CONSTANT, KIND_ACTIVATION, KIND_ALIAS, KIND_OUTPUT = range(5)
KIND_NAMES = ["input", "const", "activation", "alias", "output"]
DT_F32, DT_F16, DT_I32, DT_I64, DT_BOOL = range(5)
DTYPE_NAMES = ["float32", "float16", "int32", "int64", "bool"]
DTYPE_ITEMSIZE = [4, 2, 4, 8, 1]
NP_DTYPES = [np.float32, np.float16, np.int32, np.int64, np.bool_]

OPCODES = ("NoOp Conv2d Conv2dRelu Linear LinearRelu Add AddRelu Relu Mul MaxPool2d AvgPool2d "
           "AdaptiveAvgPool2d Transpose Size Narrow Embedding LayerNorm AddLayerNorm MHA "
           "FeedForward CrossMHA CachedMHA").split()  # CrossMHA (20) and CachedMHA (21) are this library's extensions, not in schema/graph.fbs
OP = {name: i for i, name in enumerate(OPCODES)}


@dataclass
class TensorRec:
    id: int = 0
    kind: int = KIND_INPUT
    offset: int = -1
    size_bytes: int = 0
    shape: Sequence[int] = ()
    dtype: int = DT_F32
    alias_of: int = -1
    data: Optional[object] = None  # bytes / memoryview / numpy array (raw little-endian payload)

    def numel(self) -> int:
        n = 1
        for d in self.shape:
            n *= int(d)
        return n

    def array(self) -> np.ndarray:
        """Constant payload as a numpy array of the tensor's dtype and shape."""
        if self.data is None:
            raise ValueError(f"tensor {self.id} carries no data")
        raw = self.data if isinstance(self.data, np.ndarray) else np.frombuffer(self.data, dtype=np.uint8)
        return raw.view(np.uint8).reshape(-1).view(NP_DTYPES[self.dtype]).reshape(tuple(self.shape))


@dataclass
class NodeRec:
    op_code: int = 0
    input_ids: List[int] = field(default_factory=list)
    output_ids: List[int] = field(default_factory=list)
    int_params: List[int] = field(default_factory=list)
    float_params: List[float] = field(default_factory=list)


@dataclass
class GraphRec:
    name: str = "model"
    arena_size: int = 0
    tensors: List[TensorRec] = field(default_factory=list)
    nodes: List[NodeRec] = field(default_factory=list)


# --------------------------------------------------------------------------------------
# writer
# --------------------------------------------------------------------------------------
class _Writer:
    """Front-to-back FlatBuffers emitter.  Position 0 of `buf` is 8-byte aligned by contract."""

    def __init__(self) -> None:
        self.buf = bytearray()

    def pad_to(self, align: int, bias: int = 0) -> None:
        """Pad until (len + bias) % align == 0."""
        while (len(self.buf) + bias) % align:
            self.buf.append(0)

    def patch_uoffset(self, field_pos: int, target_pos: int) -> None:
        assert target_pos > field_pos
        struct.pack_into("<I", self.buf, field_pos, target_pos - field_pos)

    def table(self, fields):
        """Emit vtable + table.  `fields` = list of (field_id, fmt_char_or_'ref', value) with
        absent fields already removed.  Returns (table_pos, {field_id: field_pos}) so callers can
        patch reference fields once the children are placed."""
        size_of = {"B": 1, "b": 1, "I": 4, "i": 4, "q": 8, "Q": 8, "f": 4, "ref": 4}
        n_slots = (max(f[0] for f in fields) + 1) if fields else 0
        # inline layout: soffset(4) pad(4) | 8-byte | 4-byte | 1-byte fields
        order = sorted(fields, key=lambda f: -size_of[f[1]])
        has8 = any(size_of[f[1]] == 8 for f in fields)
        cursor = 8 if has8 else 4
        rel = {}
        for fid, kind, _ in order:
            sz = size_of[kind]
            cursor = (cursor + sz - 1) // sz * sz
            rel[fid] = cursor
            cursor += sz
        inline_size = (cursor + 3) // 4 * 4
        vt_size = 4 + 2 * n_slots
        # vtable (2-aligned) immediately followed by padding so the table is 8-aligned
        self.pad_to(2)
        self.pad_to(8, bias=vt_size)
        vt_pos = len(self.buf)
        self.buf += struct.pack("<HH", vt_size, inline_size)
        for slot in range(n_slots):
            self.buf += struct.pack("<H", rel.get(slot, 0))
        t_pos = len(self.buf)
        assert t_pos % 8 == 0
        self.buf += bytes(inline_size)
        struct.pack_into("<i", self.buf, t_pos, t_pos - vt_pos)
        pos = {}
        for fid, kind, value in fields:
            p = t_pos + rel[fid]
            pos[fid] = p
            if kind != "ref":
                struct.pack_into("<" + kind, self.buf, p, value)
        return t_pos, pos

    def scalar_vector(self, field_pos: int, payload, count: int, elem_size: int) -> None:
        """Emit `u32 count` + payload so that the payload is `elem_size`-aligned."""
        self.pad_to(max(elem_size, 4), bias=4)
        self.pad_to(4)
        start = len(self.buf)
        self.patch_uoffset(field_pos, start)
        self.buf += struct.pack("<I", count)
        self.buf += payload

    def string(self, field_pos: int, s: str) -> None:
        raw = s.encode("utf-8")
        self.pad_to(4)
        self.patch_uoffset(field_pos, len(self.buf))
        self.buf += struct.pack("<I", len(raw)) + raw + b"\0"


def _payload_bytes(data) -> memoryview:
    if isinstance(data, np.ndarray):
        return memoryview(np.ascontiguousarray(data).reshape(-1).view(np.uint8))
    return memoryview(data).cast("B")


def _emit_tensor(w: _Writer, t: TensorRec) -> int:
    fields = []
    if t.id != 0:
        fields.append((0, "I", int(t.id)))
    if t.kind != 0:
        fields.append((1, "b", int(t.kind)))
    if t.offset != -1:
        fields.append((2, "q", int(t.offset)))
    if t.size_bytes != 0:
        fields.append((3, "Q", int(t.size_bytes)))
    fields.append((4, "ref", None))  # shape always written (reference serializer.py:283)
    if t.dtype != 0:
        fields.append((5, "b", int(t.dtype)))
    if t.alias_of != -1:
        fields.append((6, "i", int(t.alias_of)))
    if t.data is not None:
        fields.append((7, "ref", None))
    t_pos, pos = w.table(fields)
    shape = [int(d) for d in t.shape]
    w.scalar_vector(pos[4], struct.pack(f"<{len(shape)}q", *shape), len(shape), 8)
    if t.data is not None:
        raw = _payload_bytes(t.data)
        w.scalar_vector(pos[7], raw, len(raw), 1)
    return t_pos


def _emit_node(w: _Writer, n: NodeRec) -> int:
    fields = []
    if n.op_code != 0:
        fields.append((0, "b", int(n.op_code)))
    fields += [(1, "ref", None), (2, "ref", None), (3, "ref", None), (4, "ref", None)]
    t_pos, pos = w.table(fields)
    w.scalar_vector(pos[1], struct.pack(f"<{len(n.input_ids)}I", *n.input_ids), len(n.input_ids), 4)
    w.scalar_vector(pos[2], struct.pack(f"<{len(n.output_ids)}I", *n.output_ids), len(n.output_ids), 4)
    w.scalar_vector(pos[3], struct.pack(f"<{len(n.int_params)}q", *[int(v) for v in n.int_params]),
                    len(n.int_params), 8)
    w.scalar_vector(pos[4], struct.pack(f"<{len(n.float_params)}f", *n.float_params),
                    len(n.float_params), 4)
    return t_pos


def _emit_table_vector(w: _Writer, field_pos: int, items, emit) -> None:
    w.pad_to(4)
    vec_pos = len(w.buf)
    w.patch_uoffset(field_pos, vec_pos)
    w.buf += struct.pack("<I", len(items))
    slots = len(w.buf)
    w.buf += bytes(4 * len(items))
    for i, item in enumerate(items):
        t_pos = emit(w, item)
        w.patch_uoffset(slots + 4 * i, t_pos)


def dumps(g: GraphRec) -> bytearray:
    """Serialise a graph to FlatBuffers bytes with root type `Graph`."""
    w = _Writer()
    w.buf += bytes(8)  # root uoffset + padding keeps the root table 8-aligned
    fields = [(0, "ref", None)]
    if g.arena_size != 0:
        fields.append((1, "Q", int(g.arena_size)))
    fields += [(2, "ref", None), (3, "ref", None)]
    root_pos, pos = w.table(fields)
    struct.pack_into("<I", w.buf, 0, root_pos)
    w.string(pos[0], g.name)
    _emit_table_vector(w, pos[2], g.tensors, _emit_tensor)
    _emit_table_vector(w, pos[3], g.nodes, _emit_node)
    return w.buf


def dump(g: GraphRec, path) -> str:
    data = dumps(g)
    with open(path, "wb") as f:
        f.write(data)
    return str(path)


# --------------------------------------------------------------------------------------
# reader
# --------------------------------------------------------------------------------------
class WireError(ValueError):
    pass


class _Table:
    def __init__(self, buf: memoryview, pos: int) -> None:
        if pos < 0 or pos + 4 > len(buf):
            raise WireError("table position out of bounds")
        self.buf, self.pos = buf, pos
        soff = struct.unpack_from("<i", buf, pos)[0]
        self.vt = pos - soff
        if self.vt < 0 or self.vt + 4 > len(buf):
            raise WireError("vtable out of bounds")
        self.vt_size = struct.unpack_from("<H", buf, self.vt)[0]
        if self.vt_size < 4 or self.vt + self.vt_size > len(buf):
            raise WireError("bad vtable size")

    def _field(self, fid: int, size: int) -> int:
        slot = 4 + 2 * fid
        if slot + 2 > self.vt_size:
            return 0
        rel = struct.unpack_from("<H", self.buf, self.vt + slot)[0]
        if rel == 0:
            return 0
        p = self.pos + rel
        if p + size > len(self.buf):
            raise WireError("field out of bounds")
        return p

    def scalar(self, fid: int, fmt: str, default):
        p = self._field(fid, struct.calcsize(fmt))
        return default if p == 0 else struct.unpack_from("<" + fmt, self.buf, p)[0]

    def ref(self, fid: int) -> int:
        p = self._field(fid, 4)
        if p == 0:
            return 0
        return p + struct.unpack_from("<I", self.buf, p)[0]

    def vector(self, fid: int, elem_size: int):
        p = self.ref(fid)
        if p == 0:
            return 0, 0
        if p + 4 > len(self.buf):
            raise WireError("vector header out of bounds")
        n = struct.unpack_from("<I", self.buf, p)[0]
        if p + 4 + n * elem_size > len(self.buf):
            raise WireError("vector payload out of bounds")
        return p + 4, n


def _scalars(t: _Table, fid: int, fmt: str):
    start, n = t.vector(fid, struct.calcsize(fmt))
    return list(struct.unpack_from(f"<{n}{fmt}", t.buf, start)) if n else []


def loads(data, copy_constants: bool = False) -> GraphRec:
    """Parse FlatBuffers bytes.  Constant payloads are zero-copy numpy views unless asked."""
    buf = memoryview(data).cast("B")
    if len(buf) < 8:
        raise WireError("file too small to be a graph")
    root = _Table(buf, struct.unpack_from("<I", buf, 0)[0])
    g = GraphRec()
    p = root.ref(0)
    if p:
        n = struct.unpack_from("<I", buf, p)[0]
        g.name = bytes(buf[p + 4:p + 4 + n]).decode("utf-8")
    g.arena_size = root.scalar(1, "Q", 0)
    start, n = root.vector(2, 4)
    for i in range(n):
        fp = start + 4 * i
        t = _Table(buf, fp + struct.unpack_from("<I", buf, fp)[0])
        rec = TensorRec(
            id=t.scalar(0, "I", 0), kind=t.scalar(1, "b", 0), offset=t.scalar(2, "q", -1),
            size_bytes=t.scalar(3, "Q", 0), shape=tuple(_scalars(t, 4, "q")),
            dtype=t.scalar(5, "b", 0), alias_of=t.scalar(6, "i", -1))
        ds, dn = t.vector(7, 1)
        if ds:
            arr = np.frombuffer(buf, dtype=np.uint8, count=dn, offset=ds)
            rec.data = arr.copy() if copy_constants else arr
        g.tensors.append(rec)
    start, n = root.vector(3, 4)
    for i in range(n):
        fp = start + 4 * i
        t = _Table(buf, fp + struct.unpack_from("<I", buf, fp)[0])
        g.nodes.append(NodeRec(op_code=t.scalar(0, "b", 0), input_ids=_scalars(t, 1, "I"),
                               output_ids=_scalars(t, 2, "I"), int_params=_scalars(t, 3, "q"),
                               float_params=_scalars(t, 4, "f")))
    return g


def load(path, copy_constants: bool = False) -> GraphRec:
    return loads(np.fromfile(path, dtype=np.uint8), copy_constants)
