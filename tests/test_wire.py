"""Graph-file encoding: the Python writer/reader against the FlatBuffers binary layout."""
import struct

import numpy as np
import pytest

from fxfusion_b200 import wire
from fxfusion_b200.wire import GraphRec, NodeRec, TensorRec


def small_graph():
    g = GraphRec(name="tiny", arena_size=256)
    g.tensors = [
        TensorRec(id=0, kind=wire.KIND_INPUT, size_bytes=64, shape=(1, 7), dtype=wire.DT_F32),
        TensorRec(id=1, kind=wire.KIND_CONSTANT, size_bytes=1792, shape=(63, 7), dtype=wire.DT_F32,
                  data=np.arange(63 * 7, dtype=np.float32).reshape(63, 7)),
        TensorRec(id=2, kind=wire.KIND_CONSTANT, size_bytes=256, shape=(63,), dtype=wire.DT_F32, data=np.ones(63, np.float32)),
        TensorRec(id=3, kind=wire.KIND_ACTIVATION, offset=0, size_bytes=256, shape=(1, 63), dtype=wire.DT_F32),
        TensorRec(id=4, kind=wire.KIND_OUTPUT, offset=0, size_bytes=256, shape=(1, 63), dtype=wire.DT_F32, alias_of=3),
    ]
    g.nodes = [NodeRec(0, [], [0]), NodeRec(0, [], [1]), NodeRec(0, [], [2]),
               NodeRec(wire.OP["Linear"], [0, 1, 2], [3]), NodeRec(0, [3], [4])]
    return g


def test_round_trip_preserves_every_field():
    g = small_graph()
    g.nodes.append(NodeRec(wire.OP["LayerNorm"], [3, 2, 2], [3], [1, 63], [1e-5]))
    g2 = wire.loads(wire.dumps(g))
    assert (g2.name, g2.arena_size) == ("tiny", 256)
    for a, b in zip(g.tensors, g2.tensors):
        assert (a.id, a.kind, a.offset, a.size_bytes, tuple(a.shape), a.dtype, a.alias_of) == \
               (b.id, b.kind, b.offset, b.size_bytes, tuple(b.shape), b.dtype, b.alias_of)
        if a.data is not None:
            assert np.array_equal(b.array(), a.data)
        else:
            assert b.data is None
    for a, b in zip(g.nodes, g2.nodes):
        assert (a.op_code, a.input_ids, a.output_ids, a.int_params) == (b.op_code, b.input_ids, b.output_ids, b.int_params)
        assert np.allclose(a.float_params, b.float_params, rtol=1e-7)


def test_layout_follows_flatbuffers_rules():
    """Walk the bytes by hand: root uoffset, vtable via soffset, field offsets, aligned vectors."""
    buf = bytes(wire.dumps(small_graph()))
    root = struct.unpack_from("<I", buf, 0)[0]
    vt = root - struct.unpack_from("<i", buf, root)[0]
    vt_size, inline = struct.unpack_from("<HH", buf, vt)
    assert vt_size == 4 + 2 * 4  # Graph has four fields
    slots = struct.unpack_from("<4H", buf, vt + 4)
    assert all(0 < s < inline for s in slots)
    # arena_size is a ulong stored inline and 8-byte aligned
    assert (root + slots[1]) % 8 == 0
    assert struct.unpack_from("<Q", buf, root + slots[1])[0] == 256
    # name string: uoffset -> u32 length + bytes + NUL
    p = root + slots[0]
    p += struct.unpack_from("<I", buf, p)[0]
    n = struct.unpack_from("<I", buf, p)[0]
    assert buf[p + 4:p + 4 + n] == b"tiny" and buf[p + 4 + n] == 0
    # tensors vector: 5 table offsets, each pointing forward to a table with a valid vtable
    p = root + slots[2]
    p += struct.unpack_from("<I", buf, p)[0]
    assert struct.unpack_from("<I", buf, p)[0] == 5
    t1 = p + 4 + 4 + struct.unpack_from("<I", buf, p + 8)[0]  # second tensor
    vt1 = t1 - struct.unpack_from("<i", buf, t1)[0]
    f = struct.unpack_from("<8H", buf, vt1 + 4)
    assert f[2] == 0, "offset == -1 is the schema default and must be omitted"
    assert f[6] == 0, "alias_of == -1 is the schema default and must be omitted"
    assert struct.unpack_from("<I", buf, t1 + f[0])[0] == 1          # id
    assert struct.unpack_from("<b", buf, t1 + f[1])[0] == wire.KIND_CONSTANT
    sp = t1 + f[4]
    sp += struct.unpack_from("<I", buf, sp)[0]
    assert struct.unpack_from("<I", buf, sp)[0] == 2 and (sp + 4) % 8 == 0  # [long] payload 8-aligned
    assert struct.unpack_from("<2q", buf, sp + 4) == (63, 7)


def test_defaults_apply_when_fields_are_absent():
    g = GraphRec(name="d", arena_size=0, tensors=[TensorRec(shape=())], nodes=[NodeRec()])
    g2 = wire.loads(wire.dumps(g))
    t = g2.tensors[0]
    assert (t.id, t.kind, t.offset, t.size_bytes, t.dtype, t.alias_of, t.data) == (0, 0, -1, 0, 0, -1, None)
    assert g2.nodes[0].op_code == 0 and g2.nodes[0].input_ids == []


def test_empty_and_scalar_shapes():
    g = GraphRec(name="", tensors=[TensorRec(id=0, shape=(), dtype=wire.DT_I64, kind=wire.KIND_ACTIVATION, offset=0, size_bytes=64),
                                    TensorRec(id=1, shape=(0, 4), kind=wire.KIND_CONSTANT, data=np.zeros((0, 4), np.float32))])
    g2 = wire.loads(wire.dumps(g))
    assert g2.tensors[0].shape == () and g2.tensors[0].numel() == 1
    assert g2.tensors[1].shape == (0, 4) and g2.tensors[1].array().shape == (0, 4)


@pytest.mark.parametrize("cut", [0, 3, 7, 20, 100, 500])
def test_truncated_file_is_rejected_not_misread(cut):
    buf = bytes(wire.dumps(small_graph()))
    with pytest.raises((wire.WireError, struct.error)):
        wire.loads(buf[:cut])


def test_large_constant_is_zero_copy_on_read():
    data = np.random.default_rng(0).standard_normal((300, 100)).astype(np.float32)
    g = GraphRec(name="c", tensors=[TensorRec(id=0, kind=wire.KIND_CONSTANT, shape=data.shape, data=data)])
    raw = np.frombuffer(bytes(wire.dumps(g)), dtype=np.uint8)
    g2 = wire.loads(raw)
    arr = g2.tensors[0].array()
    assert np.array_equal(arr, data)
    assert np.shares_memory(arr, raw)
