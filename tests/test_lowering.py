"""Lowered-graph builders and the restated memory planner."""
import numpy as np
import pytest

from fxfusion_b200 import lowering, wire
from fxfusion_b200.lowering import GraphBuilder


def test_planner_known_answer_linear_7_63():
    """Reference known answer: Linear(7,63) on a batch of 1 -> one 256-byte buffer, arena 256
    (py/tests/test_memory_plan.py:98-120)."""
    b = GraphBuilder("lin", 64)
    x = b.input((1, 7), wire.DT_F32)
    w, bias = b.const(np.zeros((63, 7), np.float32)), b.const(np.zeros(63, np.float32))
    y = b.op("Linear", [x, w, bias], (1, 63))
    b.output(y)
    g = b.finish()
    assert g.arena_size == 256
    assert g.tensors[y].size_bytes == 256 and g.tensors[y].offset == 0
    assert g.tensors[-1].kind == wire.KIND_OUTPUT and g.tensors[-1].alias_of == y and g.tensors[-1].offset == 0


def _live_overlap_free(g):
    """No two simultaneously live arena tensors overlap (py/tests/test_memory_plan.py:123-158)."""
    last = {}
    for i, n in enumerate(g.nodes):
        for j in n.input_ids:
            last[j] = i
    acts = [t for t in g.tensors if t.kind == wire.KIND_ACTIVATION]
    for a in acts:
        for b in acts:
            if a.id >= b.id:
                continue
            a_end = last.get(a.id, a.id)
            # aliases extend the life of their source
            for t in g.tensors:
                if t.kind in (wire.KIND_ALIAS, wire.KIND_OUTPUT) and t.offset == a.offset and t.alias_of == a.id:
                    a_end = max(a_end, last.get(t.id, t.id))
            if b.id <= a_end:  # b is created while a is still live
                assert a.offset + a.size_bytes <= b.offset or b.offset + b.size_bytes <= a.offset, (a, b)


def test_mlp_config_graph():
    layers = lowering.mlp_params(16, 512, 10, seed=0)
    g = lowering.mlp_graph(layers, batch=32)
    ops = [wire.OPCODES[n.op_code] for n in g.nodes if n.op_code]
    assert ops == ["LinearRelu"] * 14 + ["FeedForward"]
    assert g.arena_size == 131072  # two 64 KB ping-pong slots
    offs = sorted({t.offset for t in g.tensors if t.kind == wire.KIND_ACTIVATION})
    assert offs == [0, 65536]
    _live_overlap_free(g)


def test_gpt_c2_graph_matches_probed_plan():
    cfg = lowering.GPT_C2
    g = lowering.gpt_graph(cfg, lowering.gpt_params(cfg, 0), batch=8, seq=64)
    ops = [wire.OPCODES[n.op_code] for n in g.nodes if n.op_code]
    assert len(ops) == 30
    assert ops[:5] == ["Embedding", "Mul", "Size", "Narrow", "Add"]
    assert ops[-2:] == ["AddLayerNorm", "Linear"] and ops.count("MHA") == 4 and ops.count("FeedForward") == 4
    assert g.arena_size == 3096576
    logits = g.tensors[-2]
    assert (logits.offset, logits.size_bytes) == (1048576, 2048000)
    for t in g.tensors:
        if t.offset >= 0:
            assert t.offset % 64 == 0 and t.offset + t.size_bytes <= g.arena_size
    _live_overlap_free(g)


def test_alignment_parameter_is_honoured():
    cfg = lowering.GPTConfig(32, 4, 128, 2, 1)
    g = lowering.gpt_graph(cfg, lowering.gpt_params(cfg, 0), batch=2, seq=8, alignment=256)
    assert all(t.offset % 256 == 0 for t in g.tensors if t.offset >= 0)
    assert all(t.size_bytes % 256 == 0 for t in g.tensors)


def _same_graph(a, b):
    assert (a.arena_size, len(a.tensors), len(a.nodes)) == (b.arena_size, len(b.tensors), len(b.nodes))
    for x, y in zip(a.tensors, b.tensors):
        assert (x.id, x.kind, x.offset, x.size_bytes, tuple(x.shape), x.dtype, x.alias_of) == \
               (y.id, y.kind, y.offset, y.size_bytes, tuple(y.shape), y.dtype, y.alias_of)
        if x.data is not None:
            assert np.array_equal(np.asarray(x.data).view(np.uint8).ravel(), np.asarray(y.data).view(np.uint8).ravel())
    for x, y in zip(a.nodes, b.nodes):
        assert (x.op_code, x.input_ids, x.output_ids, x.int_params) == (y.op_code, y.input_ids, y.output_ids, y.int_params)
        assert np.allclose(x.float_params, y.float_params, rtol=1e-7)


def load_gpt_params_into(model, cfg, p):
    import torch
    D = cfg.d_model
    sd = {"norm.weight": p["ln_f.w"], "norm.bias": p["ln_f.b"], "in_embedding.embedding.weight": p["emb"],
          "pos_encoding.pe": p["pe"], "linear.weight": p["head.w"], "linear.bias": p["head.b"]}
    for l in range(cfg.layers):
        pre = f"gpt_blocks.{l}."
        for j, n in enumerate("qkv"):
            sd[pre + f"mha.W_{n}.weight"] = p[f"l{l}.qkv.w"][j * D:(j + 1) * D]
            sd[pre + f"mha.W_{n}.bias"] = p[f"l{l}.qkv.b"][j * D:(j + 1) * D]
        for mine, theirs in (("wo", "mha.W_o"), ("ff1", "ff.linear1"), ("ff2", "ff.linear2"), ("ln1", "norm1"), ("ln2", "norm2")):
            sd[pre + theirs + ".weight"] = p[f"l{l}.{mine}.w"]
            sd[pre + theirs + ".bias"] = p[f"l{l}.{mine}.b"]
    model.load_state_dict({k: torch.from_numpy(np.array(v)) for k, v in sd.items()})


def test_gpt_builder_equals_reference_passes(reference_py):
    """The direct builder must emit exactly what the reference's FusionPass + ShapePropPass +
    MemoryPlanningPass + serializer logic produce for the reference's own GPT module."""
    import torch
    from fxfusion.models.transformer.models.gpt import GPT
    from fxfusion_b200.compile_ref import compile_with_reference
    cfg = lowering.GPTConfig(32, 4, 128, 2, 2)
    p = lowering.gpt_params(cfg, seed=3)
    model = GPT(32, 4, 128, 2, 0.0, 2).eval()
    assert np.array_equal(model.pos_encoding.pe.numpy(), p["pe"]), "positional-encoding table must be bit-identical"
    load_gpt_params_into(model, cfg, p)
    tokens = torch.zeros((2, 8), dtype=torch.int64)
    mask = torch.ones((2, 1, 8, 8), dtype=torch.bool)
    _, ref = compile_with_reference(model, [tokens, mask], model_name="gpt")
    _same_graph(ref, lowering.gpt_graph(cfg, p, 2, 8))


def test_mlp_builder_equals_reference_passes(reference_py):
    import torch
    import torch.nn as nn
    from fxfusion_b200.compile_ref import compile_with_reference
    layers = lowering.mlp_params(5, 32, 10, seed=1)
    mods = []
    for i, (w, b) in enumerate(layers):
        lin = nn.Linear(w.shape[1], w.shape[0])
        lin.weight.data = torch.from_numpy(w.copy())
        lin.bias.data = torch.from_numpy(b.copy())
        mods.append(lin)
        if i < len(layers) - 1:
            mods.append(nn.ReLU())
    _, ref = compile_with_reference(nn.Sequential(*mods).eval(), [torch.randn(4, 32)], model_name="mlp")
    _same_graph(ref, lowering.mlp_graph(layers, 4))


def test_resnet50_builder_equals_reference_passes(reference_py):
    """torchvision's ResNet-50 lowered by the reference passes == the direct builder: op sequence, params, tensor
    table, offsets and arena size (27 295 744 bytes at batch 2)."""
    torch = pytest.importorskip("torch")
    tv = pytest.importorskip("torchvision")
    from fxfusion_b200.compile_ref import compile_with_reference
    _, ref = compile_with_reference(tv.models.resnet50(weights=None).eval(), [torch.randn(2, 3, 224, 224)], model_name="r50")
    mine = lowering.resnet50_graph(lowering.resnet50_params(0), 2)
    assert ref.arena_size == mine.arena_size == 27295744
    assert [(n.op_code, n.input_ids, n.output_ids, n.int_params) for n in ref.nodes] == [(n.op_code, n.input_ids, n.output_ids, n.int_params) for n in mine.nodes]
    for a, b in zip(ref.tensors, mine.tensors):
        assert (a.id, a.kind, a.offset, a.size_bytes, tuple(a.shape), a.dtype, a.alias_of) == (b.id, b.kind, b.offset, b.size_bytes, tuple(b.shape), b.dtype, b.alias_of)
