"""Compile side: drive the reference's own, unchanged FX passes and emit a graph file.

The reference pipeline is FusionPass -> ShapePropPass -> MemoryPlanningPass -> Serializer
(py/fxfusion/compiler.py:17-48).  The first three are used as they are.  The reference
Serializer needs the `flatbuffers` package and flatc-generated `gen.fxfusion.*` modules; its
node classification (`_node_opcode_and_params`, serializer.py:114-185) and the per-node metadata
the passes leave behind (`meta["id"|"kind"|"alloc"|"shape"|"dtype"]`) are all that is needed to
fill a `wire.GraphRec`, which this package's own FlatBuffers writer then encodes.  When
`flatbuffers`/`gen` are not installed, inert stand-in modules are registered so that the
reference `serializer` module can be imported for that classification logic only.

The reference package `fxfusion` must be importable: put its `py/` directory on sys.path or
point the environment variable FXFUSION_REFERENCE_PY at it.
"""
from __future__ import annotations

import os
import sys
import types
from typing import Optional, Sequence, Tuple

from . import wire
from .wire import GraphRec, NodeRec, TensorRec


def _ensure_reference_importable() -> None:
    try:
        import fxfusion.passes.fusion_pass  # noqa: F401
        return
    except ImportError:
        pass
    path = os.environ.get("FXFUSION_REFERENCE_PY")
    if path and os.path.isdir(path):
        sys.path.insert(0, path)
    try:
        import fxfusion.passes.fusion_pass  # noqa: F401
    except ImportError as exc:
        raise RuntimeError(
            "the reference compile passes (package `fxfusion`) are not importable; install the reference or set "
            "FXFUSION_REFERENCE_PY to its py/ directory") from exc


def _install_serializer_stubs() -> None:
    """Stand-ins for `flatbuffers` and `gen.fxfusion.*` (enum values from schema/graph.fbs)."""
    if "flatbuffers" not in sys.modules:
        try:
            import flatbuffers  # noqa: F401
        except ImportError:
            fb = types.ModuleType("flatbuffers")
            fb.Builder = lambda n: None
            sys.modules["flatbuffers"] = fb
    try:
        import gen.fxfusion.OpCode  # noqa: F401
        return
    except ImportError:
        pass
    gen = types.ModuleType("gen")
    genf = types.ModuleType("gen.fxfusion")
    sys.modules["gen"], sys.modules["gen.fxfusion"] = gen, genf
    enums = {
        "OpCode": wire.OPCODES,
        "TensorKind": ["Input", "Constant", "Activation", "Alias", "Output"],
        "DType": ["Float32", "Float16", "Int32", "Int64", "Bool"],
        "Graph": [], "Node": [], "Tensor": [],
    }
    for name, members in enums.items():
        mod = types.ModuleType(f"gen.fxfusion.{name}")
        cls = type(name, (), {m: i for i, m in enumerate(members)})
        setattr(mod, name, cls)
        sys.modules[f"gen.fxfusion.{name}"] = mod
        setattr(genf, name, mod)


def lower_with_reference(model, example_inputs: Sequence, memory_alignment: int = 64, DEBUG: bool = False):
    """Runs the reference passes; returns the annotated fx GraphModule."""
    _ensure_reference_importable()
    import torch
    from fxfusion.passes.fusion_pass import FusionPass
    from fxfusion.passes.memory_plan import MemoryPlanningPass
    from fxfusion.passes.shape_prop import ShapePropPass

    if model.training:
        raise RuntimeError("FXFusion only supports inference graphs. Call model.eval() before compiling.")
    with torch.inference_mode():
        fx_model = FusionPass().run(model, device="cpu")
        if DEBUG:
            fx_model.graph.print_tabular()
        ShapePropPass(fx_model).propagate(*example_inputs)
        MemoryPlanningPass(fx_model, alignment=memory_alignment).run()
    return fx_model


def graph_from_fx(fx_model, model_name: str) -> GraphRec:
    """What the reference Serializer.run would write (serializer.py:34-69), as a GraphRec."""
    _install_serializer_stubs()
    import torch
    from fxfusion.serializer import Serializer

    ser = Serializer(fx_model, model_name=model_name)
    ser._validate_metadata()
    kind_code = {"input": wire.KIND_INPUT, "const": wire.KIND_CONSTANT, "activation": wire.KIND_ACTIVATION,
                 "alias": wire.KIND_ALIAS, "output": wire.KIND_OUTPUT}
    dtype_code = {torch.float32: wire.DT_F32, torch.float16: wire.DT_F16, torch.int32: wire.DT_I32,
                  torch.int64: wire.DT_I64, torch.bool: wire.DT_BOOL}
    g = GraphRec(name=model_name, arena_size=int(fx_model.meta["arena_size"]))
    for node in fx_model.graph.nodes:
        alloc = node.meta.get("alloc")
        dt = node.meta.get("dtype")
        if dt not in dtype_code:
            raise RuntimeError(f"Unsupported dtype: {dt}")
        rec = TensorRec(id=int(node.meta["id"]), kind=kind_code[node.meta["kind"]],
                        shape=tuple(int(d) for d in (node.meta.get("shape") or ())), dtype=dtype_code[dt])
        if alloc is not None:
            rec.offset = alloc.mem_offset if alloc.mem_offset is not None else -1
            rec.size_bytes = int(alloc.size_bytes)
            rec.alias_of = ser._alias_of(alloc)
        if node.meta.get("kind") == "const":
            value = ser._fetch_attr(str(node.target))
            if not isinstance(value, torch.Tensor):
                raise TypeError(f"Unsupported const type for {node.name}: {type(value)}")
            rec.data = value.detach().contiguous().cpu().numpy()
        g.tensors.append(rec)
        res = ser._node_opcode_and_params(node)
        if res is not None:
            opcode, ints, floats = res
            g.nodes.append(NodeRec(op_code=int(opcode), input_ids=ser._input_ids_for_node(node),
                                   output_ids=[int(node.meta["id"])], int_params=[int(v) for v in ints],
                                   float_params=[float(v) for v in floats]))
    return g


def compile_with_reference(model, example_inputs: Sequence, model_name: Optional[str] = None, DEBUG: bool = False,
                           memory_alignment: int = 64) -> Tuple[object, GraphRec]:
    name = model_name or model.__class__.__name__.lower()
    fx_model = lower_with_reference(model, example_inputs, memory_alignment, DEBUG)
    return fx_model, graph_from_fx(fx_model, name)
