"""Python face of the runtime: `ExecutionEngine` and `Engine`, as the reference exposes them.

Reference:
  * `torch.classes.fxfusion_extension.ExecutionEngine(bin_path, device)` with
    `.run(List[Tensor]) -> List[Tensor]` (csrc/bindings/python_bindings.cpp:8-12,
    csrc/runtime/execution_engine.cpp:12-43);
  * `Engine(model, example_inputs, model_name, device, DEBUG, memory_alignment)` with `.run`
    (py/fxfusion/engine.py:7-35), which compiles with the reference's FX passes first.

Here the class is a thin ctypes client of libfxf_b200.so.  PyTorch appears only as the
container of device memory the caller hands in and gets back: inputs are CUDA tensors, outputs
are CUDA tensors that VIEW engine-owned arena memory and stay valid until the next `run`
(the reference returns arena views too, execution_engine.cpp:42).
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path
from typing import List, Optional, Sequence

import numpy as np

from . import _lib, wire
from ._lib import FxfEngineOptions, FxfTensor

_TORCH_DTYPES = None


def _torch():
    import torch
    return torch


def _torch_dtype(code: int):
    global _TORCH_DTYPES
    if _TORCH_DTYPES is None:
        torch = _torch()
        _TORCH_DTYPES = [torch.float32, torch.float16, torch.int32, torch.int64, torch.bool]
    return _TORCH_DTYPES[code]


class _DeviceView:
    """Exposes raw device memory through __cuda_array_interface__ so torch can wrap it."""

    def __init__(self, ptr: int, shape, typestr: str, owner) -> None:
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False),
                                         "version": 2, "strides": None}
        self._owner = owner  # keeps the engine alive while a view exists


def _device_index(device) -> int:
    s = str(device)
    if s in ("cuda", "gpu"):
        return _torch().cuda.current_device()
    if s.startswith("cuda:"):
        return int(s.split(":", 1)[1])
    if s.isdigit():
        return int(s)
    raise RuntimeError(f"fxfusion_b200 runs on CUDA devices only (no CPU backend); got device '{device}'")


class ExecutionEngine:
    """Loads a graph file onto one GPU and runs it.  Not re-entrant (one run at a time)."""

    def __init__(self, graph_path: str, device: str = "cuda:0", *, use_cuda_graph: bool = True,
                 precision: str = "auto", comm=None, shard_output: bool = False, **options) -> None:
        """`comm`: a fxfusion_b200.tp.Communicator makes this a tensor-parallel engine (heads and FeedForward
        hidden units sharded over its ranks; construction is collective).  `shard_output` additionally shards
        the vocabulary of the final Linear: `outputs()` then holds only this rank's column block and
        `argmax_scatter` / `decode_static` combine the ranks.  `options`: further integer fields of FxfEngineOptions by
        name (no_epilogue_fusion, no_tp_fused_exchange, p2p_start_budget_ms, p2p_end_budget_ms, p2p_grid, tc_chunk_k, tc_pair, tp_push)."""
        self._h = C.c_void_p()
        lib = _lib.lib()
        if precision not in _lib.GEMM_MODES:
            raise ValueError(f"precision must be one of {sorted(_lib.GEMM_MODES)}")
        opts = FxfEngineOptions()
        opts.struct_size = C.sizeof(FxfEngineOptions)
        opts.use_cuda_graph = 1 if use_cuda_graph else 0
        opts.gemm_mode = _lib.GEMM_MODES[precision]
        opts.tp_rank, opts.tp_size = (comm.rank, comm.size) if comm is not None else (0, 1)
        opts.tp_shard_output = 1 if (shard_output and comm is not None) else 0
        for key, value in options.items():
            if key not in ("no_epilogue_fusion", "no_tp_fused_exchange", "p2p_start_budget_ms", "p2p_end_budget_ms", "p2p_grid", "tc_chunk_k", "tc_pair", "tp_push"):
                raise TypeError(f"unknown engine option '{key}'")
            setattr(opts, key, int(value))
        self.comm = comm  # keeps the communicator alive as long as the engine
        self.device_index = _device_index(device)
        self.device = f"cuda:{self.device_index}"
        _lib.check(lib.fxf_engine_create_tp(str(graph_path).encode(), self.device_index, C.byref(opts),
                                            comm.handle if comm is not None else None, C.byref(self._h)))
        self._lib = lib
        self.num_inputs = lib.fxf_engine_num_inputs(self._h)
        self.num_outputs = lib.fxf_engine_num_outputs(self._h)
        self.input_descs = [self._desc(lib.fxf_engine_input_desc, i) for i in range(self.num_inputs)]
        self.output_descs = [self._desc(lib.fxf_engine_output_desc, i) for i in range(self.num_outputs)]
        self._outputs = None
        self._input_views = None

    # -- introspection ------------------------------------------------------------------------
    def _desc(self, fn, i: int) -> FxfTensor:
        d = FxfTensor()
        _lib.check(fn(self._h, i, C.byref(d)))
        return d

    @property
    def handle(self) -> C.c_void_p:
        return self._h

    @property
    def num_nodes(self) -> int:
        return self._lib.fxf_engine_num_nodes(self._h)

    @property
    def arena_bytes(self) -> int:
        return self._lib.fxf_engine_arena_bytes(self._h)

    @property
    def device_bytes(self) -> int:
        return self._lib.fxf_engine_device_bytes(self._h)

    @property
    def launches_per_run(self) -> int:
        return self._lib.fxf_engine_launches_per_run(self._h)

    def describe(self) -> str:
        buf = C.create_string_buffer(1 << 18)
        _lib.check(self._lib.fxf_engine_describe(self._h, buf, len(buf)))
        return buf.value.decode()

    def node_info(self):
        out = []
        for i in range(self.num_nodes):
            op, fl, by = C.c_int(), C.c_double(), C.c_double()
            var = C.create_string_buffer(128)
            _lib.check(self._lib.fxf_engine_node_info(self._h, i, C.byref(op), C.byref(fl), C.byref(by), var, len(var)))
            out.append({"op": wire.OPCODES[op.value], "flops": fl.value, "bytes": by.value, "variant": var.value.decode()})
        return out

    def time_nodes(self) -> List[float]:
        n = self.num_nodes
        ms = (C.c_float * n)()
        _lib.check(self._lib.fxf_engine_time_nodes(self._h, ms, n, self._stream()))
        return list(ms)

    def profile_launches(self):
        """One traced forward: [{kernel, node, ms, flops, bytes}] per kernel launch."""
        cap = self.launches_per_run + 2 * self.num_nodes + 16  # collectives are traced too
        buf = (_lib.FxfLaunchInfo * cap)()
        n = C.c_int()
        _lib.check(self._lib.fxf_engine_profile_launches(self._h, self._stream(), buf, cap, C.byref(n)))
        return [{"kernel": buf[i].kernel.decode(), "node": buf[i].node, "ms": buf[i].ms, "flops": buf[i].flops,
                 "bytes": buf[i].bytes} for i in range(n.value)]

    def device_status(self) -> int:
        st = C.c_int()
        _lib.check(self._lib.fxf_engine_device_status(self._h, self._stream(), C.byref(st)))
        return st.value

    # -- tensors --------------------------------------------------------------------------------
    def _stream(self) -> C.c_void_p:
        return C.c_void_p(_torch().cuda.current_stream(self.device_index).cuda_stream)

    def _wrap(self, desc: FxfTensor):
        torch = _torch()
        shape = tuple(desc.shape[i] for i in range(desc.rank))
        if desc.nbytes == 0:
            return torch.empty(shape, dtype=_torch_dtype(desc.dtype), device=self.device)
        typestr = ["<f4", "<f2", "<i4", "<i8", "|u1"][desc.dtype]  # bool travels as bytes
        t = torch.as_tensor(_DeviceView(desc.ptr, shape, typestr, self), device=self.device)
        return t.view(torch.bool) if desc.dtype == wire.DT_BOOL else t

    def outputs(self):
        """Output tensors (views of the arena; contents change with every run)."""
        if self._outputs is None:
            self._outputs = [self._wrap(d) for d in self.output_descs]
        return self._outputs

    def input_slots(self):
        """The engine's static input buffers as tensors; writing them directly avoids the copy in run()."""
        if self._input_views is None:
            self._input_views = [self._wrap(d) for d in self.input_descs]
        return self._input_views

    # -- execution --------------------------------------------------------------------------------
    def run(self, inputs: Sequence) -> List:
        """ExecutionEngine::run (execution_engine.cpp:31-43): device check, bind, execute."""
        torch = _torch()
        if len(inputs) != self.num_inputs:
            raise RuntimeError(f"Input count mismatch: the graph has {self.num_inputs} inputs, {len(inputs)} were given")
        ptrs = (C.c_void_p * max(1, self.num_inputs))()
        keep = []
        for i, (t, d) in enumerate(zip(inputs, self.input_descs)):
            if not isinstance(t, torch.Tensor) or not t.is_cuda or t.device.index != self.device_index:
                raise RuntimeError(f"input engine device mismatch, index: {i}")
            if t.dtype != _torch_dtype(d.dtype):
                raise RuntimeError(f"input {i}: dtype {t.dtype} does not match the graph's {_torch_dtype(d.dtype)}")
            if t.numel() * t.element_size() != d.nbytes:
                raise RuntimeError(f"input {i}: shape {tuple(t.shape)} does not match the graph's "
                                   f"{tuple(d.shape[k] for k in range(d.rank))}")
            t = t.contiguous()
            keep.append(t)
            ptrs[i] = t.data_ptr()
        _lib.check(self._lib.fxf_engine_run(self._h, ptrs, self.num_inputs, self._stream()))
        return self.outputs()

    def run_host(self, inputs: Sequence[np.ndarray], outputs: Optional[Sequence[np.ndarray]] = None) -> None:
        """Host buffers in, host buffers out (H2D, forward, D2H, sync) through fxf_engine_run_host."""
        if len(inputs) != self.num_inputs:
            raise RuntimeError(f"Input count mismatch: the graph has {self.num_inputs} inputs, {len(inputs)} were given")
        ptrs = (C.c_void_p * max(1, self.num_inputs))()
        for i, (a, d) in enumerate(zip(inputs, self.input_descs)):
            if a.nbytes != d.nbytes:
                raise RuntimeError(f"input {i}: {a.nbytes} bytes given, the graph expects {d.nbytes}")
            ptrs[i] = a.ctypes.data
        if outputs is None:
            _lib.check(self._lib.fxf_engine_run_host(self._h, ptrs, self.num_inputs, None, 0, self._stream()))
            return
        optrs = (C.c_void_p * max(1, self.num_outputs))()
        for i, a in enumerate(outputs):
            optrs[i] = a.ctypes.data if a is not None else None
        _lib.check(self._lib.fxf_engine_run_host(self._h, ptrs, self.num_inputs, optrs, self.num_outputs, self._stream()))

    def argmax_scatter(self, tokens, current_len: int) -> None:
        """tokens[:, current_len] = argmax of output 0 at position current_len - 1 (combined over the ranks when
        the vocabulary is sharded)."""
        _lib.check(self._lib.fxf_engine_argmax_scatter(self._h, C.c_void_p(tokens.data_ptr()), int(current_len), self._stream()))

    @property
    def supports_last_row(self) -> bool:
        """True when the graph ends in the Linear that produces output 0, so decode_static(last_row_only=True) applies."""
        return bool(self._lib.fxf_engine_supports_last_row(self._h))

    def decode_static(self, tokens, initial_len: int, pad_idx: int = 0, last_row_only: bool = False):
        """Complete `tokens` (int64 CUDA tensor [B,T], prompt in the first `initial_len` columns) in
        place by greedy decoding on the device; returns it.  No host synchronisation.

        last_row_only=True evaluates the final vocabulary projection only at the position the loop reads
        (row current_len - 1 of each sequence) instead of at all T positions: the same tokens, about 30 % fewer
        flops per step at GPT-2-small shape; the engine's output 0 (full logits) is then not updated."""
        torch = _torch()
        if not (isinstance(tokens, torch.Tensor) and tokens.is_cuda and tokens.dtype == torch.int64 and tokens.is_contiguous()):
            raise RuntimeError("decode_static: tokens must be a contiguous int64 CUDA tensor")
        fn = self._lib.fxf_decode_static_last_row if last_row_only else self._lib.fxf_decode_static
        _lib.check(fn(self._h, C.c_void_p(tokens.data_ptr()), int(initial_len), int(pad_idx), self._stream()))
        return tokens

    def decode_cached(self, tokens, initial_len: int):
        """Incremental greedy decode for an engine built from `lowering.gpt_step_graph` (one position per forward,
        keys / values cached inside the engine): completes `tokens` (int64 CUDA tensor [B,T]) in place and returns it."""
        torch = _torch()
        if not (isinstance(tokens, torch.Tensor) and tokens.is_cuda and tokens.dtype == torch.int64 and tokens.is_contiguous()):
            raise RuntimeError("decode_cached: tokens must be a contiguous int64 CUDA tensor")
        _lib.check(self._lib.fxf_decode_cached(self._h, C.c_void_p(tokens.data_ptr()), int(initial_len), self._stream()))
        return tokens

    def close(self) -> None:
        if getattr(self, "_h", None) is not None and self._h.value:
            self._outputs = None
            self._input_views = None
            self._lib.fxf_engine_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Engine:
    """`Engine(model, example_inputs, ...)` of the reference (py/fxfusion/engine.py:7-35).

    Compilation is the reference's own, unchanged: its FusionPass, ShapePropPass and
    MemoryPlanningPass must be importable (package `fxfusion`).  Only the last step differs — the
    graph file is written by this package's FlatBuffers writer and loaded by the B200 runtime.
    """

    def __init__(self, model, example_inputs, model_name: Optional[str] = None, device: str = "cuda:0",
                 DEBUG: bool = False, memory_alignment: int = 64, out_dir: Optional[str] = None, **engine_kwargs) -> None:
        from .compile_ref import compile_with_reference
        self.fx_model, graph = compile_with_reference(model, example_inputs, model_name=model_name, DEBUG=DEBUG,
                                                      memory_alignment=memory_alignment)
        out = Path(out_dir) if out_dir else Path.cwd() / "data"
        out.mkdir(parents=True, exist_ok=True)
        self.bin_path = str(out / f"{graph.name}.bin")
        wire.dump(graph, self.bin_path)
        self._engine = ExecutionEngine(self.bin_path, device, **engine_kwargs)

    def run(self, inputs):
        return self._engine.run(inputs)
