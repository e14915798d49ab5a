"""Call one CUDA kernel of the backend outside any engine (fxf_kernel_invoke).

The argument contract is the reference's KernelFn (csrc/include/runtime/tensor_registry.hpp:20-26):
a registry of tensors, input ids, output ids, int and float params.  Tensors are torch CUDA
tensors; scratch memory, where an op needs it, is allocated here as a torch buffer.
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence

from . import _lib, wire
from ._lib import FxfTensor

_DT = None


def _dtype_code(t) -> int:
    global _DT
    import torch
    if _DT is None:
        _DT = {torch.float32: wire.DT_F32, torch.float16: wire.DT_F16, torch.int32: wire.DT_I32,
               torch.int64: wire.DT_I64, torch.bool: wire.DT_BOOL}
    return _DT[t.dtype]


def describe(t) -> FxfTensor:
    d = FxfTensor()
    d.ptr = t.data_ptr()
    d.dtype = _dtype_code(t)
    d.rank = t.dim()
    for i in range(t.dim()):
        d.shape[i] = t.shape[i]
        d.stride[i] = t.stride(i)
    d.nbytes = t.numel() * t.element_size()
    return d


def invoke(op: str, registry: Sequence, in_ids: Sequence[int], out_ids: Sequence[int], ints: Sequence[int] = (),
           floats: Sequence[float] = (), precision: str = "auto") -> None:
    """Runs opcode `op` (name from wire.OPCODES) on the current CUDA stream; writes registry[out_ids[0]]."""
    import torch
    lib = _lib.lib()
    n = len(registry)
    reg = (FxfTensor * n)(*[describe(t) for t in registry])
    ii = (C.c_uint32 * max(1, len(in_ids)))(*in_ids)
    oo = (C.c_uint32 * max(1, len(out_ids)))(*out_ids)
    ip = (C.c_int64 * max(1, len(ints)))(*[int(v) for v in ints])
    fp = (C.c_float * max(1, len(floats)))(*[float(v) for v in floats])
    mode = _lib.GEMM_MODES[precision]
    head = (wire.OP[op], reg, n, ii, len(in_ids), oo, len(out_ids), ip, len(ints), fp, len(floats))
    need = lib.fxf_kernel_scratch_bytes(*head, mode)
    if need < 0:
        raise RuntimeError(lib.fxf_last_error().decode())
    dev = registry[out_ids[0]].device
    scratch = torch.empty(max(int(need), 16), dtype=torch.uint8, device=dev)
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    _lib.check(lib.fxf_kernel_invoke(*head, C.c_void_p(scratch.data_ptr()), need, mode, stream))
    scratch.record_stream(torch.cuda.current_stream(dev))


def feedforward_static(x, w1, b1, w2, b2, out) -> None:
    """out = relu(x @ w1.T + b1) @ w2.T + b2 through fxf_feedforward_static: nothing is allocated, the hidden
    activation lives in the library's fixed scratch array (see include/fxf_b200.h for the limits).
    All arguments are contiguous float32 CUDA tensors on the current device."""
    import torch
    lib = _lib.lib()
    D = x.shape[-1]
    F, P = w1.shape[0], w2.shape[0]
    M = out.numel() // P if P else (x.numel() // D if D else 0)   # rows come from the output: x has no elements when D == 0
    stream = C.c_void_p(torch.cuda.current_stream(x.device).cuda_stream)
    _lib.check(lib.fxf_feedforward_static(x.data_ptr(), w1.data_ptr(), b1.data_ptr(), w2.data_ptr(), b2.data_ptr(), out.data_ptr(),
                                          M, D, F, P, stream))


def tp_exchange_emulated(partials, residuals=None, x_outs=None, y_outs=None, gamma=None, beta=None, eps: float = 1e-5,
                         replicate_x: bool = False, budget_ms: int = 200, skip_rank: int = -1, pushed: bool = False):
    """The tensor-parallel exchange (sum of the ranks' partial [M,D] + residual, LayerNorm, rows owned by rank) with all
    ranks' buffers on the current GPU and one cooperative launch (fxf_tp_exchange_emulated).  Each argument is a list with
    one float32 CUDA tensor [M,D] per rank (or None).  pushed: partials[q] is rank q's exchange window as the row-pushed
    products leave it (see linear_pushed).  Returns the ranks' status words after the call has finished."""
    import torch
    lib = _lib.lib()
    n = len(partials)
    M, D = partials[0].shape
    arr = lambda ts: (C.c_void_p * n)(*[t.data_ptr() for t in ts]) if ts is not None else None
    sync = torch.zeros(n * 8192, dtype=torch.uint8, device=partials[0].device)
    stream = C.c_void_p(torch.cuda.current_stream(partials[0].device).cuda_stream)
    _lib.check(lib.fxf_tp_exchange_emulated(n, arr(partials), arr(residuals), arr(x_outs), arr(y_outs),
                                            gamma.data_ptr() if gamma is not None else None, beta.data_ptr() if beta is not None else None,
                                            float(eps), M, D, (1 if replicate_x else 0) | (2 if pushed else 0), C.c_void_p(sync.data_ptr()), sync.numel(), int(budget_ms),
                                            int(skip_rank), stream))
    torch.cuda.synchronize()
    words = sync.view(torch.int32).view(n, 2048)[:, 4160 // 4].cpu().tolist()
    return words


def linear_pushed(x, w, bias, windows, rank: int):
    """Producer `rank`'s row-parallel product x[M,K] @ w[N,K].T (+ bias) on the tensor cores with a row-pushed output
    (fxf_linear_pushed): row g of the result, owned by rank q = g // R with R = M // len(windows), lands in windows[q] at
    row rank*R + (g - q*R).  windows: one float32 CUDA tensor [M,N] per rank, all on the current GPU."""
    import torch
    lib = _lib.lib()
    n = len(windows)
    M, K = x.shape
    N = w.shape[0]
    need = lib.fxf_linear_pushed_scratch_bytes(N, K)
    scratch = torch.empty(need + 256, dtype=torch.uint8, device=x.device)
    base = (scratch.data_ptr() + 255) // 256 * 256
    arr = (C.c_void_p * n)(*[t.data_ptr() for t in windows])
    stream = C.c_void_p(torch.cuda.current_stream(x.device).cuda_stream)
    _lib.check(lib.fxf_linear_pushed(x.data_ptr(), w.data_ptr(), bias.data_ptr() if bias is not None else None, arr, n, int(rank), M, N, K,
                                     C.c_void_p(base), need, stream))
    torch.cuda.synchronize()


def gemm_variant(M: int, N: int, K: int, precision: str = "auto", sm_count: int = 148) -> str:
    """Which GEMM kernel the dispatch rule takes for out[M,N] = x[M,K] @ w[N,K].T (host-only query)."""
    buf = C.create_string_buffer(96)
    _lib.check(_lib.lib().fxf_gemm_variant(M, N, K, _lib.GEMM_MODES[precision], sm_count, buf, len(buf)))
    return buf.value.decode()
