"""ctypes binding of libfxf_b200.so — the only way Python reaches the CUDA backend.

There is no fallback: if the shared library is missing or a call fails, an exception is
raised.  Nothing here imports PyTorch.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

MAX_DIMS = 8
LIB_PATH = Path(__file__).resolve().parent / "lib" / "libfxf_b200.so"


class FxfTensor(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("dtype", C.c_int32), ("rank", C.c_int32),
                ("shape", C.c_int64 * MAX_DIMS), ("stride", C.c_int64 * MAX_DIMS), ("nbytes", C.c_int64)]


class FxfEngineOptions(C.Structure):
    _fields_ = [("struct_size", C.c_int32), ("use_cuda_graph", C.c_int32), ("gemm_mode", C.c_int32),
                ("tp_rank", C.c_int32), ("tp_size", C.c_int32), ("tp_shard_output", C.c_int32),
                ("no_epilogue_fusion", C.c_int32), ("no_tp_fused_exchange", C.c_int32), ("p2p_start_budget_ms", C.c_int32),
                ("p2p_end_budget_ms", C.c_int32), ("p2p_grid", C.c_int32), ("tc_chunk_k", C.c_int32), ("tc_pair", C.c_int32), ("tp_push", C.c_int32), ("reserved", C.c_int32 * 2)]


class FxfLaunchInfo(C.Structure):
    _fields_ = [("kernel", C.c_char * 48), ("node", C.c_int32), ("ms", C.c_float), ("flops", C.c_double), ("bytes", C.c_double)]


GEMM_AUTO, GEMM_FP32_SIMT, GEMM_TF32X3 = 0, 1, 2
GEMM_BF16 = 3
GEMM_TF32_BF16X2 = 4
GEMM_MODES = {"auto": GEMM_AUTO, "fp32_simt": GEMM_FP32_SIMT, "fp32_3xtf32": GEMM_TF32X3, "bf16": GEMM_BF16, "fp32_tf32_bf16x2": GEMM_TF32_BF16X2}

# name -> (restype, argtypes); mirrors include/fxf_b200.h one to one
_u32p, _i64p, _f32p = C.POINTER(C.c_uint32), C.POINTER(C.c_int64), C.POINTER(C.c_float)
_kernel_args = [C.c_int, C.POINTER(FxfTensor), C.c_int, _u32p, C.c_int, _u32p, C.c_int, _i64p, C.c_int, _f32p, C.c_int]
SIGNATURES = {
    "fxf_last_error": (C.c_char_p, []),
    "fxf_version": (C.c_char_p, []),
    "fxf_engine_create": (C.c_int, [C.c_char_p, C.c_int, C.POINTER(FxfEngineOptions), C.POINTER(C.c_void_p)]),
    "fxf_comm_unique_id": (C.c_int, [C.c_void_p]),
    "fxf_comm_create": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_void_p)]),
    "fxf_comm_destroy": (None, [C.c_void_p]),
    "fxf_comm_rank": (C.c_int, [C.c_void_p]),
    "fxf_comm_size": (C.c_int, [C.c_void_p]),
    "fxf_engine_create_tp": (C.c_int, [C.c_char_p, C.c_int, C.POINTER(FxfEngineOptions), C.c_void_p, C.POINTER(C.c_void_p)]),
    "fxf_gemm_variant": (C.c_int, [C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_int, C.c_char_p, C.c_size_t]),
    "fxf_tp_exchange_emulated": (C.c_int, [C.c_int] + [C.POINTER(C.c_void_p)] * 4 + [C.c_void_p, C.c_void_p, C.c_float, C.c_int64, C.c_int64, C.c_int,
                                            C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_void_p]),
    "fxf_linear_pushed_scratch_bytes": (C.c_int64, [C.c_int64, C.c_int64]),
    "fxf_linear_pushed": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_int64, C.c_int64, C.c_int64,
                                    C.c_void_p, C.c_int64, C.c_void_p]),
    "fxf_engine_argmax_scatter": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "fxf_engine_create_from_memory": (C.c_int, [C.c_void_p, C.c_size_t, C.c_int, C.POINTER(FxfEngineOptions), C.POINTER(C.c_void_p)]),
    "fxf_engine_destroy": (None, [C.c_void_p]),
    "fxf_engine_num_inputs": (C.c_int, [C.c_void_p]),
    "fxf_engine_num_outputs": (C.c_int, [C.c_void_p]),
    "fxf_engine_input_desc": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(FxfTensor)]),
    "fxf_engine_output_desc": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(FxfTensor)]),
    "fxf_engine_num_nodes": (C.c_int, [C.c_void_p]),
    "fxf_engine_arena_bytes": (C.c_int64, [C.c_void_p]),
    "fxf_engine_device_bytes": (C.c_int64, [C.c_void_p]),
    "fxf_engine_launches_per_run": (C.c_int, [C.c_void_p]),
    "fxf_engine_run": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.c_int, C.c_void_p]),
    "fxf_engine_run_host": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.c_int, C.POINTER(C.c_void_p), C.c_int, C.c_void_p]),
    "fxf_engine_device_status": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_int)]),
    "fxf_engine_describe": (C.c_int, [C.c_void_p, C.c_char_p, C.c_size_t]),
    "fxf_engine_time_nodes": (C.c_int, [C.c_void_p, _f32p, C.c_int, C.c_void_p]),
    "fxf_engine_node_info": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_double), C.POINTER(C.c_double), C.c_char_p, C.c_size_t]),
    "fxf_engine_profile_launches": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(FxfLaunchInfo), C.c_int, C.POINTER(C.c_int)]),
    "fxf_kernel_scratch_bytes": (C.c_int64, _kernel_args + [C.c_int]),
    "fxf_kernel_invoke": (C.c_int, _kernel_args + [C.c_void_p, C.c_int64, C.c_int, C.c_void_p]),
    "fxf_feedforward_static_max_bytes": (C.c_int64, []),
    "fxf_feedforward_static": (C.c_int, [C.c_void_p] * 6 + [C.c_int64] * 4 + [C.c_void_p]),
    "fxf_decode_build_mask": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int64, C.c_void_p]),
    "fxf_decode_argmax_scatter": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int64, C.c_int, C.c_void_p]),
    "fxf_decode_static": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_void_p]),
    "fxf_decode_static_last_row": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_void_p]),
    "fxf_engine_supports_last_row": (C.c_int, [C.c_void_p]),
    "fxf_decode_cached": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
}

_lib = None


def lib() -> C.CDLL:
    """Load the shared library (once) and declare every prototype."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: the CUDA backend has not been built "
                "(run `python -m fxfusion_b200.build`); there is no CPU fallback")
        handle = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError if the symbol is not exported
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        raise RuntimeError(lib().fxf_last_error().decode("utf-8", "replace"))
