"""The C-ABI library: loads, exports every declared symbol, reports errors — no GPU needed."""
import ctypes as C
import re
from pathlib import Path

import pytest

from conftest import REPO


def declared_symbols():
    text = (REPO / "include" / "fxf_b200.h").read_text()
    return re.findall(r"FXF_API\s+[\w\s\*]+?\b(fxf_\w+)\s*\(", text)


def test_header_declares_the_expected_surface():
    names = declared_symbols()
    assert len(names) == len(set(names)) >= 24
    for must in ("fxf_engine_create", "fxf_engine_run", "fxf_engine_run_host", "fxf_kernel_invoke", "fxf_decode_static", "fxf_last_error"):
        assert must in names


def test_library_exports_every_declared_symbol(built_lib):
    from fxfusion_b200 import _lib
    for name in declared_symbols():
        assert hasattr(built_lib, name), f"{name} is declared in include/fxf_b200.h but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes prototype"
    assert set(_lib.SIGNATURES) == set(declared_symbols())


def test_struct_layout_matches_header(built_lib):
    from fxfusion_b200._lib import FxfEngineOptions, FxfTensor
    assert C.sizeof(FxfTensor) == 8 + 4 + 4 + 8 * 8 + 8 * 8 + 8
    assert C.sizeof(FxfEngineOptions) == 16 * 4
    assert built_lib.fxf_version().decode().endswith("sm_100a")


def test_missing_file_reports_the_reference_error(built_lib):
    h = C.c_void_p()
    rc = built_lib.fxf_engine_create(b"/nonexistent/graph.bin", 0, None, C.byref(h))
    assert rc != 0 and not h.value
    assert "ExecutionEngine failed to open: /nonexistent/graph.bin" in built_lib.fxf_last_error().decode()


def test_cpu_device_is_refused_by_the_wrapper():
    from fxfusion_b200.engine import ExecutionEngine
    with pytest.raises(RuntimeError, match="CUDA devices only"):
        ExecutionEngine("whatever.bin", "cpu")


def test_product_never_imports_the_oracle():
    for path in (REPO / "fxfusion_b200").rglob("*"):
        if path.suffix in (".py", ".cpp", ".cu", ".hpp", ".h") and "build" not in path.parts[len(REPO.parts):-1]:
            text = path.read_text(errors="ignore")
            assert not re.search(r"^\s*(from|import)\s+oracle\b", text, re.M), path
            assert "oracle/" not in text, path


def test_gemm_dispatch_rule_is_a_host_side_query(built_lib):
    """fxf_gemm_variant answers without a GPU which kernel a dense layer of a given shape takes: the benchmark's layer
    shapes go to CTA pairs with the default arithmetic (one TF32 product + two bf16 corrections), a K that is not a multiple
    of 8 keeps three TF32 products, batch-sized layers stay on the fp32 weight-streaming kernel."""
    from fxfusion_b200.kernels import gemm_variant
    pair = "tcgen05-tf32+2bf16-256x256-pair-smemA"
    for shape in [(8192, 3072, 768), (8192, 2304, 768), (8192, 768, 3072), (8192, 50257, 768), (8192, 768, 1536)]:
        assert gemm_variant(*shape) == pair, shape
    assert gemm_variant(8192, 768, 768) == "tcgen05-tf32+2bf16-128x192-tmemA"
    assert gemm_variant(1024, 64, 256) == "tcgen05-tf32+2bf16-128x64-tmemA"
    assert gemm_variant(5000, 1111, 500) == "tcgen05-tf32x3-128x192-tmemA"          # K % 8 != 0
    assert gemm_variant(8192, 3072, 768, precision="fp32_3xtf32") == "tcgen05-tf32x3-256x256-pair-smemA"
    assert gemm_variant(8192, 3072, 768, precision="bf16") == "tcgen05-bf16-128x192"
    assert gemm_variant(8192, 3072, 768, precision="fp32_simt") == "simt128x128"
    assert gemm_variant(32, 512, 512) == "skinny32x8"                                # the MLP of the first benchmark configuration
