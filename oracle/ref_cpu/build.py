"""TEST INFRASTRUCTURE — builds `oracle/_ref/fxf_ref_cpu.so` from the reference's own sources.

    python -m oracle.ref_cpu.build [/path/to/reference]

Without an argument the checkout is looked up in $FXFUSION_REFERENCE, then in a directory named
`reference` beside this repository.

The reference CPU kernels (csrc/kernels/cpu/*.cpp) and csrc/runtime/cache.cpp include only
LibTorch and two of the reference's headers, so they compile as they are with g++ against the
installed torch; the reference's CMake build is not used (it needs flatc-generated headers).
Sources are read from the reference checkout; only the built module lands in `oracle/_ref/`.
`load()` imports the built module if present (no reference checkout is needed for that).
"""
from __future__ import annotations

import importlib.util
import os
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE.parent / "_ref"
NAME = "fxf_ref_cpu"


def default_reference() -> str:
    """Path of the reference checkout: $FXFUSION_REFERENCE, else `<parent of this repository>/reference`."""
    return os.environ.get("FXFUSION_REFERENCE") or str(HERE.parents[2] / "reference")


def build(reference: str | None = None, verbose: bool = False):
    reference = reference or default_reference()
    ref = Path(reference)
    csrc = ref / "csrc"
    if not (csrc / "kernels" / "cpu").is_dir():
        raise FileNotFoundError(f"no reference checkout at {reference}")
    from torch.utils.cpp_extension import load as cpp_load
    OUT.mkdir(exist_ok=True)
    sources = [str(HERE / "shim.cpp")] + sorted(str(p) for p in (csrc / "kernels" / "cpu").glob("*.cpp")) + [str(csrc / "runtime" / "cache.cpp")]
    return cpp_load(name=NAME, sources=sources,
                    extra_include_paths=[str(csrc / "include" / "runtime"), str(csrc / "include" / "kernels" / "cpu")],
                    extra_cflags=["-O2", "-std=c++17"], build_directory=str(OUT), verbose=verbose)


def load():
    """Import the prebuilt module from oracle/_ref, or return None if it has not been built."""
    so = OUT / f"{NAME}.so"
    if not so.exists():
        return None
    import torch  # noqa: F401  (the module links against libtorch)
    spec = importlib.util.spec_from_file_location(NAME, so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def ensure(reference: str | None = None):
    reference = reference or default_reference()
    mod = load()
    if mod is None and os.path.isdir(reference):
        build(reference)
        mod = load()
    return mod


if __name__ == "__main__":
    build(sys.argv[1] if len(sys.argv) > 1 else None, verbose=True)
    print(OUT / f"{NAME}.so")
