"""Shared comparison helpers for the tests."""
from __future__ import annotations

import numpy as np
import torch


def compare_outputs(actual, expected, atol=1e-3, rtol=1e-3):
    """The reference's acceptance rule (py/tests/utils.py:14-90): equal count, shape and dtype;
    integer and bool tensors exactly equal; NaN positions identical; the rest allclose."""
    if isinstance(actual, torch.Tensor):
        actual, expected = [actual], [expected]
    if len(actual) != len(expected):
        return False, f"output count {len(actual)} != {len(expected)}"
    for i, (a, e) in enumerate(zip(actual, expected)):
        a, e = a.detach().cpu(), e.detach().cpu()
        if tuple(a.shape) != tuple(e.shape):
            return False, f"output {i}: shape {tuple(a.shape)} != {tuple(e.shape)}"
        if a.dtype != e.dtype:
            return False, f"output {i}: dtype {a.dtype} != {e.dtype}"
        if not a.dtype.is_floating_point:
            if not torch.equal(a, e):
                return False, f"output {i}: integer tensors differ"
            continue
        an, en = torch.isnan(a), torch.isnan(e)
        if not torch.equal(an, en):
            return False, f"output {i}: NaN masks differ ({int(an.sum())} vs {int(en.sum())} NaNs)"
        av, ev = a[~an], e[~en]
        if not torch.allclose(av, ev, atol=atol, rtol=rtol):
            d = (av - ev).abs()
            rel = d / ev.abs().clamp_min(1e-12)
            return False, f"output {i}: max abs {d.max().item():.3e}, max rel {rel.max().item():.3e} (atol {atol}, rtol {rtol})"
    return True, "ok"


def max_abs_rel(a: torch.Tensor, e: torch.Tensor):
    a, e = a.detach().cpu().double(), e.detach().cpu().double()
    ok = ~(torch.isnan(a) | torch.isnan(e))
    d = (a[ok] - e[ok]).abs()
    if d.numel() == 0:
        return 0.0, 0.0
    return d.max().item(), (d / e[ok].abs().clamp_min(1e-6)).max().item()


def reference_cpu_kernels():
    """The reference's own compiled CPU kernels (oracle/_ref) as a kernel table for GraphOracle, or None when that
    module has not been built (the restated oracle, tested bit-identical to it, is used then)."""
    from oracle.graph_oracle import KERNELS
    from oracle.ref_cpu.build import load as load_ref
    ref = load_ref()
    if ref is None:
        return None

    def bind(op):
        def fn(reg, i, o, ints, floats):
            ref.call(op, [t if t is not None else torch.empty(0) for t in reg], list(i), list(o), list(ints), list(floats))
        return fn
    return {op: bind(op) for op in KERNELS}
