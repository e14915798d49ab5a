"""TEST INFRASTRUCTURE — the CPU oracle for the FXFusion runtime hot path.

Nothing in the product (`fxfusion_b200/`) may import this package.  It is used by `tests/`,
by `__graft_entry__.smoke()` and by the CPU-baseline / reference legs of `bench.py`, always as
the checker or the baseline, never as the thing that is measured as the product.
"""
