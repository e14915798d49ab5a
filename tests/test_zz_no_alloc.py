"""fxf_feedforward_static: the FeedForward entry point that allocates nothing.

It exists for callers that cannot call cudaMalloc (their own pool owns the device, or they cannot
tolerate an allocation's implicit synchronisation); its hidden activation lives in a fixed array inside
the library.  The test calls it through the C ABI twice in a row — the second call with other data and
a smaller problem, so anything the first call left in the shared array would show — and compares each
result with the existing entry point (fxf_kernel_invoke, FeedForward, fp32 FFMA kernels) within the
tolerance the other parity tests use.  It also checks the size limit.  This file sorts last so that a run
that stops at the first failure has already executed every other test.
"""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
ATOL, RTOL = 1e-4, 1e-3


def _problem(M, D, F, P, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(M, D, generator=g).cuda(), (torch.randn(F, D, generator=g) / math.sqrt(D)).cuda(), torch.randn(F, generator=g).cuda(),
            (torch.randn(P, F, generator=g) / math.sqrt(F)).cuda(), torch.randn(P, generator=g).cuda()]


def test_static_feedforward_matches_existing_entry_point_twice(built_lib):
    from fxfusion_b200.kernels import feedforward_static, invoke
    assert built_lib.fxf_feedforward_static_max_bytes() == 8 << 20
    # the last case has at most 64 rows against a weight of a megabyte: the few-rows kernels, which must not cut K into parts
    # here because this entry point hands them no workspace
    for M, D, F, P, seed in [(300, 96, 1000, 64, 1), (130, 96, 200, 50, 2), (8, 1024, 1024, 64, 3)]:
        x, w1, b1, w2, b2 = _problem(M, D, F, P, seed)
        want = torch.zeros(M, P, device="cuda")
        invoke("FeedForward", [x, w1, b1, w2, b2, want], [0, 1, 2, 3, 4], [5], precision="fp32_simt")
        got = torch.full((M, P), float("nan"), device="cuda")
        feedforward_static(x, w1, b1, w2, b2, got)
        torch.cuda.synchronize()
        assert not torch.isnan(got).any()
        assert torch.allclose(got, want, atol=ATOL, rtol=RTOL), (got - want).abs().max().item()
        ref = torch.relu(x.cpu() @ w1.cpu().T + b1.cpu()) @ w2.cpu().T + b2.cpu()
        assert torch.allclose(got.cpu(), ref, atol=ATOL, rtol=RTOL)


def test_static_feedforward_with_empty_extents(built_lib):
    """No hidden units (F = 0): the output is the second bias; no input columns (D = 0): the hidden layer is relu(b1)."""
    from fxfusion_b200.kernels import feedforward_static
    for M, D, F, P, seed in [(40, 64, 0, 16, 4), (5, 0, 32, 7, 5)]:
        x, w1, b1, w2, b2 = _problem(M, D, F, P, seed)
        got = torch.full((M, P), float("nan"), device="cuda")
        feedforward_static(x, w1, b1, w2, b2, got)
        torch.cuda.synchronize()
        ref = torch.relu(x.cpu() @ w1.cpu().T + b1.cpu()) @ w2.cpu().T + b2.cpu()
        assert torch.allclose(got.cpu(), ref, atol=ATOL, rtol=RTOL), (M, D, F, P)


def test_static_feedforward_refuses_oversized_problems(built_lib):
    from fxfusion_b200.kernels import feedforward_static
    M, D, F, P = 1024, 16, 4096, 8  # hidden = 16 MiB > 8 MiB
    x, w1, b1, w2, b2 = _problem(M, D, F, P, 3)
    out = torch.zeros(M, P, device="cuda")
    with pytest.raises(RuntimeError, match="static scratch"):
        feedforward_static(x, w1, b1, w2, b2, out)
    assert torch.count_nonzero(out) == 0
