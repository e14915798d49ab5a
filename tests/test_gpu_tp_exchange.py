"""The tensor-parallel exchange kernel (sum of the ranks' partial outputs + residual Add + LayerNorm, rows owned by rank),
run with all ranks' buffers on ONE GPU through fxf_tp_exchange_emulated: one cooperative launch carries the blocks of every
rank, so the peer barriers, the row ownership and the bounded waits are exercised without a second GPU.  The multi-GPU
path proper (peer-mapped engines) is covered by test_tp.py where at least two GPUs are visible."""
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(n, M, D, seed):
    g = torch.Generator().manual_seed(seed)
    parts = [torch.randn(M, D, generator=g) for _ in range(n)]
    res = torch.randn(M, D, generator=g)
    gamma, beta = torch.randn(D, generator=g), torch.randn(D, generator=g)
    x = parts[0].clone()
    for q in range(1, n):
        x = x + parts[q]          # ranks in fixed order, fp32, as the kernel adds them
    return parts, res, gamma, beta, x


@pytest.mark.parametrize("n,M,D", [(2, 64, 768), (4, 37, 768), (2, 5, 256), (4, 128, 100), (8, 50, 1024), (3, 7, 4)])
def test_exchange_add_layernorm_rows_owned_by_rank(built_lib, n, M, D):
    from fxfusion_b200.kernels import tp_exchange_emulated
    parts, res, gamma, beta, x = _case(n, M, D, seed=n * 1000 + M)
    want_x = x + res
    want_y = torch.nn.functional.layer_norm(want_x, (D,), gamma, beta, 1e-5)
    R = -(-M // n)
    dp = [t.cuda() for t in parts]
    dres = [res.cuda() for _ in range(n)]
    dx = [torch.full((M, D), float("nan"), device="cuda") for _ in range(n)]
    dy = [torch.full((M, D), float("nan"), device="cuda") for _ in range(n)]
    status = tp_exchange_emulated(dp, dres, dx, dy, gamma.cuda(), beta.cuda(), 1e-5, replicate_x=False)
    assert status == [0] * n
    for r in range(n):
        lo, hi = min(M, r * R), min(M, (r + 1) * R)
        got = dx[r].cpu()
        assert torch.equal(got[lo:hi], want_x[lo:hi]), "the owner's rows of the residual stream must be the fp32 sum in rank order"
        rest = torch.cat([got[:lo], got[hi:]])
        assert torch.isnan(rest).all(), "a rank must not write residual rows it does not own"
        assert torch.allclose(dy[r].cpu(), want_y, atol=1e-4, rtol=1e-3), (dy[r].cpu() - want_y).abs().max().item()


def test_exchange_variants_and_overlapping_buffers(built_lib):
    """AddLayerNorm form (no residual stream output), plain all-reduce + Add form (every rank gets every row), and the
    buffer overlaps the arena planner produces: normalised rows written on top of the partial sums, residual updated in place."""
    from fxfusion_b200.kernels import tp_exchange_emulated
    n, M, D = 4, 96, 512
    parts, res, gamma, beta, x = _case(n, M, D, seed=7)
    want_x = x + res
    want_y = torch.nn.functional.layer_norm(want_x, (D,), gamma, beta, 1e-5)
    # y only, stored on top of each rank's partial buffer
    dp = [t.cuda() for t in parts]
    status = tp_exchange_emulated(dp, [res.cuda() for _ in range(n)], None, dp, gamma.cuda(), beta.cuda(), 1e-5)
    assert status == [0] * n
    for r in range(n):
        assert torch.allclose(dp[r].cpu(), want_y, atol=1e-4, rtol=1e-3)
    # x only, replicated, in place over the residual
    dp = [t.cuda() for t in parts]
    dres = [res.cuda() for _ in range(n)]
    status = tp_exchange_emulated(dp, dres, dres, None, None, None, 0.0, replicate_x=True)
    assert status == [0] * n
    for r in range(n):
        assert torch.equal(dres[r].cpu(), want_x)
    # no residual at all: a plain sum + LayerNorm
    dp = [t.cuda() for t in parts]
    dy = [torch.zeros(M, D, device="cuda") for _ in range(n)]
    status = tp_exchange_emulated(dp, None, None, dy, gamma.cuda(), beta.cuda(), 1e-5)
    assert status == [0] * n
    assert torch.allclose(dy[n - 1].cpu(), torch.nn.functional.layer_norm(x, (D,), gamma, beta, 1e-5), atol=1e-4, rtol=1e-3)


def test_exchange_wait_runs_out_when_a_rank_never_arrives(built_lib):
    """Failure detection without a fault: rank 1 never reaches the exchange (nothing sets its flags), the other ranks' waits
    run out after the 50 ms budget, they record status 121 and return; the GPU stays usable."""
    from fxfusion_b200.kernels import tp_exchange_emulated
    n, M, D = 4, 64, 256
    parts, res, gamma, beta, x = _case(n, M, D, seed=11)
    dp = [t.cuda() for t in parts]
    dy = [torch.zeros(M, D, device="cuda") for _ in range(n)]
    t0 = time.perf_counter()
    status = tp_exchange_emulated(dp, None, None, dy, gamma.cuda(), beta.cuda(), 1e-5, budget_ms=50, skip_rank=1)
    elapsed = time.perf_counter() - t0
    assert elapsed < 5.0, f"the bounded wait took {elapsed:.2f} s"
    assert status[1] == 0 and all(s in (121, 123) for i, s in enumerate(status) if i != 1) and 121 in status
    # the context is intact: the same exchange with every rank present succeeds
    status = tp_exchange_emulated(dp, None, None, dy, gamma.cuda(), beta.cuda(), 1e-5, budget_ms=200)
    assert status == [0] * n
    assert torch.allclose(dy[0].cpu(), torch.nn.functional.layer_norm(x, (D,), gamma, beta, 1e-5), atol=1e-4, rtol=1e-3)


@pytest.mark.parametrize("n,M,N,K", [(2, 512, 256, 128), (4, 1024, 768, 192), (2, 2048, 768, 384), (4, 512, 200, 64)])
def test_row_pushed_product_feeds_the_exchange(built_lib, n, M, N, K):
    """The row-parallel product with a row-pushed output (every producer played in turn on this GPU) followed by the exchange
    in its pushed layout: each owner finds all producers' partial rows in its own window, and the result equals the
    unsharded Linear + residual Add + LayerNorm."""
    from fxfusion_b200.kernels import linear_pushed, tp_exchange_emulated
    g = torch.Generator().manual_seed(n * 100 + K)
    xs = [torch.randn(M, K, generator=g) for _ in range(n)]            # producer p's slice of the activation columns
    ws = [torch.randn(N, K, generator=g) / K ** 0.5 for _ in range(n)]  # and of the weight columns
    bias = torch.randn(N, generator=g)
    res = torch.randn(M, N, generator=g)
    gamma, beta = torch.randn(N, generator=g), torch.randn(N, generator=g)
    R = M // n
    windows = [torch.full((M, N), float("nan"), device="cuda") for _ in range(n)]
    for p in range(n):
        linear_pushed(xs[p].cuda(), ws[p].cuda(), bias.cuda() if p == 0 else None, windows, p)
    parts = [xs[p].double() @ ws[p].double().T + (bias.double() if p == 0 else 0.0) for p in range(n)]
    for q in range(n):
        got = windows[q].cpu()
        for p in range(n):
            want = parts[p][q * R:(q + 1) * R]
            err = (got[p * R:(p + 1) * R].double() - want).abs().max().item()
            assert err < 2e-5 * max(1.0, want.abs().max().item()), (q, p, err)
    want_x = (sum(parts) + res.double()).float()
    want_y = torch.nn.functional.layer_norm(want_x, (N,), gamma, beta, 1e-5)
    dx = [torch.full((M, N), float("nan"), device="cuda") for _ in range(n)]
    dy = [torch.full((M, N), float("nan"), device="cuda") for _ in range(n)]
    status = tp_exchange_emulated(windows, [res.cuda() for _ in range(n)], dx, dy, gamma.cuda(), beta.cuda(), 1e-5, pushed=True)
    assert status == [0] * n
    for r in range(n):
        assert torch.allclose(dx[r].cpu()[r * R:(r + 1) * R], want_x[r * R:(r + 1) * R], atol=1e-4, rtol=1e-4)
        assert torch.allclose(dy[r].cpu(), want_y, atol=1e-4, rtol=1e-3), (dy[r].cpu() - want_y).abs().max().item()


def test_row_pushed_product_rejects_ragged_ownership(built_lib):
    from fxfusion_b200.kernels import linear_pushed
    windows = [torch.zeros(384, 256, device="cuda") for _ in range(2)]
    with pytest.raises(RuntimeError, match="128-row"):
        linear_pushed(torch.zeros(384, 128, device="cuda"), torch.zeros(256, 128, device="cuda"), None, windows, 0)
