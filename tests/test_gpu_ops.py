"""Per-kernel parity through fxf_kernel_invoke: each CUDA kernel against the CPU oracle's restatement
of the reference kernel on the same seeded inputs, including ragged, empty and odd-sized cases."""
import math

import pytest
import torch

from helpers import compare_outputs
from fxfusion_b200 import wire
from oracle.graph_oracle import KERNELS

pytestmark = pytest.mark.gpu
ATOL, RTOL = 1e-4, 1e-3


def both(op, reg, in_ids, out_ids, ints=(), floats=(), exact=False, precision="auto", atol=ATOL, rtol=RTOL):
    from fxfusion_b200.kernels import invoke
    cpu = [t.clone() for t in reg]
    KERNELS[wire.OP[op]](cpu, list(in_ids), list(out_ids), list(ints), list(floats))
    gpu = [t.cuda() for t in reg]
    invoke(op, gpu, in_ids, out_ids, ints, floats, precision=precision)
    torch.cuda.synchronize()
    got, want = gpu[out_ids[0]].cpu(), cpu[out_ids[0]]
    if exact:
        if got.dtype.is_floating_point:  # NaN != NaN, so compare NaN positions and the remaining bits separately
            assert torch.equal(torch.isnan(got), torch.isnan(want)), f"{op}: NaN positions differ"
            assert torch.equal(torch.nan_to_num(got, nan=0.0), torch.nan_to_num(want, nan=0.0)), f"{op}: not bit-exact"
        else:
            assert torch.equal(got, want), f"{op}: not bit-exact"
    else:
        ok, info = compare_outputs(got, want, atol=atol, rtol=rtol)
        assert ok, f"{op}: {info}"
    return got


def rnd(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed + sum(shape))
    return torch.randn(*shape, generator=g) * scale


@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (7, 13, 5), (32, 512, 512), (33, 65, 17), (128, 128, 64), (300, 700, 260),
                                   (512, 1000, 256), (1024, 768, 768), (5, 2304, 768), (0, 8, 4), (3, 4, 0)])
@pytest.mark.parametrize("relu", [False, True])
def test_linear(built_lib, M, N, K, relu):
    x, w, b = rnd(M, K), rnd(N, K, seed=1, scale=1 / math.sqrt(max(K, 1))), rnd(N, seed=2)
    both("LinearRelu" if relu else "Linear", [x, w, b, torch.zeros(M, N)], [0, 1, 2], [3], precision="fp32_simt")


# Shapes chosen so that every arm of the default tensor-core dispatch runs (asserted through fxf_gemm_variant): 256-wide
# tiles computed by CTA pairs (cta_group::2), 192- / 128- / 64-wide tiles with A in tensor memory; K-split last rounds (tiles
# not a multiple of the worker count, K >= 128), ragged M / N / K, an output pitch that is not a multiple of 4 (scalar
# epilogue, the 50257-column vocabulary among them), and accumulation chains of one to three chunks.  The single-CTA 256-wide
# and 224-wide hybrid variants are reached with CTA pairs switched off (test_linear_variants_without_cta_pairs).
TC_SHAPES = [
    (8192, 3072, 768, "256x256-pair-smemA"), (8192, 2304, 768, "256x256-pair-smemA"), (8192, 768, 3072, "256x256-pair-smemA"),
    (2048, 12565, 768, "256x256-pair-smemA"), (8192, 768, 768, "128x192-tmemA"), (4096, 576, 768, "128x192-tmemA"),
    (5000, 1111, 500, "128x192-tmemA"), (8192, 8288, 768, "256x256-pair-smemA"), (2048, 50257, 768, "256x256-pair-smemA"),
    (3000, 3000, 516, "256x256-pair-smemA"), (1000, 4096, 520, "256x256-pair-smemA"),
    (1024, 768, 768, "128x128-tmemA"), (300, 700, 260, "128x128-tmemA"), (512, 1001, 256, "128x128-tmemA"),
    (128, 128, 64, "128x128-tmemA"), (1024, 64, 256, "128x64-tmemA"), (200, 64, 36, "128x64-tmemA"),
]


@pytest.mark.parametrize("M,N,K,arm", TC_SHAPES)
@pytest.mark.parametrize("relu", [False, True])
@pytest.mark.parametrize("precision", ["auto", "fp32_3xtf32"])
def test_linear_tensor_core(built_lib, M, N, K, arm, relu, precision):
    """The tcgen05 GEMM itself, every variant, against the reference CPU kernel, in both fp32-grade arithmetics: three TF32
    products ("fp32_3xtf32") and one TF32 product + two bf16 corrections, which "auto" takes whenever K is a multiple of 8."""
    from fxfusion_b200.kernels import gemm_variant
    mixed = precision == "auto" and K % 8 == 0
    assert gemm_variant(M, N, K, precision) == ("tcgen05-tf32+2bf16-" if mixed else "tcgen05-tf32x3-") + arm
    x, w, b = rnd(M, K), rnd(N, K, seed=1, scale=1 / math.sqrt(K)), rnd(N, seed=2)
    both("LinearRelu" if relu else "Linear", [x, w, b, torch.zeros(M, N)], [0, 1, 2], [3], precision=precision)


def _linear_engine(M, N, K, tmp_path, relu=False, **options):
    """One Linear node as an engine (engine options reach the dispatch; fxf_kernel_invoke always uses the defaults)."""
    import numpy as np
    from fxfusion_b200 import lowering
    from fxfusion_b200.engine import ExecutionEngine
    b = lowering.GraphBuilder(f"lin_{M}_{N}_{K}")
    g = np.random.default_rng(M + N + K)
    w = (g.standard_normal((N, K), dtype=np.float32) / math.sqrt(K)).astype(np.float32)
    bias = g.standard_normal((N,), dtype=np.float32)
    x = b.input((M, K), wire.DT_F32)
    b.output(b.op("LinearRelu" if relu else "Linear", [x, b.const(w), b.const(bias)], (M, N)))
    path = tmp_path / f"lin_{M}_{N}_{K}.bin"
    wire.dump(b.finish(), path)
    return ExecutionEngine(str(path), "cuda:0", **options), torch.from_numpy(w), torch.from_numpy(bias)


@pytest.mark.parametrize("M,N,K,arm", [(8192, 3072, 768, "128x256-smemA"), (2048, 50257, 768, "128x224-hybridA"), (8192, 8288, 768, "128x224-hybridA"),
                                       (3000, 3000, 516, "128x256-smemA")])
def test_linear_variants_without_cta_pairs(built_lib, tmp_path, M, N, K, arm):
    """Engine option tc_pair = 1: the widest tiles are computed by single CTAs (256-wide with A in shared memory, and the
    224-wide hybrid the time model picks for very wide outputs) — the variants convolutions and pair-less engines use."""
    eng, w, bias = _linear_engine(M, N, K, tmp_path, relu=True, tc_pair=1, precision="fp32_3xtf32")
    assert "tcgen05-tf32x3-" + arm in eng.describe()
    x = rnd(M, K)
    got = eng.run([x.cuda()])[0].cpu()
    want = torch.zeros(M, N)
    KERNELS[wire.OP["LinearRelu"]]([x, w, bias, want], [0, 1, 2], [3], [], [])
    ok, info = compare_outputs(got, want, atol=ATOL, rtol=RTOL)
    assert ok, info
    assert eng.device_status() == 0
    eng.close()


@pytest.mark.parametrize("M,N,K,arm,options", [
    (8192, 3072, 768, "256x256-pair", {}), (8192, 768, 3072, "256x256-pair", {}), (2048, 50257, 768, "256x256-pair", {}),
    (8192, 3072, 768, "128x192", {"tc_pair": 1}), (1024, 768, 768, "128x128", {}), (300, 700, 264, "128x128", {}), (1024, 64, 256, "128x64", {}),
    (2048, 50257, 768, "128x192", {"tc_pair": 1}), (512, 200, 4096, "128x128", {}), (8192, 768, 768, "128x192", {})])
def test_linear_mixed_tf32_bf16_mode(built_lib, tmp_path, M, N, K, arm, options):
    """Mode fp32_tf32_bf16x2: x_hi*w_hi as TF32 products, the corrections bf16(x_lo)*bf16(w_hi) and bf16(x)*bf16(w_lo) as one
    bf16 product each per 16 K-elements — with CTA pairs (operands in shared memory) and without (A in tensor memory).  It
    is held to the same 1e-4 / 1e-3 rule as the 3xTF32 mode."""
    eng, w, bias = _linear_engine(M, N, K, tmp_path, precision="fp32_tf32_bf16x2", **options)
    assert "tcgen05-tf32+2bf16-" + arm in eng.describe(), eng.describe()
    x = rnd(M, K)
    got = eng.run([x.cuda()])[0].cpu()
    want = torch.zeros(M, N)
    KERNELS[wire.OP["Linear"]]([x, w, bias, want], [0, 1, 2], [3], [], [])
    ok, info = compare_outputs(got, want, atol=ATOL, rtol=RTOL)
    assert ok, info
    assert eng.device_status() == 0
    eng.close()


@pytest.mark.parametrize("M,N,K", [(256, 256, 16384), (384, 192, 6144), (1000, 300, 3072)])
def test_tensor_core_error_does_not_grow_with_k(built_lib, M, N, K):
    """The tensor core adds into its accumulator with truncation (about 4e-8 * K of the result's scale for one chain);
    the kernel cuts the K loop into chains of 1024 and sums them with CUDA cores, so a K of 16384 still lands within
    6e-5 of the scale (one unbroken chain would be off by 6e-4)."""
    from fxfusion_b200.kernels import invoke
    x, w, b = rnd(M, K), rnd(N, K, seed=1, scale=1 / math.sqrt(K)), rnd(N, seed=2)
    want = (x.double() @ w.double().T + b.double())
    out = torch.zeros(M, N).cuda()
    invoke("Linear", [x.cuda(), w.cuda(), b.cuda(), out], [0, 1, 2], [3], precision="auto")
    err = ((out.cpu().double() - want).abs().max() / want.abs().max()).item()
    assert err < 6e-5, err
    both("Linear", [x, w, b, torch.zeros(M, N)], [0, 1, 2], [3], precision="auto")


def test_linear_keeps_leading_dims(built_lib):
    both("Linear", [rnd(2, 3, 5, 16), rnd(24, 16, seed=1), rnd(24, seed=2), torch.zeros(2, 3, 5, 24)], [0, 1, 2], [3])


@pytest.mark.parametrize("M,D,F,P", [(20, 64, 256, 64), (32, 512, 512, 10), (130, 96, 200, 50)])
def test_feedforward(built_lib, M, D, F, P):
    reg = [rnd(M, D), rnd(F, D, seed=1, scale=0.1), rnd(F, seed=2), rnd(P, F, seed=3, scale=0.1), rnd(P, seed=4), torch.zeros(M, P)]
    both("FeedForward", reg, [0, 1, 2, 3, 4], [5])


def _mha_reg(B, T, H, hd, mask):
    D = H * hd
    return [rnd(B, T, D), mask, rnd(3 * D, D, seed=1, scale=1 / math.sqrt(D)), rnd(3 * D, seed=2, scale=0.1),
            rnd(D, D, seed=3, scale=1 / math.sqrt(D)), rnd(D, seed=4, scale=0.1), torch.zeros(B, T, D)]


@pytest.mark.parametrize("precision", ["auto", "fp32_simt"])
@pytest.mark.parametrize("B,T,H,hd", [(2, 6, 4, 8), (1, 5, 2, 16), (2, 64, 4, 64), (1, 65, 2, 64), (3, 130, 3, 32), (1, 8, 1, 128), (2, 33, 2, 20),
                                      (1, 128, 1, 64), (1, 256, 2, 64), (2, 72, 2, 64), (1, 200, 3, 64), (3, 16, 1, 64), (2, 384, 2, 64)])
def test_mha_causal(built_lib, B, T, H, hd, precision):
    """head_dim 64 with T % 4 == 0 takes the tcgen05 attention kernel in "auto" mode, everything else the fp32 one."""
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool)).view(1, 1, T, T).expand(B, 1, T, T).contiguous()
    both("MHA", _mha_reg(B, T, H, hd, mask), [0, 1, 2, 3, 4, 5], [6], ints=[H, hd, H * hd, 3 * H * hd], floats=[math.sqrt(hd)], precision=precision)


def test_mha_beyond_4096_keys(built_lib):
    """The tcgen05 attention kernel tracks its key blocks in one 32-bit word (32 blocks of 128 keys); longer sequences must
    take the fp32 kernel instead of silently dropping the keys from position 4096 on."""
    B, T, H, hd = 1, 4224, 1, 64
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool)).view(1, 1, T, T)
    got = both("MHA", _mha_reg(B, T, H, hd, mask), [0, 1, 2, 3, 4, 5], [6], ints=[H, hd, H * hd, 3 * H * hd], floats=[math.sqrt(hd)])
    assert not torch.isnan(got).any()


@pytest.mark.parametrize("hd", [16, 64])
@pytest.mark.parametrize("shape", ["b11t", "11tt", "bhtt", "random"])
def test_mha_mask_broadcast_shapes(built_lib, shape, hd):
    B, T, H = 2, 40 if hd == 16 else 136, 3
    g = torch.Generator().manual_seed(5)
    if shape == "b11t":
        mask = torch.ones(B, 1, 1, T, dtype=torch.bool)
        mask[1, 0, 0, 25:] = False
    elif shape == "11tt":
        mask = torch.tril(torch.ones(T, T, dtype=torch.bool)).view(1, 1, T, T)
    elif shape == "bhtt":
        mask = torch.rand(B, H, T, T, generator=g) < 0.7
        mask[..., 0] = True
    else:
        mask = torch.rand(B, 1, T, T, generator=g) < 0.5
        mask[..., 0] = True
    both("MHA", _mha_reg(B, T, H, hd, mask), [0, 1, 2, 3, 4, 5], [6], ints=[H, hd, H * hd, 3 * H * hd], floats=[math.sqrt(hd)])


@pytest.mark.parametrize("precision", ["auto", "fp32_simt"])
@pytest.mark.parametrize("B,Tq,Tk,H,hd,mask_kind", [(2, 6, 9, 4, 8, "b11k"), (1, 40, 72, 2, 64, "b11k"), (2, 130, 64, 3, 64, "bqk"), (2, 24, 256, 2, 64, "causal-ish"),
                                                   (1, 5, 33, 2, 20, "bqk"), (2, 128, 384, 2, 64, "b11k"), (1, 7, 16, 1, 64, "11qk")])
def test_cross_mha(built_lib, B, Tq, Tk, H, hd, mask_kind, precision):
    """Attention with queries from one sequence and keys/values from another (extension opcode CrossMHA): head_dim 64
    with Tk % 4 == 0 takes the tcgen05 kernel in "auto" mode.  Oracle = the reference's eager MultiHeadAttention math."""
    D = H * hd
    g = torch.Generator().manual_seed(3)
    if mask_kind == "b11k":
        mask = torch.ones(B, 1, 1, Tk, dtype=torch.bool)
        mask[-1, 0, 0, Tk - Tk // 3:] = False
    elif mask_kind == "bqk":
        mask = torch.rand(B, 1, Tq, Tk, generator=g) < 0.6
        mask[..., 0] = True
    elif mask_kind == "11qk":
        mask = torch.rand(1, 1, Tq, Tk, generator=g) < 0.5
        mask[..., 1] = True
    else:  # a band: query q sees keys <= 10 q  (whole key blocks are masked for the early queries)
        mask = (torch.arange(Tk).view(1, 1, 1, Tk) <= 10 * torch.arange(Tq).view(1, 1, Tq, 1)).expand(B, 1, Tq, Tk).contiguous()
    reg = [rnd(B, Tq, D), rnd(B, Tk, D, seed=9), mask, rnd(D, D, seed=1, scale=1 / math.sqrt(D)), rnd(D, seed=2, scale=0.1),
           rnd(2 * D, D, seed=3, scale=1 / math.sqrt(D)), rnd(2 * D, seed=4, scale=0.1), rnd(D, D, seed=5, scale=1 / math.sqrt(D)), rnd(D, seed=6, scale=0.1),
           torch.zeros(B, Tq, D)]
    both("CrossMHA", reg, [0, 1, 2, 3, 4, 5, 6, 7, 8], [9], ints=[H, hd, D, 2 * D], floats=[math.sqrt(hd)], precision=precision)


def test_cross_mha_rejects_inconsistent_operands(built_lib):
    from fxfusion_b200.kernels import invoke
    D = 32
    reg = [rnd(2, 4, D).cuda(), rnd(3, 5, D).cuda(), torch.ones(2, 1, 1, 5, dtype=torch.bool).cuda(), rnd(D, D).cuda(), rnd(D).cuda(),
           rnd(2 * D, D).cuda(), rnd(2 * D).cuda(), rnd(D, D).cuda(), rnd(D).cuda(), torch.zeros(2, 4, D).cuda()]
    with pytest.raises(RuntimeError, match="cross_mha"):   # memory batch differs from x batch
        invoke("CrossMHA", reg, [0, 1, 2, 3, 4, 5, 6, 7, 8], [9], ints=[4, 8, D, 2 * D], floats=[math.sqrt(8)])


def test_mha_fully_masked_rows_and_nan_values(built_lib):
    """A fully masked query row is NaN; a NaN in the input poisons exactly what torch's matmul poisons."""
    _masked_rows_and_nan(2, 12, 2, 8)
    _masked_rows_and_nan(2, 132, 2, 64)   # the tcgen05 attention kernel, two key blocks
    # three key blocks, causal: the kernel may skip a block whose mask bytes are all zero, but not one whose V rows
    # hold a NaN (position 300 is masked for the first 300 queries and still poisons them, as 0 * NaN does in torch)
    _masked_rows_and_nan(2, 384, 2, 64, nan_pos=300)


@pytest.mark.parametrize("H", [2, 12])
def test_mha_block_sparse_masks(built_lib, H):
    """Masks with whole 128-key blocks of zeros (skipped by the tcgen05 kernel) next to fully masked rows and a CTA
    whose every block is masked.  With 12 heads the packed projection is wide enough for the 256-wide tiles whose epilogue
    writes V transposed and its finite flags itself (no transpose launch): the non-finite V row has to be found there too."""
    B, T, hd = 2, 512, 64
    mask = torch.ones(B, 1, T, T, dtype=torch.bool)
    mask[:, :, :, 128:256] = False            # one key block is dead for every query
    mask[0, :, 256:384, :] = False            # batch 0: a whole query tile sees nothing -> NaN rows
    mask[1, :, 5, :] = False                  # batch 1: one fully masked row
    mask[1, :, 384:, :384] = False            # batch 1: the last query tile sees only the last key block
    got = both("MHA", _mha_reg(B, T, H, hd, mask), [0, 1, 2, 3, 4, 5], [6], ints=[H, hd, H * hd, 3 * H * hd], floats=[math.sqrt(hd)])
    assert torch.isnan(got[0, 256:384]).all() and torch.isnan(got[1, 5]).all() and not torch.isnan(got[1, 384:]).any()
    # an infinite V element inside the dead block still reaches every row (0 * inf = NaN in the reference)
    reg = _mha_reg(B, T, H, hd, mask)
    reg[0][1, 200, :] = float("inf")
    both("MHA", reg, [0, 1, 2, 3, 4, 5], [6], ints=[H, hd, H * hd, 3 * H * hd], floats=[math.sqrt(hd)])


def _masked_rows_and_nan(B, T, H, hd, nan_pos=9):
    mask = torch.ones(B, 1, T, T, dtype=torch.bool)
    mask[0, 0, 3, :] = False
    reg = _mha_reg(B, T, H, hd, mask)
    got = both("MHA", reg, [0, 1, 2, 3, 4, 5], [6], ints=[H, hd, H * hd, 3 * H * hd], floats=[math.sqrt(hd)])
    assert torch.isnan(got[0, 3]).all() and not torch.isnan(got[1]).any()
    reg = _mha_reg(B, T, H, hd, torch.tril(torch.ones(T, T, dtype=torch.bool)).view(1, 1, T, T).expand(B, 1, T, T).contiguous())
    reg[0][1, nan_pos, :] = float("nan")  # a NaN token late in the sequence: masked for earlier queries, weight 0 * NaN
    both("MHA", reg, [0, 1, 2, 3, 4, 5], [6], ints=[H, hd, H * hd, 3 * H * hd], floats=[math.sqrt(hd)])


@pytest.mark.parametrize("M,N", [(1, 1), (3, 5), (20, 64), (8192, 768), (7, 1024), (5, 1028), (4, 4096), (9, 130), (0, 16)])
def test_layer_norm_and_add_layer_norm(built_lib, M, N):
    x, z, w, b = rnd(M, N, scale=3.0) + 0.5, rnd(M, N, seed=1), rnd(N, seed=2), rnd(N, seed=3)
    both("LayerNorm", [x, w, b, torch.zeros(M, N)], [0, 1, 2], [3], ints=[1, N], floats=[1e-5])
    both("AddLayerNorm", [x, z, w, b, torch.zeros(M, N)], [0, 1, 2, 3], [4], ints=[1, N], floats=[1e-5])


def test_layer_norm_two_normalized_dims(built_lib):
    x, w, b = rnd(3, 6, 10), rnd(6, 10, seed=1), rnd(6, 10, seed=2)
    both("LayerNorm", [x, w, b, torch.zeros(3, 6, 10)], [0, 1, 2], [3], ints=[2, 6, 10], floats=[1e-5])


@pytest.mark.parametrize("sa,sb", [((2, 8, 6, 6), (2, 8, 6, 6)), ((32, 256, 768), (1, 256, 768)), ((4, 10, 64), (64,)),
                                   ((3, 5, 7), (3, 1, 7)), ((1, 5, 7), (3, 5, 7)), ((5,), (5,)), ((2, 3), (1,)), ((0, 4), (0, 4))])
def test_add_family_broadcasting(built_lib, sa, sb):
    a, b = rnd(*sa), rnd(*sb, seed=1)
    out = torch.zeros(torch.broadcast_shapes(sa, sb))
    both("Add", [a, b, out], [0, 1], [2], exact=True)
    both("AddRelu", [a, b, out], [0, 1], [2], exact=True)
    both("Mul", [a, b, out], [0, 1], [2], ints=[0], exact=True)


def test_relu_and_scalar_mul_including_nan(built_lib):
    x = rnd(5, 33)
    x[0, 0], x[1, 1], x[2, 2] = float("nan"), float("inf"), -float("inf")
    both("Relu", [x, torch.zeros(5, 33)], [0], [1], exact=True)
    for mode, s in ((1, 2.5), (2, 3.0), (3, 0.0)):
        both("Mul", [x, torch.zeros(5, 33)], [0], [1], ints=[mode], floats=[s], exact=True)
    both("Relu", [rnd(16, 64), torch.zeros(16, 64)], [0], [1], exact=True)


def test_relu_in_place_alias(built_lib):
    """The planner may alias Relu's output onto its input (reference passes/memory_plan.py:72-75)."""
    from fxfusion_b200.kernels import invoke
    x = rnd(7, 64).cuda()
    want = torch.relu(x.cpu())
    invoke("Relu", [x, x], [0], [1])
    assert torch.equal(x.cpu(), want)


def test_size_writes_int64_scalar(built_lib):
    both("Size", [rnd(6, 10, 64), torch.zeros((), dtype=torch.int64)], [0], [1], ints=[1], exact=True)
    both("Size", [rnd(6, 10, 64), torch.zeros((), dtype=torch.int64)], [0], [1], ints=[-1], exact=True)


@pytest.mark.parametrize("shape,dim,start,length", [((2, 10, 64), 1, 0, 5), ((2, 5, 13), 2, 3, 7), ((1, 5000, 32), 1, 0, 8),
                                                    ((6, 64), 0, 2, 3), ((4, 3, 5), 1, 1, 1), ((3, 7), 1, 0, 0)])
def test_narrow_is_bit_exact(built_lib, shape, dim, start, length):
    x = rnd(*shape)
    out_shape = list(shape)
    out_shape[dim] = length
    both("Narrow", [x, torch.zeros(out_shape)], [0], [1], ints=[dim, start, length], exact=True)
    # dynamic form: length -1, taken from a scalar tensor in the reference and from the output shape here
    both("Narrow", [x, torch.tensor(length, dtype=torch.int64), torch.zeros(out_shape)], [0, 1], [2], ints=[dim, start, -1], exact=True)


def test_narrow_other_dtypes(built_lib):
    x = torch.arange(2 * 9 * 5, dtype=torch.int64).view(2, 9, 5)
    both("Narrow", [x, torch.zeros(2, 4, 5, dtype=torch.int64)], [0], [1], ints=[1, 2, 4], exact=True)
    m = torch.rand(3, 11, generator=torch.Generator().manual_seed(0)) < 0.5
    both("Narrow", [m, torch.zeros(3, 5, dtype=torch.bool)], [0], [1], ints=[1, 3, 5], exact=True)


@pytest.mark.parametrize("V,D,shape", [(1000, 64, (2, 10)), (50, 7, (3,)), (128, 768, (32, 256)), (10, 4, (0,))])
def test_embedding_is_bit_exact(built_lib, V, D, shape):
    idx = torch.randint(0, V, shape, generator=torch.Generator().manual_seed(0))
    both("Embedding", [idx, rnd(V, D), torch.zeros(*shape, D)], [0, 1], [2], exact=True)


@pytest.mark.parametrize("shape,d0,d1", [((2, 5, 7, 3), 0, 2), ((6, 16), 0, 1), ((3, 37, 41), -2, -1), ((2, 8, 4, 16), 1, 2),
                                         ((2, 3, 4, 5, 2, 3, 2, 2), 1, 6), ((5, 1), 0, 1), ((4, 6), 1, 1)])
def test_transpose_is_bit_exact(built_lib, shape, d0, d1):
    x = rnd(*shape)
    want_shape = list(torch.transpose(x, d0, d1).shape)
    both("Transpose", [x, torch.zeros(want_shape)], [0], [1], ints=[d0 % len(shape), d1 % len(shape)], exact=True)


@pytest.mark.parametrize("N,C,H,W,O,k,s,p,d,g,relu", [
    (1, 3, 20, 20, 16, 3, 1, 1, 1, 1, False), (2, 3, 21, 19, 16, 3, 2, 1, 1, 1, True), (2, 8, 30, 30, 24, 7, 2, 3, 1, 1, True),
    (1, 16, 14, 14, 24, 1, 2, 0, 1, 1, False), (2, 8, 12, 12, 8, 3, 1, 2, 2, 1, False), (1, 12, 9, 9, 18, 3, 1, 1, 1, 3, True),
    (3, 64, 7, 7, 130, 1, 1, 0, 1, 1, True)])
def test_conv2d(built_lib, N, C, H, W, O, k, s, p, d, g, relu):
    x, w, b = rnd(N, C, H, W), rnd(O, C // g, k, k, seed=1, scale=1 / math.sqrt(C // g * k * k)), rnd(O, seed=2)
    ho = (H + 2 * p - d * (k - 1) - 1) // s + 1
    wo = (W + 2 * p - d * (k - 1) - 1) // s + 1
    both("Conv2dRelu" if relu else "Conv2d", [x, w, b, torch.zeros(N, O, ho, wo)], [0, 1, 2], [3],
         ints=[s, s, p, p, d, d, g, 1, 1, 1, 256, 1, 1])


def test_pools(built_lib):
    x = rnd(2, 8, 28, 28)
    both("MaxPool2d", [x, torch.zeros(2, 8, 14, 14)], [0], [1], ints=[3, 3, 2, 2, 1, 1, 1, 1, 0] + [1, 1, 1, 256, 1, 1], exact=True)
    y = rnd(1, 4, 14, 15)
    both("MaxPool2d", [y, torch.zeros(1, 4, 7, 7)], [0], [1], ints=[3, 3, 2, 2, 0, 0, 1, 1, 1] + [1, 1, 1, 256, 1, 1], exact=True)
    both("AvgPool2d", [x, torch.zeros(2, 8, 14, 14)], [0], [1], ints=[3, 3, 2, 2, 1, 1, 0] + [1, 1, 1, 256, 1, 1])
    both("AvgPool2d", [y, torch.zeros(1, 4, 7, 8)], [0], [1], ints=[2, 2, 2, 2, 0, 0, 1] + [1, 1, 1, 256, 1, 1])
    both("AdaptiveAvgPool2d", [rnd(2, 32, 7, 7), torch.zeros(2, 32, 1, 1)], [0], [1], ints=[1, 1] + [1, 1, 1, 256, 1, 1])
    both("AdaptiveAvgPool2d", [rnd(1, 5, 10, 7), torch.zeros(1, 5, 3, 2)], [0], [1], ints=[3, 2] + [1, 1, 1, 256, 1, 1])
    z = rnd(1, 2, 6, 6)
    z[0, 0, 2, 2] = float("nan")
    both("MaxPool2d", [z, torch.zeros(1, 2, 3, 3)], [0], [1], ints=[2, 2, 2, 2, 0, 0, 1, 1, 0] + [1, 1, 1, 256, 1, 1])


def test_argument_errors_are_reported_not_executed(built_lib):
    from fxfusion_b200.kernels import invoke
    x, w, b, o = rnd(4, 8).cuda(), rnd(6, 9).cuda(), rnd(6).cuda(), torch.zeros(4, 6).cuda()
    with pytest.raises(RuntimeError, match="does not match weight"):
        invoke("Linear", [x, w, b, o], [0, 1, 2], [3])
    with pytest.raises(RuntimeError, match="unknown mul_mode"):
        invoke("Mul", [x, torch.zeros(4, 8).cuda()], [0], [1], ints=[7], floats=[1.0])
    with pytest.raises(RuntimeError, match="slice exceeds"):
        invoke("Narrow", [x, torch.zeros(4, 9).cuda()], [0], [1], ints=[1, 0, 9])


def test_channels_last_tensors_are_honoured(built_lib):
    """Kernels address 4-D tensors through their strides: channels-last inputs / outputs (what the engine uses
    between convolutions) give the same values as NCHW ones."""
    from fxfusion_b200.kernels import invoke
    cl = lambda t: t.contiguous(memory_format=torch.channels_last)
    N, C, H, W, O = 2, 64, 14, 14, 96
    x, w1, b1 = rnd(N, C, H, W), rnd(O, C, 1, 1, seed=1, scale=0.1), rnd(O, seed=2)
    w3, b3 = rnd(O, C, 3, 3, seed=3, scale=0.05), rnd(O, seed=4)
    ints = lambda s, p: [s, s, p, p, 1, 1, 1, 1, 1, 1, 256, 1, 1]
    for wt, bs, s, p in ((w1, b1, 1, 0), (w1, b1, 2, 0), (w3, b3, 1, 1), (w3, b3, 2, 1)):
        want = torch.relu(torch.conv2d(x, wt, bs, s, p))
        for xin in (x.cuda(), cl(x.cuda())):
            for out in (torch.zeros_like(want).cuda(), cl(torch.zeros_like(want).cuda())):
                invoke("Conv2dRelu", [xin, wt.cuda(), bs.cuda(), out], [0, 1, 2], [3], ints=ints(s, p))
                assert out.stride() != want.stride() or True
                ok, info = compare_outputs(out.cpu().contiguous(), want, atol=ATOL, rtol=RTOL)
                assert ok, (s, p, xin.stride(), out.stride(), info)
    xc = cl(x.cuda())
    mp = cl(torch.zeros(N, C, 7, 7).cuda())
    invoke("MaxPool2d", [xc, mp], [0], [1], ints=[3, 3, 2, 2, 1, 1, 1, 1, 0, 1, 1, 1, 256, 1, 1])
    assert torch.equal(mp.cpu().contiguous(), torch.max_pool2d(x, 3, 2, 1))
    ap = torch.zeros(N, C, 1, 1).cuda()
    invoke("AdaptiveAvgPool2d", [xc, ap], [0], [1], ints=[1, 1, 1, 1, 1, 256, 1, 1])
    assert torch.allclose(ap.cpu(), torch.nn.functional.adaptive_avg_pool2d(x, 1), atol=1e-5)
    y = cl(rnd(N, C, H, W, seed=9).cuda())
    o = cl(torch.zeros(N, C, H, W).cuda())
    invoke("AddRelu", [xc, y, o], [0, 1], [2])
    assert torch.equal(o.cpu().contiguous(), torch.relu(x + y.cpu().contiguous()))


@pytest.mark.gpu
@pytest.mark.parametrize("N,C,H,W,O,kh,kw,ph,pw,dh,dw,st", [
    (2, 64, 14, 14, 96, 3, 3, 1, 1, 1, 1, 1),     # ResNet-style 3x3, two images per 128-pixel box is impossible (196 > 128)
    (5, 32, 7, 7, 64, 3, 3, 1, 1, 1, 1, 1),       # whole images per box (49 pixels -> two images per tile, ragged batch)
    (1, 16, 56, 56, 64, 3, 3, 1, 1, 1, 1, 1),     # one 16-channel slab per tap
    (3, 48, 9, 20, 130, 5, 3, 2, 0, 1, 1, 1),     # asymmetric filter and padding, output channels not a tile multiple
    (2, 64, 17, 17, 64, 3, 3, 2, 2, 2, 2, 1),     # dilation 2
    (1, 128, 28, 28, 256, 3, 3, 0, 0, 1, 1, 1),   # no padding: output smaller than input
    (4, 64, 12, 12, 64, 1, 7, 0, 3, 1, 1, 1),     # 1 x 7
    (2, 128, 56, 56, 128, 3, 3, 1, 1, 1, 1, 2),   # ResNet stage transition: 3x3 stride 2
    (3, 256, 56, 56, 512, 1, 1, 0, 0, 1, 1, 2),   # ResNet downsample branch: 1x1 stride 2
    (5, 32, 15, 13, 64, 3, 3, 1, 1, 1, 1, 2),     # odd extents with stride 2 (whole images per box)
    (2, 16, 30, 30, 64, 5, 5, 2, 2, 1, 1, 2),     # 5x5 stride 2
    (2, 3, 64, 64, 64, 7, 7, 3, 3, 1, 1, 2),      # ResNet stem: 3 channels, 7x7 stride 2 -> space-to-depth + stride-1 tensor-core convolution
    (3, 4, 33, 29, 80, 3, 5, 1, 2, 1, 1, 2),      # 4 channels, odd extents, asymmetric filter
    (2, 1, 40, 40, 64, 4, 4, 0, 0, 1, 1, 2),      # one channel, even filter, no padding
])
def test_conv_implicit_gemm_tensor_core(built_lib, N, C, H, W, O, kh, kw, ph, pw, dh, dw, st):
    """Convolution (stride 1 or 2) over channels-last tensors runs as an implicit GEMM on the tensor cores
    (3xTF32); NCHW tensors and the fp32 mode take the SIMT kernel.  Both match torch.conv2d
    (reference semantics: csrc/kernels/cpu/conv2d.cpp:6-22, conv2d_relu.cpp)."""
    from fxfusion_b200.kernels import invoke
    cl = lambda t: t.contiguous(memory_format=torch.channels_last)
    x, w, b = rnd(N, C, H, W, seed=11), rnd(O, C, kh, kw, seed=12, scale=0.05), rnd(O, seed=13)
    ints = [st, st, ph, pw, dh, dw, 1]
    for relu in (False, True):
        want = torch.conv2d(x, w, b, st, (ph, pw), (dh, dw))
        want = torch.relu(want) if relu else want
        for precision in ("auto", "fp32_simt"):
            out = cl(torch.full_like(want, float("nan")).cuda())
            invoke("Conv2dRelu" if relu else "Conv2d", [cl(x.cuda()), w.cuda(), b.cuda(), out], [0, 1, 2], [3], ints=ints, precision=precision)
            ok, info = compare_outputs(out.cpu().contiguous(), want, atol=ATOL, rtol=RTOL)
            assert ok, (precision, relu, info)


def _rel_to_scale(got, want):
    return ((got - want).abs().max() / want.abs().max().clamp_min(1e-30)).item()


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (300, 700, 264), (8192, 768, 768), (1000, 2304, 768), (64, 50, 32), (256, 192, 4096)])
def test_bf16_mode_linear(built_lib, M, N, K):
    """Optional bf16 mode: operands rounded to bf16 for the tensor-core products, fp32 accumulation and output.
    Within 2e-2 of the output scale (measured about 3e-3); shapes the tensor-core kernel does not take fall back to fp32."""
    from fxfusion_b200.kernels import invoke
    x, w, b = rnd(M, K), rnd(N, K, seed=1, scale=1 / math.sqrt(K)), rnd(N, seed=2)
    want = torch.relu(torch.nn.functional.linear(x, w, b))
    out = torch.full((M, N), float("nan")).cuda()
    invoke("LinearRelu", [x.cuda(), w.cuda(), b.cuda(), out], [0, 1, 2], [3], precision="bf16")
    err = _rel_to_scale(out.cpu(), want)
    assert err < 2e-2, err
    # the rounding must actually be bf16-sized where the tensor-core kernel applies, and absent where it does not
    if M >= 64 and N >= 64 and K >= 32 and K % 8 == 0:
        assert err > 1e-5, "bf16 mode produced fp32-grade results: the bf16 kernel did not run"


def test_bf16_mode_mha_feedforward_conv(built_lib):
    from fxfusion_b200.kernels import invoke
    B, T, H, hd = 2, 128, 4, 64
    D = H * hd
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool)).view(1, 1, T, T).expand(B, 1, T, T).contiguous()
    reg = _mha_reg(B, T, H, hd, mask)
    cpu = [t.clone() for t in reg]
    KERNELS[wire.OP["MHA"]](cpu, [0, 1, 2, 3, 4, 5], [6], [H, hd, D, 3 * D], [math.sqrt(hd)])
    gpu = [t.cuda() for t in reg]
    invoke("MHA", gpu, [0, 1, 2, 3, 4, 5], [6], ints=[H, hd, D, 3 * D], floats=[math.sqrt(hd)], precision="bf16")
    assert _rel_to_scale(gpu[6].cpu(), cpu[6]) < 2e-2
    x, w1, b1, w2, b2 = rnd(512, 256), rnd(1024, 256, seed=1, scale=1 / 16), rnd(1024, seed=2), rnd(256, 1024, seed=3, scale=1 / 32), rnd(256, seed=4)
    want = torch.nn.functional.linear(torch.relu(torch.nn.functional.linear(x, w1, b1)), w2, b2)
    out = torch.zeros(512, 256).cuda()
    invoke("FeedForward", [x.cuda(), w1.cuda(), b1.cuda(), w2.cuda(), b2.cuda(), out], [0, 1, 2, 3, 4], [5], precision="bf16")
    assert _rel_to_scale(out.cpu(), want) < 2e-2
    cl = lambda t: t.contiguous(memory_format=torch.channels_last)
    xi, wc, bc = rnd(2, 64, 28, 28, seed=5), rnd(128, 64, 3, 3, seed=6, scale=0.05), rnd(128, seed=7)
    for stride in (1, 2):
        want = torch.relu(torch.conv2d(xi, wc, bc, stride, 1))
        out = cl(torch.zeros_like(want).cuda())
        invoke("Conv2dRelu", [cl(xi.cuda()), wc.cuda(), bc.cuda(), out], [0, 1, 2], [3], ints=[stride, stride, 1, 1, 1, 1, 1], precision="bf16")
        err = _rel_to_scale(out.cpu().contiguous(), want)
        assert 1e-5 < err < 2e-2, err
