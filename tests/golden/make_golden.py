"""Generates the golden fixtures in this directory from the reference itself.

    python tests/golden/make_golden.py [/path/to/reference]

For every case (they follow the reference's own py/tests/test_ops.py, with smaller spatial sizes
so the files stay small) the UNMODIFIED reference is run twice in this process:
  * its FX passes (FusionPass, ShapePropPass, MemoryPlanningPass) lower the model and the result
    is written as `<case>.bin` with this repository's FlatBuffers writer;
  * its eager PyTorch model — the ground truth the reference's tests compare against
    (py/tests/utils.py:93-106) — produces the expected outputs, stored with the inputs in
    `<case>.npz` (`in0..`, `out0..`; decode cases store `tokens` and `expected_tokens`).
The reference checkout is not available where the GPU tests run, so these files are committed.
"""
from __future__ import annotations

import os
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REPO = HERE.parents[1]
sys.path.insert(0, str(REPO))
REFERENCE = sys.argv[1] if len(sys.argv) > 1 else (os.environ.get("FXFUSION_REFERENCE") or str(REPO.parent / "reference"))
os.environ.setdefault("FXFUSION_REFERENCE_PY", str(Path(REFERENCE) / "py"))
sys.dont_write_bytecode = True

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.nn as nn  # noqa: E402

from fxfusion_b200 import wire  # noqa: E402
from fxfusion_b200.compile_ref import _ensure_reference_importable, compile_with_reference  # noqa: E402

_ensure_reference_importable()
from fxfusion.models.transformer.blocks.gpt_block import GPTBlock  # noqa: E402
from fxfusion.models.transformer.layers.embedding import PositionalEncoding  # noqa: E402
from fxfusion.models.transformer.layers.masks import StaticDecoderMaskBuilder, make_static_buffer  # noqa: E402
from fxfusion.models.transformer.models.gpt import GPT  # noqa: E402

torch.set_grad_enabled(False)


def _np(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().numpy()


def emit(name: str, model: nn.Module, inputs, extra=None) -> None:
    model = model.eval()
    _, graph = compile_with_reference(model, inputs, model_name=name)
    wire.dump(graph, HERE / f"{name}.bin")
    out = model(*inputs)
    outs = list(out) if isinstance(out, (tuple, list)) else [out]
    arrays = {f"in{i}": _np(t) for i, t in enumerate(inputs)}
    arrays.update({f"out{i}": _np(t) for i, t in enumerate(outs)})
    if extra:
        arrays.update(extra)
    np.savez_compressed(HERE / f"{name}.npz", **arrays)
    ops = [wire.OPCODES[n.op_code] for n in graph.nodes if n.op_code]
    print(f"{name:36s} arena {graph.arena_size:8d}  ops {ops}")


def greedy_decode_static(model, tokens, mask_builder, max_seq_len):
    """The reference's eager greedy loop (py/fxfusion/models/transformer/inference.py:6-24); that module
    cannot be imported here because it pulls in the reference's compiled extension."""
    buf = make_static_buffer(tokens, max_seq_len)
    cur = tokens.shape[1]
    for _ in range(max_seq_len - tokens.shape[1]):
        logits = model(buf, mask_builder(buf, cur))
        buf[:, cur] = logits[:, cur - 1, :].argmax(dim=-1)
        cur += 1
    return buf[:, :cur]


def Lambda(fn):
    """Wraps a 1- or 2-argument tensor function in a traceable module."""
    import inspect

    if len(inspect.signature(fn).parameters) == 1:
        class M1(nn.Module):
            def forward(self, x):
                return fn(x)
        return M1()

    class M2(nn.Module):
        def forward(self, x, y):
            return fn(x, y)
    return M2()


def main() -> None:
    torch.manual_seed(0)

    class Conv(nn.Module):
        def __init__(self, relu, stride):
            super().__init__()
            self.conv = nn.Conv2d(3, 16, kernel_size=3, stride=stride, padding=1)
            self.relu = nn.ReLU()
            self.with_relu = relu

        def forward(self, x):
            return self.relu(self.conv(x)) if self.with_relu else self.conv(x)

    class ConvBnRelu(nn.Module):
        def __init__(self):
            super().__init__()
            self.conv = nn.Conv2d(8, 24, kernel_size=7, stride=2, padding=3, bias=False)
            self.bn = nn.BatchNorm2d(24)
            self.bn.running_mean.normal_(0, 0.1)
            self.bn.running_var.uniform_(0.5, 1.5)
            self.bn.weight.data.normal_(1, 0.1)
            self.bn.bias.data.normal_(0, 0.1)
            self.relu = nn.ReLU()

        def forward(self, x):
            return self.relu(self.bn(self.conv(x)))

    emit("conv2d", Conv(False, 1), [torch.randn(1, 3, 20, 20)])
    emit("conv2d_relu", Conv(True, 2), [torch.randn(2, 3, 21, 19)])
    emit("conv_bn_relu", ConvBnRelu(), [torch.randn(2, 8, 30, 30)])
    emit("max_pool2d", nn.Sequential(nn.MaxPool2d(kernel_size=3, stride=2, padding=1)), [torch.randn(1, 8, 28, 28)])
    emit("max_pool2d_ceil", nn.Sequential(nn.MaxPool2d(kernel_size=3, stride=2, padding=0, ceil_mode=True)), [torch.randn(1, 4, 14, 15)])
    emit("avg_pool2d", nn.Sequential(nn.AvgPool2d(kernel_size=3, stride=2, padding=1)), [torch.randn(1, 8, 28, 28)])
    emit("adaptive_avg_pool2d", nn.Sequential(nn.AdaptiveAvgPool2d((1, 1))), [torch.randn(2, 32, 7, 7)])
    emit("adaptive_avg_pool2d_3x2", nn.Sequential(nn.AdaptiveAvgPool2d((3, 2))), [torch.randn(1, 5, 10, 7)])
    emit("linear", nn.Sequential(nn.Linear(64, 100)), [torch.randn(1, 64)])
    emit("linear_relu", nn.Sequential(nn.Linear(64, 48), nn.ReLU()), [torch.randn(3, 64)])
    emit("add", Lambda(lambda x, y: x + y), [torch.randn(2, 8, 6, 6), torch.randn(2, 8, 6, 6)])
    emit("add_relu", Lambda(lambda x: torch.relu(x + x)), [torch.randn(1, 8, 6, 6)])
    emit("relu", Lambda(lambda x: torch.relu(x)), [torch.randn(2, 8, 6, 6)])
    emit("embedding", nn.Sequential(nn.Embedding(100, 16)), [torch.randint(1, 100, (2, 10))])
    emit("layernorm", nn.Sequential(nn.LayerNorm(64)), [torch.randn(2, 10, 64)])
    emit("layernorm_no_affine", nn.Sequential(nn.LayerNorm(64, elementwise_affine=False)), [torch.randn(2, 10, 64)])

    class AddLN(nn.Module):
        def __init__(self, affine):
            super().__init__()
            self.norm = nn.LayerNorm(64, elementwise_affine=affine)

        def forward(self, x):
            return self.norm(x + x)

    emit("add_layernorm", AddLN(True), [torch.randn(2, 10, 64)])
    emit("add_layernorm_no_affine", AddLN(False), [torch.randn(2, 10, 64)])
    emit("feedforward", nn.Sequential(nn.Linear(64, 256), nn.ReLU(), nn.Linear(256, 64)), [torch.randn(2, 10, 64)])

    class Residual(nn.Module):
        def __init__(self, down):
            super().__init__()
            c_out = 24 if down else 16
            self.conv1 = nn.Conv2d(16, c_out, kernel_size=3, stride=2 if down else 1, padding=1)
            self.conv2 = nn.Conv2d(c_out, c_out, kernel_size=3, stride=1, padding=1)
            self.down = nn.Conv2d(16, c_out, kernel_size=1, stride=2, padding=0) if down else None

        def forward(self, x):
            skip = self.down(x) if self.down is not None else x
            return torch.relu(self.conv2(torch.relu(self.conv1(x))) + skip)

    emit("residual_block", Residual(False), [torch.randn(1, 16, 14, 14)])
    emit("residual_block_downsample", Residual(True), [torch.randn(1, 16, 14, 14)])
    emit("mlp", nn.Sequential(nn.Linear(64, 64), nn.ReLU(), nn.Linear(64, 64), nn.ReLU(), nn.Linear(64, 10)), [torch.randn(4, 64)])
    emit("transpose_multidim", Lambda(lambda x: x.transpose(0, 2)), [torch.randn(2, 5, 7, 3)])
    emit("transpose_then_view", Lambda(lambda x: x.transpose(0, 2).contiguous().view(6, 16).transpose(0, 1)), [torch.randn(2, 8, 6)])
    emit("transpose_last2", Lambda(lambda x: x.transpose(-2, -1)), [torch.randn(3, 37, 41)])
    emit("mul_tensor_tensor", Lambda(lambda x: x * x), [torch.randn(4, 64)])
    emit("mul_tensor_scalar_float", Lambda(lambda x: 0.5 * (x * 2.5)), [torch.randn(4, 64)])
    emit("mul_tensor_scalar_int", Lambda(lambda x: 2 * (x * 3)), [torch.randn(4, 64)])
    emit("mul_tensor_scalar_bool", Lambda(lambda x: False * (x * True)), [torch.randn(4, 64)])
    emit("narrow", Lambda(lambda x: torch.narrow(x, 1, 0, 5)), [torch.randn(2, 10, 64)])
    emit("narrow_offset", Lambda(lambda x: torch.narrow(x, 2, 3, 7)), [torch.randn(2, 5, 13)])
    emit("narrow_dynamic_length", Lambda(lambda x, y: torch.narrow(x, 1, 0, y.size(1))), [torch.randn(2, 10, 64), torch.randn(2, 5, 64)])
    emit("size", Lambda(lambda x: torch.narrow(x, 0, 0, x.size(0))), [torch.randn(6, 64)])

    class PEAdd(nn.Module):
        def __init__(self):
            super().__init__()
            self.register_buffer("pe", torch.randn(1, 20, 64))

        def forward(self, x):
            return x + torch.narrow(self.pe, 1, 0, x.size(1))

    emit("narrow_then_add_broadcast_batch", PEAdd(), [torch.randn(2, 10, 64)])
    emit("positional_encoding_batch2", PositionalEncoding(64, max_seq_len=50, dropout=0.0), [torch.randn(2, 10, 64)])
    emit("mha_via_block_batch2", GPTBlock(32, 4, expansion_factor=2, dropout=0.0), [torch.randn(2, 6, 32), torch.ones((2, 1, 6, 6), dtype=torch.bool)])
    # head_dim 64, sequence longer than one key tile, broadcast padding-style mask [B,1,1,T]
    pad_mask = torch.ones((2, 1, 1, 70), dtype=torch.bool)
    pad_mask[1, 0, 0, 50:] = False
    emit("mha_block_hd64_padmask", GPTBlock(128, 2, expansion_factor=2, dropout=0.0), [torch.randn(2, 70, 128), pad_mask])

    # ---- GPT: forward, greedy decode, NaN parity (one model, one graph shape) ----------------
    torch.manual_seed(0)
    d_model, h, vocab, exp, layers, B, T, L0 = 32, 4, 128, 2, 1, 2, 8, 5
    model = GPT(d_model, h, vocab, exp, 0.0, layers).eval()
    tokens = torch.randint(1, vocab, (B, L0))
    builder = StaticDecoderMaskBuilder(max_seq_len=T)
    buf = make_static_buffer(tokens, max_seq_len=T, pad_idx=0)
    mask = builder(buf, current_len=L0, pad_idx=0)
    expected = greedy_decode_static(model=model, tokens=tokens.clone(), mask_builder=builder, max_seq_len=T)
    emit("gpt_forward_static_shape", model, [buf, mask], extra={"tokens": _np(tokens), "expected_tokens": _np(expected)})
    # fully masked query row -> NaN rows must match (reference test_mha_fully_masked_row_nan_parity)
    full = torch.randint(1, vocab, (B, T))
    nan_mask = torch.ones((B, 1, T, T), dtype=torch.bool)
    nan_mask[0, 0, 0, :] = False
    emit("gpt_fully_masked_row", model, [full, nan_mask])
    # a 2-layer model decoded over more steps
    torch.manual_seed(1)
    model2 = GPT(64, 4, 200, 4, 0.0, 2).eval()
    B2, T2, L2 = 3, 24, 6
    tokens2 = torch.randint(1, 200, (B2, L2))
    builder2 = StaticDecoderMaskBuilder(max_seq_len=T2)
    buf2 = make_static_buffer(tokens2, max_seq_len=T2)
    expected2 = greedy_decode_static(model=model2, tokens=tokens2.clone(), mask_builder=builder2, max_seq_len=T2)
    emit("gpt_2layer_decode", model2, [buf2, builder2(buf2, L2)], extra={"tokens": _np(tokens2), "expected_tokens": _np(expected2)})


if __name__ == "__main__":
    main()
