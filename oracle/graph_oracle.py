"""TEST INFRASTRUCTURE — CPU restatement of the reference runtime's execution of a graph file.

The reference CPU backend delegates every kernel to LibTorch (`out.copy_(torch::<op>(...))`),
so its arithmetic IS ATen's CPU arithmetic (MKL sgemm, oneDNN convolution, ATen softmax and
layer_norm) of the installed torch build.  `requirements.txt:1` of the reference lists `torch`
unpinned; parity is therefore pinned relative to the torch installed next to this file and is
unpinned in absolute terms.  This module restates, op by op, the calls those kernels make and
walks a graph file the way the reference runtime does:

  run loop      csrc/runtime/runtime_graph.cpp:20-24, runtime_node.cpp:43-45 (NoOp skipped)
  registry      csrc/runtime/memory_manager.cpp:30-111 (alias/output share the source storage)
  conv2d        csrc/kernels/cpu/conv2d.cpp:5-17          conv2d_relu  conv2d_relu.cpp:5-17
  linear        csrc/kernels/cpu/linear.cpp:5-12          linear_relu  linear_relu.cpp:5-12
  add/add_relu  csrc/kernels/cpu/add.cpp:5-10, add_relu.cpp:5-11      relu  relu.cpp:5-9
  mul           csrc/kernels/cpu/mul.cpp:5-25
  pools         csrc/kernels/cpu/max_pool2d.cpp:5-16, avg_pool2d.cpp:5-15, adaptive_avg_pool2d.cpp:5-12
  transpose     csrc/kernels/cpu/transpose.cpp:5-12       size  size.cpp:5-11
  narrow        csrc/kernels/cpu/narrow.cpp:5-13          embedding  embedding.cpp:5-11
  layer_norm    csrc/kernels/cpu/layer_norm.cpp:5-16      add_layer_norm  add_layer_norm.cpp:5-17
  mha           csrc/kernels/cpu/mha.cpp:5-52             feedforward  feedforward.cpp:5-14

`oracle/ref_cpu/` compiles the reference's own, unmodified kernel sources into
`oracle/_ref/`; tests check that this restatement is bit-identical to them, and
`tests/golden/` pins both against outputs of the reference's eager models.

Arena aliasing is not modelled (every tensor has private storage): the planner guarantees an
op's output never overlaps its live inputs, so values are the same.
"""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Optional, Sequence

import numpy as np
import torch
import torch.nn.functional as F

from fxfusion_b200 import wire  # format reader only (no CUDA code is touched)

TORCH_DTYPES = [torch.float32, torch.float16, torch.int32, torch.int64, torch.bool]

# signature: fn(reg: list[Tensor|None], in_ids, out_ids, ints, floats) -> None (writes reg[out])
KernelFn = Callable[[List[Optional[torch.Tensor]], Sequence[int], Sequence[int], Sequence[int], Sequence[float]], None]


def _conv(reg, i, o, ints, floats, relu=False):
    y = torch.conv2d(reg[i[0]], reg[i[1]], reg[i[2]], [ints[0], ints[1]], [ints[2], ints[3]], [ints[4], ints[5]], ints[6])
    reg[o[0]].copy_(torch.relu(y) if relu else y)


def _mul(reg, i, o, ints, floats):
    mode = ints[0]
    if mode == 0:
        reg[o[0]].copy_(torch.mul(reg[i[0]], reg[i[1]]))
    elif mode in (1, 2, 3):
        reg[o[0]].copy_(torch.mul(reg[i[0]], float(np.float32(floats[0]))))
    else:
        raise RuntimeError(f"mul: unknown mul_mode {mode}")


def _narrow(reg, i, o, ints, floats):
    length = ints[2]
    if length < 0:
        length = int(reg[i[1]].item())
    reg[o[0]].copy_(reg[i[0]].narrow(ints[0], ints[1], length))


def _layer_norm(reg, i, o, ints, floats):
    shape = list(ints[1:1 + ints[0]])
    reg[o[0]].copy_(torch.layer_norm(reg[i[0]], shape, reg[i[1]], reg[i[2]], float(np.float32(floats[0]))))


def _add_layer_norm(reg, i, o, ints, floats):
    shape = list(ints[1:1 + ints[0]])
    reg[o[0]].copy_(torch.layer_norm(torch.add(reg[i[0]], reg[i[1]]), shape, reg[i[2]], reg[i[3]], float(np.float32(floats[0]))))


def _mha(reg, i, o, ints, floats):
    x, mask, wqkv, bqkv, wo, bo = (reg[k] for k in i[:6])
    H, hd, D, QKV = ints[:4]
    scale = float(np.float32(floats[0]))
    qkv = F.linear(x, wqkv, bqkv)
    B, T = x.size(0), x.size(1)
    q = qkv[:, :, 0:D].view(B, T, H, hd).transpose(1, 2)
    k = qkv[:, :, D:2 * D].view(B, T, H, hd).transpose(1, 2)
    v = qkv[:, :, 2 * D:QKV].view(B, T, H, hd).transpose(1, 2)
    scores = torch.matmul(q, k.transpose(-2, -1)) / scale
    scores = scores.masked_fill(mask == 0, -math.inf)
    attn = torch.softmax(scores, -1)
    ctx = torch.matmul(attn, v).transpose(1, 2).contiguous().view(B, T, D)
    reg[o[0]].copy_(F.linear(ctx, wo, bo))


def _cross_mha(reg, i, o, ints, floats):
    """Attention with queries from x and keys/values from `memory`: the arithmetic of the reference's eager
    MultiHeadAttention.forward(q, k, v, mask) (py/fxfusion/models/transformer/layers/attention.py:19-33) called as the decoder
    block calls it (blocks/decoder_block.py:22), with Wk and Wv packed into one weight."""
    x, mem, mask, wq, bq, wkv, bkv, wo, bo = (reg[k] for k in i[:9])
    H, hd, D, KV = ints[:4]
    scale = float(np.float32(floats[0]))
    B, Tq, Tk = x.size(0), x.size(1), mem.size(1)
    q = F.linear(x, wq, bq).view(B, Tq, H, hd).transpose(1, 2)
    kv = F.linear(mem, wkv, bkv)
    k = kv[:, :, 0:D].view(B, Tk, H, hd).transpose(1, 2)
    v = kv[:, :, D:KV].view(B, Tk, H, hd).transpose(1, 2)
    scores = torch.matmul(q, k.transpose(-2, -1)) / scale
    scores = scores.masked_fill(mask == 0, -math.inf)
    attn = torch.softmax(scores, -1)
    ctx = torch.matmul(attn, v).transpose(1, 2).contiguous().view(B, Tq, D)
    reg[o[0]].copy_(F.linear(ctx, wo, bo))


_KV_STATE: Dict[tuple, torch.Tensor] = {}


def _cached_mha(reg, i, o, ints, floats):
    """One new position against cached keys / values: MHA (csrc/kernels/cpu/mha.cpp:5-52) restricted to query row `pos`
    under the static decoder mask (layers/masks.py:141-154: key j <= pos and tokens[b, j] != pad).  The cache is kept per
    (registry, output tensor), i.e. per node of one GraphOracle."""
    x, tokens, pos, wqkv, bqkv, wo, bo = (reg[k] for k in i[:7])
    H, hd, D, QKV, pad = ints[:5]
    scale = float(np.float32(floats[0]))
    B, T, p = x.size(0), tokens.size(1), int(pos.item())
    cache = _KV_STATE.setdefault((id(reg), o[0]), torch.zeros(B, T, 2 * D))
    qkv = F.linear(x, wqkv, bqkv)                      # [B,1,3D]
    cache[:, p, :] = qkv[:, 0, D:]
    q = qkv[:, :, 0:D].view(B, 1, H, hd).transpose(1, 2)                    # [B,H,1,hd]
    k = cache[:, :p + 1, 0:D].reshape(B, p + 1, H, hd).transpose(1, 2)       # [B,H,p+1,hd]
    v = cache[:, :p + 1, D:].reshape(B, p + 1, H, hd).transpose(1, 2)
    scores = torch.matmul(q, k.transpose(-2, -1)) / scale
    keep = (tokens[:, :p + 1] != pad).view(B, 1, 1, p + 1)
    scores = scores.masked_fill(keep == 0, -math.inf)
    ctx = torch.matmul(torch.softmax(scores, -1), v).transpose(1, 2).contiguous().view(B, 1, D)
    reg[o[0]].copy_(F.linear(ctx, wo, bo))


KERNELS: Dict[int, KernelFn] = {
    wire.OP["Conv2d"]: lambda r, i, o, a, f: _conv(r, i, o, a, f, False),
    wire.OP["Conv2dRelu"]: lambda r, i, o, a, f: _conv(r, i, o, a, f, True),
    wire.OP["Linear"]: lambda r, i, o, a, f: r[o[0]].copy_(F.linear(r[i[0]], r[i[1]], r[i[2]])),
    wire.OP["LinearRelu"]: lambda r, i, o, a, f: r[o[0]].copy_(torch.relu(F.linear(r[i[0]], r[i[1]], r[i[2]]))),
    wire.OP["Add"]: lambda r, i, o, a, f: r[o[0]].copy_(torch.add(r[i[0]], r[i[1]])),
    wire.OP["AddRelu"]: lambda r, i, o, a, f: r[o[0]].copy_(torch.relu(torch.add(r[i[0]], r[i[1]]))),
    wire.OP["Relu"]: lambda r, i, o, a, f: r[o[0]].copy_(torch.relu(r[i[0]])),
    wire.OP["Mul"]: _mul,
    wire.OP["MaxPool2d"]: lambda r, i, o, a, f: r[o[0]].copy_(
        torch.max_pool2d(r[i[0]], [a[0], a[1]], [a[2], a[3]], [a[4], a[5]], [a[6], a[7]], bool(a[8]))),
    wire.OP["AvgPool2d"]: lambda r, i, o, a, f: r[o[0]].copy_(
        F.avg_pool2d(r[i[0]], [a[0], a[1]], [a[2], a[3]], [a[4], a[5]], bool(a[6]))),
    wire.OP["AdaptiveAvgPool2d"]: lambda r, i, o, a, f: r[o[0]].copy_(F.adaptive_avg_pool2d(r[i[0]], [a[0], a[1]])),
    wire.OP["Transpose"]: lambda r, i, o, a, f: r[o[0]].copy_(torch.transpose(r[i[0]], a[0], a[1])),
    wire.OP["Size"]: lambda r, i, o, a, f: r[o[0]].fill_(r[i[0]].size(a[0])),
    wire.OP["Narrow"]: _narrow,
    wire.OP["Embedding"]: lambda r, i, o, a, f: r[o[0]].copy_(torch.embedding(r[i[1]], r[i[0]])),
    wire.OP["LayerNorm"]: _layer_norm,
    wire.OP["AddLayerNorm"]: _add_layer_norm,
    wire.OP["MHA"]: _mha,
    wire.OP["CrossMHA"]: _cross_mha,
    wire.OP["CachedMHA"]: _cached_mha,
    wire.OP["FeedForward"]: lambda r, i, o, a, f: r[o[0]].copy_(
        F.linear(torch.relu(F.linear(r[i[0]], r[i[1]], r[i[2]])), r[i[3]], r[i[4]])),
}


class GraphOracle:
    """Executes a graph file on the CPU, one node after another, like the reference runtime."""

    def __init__(self, graph, kernels: Optional[Dict[int, KernelFn]] = None) -> None:
        g = wire.load(graph) if isinstance(graph, (str, bytes)) or hasattr(graph, "__fspath__") else graph
        self.graph = g
        self.kernels = kernels or KERNELS
        n = len(g.tensors)
        self.reg: List[Optional[torch.Tensor]] = [None] * n
        self.input_ids: List[int] = []
        self.output_ids: List[int] = []
        for t in g.tensors:
            dt = TORCH_DTYPES[t.dtype]
            shape = list(t.shape)
            if t.kind == wire.KIND_CONSTANT:
                if t.data is None:
                    raise RuntimeError("Constant tensor missing data")
                arr = t.array()
                self.reg[t.id] = torch.from_numpy(np.array(arr, copy=True))
            elif t.kind == wire.KIND_ACTIVATION:
                if t.offset < 0:
                    raise RuntimeError("Arena-backed tensor has invalid offset")
                self.reg[t.id] = torch.zeros(shape, dtype=dt)
            elif t.kind in (wire.KIND_ALIAS, wire.KIND_OUTPUT):
                src = t.alias_of
                if src < 0 or src >= n or self.reg[src] is None:
                    if t.offset >= 0:
                        self.reg[t.id] = torch.zeros(shape, dtype=dt)
                    else:
                        raise RuntimeError("Invalid alias source ID")
                else:
                    if self.reg[src].numel() != int(np.prod(shape, dtype=np.int64)):
                        raise RuntimeError(f"Alias numel mismatch for tensor id {t.id}")
                    self.reg[t.id] = self.reg[src].view(shape)
                if t.kind == wire.KIND_OUTPUT:
                    self.output_ids.append(t.id)
            elif t.kind == wire.KIND_INPUT:
                self.input_ids.append(t.id)
                self.reg[t.id] = torch.zeros(shape, dtype=dt)
            else:
                raise RuntimeError("Unsupported TensorKind in FlatBuffer")
        self.nodes = [nd for nd in g.nodes if nd.op_code != 0]
        for nd in self.nodes:
            if nd.op_code not in self.kernels:
                raise RuntimeError(f"Unregistered OpCode: {nd.op_code}")

    @torch.no_grad()
    def run(self, inputs: Sequence[torch.Tensor]) -> List[torch.Tensor]:
        if len(inputs) != len(self.input_ids):
            raise RuntimeError("Input count mismatch")
        for tid, x in zip(self.input_ids, inputs):
            # inputs are bound by reference in the reference runtime; aliases of inputs were bound at
            # build time to a placeholder there, here they follow the data
            self.reg[tid].copy_(x.reshape(self.reg[tid].shape))
        for nd in self.nodes:
            self.kernels[nd.op_code](self.reg, nd.input_ids, nd.output_ids, list(nd.int_params), list(nd.float_params))
        return [self.reg[i] for i in self.output_ids]


# --------------------------------------------------------------------------------------
# decode loop (reference py/fxfusion/models/transformer/inference.py:28-45, layers/masks.py:70-154)
# --------------------------------------------------------------------------------------
def make_static_buffer(tokens: torch.Tensor, max_seq_len: int, pad_idx: int = 0) -> torch.Tensor:
    B, T = tokens.shape
    if T > max_seq_len:
        raise ValueError(f"Token length {T} exceeds max_seq_len {max_seq_len}")
    buf = torch.full((B, max_seq_len), pad_idx, dtype=tokens.dtype)
    buf[:, :T] = tokens
    return buf


def static_decoder_mask(tokens: torch.Tensor, current_len: int, pad_idx: int = 0) -> torch.Tensor:
    B, T = tokens.shape
    prefix = (torch.arange(T) < current_len).view(1, 1, 1, T).expand(B, 1, 1, T)
    padding = (tokens != pad_idx).unsqueeze(1).unsqueeze(2)
    causal = torch.tril(torch.ones((T, T), dtype=torch.bool))
    return prefix & padding & causal


def decode_static(run: Callable[[torch.Tensor, torch.Tensor], torch.Tensor], tokens: torch.Tensor, max_seq_len: int,
                  steps: Optional[int] = None, margins: Optional[list] = None) -> torch.Tensor:
    """Greedy full-recompute decode.  `run(buffer, mask)` returns logits [B,T,V].  If `margins` is a
    list it receives, per step, the top-1 minus top-2 logit gap of every sequence."""
    B, initial_len = tokens.shape
    buf = make_static_buffer(tokens, max_seq_len)
    cur = initial_len
    total = max_seq_len - initial_len if steps is None else min(steps, max_seq_len - initial_len)
    for _ in range(total):
        mask = static_decoder_mask(buf, cur)
        logits = run(buf, mask)
        row = logits[:, cur - 1, :]
        if margins is not None:
            top2 = torch.topk(row, 2, dim=-1).values
            margins.append((top2[:, 0] - top2[:, 1]).clone())
        buf[:, cur] = row.argmax(dim=-1)
        cur += 1
    return buf[:, :cur]


def decode_cached(run_step: Callable[[torch.Tensor, torch.Tensor, torch.Tensor], torch.Tensor], tokens: torch.Tensor, max_seq_len: int) -> torch.Tensor:
    """Greedy incremental decode with a single-position step graph: `run_step(ids [B,1], pos [1], buffer [B,T])` returns
    logits [B,1,V] for the tokens at `pos` (the step keeps keys / values of earlier positions itself).  Positions are fed
    in order from 0; prompt positions only fill the caches."""
    B, initial_len = tokens.shape
    buf = make_static_buffer(tokens, max_seq_len)
    for p in range(max_seq_len - 1):
        logits = run_step(buf[:, p:p + 1].contiguous(), torch.tensor([p], dtype=torch.int64), buf)
        if p + 1 >= initial_len:
            buf[:, p + 1] = logits[:, 0, :].argmax(dim=-1)
    return buf
