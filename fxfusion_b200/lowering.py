"""Lowered-graph builders: emit the graph file for a model family directly.

The reference obtains a graph file by tracing an nn.Module through its FX passes (fusion,
shape propagation, memory planning, serializer).  The file format is the contract the runtime
consumes; this module writes the same lowered graphs without PyTorch-FX, so a machine that has
only this package can create workloads:

  * `GraphBuilder` mirrors what the reference records per fx node: one tensor per node in graph
    order with `id == index` (reference passes/memory_plan.py:204, serializer.py:37), kinds
    input / const / activation / alias / output (memory_plan.py:87-102), NoOp nodes for
    placeholders, constants, eval-mode Dropout and `output` (serializer.py:116-133).
  * `GraphBuilder.finish` (with `_Arena`) is the reference's static planner restated: liveness by last use, first-fit
    free list with coalescing and top-of-arena shrink, sizes rounded up to the alignment, a
    buffer released right after its last user has been allocated
    (passes/memory_plan.py:147-213, passes/memory_manager.py:34-91).
  * `mlp_graph` and `gpt_graph` reproduce the node sequences the reference passes generate for
    nn.Sequential(Linear, ReLU, ...) and for its GPT model
    (py/fxfusion/models/transformer/models/gpt.py:8-28, blocks/gpt_block.py:7-19): the BOSS fusion
    turns the trailing LinearRelu + Linear into one FeedForward, every GPT block is pre-LN, and
    only the last residual add fuses with the final LayerNorm.

Tests compare these builders against the reference passes node by node where the reference is
importable.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from . import wire
from .wire import GraphRec, NodeRec, OP, TensorRec


# --------------------------------------------------------------------------------------
# planner
# --------------------------------------------------------------------------------------
class _Arena:
    """First-fit free-list allocator (reference passes/memory_manager.py:34-91)."""

    def __init__(self, alignment: int = 64) -> None:
        if alignment <= 0 or alignment & (alignment - 1):
            raise ValueError("alignment must be a positive power of two")
        self.alignment = alignment
        self.free: List[Tuple[int, int]] = []
        self.top = 0
        self.peak = 0

    def align(self, v: int) -> int:
        return (v + self.alignment - 1) // self.alignment * self.alignment

    def allocate(self, size: int) -> int:
        for idx, (off, blk) in enumerate(self.free):
            start = self.align(off)
            if start + size <= off + blk:
                self.free.pop(idx)
                front = start - off
                if front > 0:
                    self.free.append((off, front))
                back = (blk - size) - front
                if back > 0:
                    self.free.append((start + size, back))
                return start
        start = self.align(self.top)
        self.top = start + size
        self.peak = max(self.peak, self.top)
        return start

    def release(self, off: int, size: int) -> None:
        if size <= 0:
            return
        self.free.append((off, size))
        self.free.sort()
        merged: List[Tuple[int, int]] = []
        for o, s in self.free:
            if merged and merged[-1][0] + merged[-1][1] == o:
                merged[-1] = (merged[-1][0], merged[-1][1] + s)
            else:
                merged.append((o, s))
        self.free = merged
        if self.free and self.free[-1][0] + self.free[-1][1] == self.top:
            o, _ = self.free.pop()
            self.top = o


@dataclass
class _Value:
    """One fx-node-equivalent: becomes exactly one Tensor record."""
    kind: str                      # input | const | activation | alias | output
    shape: Tuple[int, ...]
    dtype: int
    inputs: List[int] = field(default_factory=list)   # ids this value reads (for liveness)
    op: int = 0                    # opcode of the node that produces it (0 = NoOp)
    ints: List[int] = field(default_factory=list)
    floats: List[float] = field(default_factory=list)
    data: Optional[np.ndarray] = None
    src: int = -1                  # alias / output source


class GraphBuilder:
    def __init__(self, name: str = "model", alignment: int = 64) -> None:
        self.name = name
        self.alignment = alignment
        self.values: List[_Value] = []

    # -- value constructors (each returns the tensor id) -----------------------------------
    def _add(self, v: _Value) -> int:
        self.values.append(v)
        return len(self.values) - 1

    def input(self, shape: Sequence[int], dtype: int) -> int:
        return self._add(_Value("input", tuple(shape), dtype))

    def const(self, array: np.ndarray) -> int:
        arr = np.ascontiguousarray(array)
        dt = {np.dtype(np.float32): wire.DT_F32, np.dtype(np.float16): wire.DT_F16, np.dtype(np.int32): wire.DT_I32,
              np.dtype(np.int64): wire.DT_I64, np.dtype(np.bool_): wire.DT_BOOL}[arr.dtype]
        return self._add(_Value("const", tuple(arr.shape), dt, data=arr))

    def op(self, opcode: str, inputs: Sequence[int], shape: Sequence[int], dtype: int = wire.DT_F32,
           ints: Sequence[int] = (), floats: Sequence[float] = ()) -> int:
        return self._add(_Value("activation", tuple(shape), dtype, list(inputs), OP[opcode], list(ints), list(floats)))

    def alias(self, src: int, shape: Optional[Sequence[int]] = None) -> int:
        """View-like node (eval Dropout, view/reshape/flatten): shares the source's storage."""
        s = self.values[src]
        return self._add(_Value("alias", tuple(shape) if shape is not None else s.shape, s.dtype, [src], src=src))

    def output(self, src: int) -> int:
        s = self.values[src]
        return self._add(_Value("output", s.shape, s.dtype, [src], src=src))

    # -- planning + serialisation ------------------------------------------------------------
    def finish(self) -> GraphRec:
        arena = _Arena(self.alignment)
        n = len(self.values)
        last_use: Dict[int, int] = {}
        for i, v in enumerate(self.values):
            for j in v.inputs:
                last_use[j] = i
        offsets: List[Optional[int]] = [None] * n
        sizes = [arena.align(int(np.prod(v.shape, dtype=np.int64)) * wire.DTYPE_ITEMSIZE[v.dtype]) for v in self.values]
        for i, v in enumerate(self.values):
            if v.kind == "activation":
                offsets[i] = arena.allocate(sizes[i])
            elif v.kind in ("alias", "output"):
                offsets[i] = offsets[v.src]
            if v.kind not in ("alias", "output"):
                released = set()
                for j in dict.fromkeys(v.inputs):
                    if last_use.get(j) != i or self.values[j].kind not in ("activation", "alias") or offsets[j] is None:
                        continue
                    key = (offsets[j], sizes[j])
                    if key in released:
                        continue
                    arena.release(*key)
                    released.add(key)
        g = GraphRec(name=self.name, arena_size=arena.peak)
        kind_code = {"input": wire.KIND_INPUT, "const": wire.KIND_CONSTANT, "activation": wire.KIND_ACTIVATION,
                     "alias": wire.KIND_ALIAS, "output": wire.KIND_OUTPUT}
        for i, v in enumerate(self.values):
            g.tensors.append(TensorRec(id=i, kind=kind_code[v.kind], offset=-1 if offsets[i] is None else offsets[i],
                                       size_bytes=sizes[i], shape=v.shape, dtype=v.dtype,
                                       alias_of=v.src if v.kind in ("alias", "output") else -1, data=v.data))
            g.nodes.append(NodeRec(op_code=v.op, input_ids=list(v.inputs), output_ids=[i],
                                   int_params=list(v.ints), float_params=list(v.floats)))
        return g


# --------------------------------------------------------------------------------------
# parameters (seeded numpy generators; torch's CPU math only for the positional-encoding table)
# --------------------------------------------------------------------------------------
def _normal(rng: np.random.Generator, shape, std: float) -> np.ndarray:
    return (rng.standard_normal(size=shape, dtype=np.float32) * np.float32(std)).astype(np.float32)


def _uniform(rng: np.random.Generator, shape, bound: float) -> np.ndarray:
    return rng.uniform(-bound, bound, size=shape).astype(np.float32)


def mlp_params(depth: int = 16, width: int = 512, n_out: int = 10, seed: int = 0) -> List[Tuple[np.ndarray, np.ndarray]]:
    """nn.Linear default init: Kaiming-uniform(a=sqrt 5) weights = U(+-1/sqrt(fan_in)), same for bias."""
    rng = np.random.default_rng(seed)
    layers = []
    for i in range(depth):
        out = n_out if i == depth - 1 else width
        bound = 1.0 / math.sqrt(width)
        layers.append((_uniform(rng, (out, width), bound), _uniform(rng, (out,), bound)))
    return layers


def mlp_graph(layers: List[Tuple[np.ndarray, np.ndarray]], batch: int, name: str = "mlp", alignment: int = 64) -> GraphRec:
    """Sequential(Linear, ReLU, ..., Linear): all but the last two layers become LinearRelu; the
    last LinearRelu + Linear pair becomes one FeedForward (reference passes/fusion/ops.py:197-203)."""
    assert len(layers) >= 2
    b = GraphBuilder(name, alignment)
    width = layers[0][0].shape[1]
    x = b.input((batch, width), wire.DT_F32)
    cur = x
    for w, bias in layers[:-2]:
        wi, bi = b.const(w), b.const(bias)
        cur = b.op("LinearRelu", [cur, wi, bi], (batch, w.shape[0]))
    (w1, b1), (w2, b2) = layers[-2], layers[-1]
    ids = [b.const(w1), b.const(b1), b.const(w2), b.const(b2)]
    cur = b.op("FeedForward", [cur] + ids, (batch, w2.shape[0]))
    b.output(cur)
    return b.finish()


@dataclass
class GPTConfig:
    d_model: int
    heads: int
    vocab: int
    expansion: int
    layers: int
    pe_len: int = 5000   # the reference's PositionalEncoding default (layers/embedding.py:18)

    @property
    def d_ff(self) -> int:
        return self.d_model * self.expansion


GPT_C2 = GPTConfig(256, 4, 1000, 4, 4)          # 4 layers, d_model 256, 4 heads, d_ff 1024
GPT2_SMALL = GPTConfig(768, 12, 50257, 4, 12)   # 12 layers, d_model 768, 12 heads, d_ff 3072


def sinusoidal_pe(pe_len: int, d_model: int) -> np.ndarray:
    """pe[0, pos, 2i] = sin(pos * w_i), pe[0, pos, 2i+1] = cos(pos * w_i), w_i = exp(-2i ln(1e4)/d),
    evaluated in float32 with torch's CPU math, the way the reference builds its buffer
    (layers/embedding.py:21-28), so the constant is bit-identical to the reference model's."""
    import torch
    pe = torch.zeros(pe_len, d_model)
    position = torch.arange(0, pe_len, dtype=torch.float).unsqueeze(1)
    div_term = torch.exp(torch.arange(0, d_model, 2).float() * (-math.log(10000.0) / d_model))
    pe[:, 0::2] = torch.sin(position * div_term)
    pe[:, 1::2] = torch.cos(position * div_term)
    return pe.unsqueeze(0).numpy()


def gpt_params(cfg: GPTConfig, seed: int = 0, std: float = 0.02) -> Dict[str, np.ndarray]:
    """Weights ~ N(0, std), biases 0, LayerNorm gamma 1 / beta 0; the Q/K/V projections are already
    packed as cat([Wq, Wk, Wv], 0) (reference passes/fusion/matchers.py:641-657)."""
    rng = np.random.default_rng(seed)
    D, F, V = cfg.d_model, cfg.d_ff, cfg.vocab
    p: Dict[str, np.ndarray] = {"emb": _normal(rng, (V, D), std), "pe": sinusoidal_pe(cfg.pe_len, D)}
    for l in range(cfg.layers):
        p[f"l{l}.ln1.w"] = np.ones(D, np.float32)
        p[f"l{l}.ln1.b"] = np.zeros(D, np.float32)
        p[f"l{l}.qkv.w"] = _normal(rng, (3 * D, D), std)
        p[f"l{l}.qkv.b"] = np.zeros(3 * D, np.float32)
        p[f"l{l}.wo.w"] = _normal(rng, (D, D), std)
        p[f"l{l}.wo.b"] = np.zeros(D, np.float32)
        p[f"l{l}.ln2.w"] = np.ones(D, np.float32)
        p[f"l{l}.ln2.b"] = np.zeros(D, np.float32)
        p[f"l{l}.ff1.w"] = _normal(rng, (F, D), std)
        p[f"l{l}.ff1.b"] = np.zeros(F, np.float32)
        p[f"l{l}.ff2.w"] = _normal(rng, (D, F), std)
        p[f"l{l}.ff2.b"] = np.zeros(D, np.float32)
    p["ln_f.w"] = np.ones(D, np.float32)
    p["ln_f.b"] = np.zeros(D, np.float32)
    p["head.w"] = _normal(rng, (V, D), std)
    p["head.b"] = np.zeros(V, np.float32)
    return p


def gpt_graph(cfg: GPTConfig, params: Dict[str, np.ndarray], batch: int, seq: int, name: str = "gpt",
              alignment: int = 64, eps: float = 1e-5) -> GraphRec:
    """Embedding, Mul(sqrt D), Size, Narrow(pe), Add, [LayerNorm, MHA, Add, LayerNorm, FeedForward,
    Add] x L with the last Add fused into AddLayerNorm, Linear head.  Inputs: token ids int64
    [B,T] and a bool mask [B,1,T,T]."""
    B, T, D, H = batch, seq, cfg.d_model, cfg.heads
    hd = D // H
    b = GraphBuilder(name, alignment)
    x = b.input((B, T), wire.DT_I64)
    mask = b.input((B, 1, T, T), wire.DT_BOOL)
    emb_w = b.const(params["emb"])
    emb = b.op("Embedding", [x, emb_w], (B, T, D))
    mul = b.op("Mul", [emb], (B, T, D), ints=[1], floats=[math.sqrt(D)])
    size = b.op("Size", [mul], (), wire.DT_I64, ints=[1])
    pe = b.const(params["pe"])
    nar = b.op("Narrow", [pe, size], (1, T, D), ints=[1, 0, -1])
    add = b.op("Add", [mul, nar], (B, T, D))
    h = b.alias(add)  # positional-encoding dropout (eval mode)
    ln_ints = [1, D]
    for l in range(cfg.layers):
        w1, b1 = b.const(params[f"l{l}.ln1.w"]), b.const(params[f"l{l}.ln1.b"])
        ln1 = b.op("LayerNorm", [h, w1, b1], (B, T, D), ints=ln_ints, floats=[eps])
        consts = [b.const(params[f"l{l}.qkv.w"]), b.const(params[f"l{l}.qkv.b"]), b.const(params[f"l{l}.wo.w"]), b.const(params[f"l{l}.wo.b"])]
        mha = b.op("MHA", [ln1, mask] + consts, (B, T, D), ints=[H, hd, D, 3 * D], floats=[math.sqrt(hd)])
        d1 = b.alias(mha)
        a1 = b.op("Add", [h, d1], (B, T, D))
        w2, b2 = b.const(params[f"l{l}.ln2.w"]), b.const(params[f"l{l}.ln2.b"])
        ln2 = b.op("LayerNorm", [a1, w2, b2], (B, T, D), ints=ln_ints, floats=[eps])
        consts = [b.const(params[f"l{l}.ff1.w"]), b.const(params[f"l{l}.ff1.b"]), b.const(params[f"l{l}.ff2.w"]), b.const(params[f"l{l}.ff2.b"])]
        ff = b.op("FeedForward", [ln2] + consts, (B, T, D))
        d2 = b.alias(ff)
        if l < cfg.layers - 1:
            h = b.op("Add", [a1, d2], (B, T, D))
        else:
            wf, bf = b.const(params["ln_f.w"]), b.const(params["ln_f.b"])
            h = b.op("AddLayerNorm", [a1, d2, wf, bf], (B, T, D), ints=ln_ints, floats=[eps])
    hw, hb = b.const(params["head.w"]), b.const(params["head.b"])
    logits = b.op("Linear", [h, hw, hb], (B, T, cfg.vocab))
    b.output(logits)
    return b.finish()


def gpt_step_graph(cfg: GPTConfig, params: Dict[str, np.ndarray], batch: int, max_len: int, name: str = "gpt_step",
                   alignment: int = 64, eps: float = 1e-5, pad_idx: int = 0) -> GraphRec:
    """One decode position of the GPT of `gpt_graph`, for incremental ("KV cache") decoding — the reference's stated
    future work (README.md:183); no reference lowering exists.  Same weights and the same per-position arithmetic as
    `gpt_graph`; the attention nodes are CachedMHA (extension opcode 21), the positional row is an Embedding gather of
    the sinusoidal table at `pos`.  Inputs: ids int64 [B,1] (the tokens at `pos`), pos int64 [1], tokens int64
    [B,max_len] (whole buffer: the pad mask of the cached keys is read from it).  Output: logits [B,1,vocab]."""
    B, T, D, H = batch, max_len, cfg.d_model, cfg.heads
    hd = D // H
    b = GraphBuilder(name, alignment)
    ids = b.input((B, 1), wire.DT_I64)
    pos = b.input((1,), wire.DT_I64)
    tokens = b.input((B, T), wire.DT_I64)
    emb = b.op("Embedding", [ids, b.const(params["emb"])], (B, 1, D))
    mul = b.op("Mul", [emb], (B, 1, D), ints=[1], floats=[math.sqrt(D)])
    pe = b.const(np.ascontiguousarray(params["pe"].reshape(-1, D)[:max(T, 1)]))   # rows 0..T-1 of the [1,P,D] table
    pe_row = b.op("Embedding", [pos, pe], (1, 1, D))
    h = b.op("Add", [mul, pe_row], (B, 1, D))
    ln_ints = [1, D]
    for l in range(cfg.layers):
        ln1 = b.op("LayerNorm", [h, b.const(params[f"l{l}.ln1.w"]), b.const(params[f"l{l}.ln1.b"])], (B, 1, D), ints=ln_ints, floats=[eps])
        consts = [b.const(params[f"l{l}.qkv.w"]), b.const(params[f"l{l}.qkv.b"]), b.const(params[f"l{l}.wo.w"]), b.const(params[f"l{l}.wo.b"])]
        att = b.op("CachedMHA", [ln1, tokens, pos] + consts, (B, 1, D), ints=[H, hd, D, 3 * D, pad_idx], floats=[math.sqrt(hd)])
        a1 = b.op("Add", [h, att], (B, 1, D))
        ln2 = b.op("LayerNorm", [a1, b.const(params[f"l{l}.ln2.w"]), b.const(params[f"l{l}.ln2.b"])], (B, 1, D), ints=ln_ints, floats=[eps])
        consts = [b.const(params[f"l{l}.ff1.w"]), b.const(params[f"l{l}.ff1.b"]), b.const(params[f"l{l}.ff2.w"]), b.const(params[f"l{l}.ff2.b"])]
        ff = b.op("FeedForward", [ln2] + consts, (B, 1, D))
        if l < cfg.layers - 1:
            h = b.op("Add", [a1, ff], (B, 1, D))
        else:
            h = b.op("AddLayerNorm", [a1, ff, b.const(params["ln_f.w"]), b.const(params["ln_f.b"])], (B, 1, D), ints=ln_ints, floats=[eps])
    logits = b.op("Linear", [h, b.const(params["head.w"]), b.const(params["head.b"])], (B, 1, cfg.vocab))
    b.output(logits)
    return b.finish()


# --------------------------------------------------------------------------------------
# Encoder-decoder Transformer (reference model: models/transformer.py:7-18, models/encoder.py, models/decoder.py,
# blocks/encoder_block.py, blocks/decoder_block.py).  The reference's compile passes cannot lower it: the decoder's
# second attention takes its queries from one tensor and its keys/values from another, the QKV packing wants three
# Linear siblings on one input (passes/fusion/matchers.py:615-621) and the unfused matmul / softmax nodes are not
# serializable (serializer.py:157,169).  This builder lowers everything the way the reference lowers a GPT stack and
# expresses that attention with the CrossMHA opcode (an extension of this library: Wq alone, Wk and Wv packed).
# --------------------------------------------------------------------------------------
@dataclass(frozen=True)
class TransformerConfig:
    d_model: int
    heads: int
    vocab: int
    expansion: int
    enc_layers: int
    dec_layers: int
    pe_len: int = 5000

    @property
    def d_ff(self) -> int:
        return self.d_model * self.expansion


TRANSFORMER_C4 = TransformerConfig(512, 8, 32000, 4, 6, 6)   # 6 + 6 layers, d_model 512, 8 heads, d_ff 2048


def transformer_params(cfg: TransformerConfig, seed: int = 0, std: float = 0.02) -> Dict[str, np.ndarray]:
    """Weights ~ N(0, std), biases 0, LayerNorm gamma 1 / beta 0.  Self-attention projections are packed as
    cat([Wq, Wk, Wv], 0); the decoder's cross-attention keeps Wq apart and packs cat([Wk, Wv], 0)."""
    rng = np.random.default_rng(seed)
    D, F, V = cfg.d_model, cfg.d_ff, cfg.vocab
    p: Dict[str, np.ndarray] = {}
    pe = sinusoidal_pe(cfg.pe_len, D)

    def ln(key):
        p[key + ".w"], p[key + ".b"] = np.ones(D, np.float32), np.zeros(D, np.float32)

    def lin(key, n_out, n_in):
        p[key + ".w"], p[key + ".b"] = _normal(rng, (n_out, n_in), std), np.zeros(n_out, np.float32)

    for side, layers in (("enc", cfg.enc_layers), ("dec", cfg.dec_layers)):
        p[f"{side}.emb"] = _normal(rng, (V, D), std)
        p[f"{side}.pe"] = pe
        for l in range(layers):
            pre = f"{side}.l{l}."
            ln(pre + "ln1"); lin(pre + "qkv", 3 * D, D); lin(pre + "wo", D, D)
            if side == "dec":
                ln(pre + "ln2"); lin(pre + "cq", D, D); lin(pre + "ckv", 2 * D, D); lin(pre + "co", D, D)
            ln(pre + "lnf"); lin(pre + "ff1", F, D); lin(pre + "ff2", D, F)
        ln(f"{side}.ln_out")
    lin("head", V, D)
    return p


def transformer_graph(cfg: TransformerConfig, params: Dict[str, np.ndarray], batch: int, src_len: int, tgt_len: int,
                      name: str = "transformer", alignment: int = 64, eps: float = 1e-5) -> GraphRec:
    """Inputs in the order of Transformer.forward: src ids int64 [B,S], tgt ids int64 [B,T], src mask bool [B,1,1,S],
    tgt mask bool [B,1,T,T]; output logits [B,T,vocab]."""
    B, S, T, D, H = batch, src_len, tgt_len, cfg.d_model, cfg.heads
    hd = D // H
    b = GraphBuilder(name, alignment)
    src = b.input((B, S), wire.DT_I64)
    tgt = b.input((B, T), wire.DT_I64)
    src_mask = b.input((B, 1, 1, S), wire.DT_BOOL)
    tgt_mask = b.input((B, 1, T, T), wire.DT_BOOL)
    ln_ints = [1, D]

    def c(key):
        return b.const(params[key])

    def embed(ids, side, L):
        emb = b.op("Embedding", [ids, c(f"{side}.emb")], (B, L, D))
        mul = b.op("Mul", [emb], (B, L, D), ints=[1], floats=[math.sqrt(D)])
        size = b.op("Size", [mul], (), wire.DT_I64, ints=[1])
        nar = b.op("Narrow", [c(f"{side}.pe"), size], (1, L, D), ints=[1, 0, -1])
        return b.alias(b.op("Add", [mul, nar], (B, L, D)))  # positional-encoding dropout (eval mode)

    def stack(h, side, layers, L, self_mask, memory=None):
        for l in range(layers):
            pre = f"{side}.l{l}."
            n1 = b.op("LayerNorm", [h, c(pre + "ln1.w"), c(pre + "ln1.b")], (B, L, D), ints=ln_ints, floats=[eps])
            att = b.op("MHA", [n1, self_mask, c(pre + "qkv.w"), c(pre + "qkv.b"), c(pre + "wo.w"), c(pre + "wo.b")], (B, L, D),
                       ints=[H, hd, D, 3 * D], floats=[math.sqrt(hd)])
            h = b.op("Add", [h, b.alias(att)], (B, L, D))
            if memory is not None:
                n2 = b.op("LayerNorm", [h, c(pre + "ln2.w"), c(pre + "ln2.b")], (B, L, D), ints=ln_ints, floats=[eps])
                cross = b.op("CrossMHA", [n2, memory, src_mask, c(pre + "cq.w"), c(pre + "cq.b"), c(pre + "ckv.w"), c(pre + "ckv.b"),
                                          c(pre + "co.w"), c(pre + "co.b")], (B, L, D), ints=[H, hd, D, 2 * D], floats=[math.sqrt(hd)])
                h = b.op("Add", [h, b.alias(cross)], (B, L, D))
            nf = b.op("LayerNorm", [h, c(pre + "lnf.w"), c(pre + "lnf.b")], (B, L, D), ints=ln_ints, floats=[eps])
            ff = b.op("FeedForward", [nf, c(pre + "ff1.w"), c(pre + "ff1.b"), c(pre + "ff2.w"), c(pre + "ff2.b")], (B, L, D))
            if l < layers - 1:
                h = b.op("Add", [h, b.alias(ff)], (B, L, D))
            else:  # the last residual add fuses with the stack's output LayerNorm
                h = b.op("AddLayerNorm", [h, b.alias(ff), c(f"{side}.ln_out.w"), c(f"{side}.ln_out.b")], (B, L, D), ints=ln_ints, floats=[eps])
        return h

    memory = stack(embed(src, "enc", S), "enc", cfg.enc_layers, S, src_mask)
    dec = stack(embed(tgt, "dec", T), "dec", cfg.dec_layers, T, tgt_mask, memory)
    logits = b.op("Linear", [dec, c("head.w"), c("head.b")], (B, T, cfg.vocab))
    b.output(logits)
    return b.finish()


def decode_prompt(batch: int, prompt_len: int, vocab: int, seed: int = 0) -> np.ndarray:
    """Prompt ids uniform in [1, vocab): id 0 is the pad id that the decode mask blocks
    (reference py/tests/test_ops.py:423, layers/masks.py:52-55)."""
    rng = np.random.default_rng(seed + 1)
    return rng.integers(1, vocab, size=(batch, prompt_len), dtype=np.int64)


# --------------------------------------------------------------------------------------
# ResNet-50 (Conv+BN folded, NCHW) — reference lowering: 33 Conv2dRelu, 20 Conv2d, 16 AddRelu, MaxPool2d,
# AdaptiveAvgPool2d, flatten (alias), Linear.  BatchNorm is folded into the convolution the way the
# reference fusion pass does it (passes/fusion/matchers.py:125-174): w' = w * g / sqrt(var + eps) per output
# channel, b' = beta - mean * g / sqrt(var + eps).
# --------------------------------------------------------------------------------------
_GRID_BLOCK = [1, 1, 1, 256, 1, 1]  # unused launch placeholders the reference serializer appends (serializer.py:188-203)
RESNET50_LAYERS = ((64, 3, 1), (128, 4, 2), (256, 6, 2), (512, 3, 2))  # (width, blocks, stride of the first block)


def _folded_conv(rng: np.random.Generator, c_out: int, c_in: int, k: int, eps: float = 1e-5) -> Tuple[np.ndarray, np.ndarray]:
    w = _normal(rng, (c_out, c_in, k, k), math.sqrt(2.0 / (c_out * k * k)))          # Kaiming normal, fan_out
    gamma, beta = 1.0 + _normal(rng, (c_out,), 0.1), _normal(rng, (c_out,), 0.1)
    mean, var = _normal(rng, (c_out,), 0.1), rng.uniform(0.5, 1.5, size=(c_out,)).astype(np.float32)
    scale = (gamma / np.sqrt(var + np.float32(eps))).astype(np.float32)
    return (w * scale[:, None, None, None]).astype(np.float32), (beta - mean * scale).astype(np.float32)


def resnet50_params(seed: int = 0, num_classes: int = 1000) -> Dict[str, np.ndarray]:
    rng = np.random.default_rng(seed)
    p: Dict[str, np.ndarray] = {}
    p["stem.w"], p["stem.b"] = _folded_conv(rng, 64, 3, 7)
    c_in = 64
    for li, (width, blocks, _) in enumerate(RESNET50_LAYERS):
        for bi in range(blocks):
            pre = f"l{li}.b{bi}."
            p[pre + "c1.w"], p[pre + "c1.b"] = _folded_conv(rng, width, c_in, 1)
            p[pre + "c2.w"], p[pre + "c2.b"] = _folded_conv(rng, width, width, 3)
            p[pre + "c3.w"], p[pre + "c3.b"] = _folded_conv(rng, width * 4, width, 1)
            if bi == 0:
                p[pre + "down.w"], p[pre + "down.b"] = _folded_conv(rng, width * 4, c_in, 1)
            c_in = width * 4
    bound = 1.0 / math.sqrt(c_in)
    p["fc.w"], p["fc.b"] = _uniform(rng, (num_classes, c_in), bound), _uniform(rng, (num_classes,), bound)
    return p


def resnet50_graph(params: Dict[str, np.ndarray], batch: int, image: int = 224, name: str = "resnet50", alignment: int = 64) -> GraphRec:
    b = GraphBuilder(name, alignment)

    def conv(x, shape, w, bias, stride, pad, relu):
        n, _, h, wd = shape
        o, _, k, _ = w.shape
        ho, wo = (h + 2 * pad - k) // stride + 1, (wd + 2 * pad - k) // stride + 1
        wi, bi = b.const(w), b.const(bias)
        out_shape = (n, o, ho, wo)
        y = b.op("Conv2dRelu" if relu else "Conv2d", [x, wi, bi], out_shape, ints=[stride, stride, pad, pad, 1, 1, 1] + _GRID_BLOCK)
        return y, out_shape

    shape = (batch, 3, image, image)
    x = b.input(shape, wire.DT_F32)
    x, shape = conv(x, shape, params["stem.w"], params["stem.b"], 2, 3, True)
    n, c, h, w = shape
    shape = (n, c, (h + 2 - 3) // 2 + 1, (w + 2 - 3) // 2 + 1)
    x = b.op("MaxPool2d", [x], shape, ints=[3, 3, 2, 2, 1, 1, 1, 1, 0] + _GRID_BLOCK)
    for li, (width, blocks, stride) in enumerate(RESNET50_LAYERS):
        for bi in range(blocks):
            pre = f"l{li}.b{bi}."
            s = stride if bi == 0 else 1
            y, ys = conv(x, shape, params[pre + "c1.w"], params[pre + "c1.b"], 1, 0, True)
            y, ys = conv(y, ys, params[pre + "c2.w"], params[pre + "c2.b"], s, 1, True)
            y, ys = conv(y, ys, params[pre + "c3.w"], params[pre + "c3.b"], 1, 0, False)
            identity = x
            if bi == 0:
                identity, _ = conv(x, shape, params[pre + "down.w"], params[pre + "down.b"], s, 0, False)
            x = b.op("AddRelu", [y, identity], ys)
            shape = ys
    n, c, _, _ = shape
    x = b.op("AdaptiveAvgPool2d", [x], (n, c, 1, 1), ints=[1, 1] + _GRID_BLOCK)
    x = b.alias(x, (n, c))  # torch.flatten(x, 1)
    wi, bi_ = b.const(params["fc.w"]), b.const(params["fc.b"])
    x = b.op("Linear", [x, wi, bi_], (n, params["fc.w"].shape[0]))
    b.output(x)
    return b.finish()
