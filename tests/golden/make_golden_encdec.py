"""Generates the encoder-decoder fixtures (`encdec_*.bin` / `.npz`) in this directory.

    python tests/golden/make_golden_encdec.py [/path/to/reference]

The reference's compile passes cannot lower its own encoder-decoder Transformer (the decoder's cross-attention does
not fit its QKV packing), so unlike make_golden.py only the EXPECTED OUTPUTS come from the reference here: its
unmodified eager model `Transformer(Encoder(...), Decoder(...))` (py/fxfusion/models/transformer/models/) is
instantiated, its weights are copied into this repository's parameter layout (Wq/Wk/Wv packed the way the reference's
packing pass packs them, matchers.py:641-657), `lowering.transformer_graph` builds the graph file, and the eager
model's logits are stored as `out0`.  The tests then require oracle(graph) == out0 and GPU(graph) == oracle.
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

from fxfusion_b200 import lowering, wire  # noqa: E402
from fxfusion_b200.compile_ref import _ensure_reference_importable  # noqa: E402

_ensure_reference_importable()
from fxfusion.models.transformer.models.decoder import Decoder  # noqa: E402
from fxfusion.models.transformer.models.encoder import Encoder  # noqa: E402
from fxfusion.models.transformer.models.transformer import Transformer  # noqa: E402

torch.set_grad_enabled(False)


def params_of(model: Transformer, cfg: lowering.TransformerConfig):
    """state_dict of the reference model -> the parameter names of lowering.transformer_params."""
    sd = {k: v.detach().clone() for k, v in model.state_dict().items()}
    p = {}

    def lin(dst, src):
        p[dst + ".w"], p[dst + ".b"] = sd[src + ".weight"].numpy(), sd[src + ".bias"].numpy()

    def packed(dst, mod, names):
        p[dst + ".w"] = torch.cat([sd[f"{mod}.{n}.weight"] for n in names], 0).numpy()
        p[dst + ".b"] = torch.cat([sd[f"{mod}.{n}.bias"] for n in names], 0).numpy()

    for side, blocks, layers in (("enc", "encoder.encoder_blocks", cfg.enc_layers), ("dec", "decoder.decoder_blocks", cfg.dec_layers)):
        top = "encoder" if side == "enc" else "decoder"
        p[f"{side}.emb"] = sd[f"{top}.in_embedding.embedding.weight"].numpy()
        # the reference buffer has 5000 rows; the fixture keeps the first pe_len (Narrow reads only the first L of them)
        p[f"{side}.pe"] = sd[f"{top}.pos_encoding.pe"][:, :cfg.pe_len].numpy()
        for l in range(layers):
            src, dst = f"{blocks}.{l}", f"{side}.l{l}."
            att = "mha" if side == "enc" else "self_attn"
            lin(dst + "ln1", f"{src}.norm1")
            packed(dst + "qkv", f"{src}.{att}", ("W_q", "W_k", "W_v"))
            lin(dst + "wo", f"{src}.{att}.W_o")
            if side == "dec":
                lin(dst + "ln2", f"{src}.norm2")
                lin(dst + "cq", f"{src}.cross_attn.W_q")
                packed(dst + "ckv", f"{src}.cross_attn", ("W_k", "W_v"))
                lin(dst + "co", f"{src}.cross_attn.W_o")
                lin(dst + "lnf", f"{src}.norm3")
            else:
                lin(dst + "lnf", f"{src}.norm2")
            lin(dst + "ff1", f"{src}.ff.{FF1}")
            lin(dst + "ff2", f"{src}.ff.{FF2}")
        lin(f"{side}.ln_out", f"{top}.norm")
    lin("head", "decoder.linear")
    return {k: np.ascontiguousarray(v, dtype=np.float32) for k, v in p.items()}


def emit(name, cfg, B, S, T, seed, pad_from=None):
    torch.manual_seed(seed)
    model = Transformer(Encoder(cfg.d_model, cfg.heads, cfg.vocab, cfg.expansion, 0.0, cfg.enc_layers),
                        Decoder(cfg.d_model, cfg.heads, cfg.vocab, cfg.expansion, 0.0, cfg.dec_layers)).eval()
    for prm in model.parameters():           # non-trivial biases and LayerNorm affines
        if prm.dim() == 1:
            prm.add_(torch.randn_like(prm) * 0.05)
    src, tgt = torch.randint(1, cfg.vocab, (B, S)), torch.randint(1, cfg.vocab, (B, T))
    src_mask = torch.ones(B, 1, 1, S, dtype=torch.bool)
    if pad_from is not None:
        src_mask[-1, 0, 0, pad_from:] = False   # padded tail of the last source sequence
    tgt_mask = torch.tril(torch.ones(T, T, dtype=torch.bool)).view(1, 1, T, T).expand(B, 1, T, T).contiguous()
    want = model(src, tgt, src_mask, tgt_mask)
    graph = lowering.transformer_graph(cfg, params_of(model, cfg), batch=B, src_len=S, tgt_len=T, name=name)
    wire.dump(graph, HERE / f"{name}.bin")
    np.savez_compressed(HERE / f"{name}.npz", in0=src.numpy(), in1=tgt.numpy(), in2=src_mask.numpy(), in3=tgt_mask.numpy(), out0=want.numpy())
    ops = [wire.OPCODES[n.op_code] for n in graph.nodes if n.op_code]
    print(f"{name:24s} arena {graph.arena_size:8d}  nodes {len(ops)}  CrossMHA x{ops.count('CrossMHA')}")


def ff_names():
    """Attribute names of the two Linear layers inside the reference FeedForward module."""
    from fxfusion.models.transformer.layers.feedforward import FeedForward
    lin = [n for n, m in FeedForward(8, 2).named_modules() if isinstance(m, torch.nn.Linear)]
    assert len(lin) == 2, lin
    return lin


FF1, FF2 = ff_names()

if __name__ == "__main__":
    emit("encdec_small", lowering.TransformerConfig(32, 4, 64, 2, 2, 2, pe_len=16), B=2, S=9, T=6, seed=0, pad_from=6)
    emit("encdec_hd64", lowering.TransformerConfig(128, 2, 96, 2, 1, 2, pe_len=48), B=2, S=40, T=24, seed=1, pad_from=33)
