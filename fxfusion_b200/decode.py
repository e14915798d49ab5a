"""Greedy static decode, host loop — the reference's `engine_decode_static` call for call.

Reference: py/fxfusion/models/transformer/inference.py:27-45 (loop), layers/masks.py:70-154
(static buffer and mask).  Every step rebuilds the [B,1,T,T] mask, runs the whole graph on the
fixed [B, max_seq_len] token buffer and takes the argmax of one logits row; there is no KV cache.
The mask and the argmax run on the GPU (fxf_decode_build_mask / fxf_decode_argmax_scatter), so the
loop never synchronises; `ExecutionEngine.decode_static` is the same loop issued from C++.
"""
from __future__ import annotations

import ctypes as C

from . import _lib


def make_static_buffer(tokens, max_seq_len: int, pad_idx: int = 0):
    import torch
    B, T = tokens.shape
    if T > max_seq_len:
        raise ValueError(f"Token length {T} exceeds max_seq_len {max_seq_len}")
    buf = torch.full((B, max_seq_len), pad_idx, dtype=tokens.dtype, device=tokens.device)
    buf[:, :T] = tokens
    return buf


class StaticDecoderMaskBuilder:
    """mask[b,0,q,k] = (k < current_len) & (tokens[b,k] != pad_idx) & (k <= q), bool [B,1,T,T]."""

    def __init__(self, max_seq_len: int) -> None:
        self.max_seq_len = max_seq_len
        self._out = None

    def __call__(self, tokens, current_len: int, pad_idx: int = 0, out=None):
        import torch
        B, T = tokens.shape
        if T > self.max_seq_len:
            raise ValueError(f"Token length {T} exceeds max_seq_len {self.max_seq_len}")
        if current_len > T:
            raise ValueError(f"current_len {current_len} exceeds static length {T}")
        if out is None:
            out = torch.empty((B, 1, T, T), dtype=torch.bool, device=tokens.device)
        stream = C.c_void_p(torch.cuda.current_stream(tokens.device).cuda_stream)
        _lib.check(_lib.lib().fxf_decode_build_mask(C.c_void_p(tokens.data_ptr()), C.c_void_p(out.data_ptr()), B, T,
                                                    int(current_len), int(pad_idx), stream))
        return out


def engine_decode_static(engine, tokens, mask_builder: StaticDecoderMaskBuilder = None, max_seq_len: int = 50):
    """tokens: int64 CUDA tensor [B, initial_len]; returns [B, max_seq_len] completed greedily."""
    import torch
    B, initial_len = tokens.shape
    mask_builder = mask_builder or StaticDecoderMaskBuilder(max_seq_len)
    buf = make_static_buffer(tokens, max_seq_len)
    lib = _lib.lib()
    cur = initial_len
    for _ in range(max_seq_len - initial_len):
        mask = mask_builder(buf, cur)
        logits = engine.run([buf, mask])[0]
        stream = C.c_void_p(torch.cuda.current_stream(tokens.device).cuda_stream)
        _lib.check(lib.fxf_decode_argmax_scatter(C.c_void_p(logits.data_ptr()), C.c_void_p(buf.data_ptr()), B, max_seq_len,
                                                 logits.shape[-1], cur, stream))
        cur += 1
    return buf[:, :cur]
