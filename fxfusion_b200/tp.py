"""Tensor parallelism: communicator set-up and the sharding rule, in one place.

The reference is single-device; this layer is new.  One process drives one GPU.  A `Communicator` wraps the
NCCL communicator the C++ engine uses for its all-reduces (fxf_comm_*); its 128-byte unique id is created on
rank 0 and shipped to the other ranks through whatever `torch.distributed` process group is active (NCCL on
GPUs, gloo in CPU tests).  `head_range`, `shard_mha`, `shard_feedforward` and `vocab_range` state the
sharding rule the engine applies on the device (fxfusion_b200/csrc/kernels/ops_dense.cu); they are what the
CPU tests check against the unsharded computation.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, Tuple

import numpy as np

from . import _lib


class Communicator:
    def __init__(self, unique_id: bytes, rank: int, size: int, device_index: int) -> None:
        self.rank, self.size = rank, size
        self.handle = C.c_void_p()
        buf = C.create_string_buffer(unique_id, 128)
        _lib.check(_lib.lib().fxf_comm_create(buf, rank, size, device_index, C.byref(self.handle)))

    @staticmethod
    def unique_id() -> bytes:
        buf = C.create_string_buffer(128)
        _lib.check(_lib.lib().fxf_comm_unique_id(buf))
        return buf.raw

    @classmethod
    def from_process_group(cls, device_index: int, ranks=None, group=None) -> "Communicator":
        """Collective over `group` (default: the world).  `ranks`: global ranks that form this communicator, in
        order (default: all ranks of the group); rank `ranks[0]` creates the id."""
        import torch.distributed as dist
        me = dist.get_rank()
        ranks = list(range(dist.get_world_size())) if ranks is None else list(ranks)
        box = [cls.unique_id() if me == ranks[0] else None]
        dist.broadcast_object_list(box, src=ranks[0], group=group)
        return cls(box[0], ranks.index(me), len(ranks), device_index)

    def close(self) -> None:
        if self.handle:
            _lib.lib().fxf_comm_destroy(self.handle)
            self.handle = C.c_void_p()


# ---- the sharding rule ---------------------------------------------------------------------------------------
def head_range(num_heads: int, rank: int, size: int) -> Tuple[int, int]:
    """Heads [h0, h1) owned by `rank`; heads that do not divide evenly are not sharded (every rank keeps all)."""
    if size <= 1 or num_heads % size:
        return 0, num_heads
    per = num_heads // size
    return rank * per, (rank + 1) * per


def hidden_range(hidden: int, rank: int, size: int) -> Tuple[int, int]:
    if size <= 1 or hidden % size:
        return 0, hidden
    per = hidden // size
    return rank * per, (rank + 1) * per


def vocab_range(vocab: int, rank: int, size: int) -> Tuple[int, int]:
    """Rows [v0, v1) of the final Linear owned by `rank`: blocks of ceil(V / size), the last ones shorter or empty."""
    c = -(-vocab // size)
    v0 = min(vocab, c * rank)
    return v0, min(vocab, v0 + c)


def shard_mha(wqkv: np.ndarray, bqkv: np.ndarray, wo: np.ndarray, bo: np.ndarray, num_heads: int, rank: int, size: int) -> Dict[str, np.ndarray]:
    """Local operands of a head-sharded MHA: rows of each of the Q, K, V thirds for the local heads, the matching
    columns of the output projection, and the output bias on rank 0 only (the partial outputs are summed)."""
    D = wo.shape[0]
    hd = D // num_heads
    h0, h1 = head_range(num_heads, rank, size)
    rows = np.concatenate([np.arange(t * D + h0 * hd, t * D + h1 * hd) for t in range(3)])
    sharded = (h1 - h0) != num_heads
    return {"wqkv": wqkv[rows], "bqkv": bqkv[rows], "wo": wo[:, h0 * hd:h1 * hd],
            "bo": bo if (rank == 0 or not sharded) else np.zeros_like(bo), "heads": h1 - h0, "head0": h0, "sharded": sharded}


def shard_cross_mha(wq: np.ndarray, bq: np.ndarray, wkv: np.ndarray, bkv: np.ndarray, wo: np.ndarray, bo: np.ndarray,
                    num_heads: int, rank: int, size: int) -> Dict[str, np.ndarray]:
    """Local operands of a head-sharded CrossMHA: rows of Wq, of the K half and of the V half of the packed Wkv for the
    local heads, the matching columns of the output projection, the output bias on rank 0 only."""
    D = wo.shape[0]
    hd = D // num_heads
    h0, h1 = head_range(num_heads, rank, size)
    q_rows = np.arange(h0 * hd, h1 * hd)
    kv_rows = np.concatenate([np.arange(t * D + h0 * hd, t * D + h1 * hd) for t in range(2)])
    sharded = (h1 - h0) != num_heads
    return {"wq": wq[q_rows], "bq": bq[q_rows], "wkv": wkv[kv_rows], "bkv": bkv[kv_rows], "wo": wo[:, h0 * hd:h1 * hd],
            "bo": bo if (rank == 0 or not sharded) else np.zeros_like(bo), "heads": h1 - h0, "head0": h0, "sharded": sharded}


def shard_feedforward(w1: np.ndarray, b1: np.ndarray, w2: np.ndarray, b2: np.ndarray, rank: int, size: int) -> Dict[str, np.ndarray]:
    f0, f1 = hidden_range(w1.shape[0], rank, size)
    sharded = (f1 - f0) != w1.shape[0]
    return {"w1": w1[f0:f1], "b1": b1[f0:f1], "w2": w2[:, f0:f1], "b2": b2 if (rank == 0 or not sharded) else np.zeros_like(b2),
            "sharded": sharded}
