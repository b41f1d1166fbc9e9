"""Token sharding of the projection path across the GPUs of one node (host logic only).

The reference is single-GPU (one CudaContext, one stream: src/training/runtime.rs:58-59); this
layer is new.  Forward Y = X.W^T + b and dX = dY.W are row independent, so ranks hold
contiguous token shards with replicated weights and exchange nothing; dW = dY^T.X (and dbias)
contract over tokens, so every rank produces a partial sum and ONE all-reduce(sum) per layer
bucket finishes it.  Two index spaces of the MS-EDEN quantizer are global and must be offset
on a shard to reproduce single-GPU bits: the sign hash is indexed by the K position (the token
index for the transposed operands) and the stochastic scale RNG by the flat group id.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

SHARD_MULTIPLE = 128  # scale tiles (128 rows), 32-chunks and 16-blocks stay whole


def shard_tokens(total_tokens: int, world: int, rank: int) -> Tuple[int, int]:
    """(tokens, first_token) of `rank`: equal contiguous shards, each a multiple of 128 rows."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} for world size {world}")
    if total_tokens % (world * SHARD_MULTIPLE) != 0:
        raise ValueError(f"{total_tokens} tokens do not split into {world} shards of whole {SHARD_MULTIPLE}-row tiles")
    tokens = total_tokens // world
    return tokens, rank * tokens


def padded_k(k: int) -> int:
    return (k + 63) // 64 * 64


def dy_rows_group_offset(first_token: int, out_dim: int) -> int:
    """Flat 16-group id of the first group of this shard's dY rows (K = padded out_dim)."""
    return first_token * (padded_k(out_dim) // 16)


def dy_transposed_col_offset(first_token: int) -> int:
    """K index (token) of the first column of this shard's dY^T / X^T operands."""
    return first_token


def sync_amax(local_amax: torch.Tensor, group=None) -> torch.Tensor:
    """All-reduce(max) of a tensor amax so every shard derives the same global scale (optional:
    without it shards use their own scales, statistically equivalent but not bit-identical)."""
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(local_amax, op=dist.ReduceOp.MAX, group=group)
    return local_amax


class GradBuckets:
    """Per-layer flat f32 buffers holding dW (+dbias) of the layer's linears as views, reduced
    with one all-reduce each as soon as the layer's backward has been enqueued."""

    def __init__(self, layer_shapes: Sequence[Sequence[Tuple[int, int, bool]]], device):
        """layer_shapes[l] = [(out_dim, in_dim, has_bias), ...]."""
        self.buffers: List[torch.Tensor] = []
        self.views: List[List[Tuple[torch.Tensor, Optional[torch.Tensor]]]] = []
        for shapes in layer_shapes:
            size = sum(o * i + (o if b else 0) for o, i, b in shapes)
            buf = torch.zeros(size, dtype=torch.float32, device=device)
            off, views = 0, []
            for o, i, b in shapes:
                dw = buf[off: off + o * i].view(o, i)
                off += o * i
                db = None
                if b:
                    db = buf[off: off + o]
                    off += o
                views.append((dw, db))
            self.buffers.append(buf)
            self.views.append(views)
        self._pending = []

    def reduce_async(self, layer: int, group=None) -> None:
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
            self._pending.append(dist.all_reduce(self.buffers[layer], group=group, async_op=True))

    def wait(self) -> None:
        for work in self._pending:
            work.wait()
        self._pending.clear()
