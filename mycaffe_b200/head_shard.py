"""Head-parallel execution of the attention path over the GPUs of one node.

Heads are independent in every variant of the path (per-(batch, head) scaled-dot-product attention;
the llama2 decode owns the KV-cache slice of its heads), so rank r of N computes heads
[r*H/N, (r+1)*H/N) and the only exchange is an all-gather of the head outputs.  The reference has no
counterpart: its only multi-GPU mode is data-parallel training (MyCaffe/common/Parallel.cs:351-508).

`torch.distributed` is the plumbing (NCCL over NVLink on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def head_range(rank: int, world: int, n_heads: int, n_kv_heads: int | None = None) -> tuple[int, int]:
    """Heads owned by `rank`.  With grouped-query attention the split is by kv head, so that a rank
    owns whole groups of query heads together with their cache slice."""
    groups = n_kv_heads if n_kv_heads is not None else n_heads
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    if groups % world != 0:
        raise ValueError(f"{groups} head groups do not divide over {world} ranks")
    per = (n_heads // groups) * (groups // world)
    return rank * per, (rank + 1) * per


def shard_heads(x: torch.Tensor, rank: int, world: int, head_dim: int = 1) -> torch.Tensor:
    """The slice of a (B, H, ...) tensor that `rank` owns (a contiguous copy)."""
    lo, hi = head_range(rank, world, x.shape[head_dim])
    return x.narrow(head_dim, lo, hi - lo).contiguous()


def gather_heads(y_local: torch.Tensor, group=None, out: torch.Tensor | None = None,
                 strided: bool = False) -> torch.Tensor:
    """All-gather the (B, H/N, T, D) head outputs of every rank into (B, H, T, D).

    One collective per call: the ranks' slices land in a (N, B, H/N, T, D) buffer (`out`, reused when
    given).  By default they are copied back into head order; with `strided` the result is the
    (B, N, H/N, T, D) view of that buffer (head h = [h // (H/N), h % (H/N)]) and nothing is copied."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return y_local
    y_local = y_local.contiguous()
    if out is None:
        out = torch.empty((world,) + tuple(y_local.shape), dtype=y_local.dtype, device=y_local.device)
    dist.all_gather_into_tensor(out.view(-1), y_local.view(-1), group=group)
    B, Hl = y_local.shape[0], y_local.shape[1]
    if strided:
        return out.transpose(0, 1)
    # (N, B, Hl, ...) -> (B, N*Hl, ...)
    return out.transpose(0, 1).reshape((B, world * Hl) + tuple(y_local.shape[2:]))


def gather_decode_outputs(o_local: torch.Tensor, group=None, out: torch.Tensor | None = None) -> torch.Tensor:
    """Decode step: (B, dim/N) per rank -> (B, dim), the input of the Wo projection."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return o_local
    o_local = o_local.contiguous()
    if out is None:
        out = torch.empty((world,) + tuple(o_local.shape), dtype=o_local.dtype, device=o_local.device)
    dist.all_gather_into_tensor(out.view(-1), o_local.view(-1), group=group)
    return out.transpose(0, 1).reshape(o_local.shape[0], world * o_local.shape[1])
