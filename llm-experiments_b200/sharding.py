"""Multi-GPU sharding of the KV-cache path: one process per GPU, ``torch.distributed``.

The reference is single-device throughout (it has no collective of any kind), so this module
has no counterpart there.  Every (sequence, head) pair is independent in append, decode and
prefill (one workgroup per pair in the reference kernels, simple-llm/src/gpu/gpu_kernels.py:2838-2839
and :612-614), which gives two ways to cut the work:

* **batch sharding** (default): rank r owns a contiguous slice of the sequences together with
  their cache; a step needs no communication at all.
* **head splitting** (long contexts with few sequences): rank r owns heads ``[r*H/W, (r+1)*H/W)`` of
  every sequence; after the local decode the ranks exchange their ``[B, H/W * D]`` outputs with
  one all-gather (NCCL over NVLink on GPUs, gloo in CPU tests) and interleave them back to
  ``[B, H*D]``.

The local attention is passed in as a callable, so the exchange logic runs unchanged on CPU
ranks in tests.
"""
from __future__ import annotations

from typing import Callable, Tuple

import torch
import torch.distributed as dist


def shard_range(total: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous ``[start, stop)`` of `total` items for `rank`; sizes differ by at most one."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world: {rank}/{world}")
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def head_range(n_heads: int, rank: int, world: int) -> Tuple[int, int]:
    """Heads owned by `rank` in the head-split configuration (needs ``n_heads % world == 0``)."""
    if n_heads % world != 0:
        raise ValueError(f"n_heads {n_heads} is not divisible by the number of ranks {world}")
    per = n_heads // world
    return rank * per, (rank + 1) * per


def slice_heads(x: torch.Tensor, n_heads: int, head_dim: int, rank: int, world: int) -> torch.Tensor:
    """Columns of a ``[B, H*D]`` matrix that belong to this rank's heads (contiguous copy)."""
    h0, h1 = head_range(n_heads, rank, world)
    return x[:, h0 * head_dim : h1 * head_dim].contiguous()


def gather_heads(local_out: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather ``[B, H/W * D]`` outputs of every rank into ``[B, H*D]`` (rank-major heads)."""
    world = dist.get_world_size(group)
    B, cols = local_out.shape
    gathered = torch.empty((world * B, cols), dtype=local_out.dtype, device=local_out.device)
    dist.all_gather_into_tensor(gathered, local_out.contiguous(), group=group)  # rank r -> rows [r*B, (r+1)*B)
    return gathered.reshape(world, B, cols).permute(1, 0, 2).reshape(B, world * cols)


def head_split_decode(local_attention: Callable[[torch.Tensor], torch.Tensor], q_full: torch.Tensor, n_heads: int,
                      head_dim: int, group=None) -> torch.Tensor:
    """Decode step of the head-split configuration.

    `local_attention` maps this rank's query slice ``[B, H/W * D]`` to its attention output of
    the same shape (over this rank's slice of the cache).  Returns the full ``[B, H*D]`` output
    on every rank.
    """
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    q_local = slice_heads(q_full, n_heads, head_dim, rank, world)
    return gather_heads(local_attention(q_local), group)
