"""Multi-GPU sharding of the KV-cache path: one process per GPU, ``torch.distributed``.

The reference is single-device throughout (it has no collective of any kind), so this module
has no counterpart there.  Every (sequence, head) pair is independent in append, decode and
prefill (one workgroup per pair in the reference kernels, simple-llm/src/gpu/gpu_kernels.py:2838-2839
and :612-614), which gives two ways to cut the work:

* **batch sharding** (default): rank r owns a contiguous slice of the sequences (``shard_range``), or a set
  chosen so that the ranks attend equally many tokens (``balanced_assignment``), together with their
  cache; a step needs no communication at all.
* **head splitting** (long contexts with few sequences): rank r owns heads ``[r*H/W, (r+1)*H/W)`` of
  every sequence; after the local decode the ranks exchange their ``[B, H/W * D]`` outputs with
  one all-gather (NCCL over NVLink on GPUs, gloo in CPU tests) and interleave them back to
  ``[B, H*D]``.

The local attention is passed in as a callable, so the exchange logic runs unchanged on CPU
ranks in tests.
"""
from __future__ import annotations

from typing import Callable, List, Sequence, Tuple

import torch
import torch.distributed as dist


def shard_range(total: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous ``[start, stop)`` of `total` items for `rank`; sizes differ by at most one."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world: {rank}/{world}")
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def balanced_assignment(lengths: Sequence[int], world: int) -> List[List[int]]:
    """Sequences for every rank such that the ranks attend about the same number of tokens: longest sequence
    first, each to the rank with the fewest tokens so far among those that still have room (every rank gets
    ``len(lengths) // world`` sequences, the first ``len(lengths) % world`` ranks one more).  A decode step
    is as slow as its heaviest rank, and contiguous slices of a ragged batch can differ by a quarter."""
    if world <= 0:
        raise ValueError(f"bad world: {world}")
    n = len(lengths)
    room = [n // world + (1 if r < n % world else 0) for r in range(world)]
    load = [0] * world
    out: List[List[int]] = [[] for _ in range(world)]
    for i in sorted(range(n), key=lambda i: (-int(lengths[i]), i)):
        r = min((r for r in range(world) if len(out[r]) < room[r]), key=lambda r: (load[r], r))
        out[r].append(i)
        load[r] += int(lengths[i])
    return [sorted(ids) for ids in out]


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


class FusedHeadGather:
    """Head-split decode whose all-gather is fused into the decode kernel (``b2kv_decode_allgather``).

    Every rank owns ``H/W`` heads.  The decode kernel of each rank stores its output rows, as they
    are finished, directly into the ``[B, H*D]`` result buffers of all ranks over NVLink (symmetric
    memory obtained from ``torch.distributed._symmetric_memory``); its last CTA raises a flag on every
    rank, and a bounded wait on the rank's own flags ends the call: no NCCL collective, no second
    kernel, no extra pass over the data.  Two
    result buffers are used alternately, so a rank that runs one step ahead never overwrites a
    result that a slower peer is still reading.
    """

    def __init__(self, device: torch.device, batch: int, n_heads_total: int, head_dim: int, dtype: torch.dtype,
                 group=None):
        import torch.distributed._symmetric_memory as symm_mem

        group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.B, self.H_total, self.D, self.dtype = batch, n_heads_total, head_dim, dtype
        self.H_local = head_range(n_heads_total, self.rank, self.world)[1] - head_range(n_heads_total, self.rank,
                                                                                           self.world)[0]
        cols = n_heads_total * head_dim
        self.out = symm_mem.empty((2, batch, cols), dtype=dtype, device=device)
        self.flags = symm_mem.empty((self.world,), dtype=torch.int32, device=device)
        self.flags.zero_()
        out_hdl = symm_mem.rendezvous(self.out, group.group_name)
        flag_hdl = symm_mem.rendezvous(self.flags, group.group_name)
        buf_bytes = batch * cols * self.out.element_size()
        self._setup_tables(device, [[int(ptr) + i * buf_bytes for ptr in out_hdl.buffer_ptrs] for i in range(2)],
                           [int(ptr) for ptr in flag_hdl.buffer_ptrs])
        torch.cuda.synchronize(device)
        dist.barrier(group)  # every rank's flags are zero before anyone writes them

    @classmethod
    def from_buffers(cls, device: torch.device, rank: int, world: int, batch: int, n_heads_total: int, head_dim: int,
                     dtype: torch.dtype, out_buffers, flag_buffers):
        """Builds a rank from buffers that the caller has already made visible to every rank
        (its own peer mapping, or several emulated ranks on one device): ``out_buffers[w]`` is rank
        w's ``[2, B, H*D]`` result tensor, ``flag_buffers[w]`` its zeroed ``int32[world]`` flags."""
        self = object.__new__(cls)
        self.rank, self.world = rank, world
        self.B, self.H_total, self.D, self.dtype = batch, n_heads_total, head_dim, dtype
        self.H_local = n_heads_total // world
        self.out, self.flags = out_buffers[rank], flag_buffers[rank]
        buf_bytes = batch * n_heads_total * head_dim * self.out.element_size()
        self._setup_tables(device, [[t.data_ptr() + i * buf_bytes for t in out_buffers] for i in range(2)],
                           [t.data_ptr() for t in flag_buffers])
        return self

    def _setup_tables(self, device, out_ptrs, flag_ptrs):
        self._out_tables = [torch.tensor(ptrs, dtype=torch.int64, device=device) for ptrs in out_ptrs]
        self._flag_table = torch.tensor(flag_ptrs, dtype=torch.int64, device=device)
        self.epoch = 0

    def decode(self, ctx, cache, layer_idx: int, q_local, wait: bool = True) -> torch.Tensor:
        """Attention of this rank's heads over its cache slice; returns the ``[B, H*D]`` result of
        all ranks (a view of the symmetric buffer used for this step)."""
        from . import _native
        from .batch import batch_op_begin, dev_status_ptr
        from .kv_cache import cache_strides, decode_workspace, dtype_code

        if cache.block_table is not None:
            raise ValueError("the fused head gather takes contiguous caches")
        if (cache.batch_size, cache.n_heads, cache.head_dim) != (self.B, self.H_local, self.D):
            raise ValueError("cache does not hold this rank's heads")
        if cache.current_len == 0:
            raise ValueError("Cache is empty: current_len=0")
        self.epoch = (self.epoch + 1) & 0xFFFFFFFF
        buf = self.epoch & 1
        ws = decode_workspace(cache)
        stream = batch_op_begin(ctx)
        s0, st, sh = cache_strides(cache)
        layer = cache.layers[layer_idx]
        rc = _native.lib.b2kv_decode_allgather(
            q_local.buffer.data_ptr(), layer.k_cache.buffer.data_ptr(), layer.v_cache.buffer.data_ptr(),
            None if cache.seq_lens is None else cache.seq_lens.data_ptr(), cache.current_len, 0, self.B, self.H_local,
            self.D, min(cache.current_len, cache.max_seq_len), s0, st, sh, dtype_code(cache.dtype), ws.data_ptr(),
            ws.numel(), self._out_tables[buf].data_ptr(), self._flag_table.data_ptr(),
            self.flags.data_ptr() if wait else None, None, 0, self.rank,
            self.world, self.H_total, self.epoch, dev_status_ptr(ctx), stream)
        _native.check(rc)
        return self.out[buf]


# ------------------------------------------------------------------------------------------
# sequence split (context parallel): every rank holds a slice of each sequence's tokens
# ------------------------------------------------------------------------------------------


def decode_partial(ctx, cache, layer_idx: int, q_new) -> torch.Tensor:
    """Attention of ``q_new [B, H*D]`` over THIS rank's slice of the cache, left unnormalised:
    returns float32 ``[B*H, D + 2]`` (row sums, then the maximum in the log2 domain - ``-inf`` when
    the slice holds no token of that sequence - then the sum of weights), ready for ``merge_partials``."""
    from . import _native
    from .batch import batch_op_begin, dev_status_ptr
    from .kv_cache import cache_strides, decode_workspace, dtype_code

    if cache.block_table is not None:
        raise ValueError("the sequence-split decode takes contiguous caches")
    B, H, D = cache.batch_size, cache.n_heads, cache.head_dim
    part = torch.empty((B * H, D + 2), dtype=torch.float32, device=q_new.buffer.device)
    ws = decode_workspace(cache)
    stream = batch_op_begin(ctx)
    s0, st, sh = cache_strides(cache)
    layer = cache.layers[layer_idx]
    t_upper = max(1, min(cache.current_len, cache.max_seq_len))
    rc = _native.lib.b2kv_decode_partial(
        q_new.buffer.data_ptr(), layer.k_cache.buffer.data_ptr(), layer.v_cache.buffer.data_ptr(), part.data_ptr(),
        None if cache.seq_lens is None else cache.seq_lens.data_ptr(), cache.current_len, 0, B, H, D, t_upper, s0, st,
        sh, dtype_code(cache.dtype), ws.data_ptr(), ws.numel(), dev_status_ptr(ctx), stream)
    _native.check(rc)
    return part


def merge_partials(ctx, parts: torch.Tensor, batch: int, n_heads: int, head_dim: int, dtype: torch.dtype) -> torch.Tensor:
    """Combines ``parts [R, B*H, D + 2]`` (one ``decode_partial`` result per slice) into ``[B, H*D]``."""
    from . import _native
    from .batch import batch_op_begin
    from .kv_cache import dtype_code

    parts = parts.contiguous()
    R = parts.shape[0]
    out = torch.empty((batch, n_heads * head_dim), dtype=dtype, device=parts.device)
    stream = batch_op_begin(ctx)
    _native.check(_native.lib.b2kv_merge_partials(parts.data_ptr(), R, batch, n_heads, head_dim, out.data_ptr(),
                                                  dtype_code(dtype), stream))
    return out


def exchange_partials(part: torch.Tensor, merge: Callable[[torch.Tensor], torch.Tensor], group=None) -> torch.Tensor:
    """The exchange of the sequence-split decode: all-gathers every rank's ``[B*H, D + 2]`` float partials
    and hands the ``[world, B*H, D + 2]`` stack to `merge`, whose result is returned.  The merge is passed in
    as a callable so that the exchange runs unchanged on CPU ranks in tests."""
    world = dist.get_world_size(group)
    gathered = torch.empty((world * part.shape[0], part.shape[1]), dtype=part.dtype, device=part.device)
    dist.all_gather_into_tensor(gathered, part.contiguous(), group=group)
    return merge(gathered.reshape(world, part.shape[0], part.shape[1]))


def sequence_split_decode(ctx, cache, layer_idx: int, q_new, group=None) -> torch.Tensor:
    """Decode step when each rank caches a different slice of every sequence's tokens (all heads):
    local unnormalised attention, one all-gather of the ``[B*H, D + 2]`` float partials, merge.
    Returns the full ``[B, H*D]`` output on every rank."""
    part = decode_partial(ctx, cache, layer_idx, q_new)
    return exchange_partials(
        part, lambda parts: merge_partials(ctx, parts, cache.batch_size, cache.n_heads, cache.head_dim, cache.dtype),
        group)
