"""KV-cache operations behind the reference's own API.

Mirrors simple-llm/src/gpu/gpu_kv_cache.py: ``kv_cache_create`` (:26-87), ``kv_cache_reset``
(:90-105), ``kv_cache_update`` (:113-186) and ``attention_with_kv_cache`` (:194-289) keep their
names, positional arguments, return value (``None``) and the conditions and texts of their
``ValueError``s.  The WGSL dispatch inside them is replaced by calls into the C-ABI CUDA
library (include/b2kv.h).

Behaviour kept from the reference, including its quirk: ``kv_cache_update`` advances
``cache.current_len`` itself on every call (:186), although its docstring tells the caller to
do so after all layers.  A multi-layer decode loop therefore either sets ``current_len`` back
before each layer's update or passes ``advance=False`` for all but one layer.

Extensions (off unless asked for through ``KVCacheConfig``): bf16 storage, the ``[B, H, T, D]``
layout, per-sequence lengths kept on the device (``ragged``), paged caches with a block
table.  The reference's 256-token limit of ``attention_with_kv_cache`` (:250-257) is not
enforced unless ``ctx.config.enforce_reference_decode_limit`` is set.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from . import _native
from .batch import batch_op_begin, dev_status_ptr, validate_buffer_shape_2d, reference_op
from .buffers import gpu_buffer_2d_create, gpu_buffer_zerofy
from .types import GPUBuffer2D, GPUContext, KVCache, KVCacheConfig, KVCacheLayer

_DTYPES = {torch.float32: _native.DTYPE_F32, torch.bfloat16: _native.DTYPE_BF16}


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise ValueError(f"Unsupported cache dtype {dtype}; supported: float32, bfloat16") from None


def cache_strides(cache: KVCache) -> Tuple[int, int, int]:
    """(stride of a sequence or block, stride of a token, stride of a head), in elements."""
    H, D, T = cache.n_heads, cache.head_dim, cache.max_seq_len
    if cache.block_table is not None:
        return H * cache.block_size * D, D, cache.block_size * D
    if cache.layout == "bthd":
        return T * H * D, H * D, D
    return H * T * D, D, T * D


def kv_cache_create(ctx: GPUContext, config: KVCacheConfig) -> KVCache:
    if config.batch_size <= 0:
        raise ValueError(f"batch_size must be > 0, got {config.batch_size}")
    if config.max_seq_len <= 0:
        raise ValueError(f"max_seq_len must be > 0, got {config.max_seq_len}")
    if config.n_layers <= 0:
        raise ValueError(f"n_layers must be > 0, got {config.n_layers}")
    if config.n_heads <= 0:
        raise ValueError(f"n_heads must be > 0, got {config.n_heads}")
    if config.head_dim <= 0:
        raise ValueError(f"head_dim must be > 0, got {config.head_dim}")
    if config.layout not in ("bthd", "bhtd"):
        raise ValueError(f"layout must be 'bthd' or 'bhtd', got {config.layout!r}")
    dtype_code(config.dtype)

    B, T, H, D = config.batch_size, config.max_seq_len, config.n_heads, config.head_dim
    paged = config.block_size > 0
    block_table = None
    n_blocks = 0
    if paged:
        max_blocks = (T + config.block_size - 1) // config.block_size
        n_blocks = config.n_blocks if config.n_blocks > 0 else B * max_blocks
        if n_blocks < B * max_blocks:
            raise ValueError(f"n_blocks {n_blocks} cannot hold {B} sequences of {max_blocks} blocks")
        # identity placement; callers may overwrite the table with their own allocation
        block_table = torch.arange(B * max_blocks, dtype=torch.int32, device=ctx.device).reshape(B, max_blocks)
        rows, cols = n_blocks * H * config.block_size, D
    elif config.layout == "bthd":
        rows, cols = B * T, H * D
    else:
        rows, cols = B * H * T, D

    layers: List[KVCacheLayer] = []
    for _ in range(config.n_layers):
        k_cache = gpu_buffer_2d_create(ctx, rows, cols, dtype=config.dtype)
        v_cache = gpu_buffer_2d_create(ctx, rows, cols, dtype=config.dtype)
        gpu_buffer_zerofy(ctx, k_cache)
        gpu_buffer_zerofy(ctx, v_cache)
        layers.append(KVCacheLayer(k_cache=k_cache, v_cache=v_cache))

    seq_lens = torch.zeros(B, dtype=torch.int32, device=ctx.device) if config.ragged else None
    return KVCache(layers=layers, batch_size=B, max_seq_len=T, current_len=0, n_heads=H, head_dim=D,
                   dtype=config.dtype, layout=config.layout, seq_lens=seq_lens, block_table=block_table,
                   block_size=config.block_size if paged else 0, n_blocks=n_blocks)


def kv_cache_reset(cache: KVCache) -> None:
    cache.current_len = 0
    if cache.seq_lens is not None:
        cache.seq_lens.zero_()


def kv_cache_set_lengths(cache: KVCache, lens) -> None:
    """Extension: install per-sequence lengths (host list / array / tensor of B ints)."""
    host = torch.as_tensor(lens, dtype=torch.int32).reshape(cache.batch_size).cpu()
    if int(host.min()) < 0 or int(host.max()) > cache.max_seq_len:
        raise ValueError(f"lengths must lie in [0, {cache.max_seq_len}]")
    device = cache.layers[0].k_cache.buffer.device
    if cache.seq_lens is None:
        cache.seq_lens = host.to(device)
    else:
        cache.seq_lens.copy_(host, non_blocking=True)
    cache.current_len = int(host.max())


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


@reference_op("kv_cache_update")
def kv_cache_update(ctx: GPUContext, cache: KVCache, layer_idx: int, new_k: GPUBuffer2D, new_v: GPUBuffer2D,
                    advance: bool = True) -> None:
    if layer_idx < 0 or layer_idx >= len(cache.layers):
        raise ValueError(f"layer_idx {layer_idx} out of range [0, {len(cache.layers)})")
    if cache.current_len >= cache.max_seq_len:
        raise ValueError(f"Cache is full: current_len={cache.current_len}, max_seq_len={cache.max_seq_len}")
    embedding_dim = cache.n_heads * cache.head_dim
    expected_rows = cache.batch_size * 1
    validate_buffer_shape_2d(new_k, (expected_rows, embedding_dim), "new_k")
    validate_buffer_shape_2d(new_v, (expected_rows, embedding_dim), "new_v")
    if new_k.buffer.dtype != cache.dtype or new_v.buffer.dtype != cache.dtype:
        raise ValueError(f"new_k/new_v dtype must match the cache dtype {cache.dtype}")

    layer = cache.layers[layer_idx]
    stream = batch_op_begin(ctx)
    s0, st, sh = cache_strides(cache)
    dt = dtype_code(cache.dtype)
    adv = 1 if (advance and cache.seq_lens is not None) else 0
    if cache.block_table is None:
        rc = _native.lib.b2kv_append(new_k.buffer.data_ptr(), new_v.buffer.data_ptr(), layer.k_cache.buffer.data_ptr(),
                                     layer.v_cache.buffer.data_ptr(), _ptr(cache.seq_lens), cache.current_len, adv,
                                     cache.batch_size, cache.n_heads, cache.head_dim, cache.max_seq_len, s0, st, sh,
                                     dt, dev_status_ptr(ctx), stream)
    else:
        rc = _native.lib.b2kv_append_paged(new_k.buffer.data_ptr(), new_v.buffer.data_ptr(),
                                           layer.k_cache.buffer.data_ptr(), layer.v_cache.buffer.data_ptr(),
                                           _ptr(cache.seq_lens), cache.current_len, adv, cache.block_table.data_ptr(),
                                           cache.block_table.shape[1], cache.block_size, cache.n_blocks,
                                           cache.batch_size, cache.n_heads, cache.head_dim, s0, st, sh, dt,
                                           dev_status_ptr(ctx), stream)
    _native.check(rc)
    if advance:
        cache.current_len += 1


def decode_workspace(cache: KVCache) -> torch.Tensor:
    """Scratch for the split-K partials, sized by the library for this cache's largest length;
    allocated on first use and grown if a tuning knob later asks for a finer split."""
    nbytes = _native.lib.b2kv_decode_workspace_bytes(cache.batch_size, cache.n_heads, cache.head_dim,
                                                     cache.max_seq_len, dtype_code(cache.dtype))
    if cache.workspace is None or cache.workspace.numel() < nbytes:
        cache.workspace = torch.empty(nbytes, dtype=torch.uint8, device=cache.layers[0].k_cache.buffer.device)
    return cache.workspace


@reference_op("attention_with_kv_cache")
def attention_with_kv_cache(ctx: GPUContext, cache: KVCache, layer_idx: int, q_new: GPUBuffer2D,
                            output: GPUBuffer2D) -> None:
    if layer_idx < 0 or layer_idx >= len(cache.layers):
        raise ValueError(f"layer_idx {layer_idx} out of range [0, {len(cache.layers)})")
    if cache.current_len == 0:
        raise ValueError("Cache is empty: current_len=0")
    if ctx.config.enforce_reference_decode_limit:
        workgroup_size = ctx.config.attention_workgroup_size
        if cache.current_len > workgroup_size:
            raise ValueError(
                f"current_len ({cache.current_len}) exceeds maximum supported "
                f"sequence length ({workgroup_size}) for attention_with_kv_cache. "
                f"Use chunked attention or increase workgroup_size in config."
            )
    embedding_dim = cache.n_heads * cache.head_dim
    expected_q_rows = cache.batch_size * 1
    validate_buffer_shape_2d(q_new, (expected_q_rows, embedding_dim), "q_new")
    validate_buffer_shape_2d(output, (expected_q_rows, embedding_dim), "output")
    if q_new.buffer.dtype != cache.dtype or output.buffer.dtype != cache.dtype:
        raise ValueError(f"q_new/output dtype must match the cache dtype {cache.dtype}")

    layer = cache.layers[layer_idx]
    ws = decode_workspace(cache)
    stream = batch_op_begin(ctx)
    s0, st, sh = cache_strides(cache)
    dt = dtype_code(cache.dtype)
    t_upper = min(cache.current_len, cache.max_seq_len)
    if cache.block_table is None:
        rc = _native.lib.b2kv_decode(q_new.buffer.data_ptr(), layer.k_cache.buffer.data_ptr(),
                                     layer.v_cache.buffer.data_ptr(), output.buffer.data_ptr(), _ptr(cache.seq_lens),
                                     cache.current_len, 0, cache.batch_size, cache.n_heads, cache.head_dim, t_upper,
                                     s0, st, sh, dt, ws.data_ptr(), ws.numel(), dev_status_ptr(ctx), stream)
    else:
        rc = _native.lib.b2kv_decode_paged(q_new.buffer.data_ptr(), layer.k_cache.buffer.data_ptr(),
                                           layer.v_cache.buffer.data_ptr(), output.buffer.data_ptr(),
                                           _ptr(cache.seq_lens), cache.current_len, 0, cache.block_table.data_ptr(),
                                           cache.block_table.shape[1], cache.block_size, cache.n_blocks,
                                           cache.batch_size, cache.n_heads, cache.head_dim, t_upper, s0, st, sh, dt,
                                           ws.data_ptr(), ws.numel(), dev_status_ptr(ctx), stream)
    _native.check(rc)


def kv_cache_gather(ctx: GPUContext, cache: KVCache, layer_idx: int, which: str = "k",
                    length: Optional[int] = None) -> torch.Tensor:
    """Extension: the logical view ``[B, length, H, D]`` of one layer's K or V (zero past each
    sequence's length), whatever the physical layout.  Used for bit-exact append checks."""
    if layer_idx < 0 or layer_idx >= len(cache.layers):
        raise ValueError(f"layer_idx {layer_idx} out of range [0, {len(cache.layers)})")
    T_out = cache.max_seq_len if length is None else int(length)
    layer = cache.layers[layer_idx]
    src = layer.k_cache if which == "k" else layer.v_cache
    out = torch.empty((cache.batch_size, T_out, cache.n_heads, cache.head_dim), dtype=cache.dtype,
                      device=src.buffer.device)
    stream = batch_op_begin(ctx)
    s0, st, sh = cache_strides(cache)
    dt = dtype_code(cache.dtype)
    n = min(cache.current_len, T_out)
    if cache.block_table is None:
        rc = _native.lib.b2kv_gather(src.buffer.data_ptr(), out.data_ptr(), _ptr(cache.seq_lens), n,
                                     cache.batch_size, cache.n_heads, cache.head_dim, T_out, s0, st, sh, dt, stream)
    else:
        rc = _native.lib.b2kv_gather_paged(src.buffer.data_ptr(), out.data_ptr(), _ptr(cache.seq_lens), n,
                                           cache.block_table.data_ptr(), cache.block_table.shape[1], cache.block_size,
                                           cache.n_blocks, cache.batch_size, cache.n_heads, cache.head_dim, T_out,
                                           s0, st, sh, dt, dev_status_ptr(ctx), stream)
    _native.check(rc)
    return out
