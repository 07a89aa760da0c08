"""Causal flash-attention prefill behind the reference's ``flash_attention`` signature.

Mirrors simple-llm/src/gpu/gpu_pass_forward.py:497-588: same positional arguments, the same
checks and ``ValueError`` texts (:531-555), ``None`` returned, O / L / M written in place.
``flash_attn_bc`` / ``flash_attn_br`` are ignored (the CUDA kernels choose their own tiles).
Extension: ``cache`` / ``layer_idx`` also write K and V rows 0..N-1 of every sequence into
that cache layer (in the same kernel for a contiguous cache and for the whole blocks of a paged one
on the tensor-core path; through the block table by a copy kernel behind it otherwise) and set the cache length to N, which the reference can only
do token by token through ``kv_cache_update``.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _native
from .batch import batch_op_begin, dev_status_ptr, reference_op, validate_buffer_shape_1d, validate_buffer_shape_2d
from .kv_cache import cache_strides, dtype_code
from .types import GPUBuffer1D, GPUBuffer2D, GPUContext, KVCache


@reference_op("flash_attention")
def flash_attention(ctx: GPUContext, Q: GPUBuffer2D, K: GPUBuffer2D, V: GPUBuffer2D, O: GPUBuffer2D,
                    L: Optional[GPUBuffer1D], M: Optional[GPUBuffer1D], batch_size: int, seq_len: int, n_heads: int,
                    head_dim: int, cache: Optional[KVCache] = None, layer_idx: int = 0) -> None:
    if head_dim > ctx.config.flash_attn_max_head_dim:
        raise ValueError(
            f"head_dim {head_dim} exceeds maximum supported by config: "
            f"{ctx.config.flash_attn_max_head_dim}. "
            f"Increase flash_attn_max_head_dim in GPUConfig or use smaller head_dim."
        )
    if batch_size <= 0 or seq_len <= 0 or n_heads <= 0 or head_dim <= 0:
        raise ValueError(
            f"Invalid dimensions: batch_size={batch_size}, seq_len={seq_len}, "
            f"n_heads={n_heads}, head_dim={head_dim}"
        )
    embedding_dim = n_heads * head_dim
    total_tokens = batch_size * seq_len
    validate_buffer_shape_2d(Q, (total_tokens, embedding_dim), "Q")
    validate_buffer_shape_2d(K, (total_tokens, embedding_dim), "K")
    validate_buffer_shape_2d(V, (total_tokens, embedding_dim), "V")
    validate_buffer_shape_2d(O, (total_tokens, embedding_dim), "O")
    stats_size = batch_size * seq_len * n_heads
    if L is not None:
        validate_buffer_shape_1d(L, stats_size, "L")
    if M is not None:
        validate_buffer_shape_1d(M, stats_size, "M")
    dtype = Q.buffer.dtype
    if any(x.buffer.dtype != dtype for x in (K, V, O)):
        raise ValueError("Q, K, V and O must share one dtype")

    kc = vc = None
    s0 = st = sh = 0
    t_max = 0
    if cache is not None:
        if layer_idx < 0 or layer_idx >= len(cache.layers):
            raise ValueError(f"layer_idx {layer_idx} out of range [0, {len(cache.layers)})")
        if (cache.batch_size, cache.n_heads, cache.head_dim) != (batch_size, n_heads, head_dim):
            raise ValueError("cache dimensions do not match the attention call")
        if seq_len > cache.max_seq_len:
            raise ValueError(f"Cache is full: seq_len={seq_len}, max_seq_len={cache.max_seq_len}")
        if cache.dtype != dtype:
            raise ValueError(f"cache dtype {cache.dtype} does not match {dtype}")
        layer = cache.layers[layer_idx]
        s0, st, sh = cache_strides(cache)
        if cache.block_table is None:  # contiguous: the attention kernel writes the rows itself
            kc, vc = layer.k_cache.buffer.data_ptr(), layer.v_cache.buffer.data_ptr()
            t_max = cache.max_seq_len

    stream = batch_op_begin(ctx)
    lm = (None if L is None else L.buffer.data_ptr(), None if M is None else M.buffer.data_ptr())
    if cache is not None and cache.block_table is not None:
        # paged: whole blocks are stored by the attention kernel, the rest by a copy kernel behind it
        rc = _native.lib.b2kv_prefill_paged(Q.buffer.data_ptr(), K.buffer.data_ptr(), V.buffer.data_ptr(),
                                            O.buffer.data_ptr(), *lm, layer.k_cache.buffer.data_ptr(),
                                            layer.v_cache.buffer.data_ptr(), cache.block_table.data_ptr(),
                                            cache.block_table.shape[1], cache.block_size, cache.n_blocks, s0, st, sh,
                                            batch_size, seq_len, n_heads, head_dim, dtype_code(dtype),
                                            dev_status_ptr(ctx), stream)
    else:
        # fp32 prompts of head_dim 128 / 64 run on the tensor cores when given scratch for their bfloat16 halves
        ws_bytes = _native.lib.b2kv_prefill_workspace_bytes(batch_size, seq_len, n_heads, head_dim, dtype_code(dtype))
        ws = None
        if ws_bytes:
            if ctx.prefill_workspace is None or ctx.prefill_workspace.numel() < ws_bytes:
                ctx.prefill_workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=ctx.device)
            ws = ctx.prefill_workspace.data_ptr()
        rc = _native.lib.b2kv_prefill_ws(Q.buffer.data_ptr(), K.buffer.data_ptr(), V.buffer.data_ptr(), O.buffer.data_ptr(),
                                         *lm, kc, vc, s0, st, sh, t_max, batch_size, seq_len, n_heads, head_dim,
                                         dtype_code(dtype), ws, ws_bytes, dev_status_ptr(ctx), stream)
    _native.check(rc)
    if cache is not None:
        cache.current_len = seq_len
        if cache.seq_lens is not None:
            cache.seq_lens.fill_(seq_len)
