"""Q / K / V projection of one decode step fused with the KV-cache append.

The reference's attention block runs three ``matmul`` dispatches on the normalised hidden state
(simple-llm/src/wgpu_backend.py:812-831; ``matmul(ctx, A, B, C)`` of
src/gpu/gpu_pass_forward.py:35-82 computes C = A @ B) and a cached decode would follow them with
``kv_cache_update`` (src/gpu/gpu_kv_cache.py:113-186).  ``qkv_project_append`` does the four steps in
one kernel for the rows of a decode step: Q goes to its buffer, the new K / V rows go straight into
the cache.  Checks and texts follow ``kv_cache_update``; bf16 caches with a contiguous layout only
(other cases: project with matmuls, then ``kv_cache_update``).
"""
from __future__ import annotations

import torch

from . import _native
from .batch import batch_op_begin, dev_status_ptr, reference_op, validate_buffer_shape_2d
from .kv_cache import _ptr, cache_strides, dtype_code
from .types import GPUBuffer2D, GPUContext, KVCache


@reference_op("matmul")
def matmul(ctx: GPUContext, A: GPUBuffer2D, B: GPUBuffer2D, C: GPUBuffer2D, residual: GPUBuffer2D = None,
           bias=None, activation: str = None) -> None:
    """``C = A @ B`` with the reference's argument order and shape check
    (simple-llm/src/gpu/gpu_pass_forward.py:35-82), bfloat16, inner and outer dimensions multiples of 8.
    The rows of a cached decode step (at most 128 rows in ``A``, dimensions multiples of 128) go to the
    weight-streaming kernel, every other shape (the prompt-side projections) to the tiled tensor-core
    GEMM.  Extensions that fold the
    dispatches which follow a matmul in the reference's block (src/wgpu_backend.py:857-930) into
    it: ``bias`` (a ``GPUBuffer1D`` of N values, ``bias_add``), ``activation="gelu"``
    (``x * sigmoid(1.702 x)``, ``gelu``) and ``residual`` (``residual_add``), applied in that order:
    ``C = act(A @ B + bias) + residual``."""
    M, K = A.shape
    K2, N = B.shape
    # same checks and texts as validate_matmul_shapes (simple-llm/src/gpu/gpu_ops.py:84-99)
    if M <= 0 or K <= 0 or N <= 0 or K2 <= 0:
        raise ValueError(f"matmul: Invalid dimensions A=({M}, {K}), B=({K2}, {N})")
    if K != K2:
        raise ValueError(f"matmul: Dimension mismatch A.shape[1]={K} != B.shape[0]={K2}")
    if tuple(C.shape) != (M, N):
        raise ValueError(f"matmul: Output shape {C.shape} doesn't match expected ({M}, {N})")
    if residual is not None:
        validate_buffer_shape_2d(residual, (M, N), "residual")
    if bias is not None and tuple(bias.shape) != (N,):
        raise ValueError(f"bias shape mismatch: expected ({N},), got {tuple(bias.shape)}")
    if activation not in (None, "gelu"):
        raise ValueError(f"unknown activation {activation!r}")
    bufs = [A, B, C] + [t for t in (residual, bias) if t is not None]
    if any(t.buffer.dtype != torch.bfloat16 for t in bufs):
        raise ValueError("matmul takes bfloat16 buffers")
    if K % 8 != 0 or N % 8 != 0:
        raise ValueError("matmul needs inner and outer dimensions that are multiples of 8 (16-byte rows)")
    # the rows of a decode step stream the weights once (b2kv_matmul_rows); everything else is a tiled GEMM
    rows_kernel = M <= 128 and K % 128 == 0 and N % 128 == 0
    stream = batch_op_begin(ctx)
    args = (A.buffer.data_ptr(), B.buffer.data_ptr(), None if bias is None else bias.buffer.data_ptr(),
            None if residual is None else residual.buffer.data_ptr(), C.buffer.data_ptr(), M, K, N,
            1 if activation == "gelu" else 0, dtype_code(torch.bfloat16))
    if rows_kernel:
        rc = _native.lib.b2kv_matmul_rows(*args, stream)
    else:
        rc = _native.lib.b2kv_matmul(*args, dev_status_ptr(ctx), stream)
    _native.check(rc)


@reference_op("qkv_project_append")
def qkv_project_append(ctx: GPUContext, cache: KVCache, layer_idx: int, x: GPUBuffer2D, wq: GPUBuffer2D,
                       wk: GPUBuffer2D, wv: GPUBuffer2D, q_out: GPUBuffer2D, advance: bool = True) -> None:
    """``q_out = x @ wq``; row ``current_len`` (or ``seq_lens[b]``) of the layer's K / V cache
    ``= x @ wk`` / ``x @ wv``; then, like ``kv_cache_update``, the length advances by one."""
    if layer_idx < 0 or layer_idx >= len(cache.layers):
        raise ValueError(f"layer_idx {layer_idx} out of range [0, {len(cache.layers)})")
    if cache.current_len >= cache.max_seq_len:
        raise ValueError(f"Cache is full: current_len={cache.current_len}, max_seq_len={cache.max_seq_len}")
    embedding_dim = cache.n_heads * cache.head_dim
    validate_buffer_shape_2d(x, (cache.batch_size, embedding_dim), "x")
    validate_buffer_shape_2d(q_out, (cache.batch_size, embedding_dim), "q_out")
    for name, w in (("wq", wq), ("wk", wk), ("wv", wv)):
        validate_buffer_shape_2d(w, (embedding_dim, embedding_dim), name)
    if cache.dtype != torch.bfloat16 or any(t.buffer.dtype != torch.bfloat16 for t in (x, wq, wk, wv, q_out)):
        raise ValueError("qkv_project_append takes bfloat16 buffers and a bfloat16 cache")
    if cache.block_table is not None:
        raise ValueError("qkv_project_append does not take a paged cache; project, then kv_cache_update")
    if cache.batch_size > 128 or embedding_dim % 128 != 0:
        raise ValueError("qkv_project_append needs batch_size <= 128 and an embedding_dim that is a multiple of 128")
    layer = cache.layers[layer_idx]
    s0, st, sh = cache_strides(cache)
    stream = batch_op_begin(ctx)
    rc = _native.lib.b2kv_qkv_append(x.buffer.data_ptr(), wq.buffer.data_ptr(), wk.buffer.data_ptr(), wv.buffer.data_ptr(),
                                     q_out.buffer.data_ptr(), layer.k_cache.buffer.data_ptr(),
                                     layer.v_cache.buffer.data_ptr(), _ptr(cache.seq_lens), cache.current_len,
                                     cache.batch_size, embedding_dim, cache.n_heads, cache.head_dim, cache.max_seq_len,
                                     s0, st, sh, dtype_code(cache.dtype), dev_status_ptr(ctx), stream)
    _native.check(rc)
    if advance:
        if cache.seq_lens is not None:
            # stream-ordered after the kernel, which read the old positions
            _native.check(_native.lib.b2kv_advance_lengths(cache.seq_lens.data_ptr(), cache.batch_size, 1, stream))
        cache.current_len += 1
