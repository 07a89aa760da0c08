"""The head and the tail of a cached generation step behind the reference's operator names.

Mirrors simple-llm/src/gpu/gpu_pass_forward.py: ``embedding`` (:84-137), ``layernorm`` (:140-176),
``extract_last_tokens`` (:285-328) and ``softmax`` (:462-494): same positional arguments, the same checks
and ``ValueError`` texts, ``None`` returned, outputs written in place, recorded between ``batch_begin`` and
``batch_commit``.  Buffers are fp32 like the reference's; ``embedding``, ``layernorm``,
``extract_last_tokens`` and ``argmax`` also take bfloat16 buffers (a bf16 decoder's hidden rows and logits).
``argmax`` is an extension: the greedy choice of the next token stays on the device (the reference reads the
probabilities back and samples on the host, src/generate.py:8-72).
"""
from __future__ import annotations

import torch

from . import _native
from .batch import batch_op_begin, dev_status_ptr, reference_op, validate_buffer_shape_1d, validate_buffer_shape_2d
from .types import GPUBuffer1D, GPUBuffer2D, GPUContext

_DTYPE_CODES = {torch.float32: _native.DTYPE_F32, torch.bfloat16: _native.DTYPE_BF16}


@reference_op("embedding")
def embedding(ctx: GPUContext, embedding_table: GPUBuffer2D, pos_encoding: GPUBuffer2D, input_ids: GPUBuffer1D,
              output: GPUBuffer2D, batch_size: int, seq_len: int, start_pos=0) -> None:
    """``output[b*seq_len + s] = embedding_table[input_ids[b*seq_len + s]] + pos_encoding[start + s]``.
    ``start_pos`` is an extension for cached decoding (the reference always starts at 0): an int, or an int32
    device tensor of ``batch_size`` positions (a ragged cache's ``seq_lens``)."""
    if batch_size <= 0 or seq_len <= 0:
        raise ValueError(f"Invalid batch_size={batch_size} or seq_len={seq_len}")
    vocab_size, embedding_dim = embedding_table.shape
    context_size, embedding_dim2 = pos_encoding.shape
    if embedding_dim != embedding_dim2:
        raise ValueError(
            f"Embedding dimension mismatch: table has {embedding_dim}, "
            f"pos_encoding has {embedding_dim2}"
        )
    if seq_len > context_size:
        raise ValueError(f"Sequence length {seq_len} exceeds context size {context_size}")
    total_tokens = batch_size * seq_len
    validate_buffer_shape_1d(input_ids, total_tokens, "input_ids")
    validate_buffer_shape_2d(output, (total_tokens, embedding_dim), "output")
    dtype = embedding_table.buffer.dtype
    if dtype not in _DTYPE_CODES or pos_encoding.buffer.dtype != dtype or output.buffer.dtype != dtype:
        raise ValueError("embedding_table, pos_encoding and output must share one dtype (float32 or bfloat16)")
    if input_ids.buffer.dtype != torch.int32:
        raise ValueError(f"input_ids must be int32, got {input_ids.buffer.dtype}")
    if embedding_dim % 8 != 0:
        raise ValueError("embedding needs an embedding_dim that is a multiple of 8 (16-byte rows)")
    seq_pos, pos0 = None, 0
    if isinstance(start_pos, torch.Tensor):
        if start_pos.dtype != torch.int32 or start_pos.numel() != batch_size:
            raise ValueError("start_pos must hold batch_size int32 positions")
        seq_pos = start_pos.data_ptr()
    else:
        pos0 = int(start_pos)
        if pos0 < 0 or pos0 + seq_len > context_size:
            raise ValueError(f"Sequence length {pos0 + seq_len} exceeds context size {context_size}")
    stream = batch_op_begin(ctx)
    _native.check(_native.lib.b2kv_embedding(embedding_table.buffer.data_ptr(), pos_encoding.buffer.data_ptr(),
                                             input_ids.buffer.data_ptr(), seq_pos, pos0, output.buffer.data_ptr(),
                                             batch_size, seq_len, embedding_dim, vocab_size, context_size,
                                             _DTYPE_CODES[dtype], dev_status_ptr(ctx), stream))


def _f32(buf, name: str) -> int:
    if buf.buffer.dtype != torch.float32:
        raise ValueError(f"{name} must be float32, got {buf.buffer.dtype}")
    if not buf.buffer.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    return buf.buffer.data_ptr()


@reference_op("layernorm")
def layernorm(ctx: GPUContext, input_buf: GPUBuffer2D, gamma: GPUBuffer1D, beta: GPUBuffer1D,
              output: GPUBuffer2D) -> None:
    n_elements, size = input_buf.shape
    if n_elements == 0 or size == 0:
        raise ValueError(f"Invalid input_buf shape: {(n_elements, size)}")
    validate_buffer_shape_1d(gamma, size, "gamma")
    validate_buffer_shape_1d(beta, size, "beta")
    validate_buffer_shape_2d(output, (n_elements, size), "output")
    bufs = (input_buf, gamma, beta, output)
    if all(t.buffer.dtype == torch.bfloat16 for t in bufs):
        # extension: bf16 rows and parameters, fp32 arithmetic
        if not all(t.buffer.is_contiguous() for t in bufs):
            raise ValueError("layernorm buffers must be contiguous")
        fn, ptrs = _native.lib.b2kv_layernorm_bf16, tuple(t.buffer.data_ptr() for t in bufs)
    else:
        fn = _native.lib.b2kv_layernorm
        ptrs = (_f32(input_buf, "input_buf"), _f32(gamma, "gamma"), _f32(beta, "beta"), _f32(output, "output"))
    stream = batch_op_begin(ctx)
    _native.check(fn(*ptrs, n_elements, size, float(ctx.config.layernorm_epsilon), stream))


@reference_op("extract_last_tokens")
def extract_last_tokens(ctx: GPUContext, input_buf: GPUBuffer2D, output: GPUBuffer2D, batch_size: int, seq_len: int,
                        embedding_dim: int) -> None:
    if batch_size <= 0 or seq_len <= 0 or embedding_dim <= 0:
        raise ValueError(
            f"Invalid dimensions: batch_size={batch_size}, seq_len={seq_len}, "
            f"embedding_dim={embedding_dim}"
        )
    total_tokens = batch_size * seq_len
    validate_buffer_shape_2d(input_buf, (total_tokens, embedding_dim), "input_buf")
    validate_buffer_shape_2d(output, (batch_size, embedding_dim), "output")
    if input_buf.buffer.dtype == torch.bfloat16 and output.buffer.dtype == torch.bfloat16:
        # extension: bf16 rows
        if not (input_buf.buffer.is_contiguous() and output.buffer.is_contiguous()) or embedding_dim % 8 != 0:
            raise ValueError("bfloat16 extract_last_tokens needs contiguous buffers and embedding_dim % 8 == 0")
        fn, src, dst = _native.lib.b2kv_extract_last_tokens_bf16, input_buf.buffer.data_ptr(), output.buffer.data_ptr()
    else:
        fn, src, dst = _native.lib.b2kv_extract_last_tokens, _f32(input_buf, "input_buf"), _f32(output, "output")
    stream = batch_op_begin(ctx)
    _native.check(fn(src, dst, batch_size, seq_len, embedding_dim, stream))


@reference_op("softmax")
def softmax(ctx: GPUContext, logits: GPUBuffer2D, probs: GPUBuffer2D) -> None:
    if logits.shape != probs.shape:
        raise ValueError(f"Softmax shape mismatch: logits {logits.shape} != probs {probs.shape}")
    batch_size, vocab_size = logits.shape
    src, dst = _f32(logits, "logits"), _f32(probs, "probs")
    stream = batch_op_begin(ctx)
    _native.check(_native.lib.b2kv_softmax(src, dst, batch_size, vocab_size, stream))


@reference_op("argmax")
def argmax(ctx: GPUContext, values: GPUBuffer2D, indices: GPUBuffer1D) -> None:
    """``indices[b]`` = index of the largest value of row b (int32; the lowest index among equals)."""
    batch_size, vocab_size = values.shape
    validate_buffer_shape_1d(indices, batch_size, "indices")
    if indices.buffer.dtype != torch.int32:
        raise ValueError(f"indices must be int32, got {indices.buffer.dtype}")
    if values.buffer.dtype == torch.bfloat16:
        if not values.buffer.is_contiguous():
            raise ValueError("values must be contiguous")
        fn, src = _native.lib.b2kv_argmax_bf16, values.buffer.data_ptr()
    else:
        fn, src = _native.lib.b2kv_argmax, _f32(values, "values")
    stream = batch_op_begin(ctx)
    _native.check(fn(src, indices.buffer.data_ptr(), batch_size, vocab_size, stream))
