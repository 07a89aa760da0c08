"""The tail of a cached generation step behind the reference's operator names.

Mirrors simple-llm/src/gpu/gpu_pass_forward.py: ``layernorm`` (:140-176), ``extract_last_tokens``
(:285-328) and ``softmax`` (:462-494): same positional arguments, the same checks and ``ValueError``
texts, ``None`` returned, outputs written in place, recorded between ``batch_begin`` and
``batch_commit``.  Buffers are fp32 like the reference's.  ``argmax`` is an extension: the greedy
choice of the next token stays on the device (the reference reads the probabilities back and
samples on the host, src/generate.py:8-72).
"""
from __future__ import annotations

import torch

from . import _native
from .batch import batch_op_begin, reference_op, validate_buffer_shape_1d, validate_buffer_shape_2d
from .types import GPUBuffer1D, GPUBuffer2D, GPUContext


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
    src, dst = _f32(input_buf, "input_buf"), _f32(output, "output")
    stream = batch_op_begin(ctx)
    _native.check(_native.lib.b2kv_extract_last_tokens(src, dst, batch_size, seq_len, embedding_dim, stream))


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
    src = _f32(values, "values")
    stream = batch_op_begin(ctx)
    _native.check(_native.lib.b2kv_argmax(src, indices.buffer.data_ptr(), batch_size, vocab_size, stream))
