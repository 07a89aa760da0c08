"""One transformer decoder layer of a cached decode step, entirely on this library's kernels.

Follows the reference's block for the rows of one new token per sequence
(simple-llm/src/wgpu_backend.py:794-935: pre-LN attention with residual, pre-LN MLP with biases, GELU
``x * sigmoid(1.702 x)`` and residual), with the cached attention in place of the reference's full
recompute:

    h1 = layernorm(x; ln1)                                   layernorm
    q  = h1 @ wq ; cache row <- h1 @ wk, h1 @ wv             qkv_project_append   (lengths advance)
    a  = attention over the cache                            attention_with_kv_cache
    x2 = x + a @ wo                                          matmul(residual=)
    h2 = layernorm(x2; ln2)                                  layernorm
    m  = gelu(h2 @ w1 + b1)                                  matmul(bias=, activation="gelu")
    y  = x2 + m @ w2 + b2                                    matmul(bias=, residual=)

Seven launches per layer (eight with a ragged cache, whose device-side lengths a small kernel advances after the
projection), bfloat16 storage, fp32 arithmetic.  Each launch is scheduled ahead of the end of the one before it
and waits inside the kernel for that one to complete; the weight-streaming kernels ask for their first weight
tiles before that wait.  Every
layer owns its own ``KVCache`` object (``n_layers=1``), so that the lengths advance once per layer
step; a ragged (per-sequence length) cache works like a shared-length one.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .attention import flash_attention
from .kv_cache import attention_with_kv_cache
from .projection import matmul, qkv_project_append
from .step_tail import layernorm
from .types import GPUBuffer1D, GPUBuffer2D, GPUContext, KVCache


@dataclass
class DecoderLayerWeights:
    """bfloat16 parameters of one layer; matrices are ``[in, out]`` as the reference stores them."""

    ln1_gamma: GPUBuffer1D
    ln1_beta: GPUBuffer1D
    wq: GPUBuffer2D
    wk: GPUBuffer2D
    wv: GPUBuffer2D
    wo: GPUBuffer2D
    ln2_gamma: GPUBuffer1D
    ln2_beta: GPUBuffer1D
    w1: GPUBuffer2D
    b1: GPUBuffer1D
    w2: GPUBuffer2D
    b2: GPUBuffer1D


@dataclass
class DecoderLayerScratch:
    """Intermediate rows of a layer step, allocated once and reused by every layer and step."""

    h: GPUBuffer2D     # normalised rows (both layer norms)
    q: GPUBuffer2D
    a: GPUBuffer2D     # attention output
    x2: GPUBuffer2D
    m: GPUBuffer2D     # MLP hidden rows [B, 4E]


def _buf(ctx: GPUContext, rows: int, cols: int) -> GPUBuffer2D:
    t = torch.empty((rows, cols), dtype=torch.bfloat16, device=ctx.device)
    return GPUBuffer2D(buffer=t, shape=(rows, cols), size=rows * cols)


def decoder_layer_scratch(ctx: GPUContext, batch_size: int, embedding_dim: int, hidden_dim: Optional[int] = None) -> DecoderLayerScratch:
    hidden_dim = hidden_dim or 4 * embedding_dim
    mk = lambda c: _buf(ctx, batch_size, c)  # noqa: E731
    return DecoderLayerScratch(h=mk(embedding_dim), q=mk(embedding_dim), a=mk(embedding_dim), x2=mk(embedding_dim),
                               m=mk(hidden_dim))


def decoder_layer_step(ctx: GPUContext, cache: KVCache, x: GPUBuffer2D, w: DecoderLayerWeights, s: DecoderLayerScratch,
                       y: GPUBuffer2D) -> None:
    """Writes the layer's output rows for one new token per sequence into ``y`` and appends the token's
    K / V to ``cache`` (layer 0 of that cache object).  To be called between ``batch_begin`` and
    ``batch_commit``; seven operations are recorded."""
    layernorm(ctx, x, w.ln1_gamma, w.ln1_beta, s.h)
    qkv_project_append(ctx, cache, 0, s.h, w.wq, w.wk, w.wv, s.q)
    attention_with_kv_cache(ctx, cache, 0, s.q, s.a)
    matmul(ctx, s.a, w.wo, s.x2, residual=x)
    layernorm(ctx, s.x2, w.ln2_gamma, w.ln2_beta, s.h)
    matmul(ctx, s.h, w.w1, s.m, bias=w.b1, activation="gelu")
    matmul(ctx, s.m, w.w2, y, bias=w.b2, residual=s.x2)


@dataclass
class PromptLayerScratch:
    """Intermediate rows of a prompt-side layer pass (``batch_size * seq_len`` rows each)."""

    h: GPUBuffer2D     # normalised rows (both layer norms)
    q: GPUBuffer2D
    k: GPUBuffer2D
    v: GPUBuffer2D
    a: GPUBuffer2D     # attention output
    x2: GPUBuffer2D
    m: GPUBuffer2D     # MLP hidden rows [rows, 4E]


def prompt_layer_scratch(ctx: GPUContext, rows: int, embedding_dim: int, hidden_dim: Optional[int] = None) -> PromptLayerScratch:
    hidden_dim = hidden_dim or 4 * embedding_dim
    mk = lambda c: _buf(ctx, rows, c)  # noqa: E731
    return PromptLayerScratch(h=mk(embedding_dim), q=mk(embedding_dim), k=mk(embedding_dim), v=mk(embedding_dim),
                              a=mk(embedding_dim), x2=mk(embedding_dim), m=mk(hidden_dim))


def prompt_layer_step(ctx: GPUContext, cache: KVCache, x: GPUBuffer2D, w: DecoderLayerWeights, s: PromptLayerScratch,
                      y: GPUBuffer2D, batch_size: int, seq_len: int) -> None:
    """The same layer for a whole prompt: ``x`` and ``y`` are ``[batch_size * seq_len, E]``.  The reference's
    block as it stands (simple-llm/src/wgpu_backend.py:794-935: three projections, causal
    ``flash_attention``, output projection, MLP), with the prompt's K / V rows written into ``cache``
    (layer 0 of that cache object; its length becomes ``seq_len``) by the attention kernel.  Nine
    operations are recorded; the projections run on the tiled tensor-core GEMM."""
    layernorm(ctx, x, w.ln1_gamma, w.ln1_beta, s.h)
    matmul(ctx, s.h, w.wq, s.q)
    matmul(ctx, s.h, w.wk, s.k)
    matmul(ctx, s.h, w.wv, s.v)
    flash_attention(ctx, s.q, s.k, s.v, s.a, None, None, batch_size, seq_len, cache.n_heads, cache.head_dim,
                    cache=cache, layer_idx=0)
    matmul(ctx, s.a, w.wo, s.x2, residual=x)
    layernorm(ctx, s.x2, w.ln2_gamma, w.ln2_beta, s.h)
    matmul(ctx, s.h, w.w1, s.m, bias=w.b1, activation="gelu")
    matmul(ctx, s.m, w.w2, y, bias=w.b2, residual=s.x2)
