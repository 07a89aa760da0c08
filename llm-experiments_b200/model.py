"""A whole bfloat16 GPT decoder on this library's kernels, with a KV cache.

The reference's forward (simple-llm/src/wgpu_backend.py:728-990: embedding + positions, pre-LN blocks
:794-935, final LayerNorm, last-token extraction, output projection) recomputes the whole context for
every new token (simple-llm/src/generate.py:26-50).  Here the same model runs as a prompt pass followed by
cached decode steps, and every operation is one of this package's operators (no torch arithmetic):

    prompt   embedding -> L x prompt_layer_step (GEMMs, causal attention + cache write) ->
             extract_last_tokens -> layernorm -> matmul (logits) -> argmax
    step     embedding at each sequence's position -> L x decoder_layer_step (fused Q/K/V + append, cached
             attention, Wo, MLP) -> layernorm -> matmul (logits) -> argmax

Storage is bfloat16, arithmetic fp32.  Every layer owns a ``KVCache`` object of one layer, so lengths advance
once per layer step; positions of a decode step come from layer 0's lengths before it advances them.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch

from . import decode_layer
from .batch import batch_begin, batch_commit
from .decode_layer import DecoderLayerScratch, DecoderLayerWeights, PromptLayerScratch
from .kv_cache import kv_cache_create, kv_cache_reset
from .projection import matmul
from .step_tail import argmax, embedding, extract_last_tokens, layernorm
from .types import GPUBuffer1D, GPUBuffer2D, GPUContext, KVCache, KVCacheConfig


@dataclass
class DecoderConfig:
    vocab_size: int
    context_size: int
    embedding_dim: int
    n_heads: int
    n_layers: int

    @property
    def head_dim(self) -> int:
        return self.embedding_dim // self.n_heads


@dataclass
class DecoderWeights:
    """bfloat16 parameters; matrices are ``[in, out]`` as the reference stores them (wgpu_backend.py:129-212)."""

    embedding: GPUBuffer2D     # [vocab, E]
    pos_encoding: GPUBuffer2D  # [context, E], interleaved sin / cos (wgpu_backend.py:98-115)
    layers: List[DecoderLayerWeights]
    lnf_gamma: GPUBuffer1D
    lnf_beta: GPUBuffer1D
    out_proj: GPUBuffer2D      # [E, vocab]


@dataclass
class DecoderState:
    """Caches and the row buffers of a decode step, allocated once; prompt buffers are sized on first use."""

    cfg: DecoderConfig
    weights: DecoderWeights
    batch_size: int
    caches: List[KVCache]
    x: GPUBuffer2D
    y: GPUBuffer2D
    h: GPUBuffer2D
    logits: GPUBuffer2D
    scratch: DecoderLayerScratch
    prompt_rows: int = 0
    prompt_x: Optional[GPUBuffer2D] = None
    prompt_y: Optional[GPUBuffer2D] = None
    prompt_scratch: Optional[PromptLayerScratch] = None
    last: Optional[GPUBuffer2D] = field(default=None)


def _b2(t: torch.Tensor) -> GPUBuffer2D:
    return GPUBuffer2D(buffer=t, shape=tuple(t.shape), size=t.numel())


def _b1(t: torch.Tensor) -> GPUBuffer1D:
    return GPUBuffer1D(buffer=t, shape=tuple(t.shape), size=t.numel())


def positional_encoding(context_size: int, embedding_dim: int) -> np.ndarray:
    """Interleaved sin / cos table of simple-llm/src/wgpu_backend.py:98-115 (float32)."""
    position = np.arange(context_size)[:, None]
    div = np.exp(np.arange(0, embedding_dim, 2) * -(math.log(10000.0) / embedding_dim))
    pe = np.zeros((context_size, embedding_dim))
    pe[:, 0::2] = np.sin(position * div)
    pe[:, 1::2] = np.cos(position * div)
    return pe.astype(np.float32)


def weights_from_numpy(ctx: GPUContext, cfg: DecoderConfig, params: dict) -> DecoderWeights:
    """``params``: float arrays under the names of ``DecoderWeights`` / ``DecoderLayerWeights`` (``layers`` a list
    of dicts); values are rounded to bfloat16."""
    dev = ctx.device
    to = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(dev).to(torch.bfloat16)  # noqa: E731
    wrap = lambda a: (_b1 if np.ndim(a) == 1 else _b2)(to(a))  # noqa: E731
    layers = [DecoderLayerWeights(**{k: wrap(v) for k, v in layer.items()}) for layer in params["layers"]]
    return DecoderWeights(embedding=wrap(params["embedding"]), pos_encoding=wrap(params["pos_encoding"]), layers=layers,
                          lnf_gamma=wrap(params["lnf_gamma"]), lnf_beta=wrap(params["lnf_beta"]),
                          out_proj=wrap(params["out_proj"]))


def random_weights(ctx: GPUContext, cfg: DecoderConfig, seed: int = 0) -> DecoderWeights:
    """Random parameters drawn on the device (benchmarks): matrices N(0, 1 / fan_in), LayerNorm near identity."""
    dev, E, V = ctx.device, cfg.embedding_dim, cfg.vocab_size
    gen = torch.Generator(device=dev).manual_seed(seed)
    rnd = lambda shape, scale=1.0: (torch.randn(shape, generator=gen, device=dev) * scale).to(torch.bfloat16)  # noqa: E731

    def layer():
        return DecoderLayerWeights(
            ln1_gamma=_b1(rnd((E,), 0.1) + 1), ln1_beta=_b1(rnd((E,), 0.1)), wq=_b2(rnd((E, E), E ** -0.5)),
            wk=_b2(rnd((E, E), E ** -0.5)), wv=_b2(rnd((E, E), E ** -0.5)), wo=_b2(rnd((E, E), E ** -0.5)),
            ln2_gamma=_b1(rnd((E,), 0.1) + 1), ln2_beta=_b1(rnd((E,), 0.1)), w1=_b2(rnd((E, 4 * E), E ** -0.5)),
            b1=_b1(rnd((4 * E,), 0.1)), w2=_b2(rnd((4 * E, E), (4 * E) ** -0.5)), b2=_b1(rnd((E,), 0.1)))

    pos = torch.from_numpy(positional_encoding(cfg.context_size, E)).to(dev).to(torch.bfloat16)
    return DecoderWeights(embedding=_b2(rnd((V, E))), pos_encoding=_b2(pos), layers=[layer() for _ in range(cfg.n_layers)],
                          lnf_gamma=_b1(rnd((E,), 0.1) + 1), lnf_beta=_b1(rnd((E,), 0.1)),
                          out_proj=_b2(rnd((E, V), E ** -0.5)))


def decoder_state_create(ctx: GPUContext, cfg: DecoderConfig, weights: DecoderWeights, batch_size: int,
                         max_seq_len: Optional[int] = None, ragged: bool = False) -> DecoderState:
    if cfg.embedding_dim % cfg.n_heads != 0:
        raise ValueError(f"embedding_dim {cfg.embedding_dim} is not divisible by n_heads {cfg.n_heads}")
    T = cfg.context_size if max_seq_len is None else max_seq_len
    if T > cfg.context_size:
        raise ValueError(f"Sequence length {T} exceeds context size {cfg.context_size}")
    E, dev = cfg.embedding_dim, ctx.device
    caches = [kv_cache_create(ctx, KVCacheConfig(batch_size=batch_size, max_seq_len=T, n_layers=1, n_heads=cfg.n_heads,
                                                 head_dim=cfg.head_dim, dtype=torch.bfloat16, layout="bhtd",
                                                 ragged=ragged)) for _ in range(cfg.n_layers)]
    mk = lambda cols: _b2(torch.empty((batch_size, cols), dtype=torch.bfloat16, device=dev))  # noqa: E731
    ctx.config.flash_attn_max_head_dim = max(ctx.config.flash_attn_max_head_dim, cfg.head_dim)
    return DecoderState(cfg=cfg, weights=weights, batch_size=batch_size, caches=caches, x=mk(E), y=mk(E), h=mk(E),
                        logits=mk(cfg.vocab_size), scratch=decode_layer.decoder_layer_scratch(ctx, batch_size, E),
                        last=mk(E))


def decoder_state_reset(state: DecoderState) -> None:
    for cache in state.caches:
        kv_cache_reset(cache)


def launches_per_decode_step(cfg: DecoderConfig) -> int:
    """Kernels of this library launched by one ``decode_step``: the embedding, eight per layer (seven operations
    and the advance of the layer cache's device-side lengths), the final layernorm, the logits projection and the
    argmax."""
    return 1 + 8 * cfg.n_layers + 3


def _head(ctx: GPUContext, state: DecoderState, rows: GPUBuffer2D, next_ids: Optional[GPUBuffer1D]) -> None:
    """Final layernorm, logits projection and (optionally) the greedy choice for the ``[B, E]`` rows."""
    w = state.weights
    layernorm(ctx, rows, w.lnf_gamma, w.lnf_beta, state.h)
    matmul(ctx, state.h, w.out_proj, state.logits)
    if next_ids is not None:
        argmax(ctx, state.logits, next_ids)


def decode_step(ctx: GPUContext, state: DecoderState, token_ids: GPUBuffer1D,
                next_ids: Optional[GPUBuffer1D] = None) -> None:
    """One cached decode step for one new token per sequence (``token_ids`` int32 ``[B]``): appends the token's
    K / V to every layer's cache, leaves the logits in ``state.logits`` and, when ``next_ids`` is given, the
    greedy next token of every sequence there.  To be called between ``batch_begin`` and ``batch_commit``."""
    cfg, w, B = state.cfg, state.weights, state.batch_size
    first = state.caches[0]
    if first.current_len >= first.max_seq_len:
        raise ValueError(f"Cache is full: current_len={first.current_len}, max_seq_len={first.max_seq_len}")
    start = first.seq_lens if first.seq_lens is not None else first.current_len
    embedding(ctx, w.embedding, w.pos_encoding, token_ids, state.x, B, 1, start_pos=start)
    src, dst = state.x, state.y
    for cache, lw in zip(state.caches, w.layers):
        decode_layer.decoder_layer_step(ctx, cache, src, lw, state.scratch, dst)
        src, dst = dst, src
    _head(ctx, state, src, next_ids)


def prefill(ctx: GPUContext, state: DecoderState, prompt_ids: GPUBuffer1D, seq_len: int,
            next_ids: Optional[GPUBuffer1D] = None) -> None:
    """The prompt pass: ``prompt_ids`` int32 ``[B * seq_len]`` (every sequence ``seq_len`` tokens) fills every
    layer's cache (lengths become ``seq_len``) and leaves the last position's logits in ``state.logits``."""
    cfg, w, B = state.cfg, state.weights, state.batch_size
    rows, E = B * seq_len, cfg.embedding_dim
    if state.prompt_rows != rows:
        mk = lambda: _b2(torch.empty((rows, E), dtype=torch.bfloat16, device=ctx.device))  # noqa: E731
        state.prompt_x, state.prompt_y = mk(), mk()
        state.prompt_scratch = decode_layer.prompt_layer_scratch(ctx, rows, E)
        state.prompt_rows = rows
    embedding(ctx, w.embedding, w.pos_encoding, prompt_ids, state.prompt_x, B, seq_len)
    src, dst = state.prompt_x, state.prompt_y
    for cache, lw in zip(state.caches, w.layers):
        decode_layer.prompt_layer_step(ctx, cache, src, lw, state.prompt_scratch, dst, B, seq_len)
        src, dst = dst, src
    extract_last_tokens(ctx, src, state.last, B, seq_len, E)
    _head(ctx, state, state.last, next_ids)


class GraphedDecodeStep:
    """``decode_step`` captured once into a CUDA graph and replayed: one graph launch per generated token instead
    of ``launches_per_decode_step`` kernel launches issued from Python, which is what bounds small batches and
    short contexts (a step of a few hundred microseconds on the GPU against about ten microseconds of host work
    per launch).  The reference records its operations into one command encoder per batch and submits them
    together (simple-llm/src/gpu/gpu_ops.py:226-360); a replayed graph is the CUDA form of re-submitting that
    encoder.

    The state must keep its lengths on the device (``ragged=True``): the kernels of the captured step read the
    positions and lengths from there, so the same graph serves every step.  The host-side ``current_len`` of the
    caches, which sizes launches, is pinned to the cache capacity while capturing; ``step()`` advances it afterwards
    like the eager call does.  ``token_ids`` and ``next_ids`` are fixed buffers: write the step's tokens into
    ``token_ids`` (or pass ``feed_back=True`` to copy ``next_ids`` there on the device after every step).
    """

    def __init__(self, ctx: GPUContext, state: DecoderState, feed_back: bool = False):
        if any(c.seq_lens is None for c in state.caches):
            raise ValueError("a graphed decode step needs per-sequence lengths on the device (ragged=True)")
        self.ctx, self.state, self.feed_back = ctx, state, feed_back
        B = state.batch_size
        self.token_ids = _b1(torch.zeros(B, dtype=torch.int32, device=ctx.device))
        self.next_ids = _b1(torch.zeros(B, dtype=torch.int32, device=ctx.device))
        self.graph: Optional[torch.cuda.CUDAGraph] = None

    def _record(self) -> None:
        ctx, state = self.ctx, self.state
        batch_begin(ctx)
        decode_step(ctx, state, self.token_ids, self.next_ids)
        batch_commit(ctx)
        if self.feed_back:
            self.token_ids.buffer.copy_(self.next_ids.buffer)

    def capture(self) -> None:
        """Runs one eager step on a side stream (first-use set-up of every kernel, scratch allocations), restores the
        lengths it advanced, then captures the step.  Call it when at least one more token fits every cache."""
        ctx, state = self.ctx, self.state
        if ctx.config.check_device_status:
            raise ValueError("check_device_status synchronises in batch_commit, which a graph capture cannot hold")
        caches = state.caches
        cap = caches[0].max_seq_len
        keep_len = [c.current_len for c in caches]
        if max(keep_len) >= cap:
            raise ValueError(f"Cache is full: current_len={max(keep_len)}, max_seq_len={cap}")
        keep_dev = [c.seq_lens.clone() for c in caches]
        keep_tok = self.token_ids.buffer.clone()
        side = torch.cuda.Stream(device=ctx.device)
        side.wait_stream(torch.cuda.current_stream(ctx.device))
        with torch.cuda.stream(side):
            self._record()  # warm-up: nothing allocates or configures a kernel inside the capture
            for c, n, dev in zip(caches, keep_len, keep_dev):
                c.current_len = cap - 1  # launches sized for the longest sequence the cache can hold
                c.seq_lens.copy_(dev)
            self.token_ids.buffer.copy_(keep_tok)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                self._record()
            for c, dev in zip(caches, keep_dev):
                c.seq_lens.copy_(dev)  # (the capture itself ran nothing)
            self.token_ids.buffer.copy_(keep_tok)
        torch.cuda.current_stream(ctx.device).wait_stream(side)
        for c, n in zip(caches, keep_len):
            c.current_len = n
        self.graph = graph

    def step(self) -> None:
        """One decode step: replays the graph on torch's current stream and advances the host-side lengths."""
        if self.graph is None:
            self.capture()
        caches = self.state.caches
        if caches[0].current_len >= caches[0].max_seq_len:
            raise ValueError(f"Cache is full: current_len={caches[0].current_len}, max_seq_len={caches[0].max_seq_len}")
        self.graph.replay()
        for c in caches:
            c.current_len += 1


class CachedDecoder:
    """Batch-of-one adapter with the interface ``generate_text`` drives: ``cache``, ``context``,
    ``prefill(tokens) -> logits [1, vocab]`` and ``decode_step(token) -> logits [1, vocab]`` (float32)."""

    def __init__(self, ctx: GPUContext, cfg: DecoderConfig, weights: DecoderWeights):
        self.ctx, self.cfg = ctx, cfg
        self.state = decoder_state_create(ctx, cfg, weights, batch_size=1)
        self.context = cfg.context_size
        self.cache = _CacheGroup(self.state)
        self._tok = _b1(torch.zeros(1, dtype=torch.int32, device=ctx.device))

    def prefill(self, tokens: Sequence[int]) -> torch.Tensor:
        ids = _b1(torch.tensor(list(tokens), dtype=torch.int32, device=self.ctx.device))
        batch_begin(self.ctx)
        prefill(self.ctx, self.state, ids, len(tokens))
        batch_commit(self.ctx)
        return self.state.logits.buffer.float()

    def decode_step(self, token: int) -> torch.Tensor:
        self._tok.buffer.fill_(int(token))
        batch_begin(self.ctx)
        decode_step(self.ctx, self.state, self._tok)
        batch_commit(self.ctx)
        return self.state.logits.buffer.float()


class _CacheGroup:
    """What ``generate_text`` resets before a generation: every layer's cache at once."""

    def __init__(self, state: DecoderState):
        self.state = state
        self.seq_lens = None

    @property
    def current_len(self) -> int:
        return self.state.caches[0].current_len

    @current_len.setter
    def current_len(self, value: int) -> None:
        for cache in self.state.caches:
            cache.current_len = value
