"""A small GPT decoder that drives the KV-cache path the way model code would.

The reference has no cached generation loop (its generate.py recomputes the whole context per
token, simple-llm/src/generate.py:28-49); this module is the missing caller: prompt prefill
through ``flash_attention`` fused with the cache write, then token-by-token decode through
``kv_cache_update`` and ``attention_with_kv_cache``; LayerNorm, the last-token extraction and the
greedy argmax run through the step-tail operators (``layernorm``, ``extract_last_tokens``,
``argmax``).  What is left (embedding, the projections, the MLP) is plain torch, standing in for
the reference's other forward ops; model structure and initialisation follow
simple-llm/src/wgpu_backend.py:98-212 and :794-977 (pre-LN blocks, interleaved sin/cos positions,
GELU = x*sigmoid(1.702x), separate output projection, LayerNorm epsilon 1e-5).

``kv_cache_update`` advances ``current_len`` on every call (reference behaviour), so the layer
loop passes ``advance=False`` for all layers but the last.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import numpy as np
import torch

from . import gpu
from .types import GPUBuffer2D, GPUContext

LN_EPS = 1e-5


def init_params(vocab: int = 256, E: int = 256, n_layers: int = 4, context: int = 256, seed: int = 0) -> Dict:
    """``randn * 0.02`` in the reference's draw order (embedding; wq wk wv wo w1 w2 per layer;
    output projection) from the legacy numpy generator; biases zero, LayerNorm affine identity."""
    rs = np.random.RandomState(seed)
    draw = lambda *shape: (rs.randn(*shape).astype(np.float32) * np.float32(0.02))  # noqa: E731
    params = {"embedding": draw(vocab, E), "layers": []}
    for _ in range(n_layers):
        layer = {}
        for name, shape in [("wq", (E, E)), ("wk", (E, E)), ("wv", (E, E)), ("wo", (E, E)), ("w1", (E, 4 * E)),
                            ("w2", (4 * E, E))]:
            layer[name] = draw(*shape)
        params["layers"].append(layer)
    params["out_proj"] = draw(E, vocab)
    position = np.arange(context)[:, None]
    div = np.exp(np.arange(0, E, 2) * -(np.log(10000.0) / E))
    pe = np.zeros((context, E))
    pe[:, 0::2] = np.sin(position * div)
    pe[:, 1::2] = np.cos(position * div)
    params["pos"] = pe.astype(np.float32)
    return params


def _gelu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(1.702 * x)


def _wrap(t: torch.Tensor) -> GPUBuffer2D:
    return GPUBuffer2D(buffer=t, shape=tuple(t.shape), size=t.numel())


class TinyGPT:
    """Batch-of-one greedy decoder with a KV cache (fp32, reference cache layout)."""

    def __init__(self, ctx: GPUContext, params: Dict, n_heads: int, context: int):
        self.ctx = ctx
        dev = ctx.device
        self.n_heads = n_heads
        self.E = params["embedding"].shape[1]
        self.D = self.E // n_heads
        self.context = context
        to = lambda a: torch.from_numpy(a).to(dev)  # noqa: E731
        self.embedding, self.pos, self.out_proj = to(params["embedding"]), to(params["pos"]), to(params["out_proj"])
        self.layers = [{k: to(v) for k, v in layer.items()} for layer in params["layers"]]
        # LayerNorm scale 1 and shift 0, as the reference initialises them (wgpu_backend.py:129-212)
        self.ln_gamma = gpu.gpu_buffer_1d_create(ctx, self.E, torch.ones(self.E))
        self.ln_beta = gpu.gpu_buffer_1d_create(ctx, self.E, torch.zeros(self.E))
        self.next_id = gpu.gpu_buffer_1d_create(ctx, 1, dtype=torch.int32)
        ctx.config.layernorm_epsilon = LN_EPS
        self.cache = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=1, max_seq_len=context,
                                                                n_layers=len(self.layers), n_heads=n_heads,
                                                                head_dim=self.D))

    def _ln(self, x: torch.Tensor) -> torch.Tensor:
        x = x.contiguous()
        out = torch.empty_like(x)
        gpu.batch_begin(self.ctx)
        gpu.layernorm(self.ctx, _wrap(x), self.ln_gamma, self.ln_beta, _wrap(out))
        gpu.batch_commit(self.ctx)
        return out

    def greedy(self, logits: torch.Tensor) -> int:
        """Index of the largest logit of row 0, chosen on the device."""
        gpu.batch_begin(self.ctx)
        gpu.argmax(self.ctx, _wrap(logits.contiguous()), self.next_id)
        gpu.batch_commit(self.ctx)
        return int(self.next_id.buffer.item())

    def prefill(self, prompt: List[int]) -> torch.Tensor:
        """Runs the prompt through the model, fills the cache, returns the last position's logits."""
        ctx, N = self.ctx, len(prompt)
        tok = torch.tensor(prompt, device=ctx.device, dtype=torch.long)
        x = self.embedding[tok] + self.pos[:N]
        ctx.config.flash_attn_max_head_dim = max(ctx.config.flash_attn_max_head_dim, self.D)
        for li, layer in enumerate(self.layers):
            h = self._ln(x)
            q, k, v = (h @ layer["wq"]).contiguous(), (h @ layer["wk"]).contiguous(), (h @ layer["wv"]).contiguous()
            o = torch.empty_like(q)
            gpu.batch_begin(ctx)
            gpu.flash_attention(ctx, _wrap(q), _wrap(k), _wrap(v), _wrap(o), None, None, 1, N, self.n_heads, self.D,
                                cache=self.cache, layer_idx=li)
            gpu.batch_commit(ctx)
            x = x + o @ layer["wo"]
            h = self._ln(x)
            x = x + _gelu(h @ layer["w1"]) @ layer["w2"]
        last_row = torch.empty((1, self.E), dtype=x.dtype, device=x.device)
        gpu.batch_begin(ctx)
        gpu.extract_last_tokens(ctx, _wrap(x.contiguous()), _wrap(last_row), 1, N, self.E)
        gpu.batch_commit(ctx)
        return self._ln(last_row) @ self.out_proj

    def decode_step(self, token: int) -> torch.Tensor:
        """Appends one token at position ``current_len`` and returns its logits ``[1, vocab]``."""
        ctx, cache = self.ctx, self.cache
        pos = cache.current_len
        x = self.embedding[token : token + 1] + self.pos[pos : pos + 1]
        last = len(self.layers) - 1
        for li, layer in enumerate(self.layers):
            h = self._ln(x)
            q, k, v = (h @ layer["wq"]).contiguous(), (h @ layer["wk"]).contiguous(), (h @ layer["wv"]).contiguous()
            o = torch.empty_like(q)
            gpu.batch_begin(ctx)
            gpu.kv_cache_update(ctx, cache, li, _wrap(k), _wrap(v), advance=False)
            cache.current_len = pos + 1  # attend over the row just written
            gpu.attention_with_kv_cache(ctx, cache, li, _wrap(q), _wrap(o))
            gpu.batch_commit(ctx)
            if li != last:
                cache.current_len = pos  # the next layer writes at the same position
            x = x + o @ layer["wo"]
            h = self._ln(x)
            x = x + _gelu(h @ layer["w1"]) @ layer["w2"]
        return self._ln(x) @ self.out_proj

    def generate(self, prompt: List[int], n_new: int) -> Tuple[List[int], torch.Tensor]:
        """Greedy decode; returns (all tokens, logits of every generated position ``[n_new, vocab]``)."""
        gpu.kv_cache_reset(self.cache)
        tokens = list(prompt)
        logits = self.prefill(tokens)
        all_logits = [logits]
        tokens.append(self.greedy(logits))
        for _ in range(n_new - 1):
            logits = self.decode_step(tokens[-1])
            all_logits.append(logits)
            tokens.append(self.greedy(logits))
        return tokens, torch.cat(all_logits, dim=0)
