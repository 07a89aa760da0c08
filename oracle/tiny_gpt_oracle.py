"""CPU oracle of the tiny GPT decoder used as the end-to-end correctness case.  TEST ONLY.

A numpy restatement of the reference's transformer forward WITHOUT any cache: the whole
context is recomputed for every new token, which is what the reference's generation does today
(simple-llm/src/generate.py:28-49; forward structure simple-llm/src/wgpu_backend.py:794-977).

* parameters: drawn as the reference draws them (wgpu_backend.py:129-212): ``randn * 0.02`` for the
  embedding, then per layer wq, wk, wv, wo, w1, w2, then the output projection; biases zero,
  LayerNorm gamma one and beta zero.  The reference does not seed; this case uses the legacy
  numpy generator seeded with 0.
* positions: interleaved sin / cos (wgpu_backend.py:98-115).
* block: pre-LN attention + residual, pre-LN MLP (W1 + b1, GELU, W2 + b2) + residual; final LN;
  separate output projection ``[E, vocab]``.  LayerNorm epsilon 1e-5
  (simple-llm/src/gpu/gpu_types.py:197); GELU is ``x * sigmoid(1.702 x)``
  (simple-llm/src/gpu/gpu_kernels.py:285-293).
* attention: dense causal softmax (kv_oracle.flash_attention_dense).
* unlike generate.py:33-35 the context is not left-padded with token 0: padding is an artefact of
  the fixed-size uncached forward, not part of the cache path.
"""
from __future__ import annotations

import numpy as np

from . import kv_oracle

LN_EPS = 1e-5


def init_params(vocab=256, E=256, n_layers=4, context=256, seed=0):
    rs = np.random.RandomState(seed)
    draw = lambda *shape: (rs.randn(*shape).astype(np.float32) * np.float32(0.02))  # noqa: E731
    params = {"embedding": draw(vocab, E), "layers": []}
    for _ in range(n_layers):
        params["layers"].append({k: draw(*shape) for k, shape in
                                 [("wq", (E, E)), ("wk", (E, E)), ("wv", (E, E)), ("wo", (E, E)),
                                  ("w1", (E, 4 * E)), ("w2", (4 * E, E))]})
    params["out_proj"] = draw(E, vocab)
    position = np.arange(context)[:, None]
    div = np.exp(np.arange(0, E, 2) * -(np.log(10000.0) / E))
    pe = np.zeros((context, E))
    pe[:, 0::2] = np.sin(position * div)
    pe[:, 1::2] = np.cos(position * div)
    params["pos"] = pe.astype(np.float32)
    return params


def layernorm(x):
    mu = x.mean(axis=-1, keepdims=True)
    var = ((x - mu) ** 2).mean(axis=-1, keepdims=True)
    return ((x - mu) / np.sqrt(var + LN_EPS)).astype(np.float32)


def gelu(x):
    return (x / (1.0 + np.exp(-1.702 * x))).astype(np.float32)


def forward_uncached(params, tokens, n_heads):
    """tokens int [N] -> logits float32 [N, vocab] (batch of one)."""
    N = len(tokens)
    E = params["embedding"].shape[1]
    D = E // n_heads
    x = params["embedding"][tokens] + params["pos"][:N]
    for layer in params["layers"]:
        h = layernorm(x)
        q, k, v = h @ layer["wq"], h @ layer["wk"], h @ layer["wv"]
        a = kv_oracle.flash_attention_dense(q[None], k[None], v[None], 1, N, n_heads, D)[0]
        x = x + a @ layer["wo"]
        h = layernorm(x)
        x = x + gelu(h @ layer["w1"]) @ layer["w2"]
    return (layernorm(x) @ params["out_proj"]).astype(np.float32)


def greedy_generate_uncached(params, prompt, n_new, n_heads):
    """Greedy decode by full recomputation; returns (tokens list, last-position logits per step)."""
    tokens = list(int(t) for t in prompt)
    step_logits = []
    for _ in range(n_new):
        logits = forward_uncached(params, np.asarray(tokens), n_heads)[-1]
        step_logits.append(logits)
        tokens.append(int(np.argmax(logits)))
    return tokens, np.stack(step_logits)
