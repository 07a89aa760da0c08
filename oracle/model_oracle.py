"""CPU restatement of the whole bfloat16 decoder with a KV cache (numpy).  TEST INFRASTRUCTURE ONLY.

Stacks the layer restatements of oracle/decode_layer_oracle.py (which follow the reference's block,
simple-llm/src/wgpu_backend.py:794-935) between the reference's embedding with positions added
(simple-llm/src/gpu/gpu_kernels.py:384-449, wgpu_backend.py:98-115) and its final LayerNorm, last-token
extraction and output projection (wgpu_backend.py:937-977), rounding to bfloat16 wherever the kernels
store bfloat16, so that a comparison measures the kernels and not the storage type.  The cache here is
the plain list of every sequence's K / V rows per layer.
"""
from __future__ import annotations

import numpy as np

from .decode_layer_oracle import bf16_round, decoder_layer_step, prompt_layer_step
from .step_tail_oracle import layernorm


def _head(params, rows):
    h = bf16_round(layernorm(rows, params["lnf_gamma"], params["lnf_beta"]))
    return bf16_round(h.astype(np.float64) @ params["out_proj"].astype(np.float64))


def prefill(params, prompt_ids, B, N, n_heads):
    """prompt_ids int [B*N] -> (logits [B, vocab] of the last position, cache: per layer (K rows, V rows), each a
    list of B float32 arrays [N, E])."""
    ids = np.asarray(prompt_ids).reshape(B * N)
    pos = np.tile(np.arange(N), B)
    x = bf16_round(params["embedding"][ids] + params["pos_encoding"][pos])
    cache = []
    for w in params["layers"]:
        x, k, v = prompt_layer_step(x, w, B, N, n_heads)
        cache.append(([k[b * N:(b + 1) * N].copy() for b in range(B)], [v[b * N:(b + 1) * N].copy() for b in range(B)]))
    last = x.reshape(B, N, -1)[:, -1, :]
    return _head(params, last), cache


def decode_step(params, token_ids, cache, n_heads):
    """One new token per sequence; appends its K / V rows to `cache` in place and returns logits [B, vocab]."""
    ids = np.asarray(token_ids)
    B = len(ids)
    lens = [len(cache[0][0][b]) for b in range(B)]
    x = bf16_round(params["embedding"][ids] + params["pos_encoding"][np.asarray(lens)])
    for w, (k_rows, v_rows) in zip(params["layers"], cache):
        x, k_new, v_new = decoder_layer_step(x, w, k_rows, v_rows, lens, n_heads)
        for b in range(B):
            k_rows[b] = np.concatenate([k_rows[b], k_new[b:b + 1]], axis=0)
            v_rows[b] = np.concatenate([v_rows[b], v_new[b:b + 1]], axis=0)
    return _head(params, x)
