"""CPU restatement of one decoder layer of a cached decode step (numpy).  TEST INFRASTRUCTURE ONLY.

Follows the reference's block (simple-llm/src/wgpu_backend.py:794-935) for one new token per sequence,
with the cached attention of oracle/kv_oracle.py, and rounds to bfloat16 where the kernels store
bfloat16 (every intermediate buffer), so that the comparison measures the kernels and not the
storage type.
"""
from __future__ import annotations

import numpy as np

from . import kv_oracle
from .step_tail_oracle import layernorm


def bf16_round(a):
    """float32 array rounded to the nearest bfloat16 (ties to even), returned as float32."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32).reshape(a.shape)


def decoder_layer_step(x, w, k_rows, v_rows, lens, n_heads):
    """x [B, E] float32 (bf16 values); w: dict of float32 arrays (bf16 values); k_rows / v_rows:
    per sequence, float32 [len_b, E] of the cached K / V rows (bf16 values); returns
    (y [B, E], new K rows [B, E], new V rows [B, E]) as float32 arrays of bf16 values."""
    B, E = x.shape
    D = E // n_heads
    h1 = bf16_round(layernorm(x, w["ln1_gamma"], w["ln1_beta"]))
    q, k_new, v_new = (bf16_round(t) for t in kv_oracle.qkv_project(h1, w["wq"], w["wk"], w["wv"]))
    a = np.zeros((B, E), dtype=np.float32)
    for b in range(B):
        K = np.concatenate([k_rows[b][: lens[b]], k_new[b : b + 1]], axis=0).reshape(-1, n_heads, D)
        V = np.concatenate([v_rows[b][: lens[b]], v_new[b : b + 1]], axis=0).reshape(-1, n_heads, D)
        qb = q[b].reshape(n_heads, D).astype(np.float64)
        s = np.einsum("hd,thd->ht", qb, K.astype(np.float64)) / np.sqrt(D)
        p = np.exp(s - s.max(axis=1, keepdims=True))
        p /= p.sum(axis=1, keepdims=True)
        a[b] = np.einsum("ht,thd->hd", p, V.astype(np.float64)).reshape(E)
    a = bf16_round(a)
    x2 = bf16_round(a.astype(np.float64) @ w["wo"].astype(np.float64) + x)
    h2 = bf16_round(layernorm(x2, w["ln2_gamma"], w["ln2_beta"]))
    z = h2.astype(np.float64) @ w["w1"].astype(np.float64) + w["b1"]
    m = bf16_round(z / (1.0 + np.exp(-1.702 * z)))
    y = bf16_round(m.astype(np.float64) @ w["w2"].astype(np.float64) + w["b2"] + x2)
    return y, k_new, v_new


def prompt_layer_step(x, w, B, N, n_heads):
    """The same layer over a whole prompt (simple-llm/src/wgpu_backend.py:794-935 as it stands: projections,
    causal attention as src/gpu_test.py:794-810, output projection, MLP).  x [B*N, E] float32 (bf16
    values); returns (y [B*N, E], K rows [B*N, E], V rows [B*N, E]) as float32 arrays of bf16 values."""
    E = x.shape[1]
    D = E // n_heads
    h1 = bf16_round(layernorm(x, w["ln1_gamma"], w["ln1_beta"]))
    q, k, v = (bf16_round(t) for t in kv_oracle.qkv_project(h1, w["wq"], w["wk"], w["wv"]))
    a = np.zeros_like(x)
    mask = np.tril(np.ones((N, N), dtype=bool))
    for b in range(B):
        rows = slice(b * N, (b + 1) * N)
        qb = q[rows].reshape(N, n_heads, D).astype(np.float64)
        kb = k[rows].reshape(N, n_heads, D).astype(np.float64)
        vb = v[rows].reshape(N, n_heads, D).astype(np.float64)
        sc = np.einsum("qhd,thd->hqt", qb, kb) / np.sqrt(D)
        sc = np.where(mask[None], sc, -1e10)
        pr = np.exp(sc - sc.max(axis=2, keepdims=True))
        pr /= pr.sum(axis=2, keepdims=True)
        a[rows] = np.einsum("hqt,thd->qhd", pr, vb).reshape(N, E)
    a = bf16_round(a)
    x2 = bf16_round(a.astype(np.float64) @ w["wo"].astype(np.float64) + x)
    h2 = bf16_round(layernorm(x2, w["ln2_gamma"], w["ln2_beta"]))
    z = h2.astype(np.float64) @ w["w1"].astype(np.float64) + w["b1"]
    m = bf16_round(z / (1.0 + np.exp(-1.702 * z)))
    y = bf16_round(m.astype(np.float64) @ w["w2"].astype(np.float64) + w["b2"] + x2)
    return y, k, v
