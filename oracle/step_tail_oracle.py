"""CPU restatement of the tail of a generation step (numpy, fp32).  TEST INFRASTRUCTURE ONLY:
the product never imports this module.

Follows the reference's WGSL kernels in simple-llm/src/gpu/gpu_kernels.py, in their order of
operations, and is pinned against the reference's own seeded test recipes
(tests/golden/reference_recipes.npz, made by tests/golden/make_golden.py from
simple-llm/src/gpu_test.py:519-574, :1644-1729 and :2057-2110).
"""
from __future__ import annotations

import numpy as np

# (n_elements, size) of gpu_test.py:521-527
LAYERNORM_RECIPE_SHAPES = [(32, 768), (1, 512), (128, 1024), (1024, 64), (10, 100)]
# (batch_size, vocab_size, transform) of gpu_test.py:1647-1657
SOFTMAX_RECIPES = [
    (2, 10, None), (4, 100, None), (2, 1000, None), (1, 50000, None),
    (2, 100, "plus50"), (2, 100, "minus50"), (2, 100, "times100"), (2, 100, "zeros"),
]
# (batch_size, seq_len, emb_dim) of gpu_test.py:2059-2066
EXTRACT_RECIPE_SHAPES = [(1, 10, 64), (4, 32, 128), (8, 64, 256), (32, 16, 512), (2, 128, 768), (1, 1, 64)]
# rows of a recipe's output kept in the fixture (all rows when there are fewer)
GOLDEN_ROWS = 8


def recipe_layernorm_inputs(n_elements, size, seed=42):
    """gpu_test.py:536-539."""
    np.random.seed(seed)
    x = np.random.randn(n_elements, size).astype(np.float32)
    gamma = np.random.randn(size).astype(np.float32)
    beta = np.random.randn(size).astype(np.float32)
    return x, gamma, beta


def recipe_softmax_inputs(batch_size, vocab_size, transform, seed=42):
    """gpu_test.py:1674-1678 with the transforms of :1652-1656."""
    np.random.seed(seed)
    x = np.random.randn(batch_size, vocab_size).astype(np.float32)
    if transform == "plus50":
        x = x + 50
    elif transform == "minus50":
        x = x - 50
    elif transform == "times100":
        x = x * 100
    elif transform == "zeros":
        x = np.zeros_like(x)
    return x.astype(np.float32)


def recipe_extract_inputs(batch_size, seq_len, emb_dim, seed=42):
    """gpu_test.py:2076-2078."""
    np.random.seed(seed)
    return np.random.randn(batch_size * seq_len, emb_dim).astype(np.float32)


def layernorm(x, gamma, beta, eps=1e-5):
    """gpu_kernels.py:196-245: mean, then the mean of (x - mean)^2, then the affine map."""
    x = np.asarray(x, dtype=np.float32)
    size = np.float32(x.shape[-1])
    mean = x.sum(axis=-1, keepdims=True, dtype=np.float32) / size
    diff = x - mean
    var = (diff * diff).sum(axis=-1, keepdims=True, dtype=np.float32) / size
    inv_std = np.float32(1.0) / np.sqrt(var + np.float32(eps))
    return (diff * inv_std * np.asarray(gamma, np.float32) + np.asarray(beta, np.float32)).astype(np.float32)


def extract_last_tokens(x, batch_size, seq_len, emb_dim):
    """gpu_kernels.py:879-884: row b*seq_len + seq_len - 1."""
    return np.ascontiguousarray(np.asarray(x).reshape(batch_size, seq_len, emb_dim)[:, -1, :])


def softmax(x):
    """gpu_kernels.py:946-988: maximum starting from -1e10, exp(x - max) / sum."""
    x = np.asarray(x, dtype=np.float32)
    m = np.maximum(x.max(axis=-1, keepdims=True), np.float32(-1e10))
    e = np.exp(x - m, dtype=np.float32)
    return (e / e.sum(axis=-1, keepdims=True, dtype=np.float32)).astype(np.float32)


def argmax(x):
    return np.argmax(np.asarray(x), axis=-1).astype(np.int32)
