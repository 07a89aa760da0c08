"""CPU oracle (numpy) for the KV-cache attention path.  TEST INFRASTRUCTURE ONLY.

This module restates, on the CPU, the arithmetic of the reference's KV-cache
path so that the CUDA kernels can be checked against it.  Nothing in the
product package may import it: only tests, the smoke check and the
``cpu_baseline`` / ``--impl reference`` legs of the benchmark do.

What each function follows (paths inside the reference project):

* ``kv_update``            simple-llm/src/gpu/gpu_kernels.py:2784-2796 (index math)
* ``decode_attention``     simple-llm/src/gpu_test.py:2328-2367 (the numpy loop the
                           reference's own test compares its kernel with)
* ``decode_attention_shader_order``
                           simple-llm/src/gpu/gpu_kernels.py:2846-2936 (the WGSL
                           shader's own order of operations: scale after the dot,
                           max seeded with -1e10, weight = exp/sum before the V sum)
* ``flash_attention_dense`` simple-llm/src/gpu_test.py:794-810 (dense causal softmax
                           with masked scores set to -1e10)
* ``flash_attention_tiled`` simple-llm/src/gpu/gpu_kernels.py:621-768 (tiled online
                           softmax, including the L / M statistics and their layout
                           ``[b*N*H + row*H + h]`` and the ``max(l, 1e-8)`` guard)

Parity pin: the reference stores no golden output files.  Its tests pin the path
by seeded recipes (``np.random.seed(42)`` + ``randn`` in a fixed order) and compare
with reference math written inside the test.  ``tests/golden/make_golden.py`` runs
those very lines of the reference's test file (the numpy ones, executed from the
reference tree) on the recipes' inputs and stores the outputs; the oracle is
checked against these fixtures in ``tests/test_oracle.py``.  Extensions that the
reference does not have (bf16 storage, per-sequence lengths, paged block tables,
lengths beyond 256, prefill fused with the cache write) are defined by this oracle
on the logical ``[B, T, H, D]`` view; for them parity is unpinned by the reference.
"""

from __future__ import annotations

import numpy as np

MASK_VALUE = np.float32(-1e10)  # gpu_kernels.py:593 and :2872


# ----------------------------------------------------------------------------
# bf16 storage helpers (the reference is fp32 only; bf16 is an extension)
# ----------------------------------------------------------------------------


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round float32 to bfloat16 (round-to-nearest-even), returned as uint16 bits."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounding = ((u >> 16) & 1) + np.uint32(0x7FFF)
    out = ((u + rounding) >> 16).astype(np.uint16)
    nan = np.isnan(x)
    if np.any(nan):
        out = np.where(nan, np.uint16(0x7FC0), out)
    return out


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    """Widen bfloat16 bits (uint16) to float32 exactly."""
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def round_to_bf16(x: np.ndarray) -> np.ndarray:
    """float32 values rounded to the nearest bf16, kept as float32."""
    return bf16_bits_to_f32(f32_to_bf16_bits(x))


# ----------------------------------------------------------------------------
# cache append / gather
# ----------------------------------------------------------------------------


def kv_update(k_cache, v_cache, new_k, new_v, pos, batch_size, max_seq_len):
    """Copy ``new_k/new_v [B, E]`` into rows ``b*T_max + pos`` of ``[B*T_max, E]`` caches.

    ``pos`` is one int (the reference's single ``current_len``) or an int array [B]
    (per-sequence positions, an extension).  In place; returns nothing.
    """
    pos = np.broadcast_to(np.asarray(pos, dtype=np.int64), (batch_size,))
    for b in range(batch_size):
        row = b * max_seq_len + int(pos[b])
        k_cache[row, :] = new_k[b, :]
        v_cache[row, :] = new_v[b, :]


def paged_slot(block_table, b, t, block_size):
    """(block id, row inside the block) of token ``t`` of sequence ``b``."""
    return int(block_table[b, t // block_size]), t % block_size


def kv_update_paged(k_pool, v_pool, new_k, new_v, pos, block_table, block_size, n_heads, head_dim):
    """Paged append: pools are ``[n_blocks, H, block_size, D]``; ``new_* [B, H*D]``."""
    B = new_k.shape[0]
    pos = np.broadcast_to(np.asarray(pos, dtype=np.int64), (B,))
    for b in range(B):
        blk, r = paged_slot(block_table, b, int(pos[b]), block_size)
        k_pool[blk, :, r, :] = new_k[b].reshape(n_heads, head_dim)
        v_pool[blk, :, r, :] = new_v[b].reshape(n_heads, head_dim)


def paged_gather(pool, block_table, lens, block_size, max_len):
    """Logical view ``[B, max_len, H, D]`` of a paged pool (rows past ``lens[b]`` zero)."""
    B = block_table.shape[0]
    _, H, _, D = pool.shape
    out = np.zeros((B, max_len, H, D), dtype=pool.dtype)
    for b in range(B):
        n = int(lens[b])
        for j in range((n + block_size - 1) // block_size):
            t0 = j * block_size
            cnt = min(block_size, n - t0)
            blk = int(block_table[b, j])
            out[b, t0 : t0 + cnt] = pool[blk, :, :cnt, :].transpose(1, 0, 2)
    return out


# ----------------------------------------------------------------------------
# single-token decode attention over the cache
# ----------------------------------------------------------------------------


def decode_attention(q, k_logical, v_logical, lens, out_dtype=np.float32):
    """softmax(q K^T / sqrt(D)) V per (sequence, head) over the first ``lens[b]`` rows.

    ``q [B, H, D]``; ``k_logical, v_logical [B, T, H, D]`` (float32 values; for the bf16
    extension pass values already rounded to bf16).  Follows the per-(b, h) loop of
    the reference test: matmul, scale, max-subtracted exp, divide, matmul.
    Sequences with ``lens[b] == 0`` give zeros (the reference refuses an empty cache
    on the host; with per-sequence lengths the kernel defines the row as zero).
    """
    B, H, D = q.shape
    lens = np.broadcast_to(np.asarray(lens, dtype=np.int64), (B,))
    scale = np.float32(1.0 / np.sqrt(D))
    out = np.zeros((B, H, D), dtype=np.float32)
    for b in range(B):
        n = int(lens[b])
        if n == 0:
            continue
        for h in range(H):
            q_bh = q[b, h][None, :].astype(np.float32)
            k_bh = k_logical[b, :n, h, :].astype(np.float32)
            v_bh = v_logical[b, :n, h, :].astype(np.float32)
            scores = np.matmul(q_bh, k_bh.T) * scale
            scores_max = np.max(scores, axis=-1, keepdims=True)
            scores_exp = np.exp(scores - scores_max)
            scores_sum = np.sum(scores_exp, axis=-1, keepdims=True)
            out[b, h] = np.matmul(scores_exp / scores_sum, v_bh)[0]
    return out.astype(out_dtype)


def decode_attention_shader_order(q, k_logical, v_logical, lens):
    """Same result computed in the order the WGSL shader uses (cross-check only)."""
    B, H, D = q.shape
    lens = np.broadcast_to(np.asarray(lens, dtype=np.int64), (B,))
    scale = np.float32(1.0) / np.sqrt(np.float32(D))
    out = np.zeros((B, H, D), dtype=np.float32)
    for b in range(B):
        n = int(lens[b])
        for h in range(H):
            s = np.zeros(n, dtype=np.float32)
            for t in range(n):
                s[t] = np.dot(q[b, h].astype(np.float32), k_logical[b, t, h].astype(np.float32)) * scale
            m = max(MASK_VALUE, s.max()) if n else MASK_VALUE
            e = np.exp(s - m)
            total = e.sum(dtype=np.float32)
            for t in range(n):
                out[b, h] += (e[t] / total) * v_logical[b, t, h].astype(np.float32)
    return out


# ----------------------------------------------------------------------------
# causal prefill attention
# ----------------------------------------------------------------------------


def flash_attention_dense(Q, K, V, batch, seq_len, n_heads, head_dim):
    """Dense causal attention of the reference test.  Q, K, V ``[B, N, H*D]`` -> O same shape."""
    def heads(x):
        return np.asarray(x, dtype=np.float32).reshape(batch, seq_len, n_heads, head_dim).transpose(0, 2, 1, 3)

    q, k, v = heads(Q), heads(K), heads(V)
    scale = np.float32(1.0 / np.sqrt(float(head_dim)))
    scores = np.einsum("bhqd,bhkd->bhqk", q, k) * scale
    causal = np.tril(np.ones((seq_len, seq_len)))[None, None, :, :]
    scores = np.where(causal == 1, scores, MASK_VALUE)
    scores = scores - scores.max(axis=-1, keepdims=True)
    w = np.exp(scores)
    w = w / w.sum(axis=-1, keepdims=True)
    out = np.einsum("bhqk,bhkd->bhqd", w.astype(np.float32), v)
    return out.transpose(0, 2, 1, 3).reshape(batch, seq_len, n_heads * head_dim).astype(np.float32)


def flash_attention_tiled(Q, K, V, batch, seq_len, n_heads, head_dim, Br=32, Bc=32):
    """Tiled online-softmax forward in the shader's order; returns ``(O, L, M)``.

    ``L`` (row sums) and ``M`` (row maxima) are flat ``[B*N*H]`` arrays indexed
    ``b*N*H + row*H + h``.  A K/V block is visited while ``kv_start <= q_end``
    (``q_end`` exclusive), so one fully masked block may be visited; its entries carry
    the mask value and contribute ``exp(-1e10 - m) == 0``.
    """
    E = n_heads * head_dim
    Qr = np.asarray(Q, dtype=np.float32).reshape(batch, seq_len, n_heads, head_dim)
    Kr = np.asarray(K, dtype=np.float32).reshape(batch, seq_len, n_heads, head_dim)
    Vr = np.asarray(V, dtype=np.float32).reshape(batch, seq_len, n_heads, head_dim)
    scale = np.float32(1.0) / np.sqrt(np.float32(head_dim))
    O = np.zeros((batch, seq_len, n_heads, head_dim), dtype=np.float32)
    L = np.zeros(batch * seq_len * n_heads, dtype=np.float32)
    M = np.zeros(batch * seq_len * n_heads, dtype=np.float32)
    for b in range(batch):
        for h in range(n_heads):
            for q_start in range(0, seq_len, Br):
                q_end = min(q_start + Br, seq_len)
                rows = q_end - q_start
                qi = Qr[b, q_start:q_end, h]
                mi = np.full(rows, MASK_VALUE, dtype=np.float32)
                li = np.zeros(rows, dtype=np.float32)
                oi = np.zeros((rows, head_dim), dtype=np.float32)
                for kv_start in range(0, seq_len, Bc):
                    if kv_start > q_end:
                        break
                    kv_end = min(kv_start + Bc, seq_len)
                    s = (qi @ Kr[b, kv_start:kv_end, h].T) * scale
                    q_pos = np.arange(q_start, q_end)[:, None]
                    kv_pos = np.arange(kv_start, kv_end)[None, :]
                    s = np.where(kv_pos <= q_pos, s, MASK_VALUE).astype(np.float32)
                    mi_new = np.maximum(mi, s.max(axis=1))
                    p = np.exp(s - mi_new[:, None]).astype(np.float32)
                    corr = np.exp(mi - mi_new).astype(np.float32)
                    li = li * corr + p.sum(axis=1, dtype=np.float32)
                    oi = oi * corr[:, None] + p @ Vr[b, kv_start:kv_end, h]
                    mi = mi_new
                O[b, q_start:q_end, h] = oi / np.maximum(li, np.float32(1e-8))[:, None]
                idx = b * seq_len * n_heads + np.arange(q_start, q_end) * n_heads + h
                L[idx] = li
                M[idx] = mi
    return O.reshape(batch, seq_len, E), L, M


# ----------------------------------------------------------------------------
# seeded recipes of the reference's tests (inputs only)
# ----------------------------------------------------------------------------


def recipe_kv_cache_inputs(batch_size=2, n_heads=4, head_dim=64, num_tokens=5, seed=42):
    """Inputs of the reference's KV test (gpu_test.py:2267-2289, :2317): returns
    ``(k_list, v_list, Q)`` with ``k_list[i], v_list[i] [B, 1, H, D]`` and ``Q [B, 1, H, D]``,
    drawn in the reference's order: per step new_k then new_v, finally Q."""
    np.random.seed(seed)
    ks, vs = [], []
    for _ in range(num_tokens):
        ks.append(np.random.randn(batch_size, 1, n_heads, head_dim).astype(np.float32))
        vs.append(np.random.randn(batch_size, 1, n_heads, head_dim).astype(np.float32))
    Q = np.random.randn(batch_size, 1, n_heads, head_dim).astype(np.float32)
    return ks, vs, Q


# (batch, seq_len, n_heads, head_dim) of the reference's flash test, gpu_test.py:747-756
FLASH_RECIPE_SHAPES = [
    (2, 8, 2, 16),
    (2, 4, 2, 16),
    (2, 16, 2, 16),
    (4, 16, 4, 64),
    (8, 32, 8, 64),
    (4, 32, 4, 32),
    (2, 64, 2, 32),
]


def recipe_flash_inputs(batch, seq_len, n_heads, head_dim, seed=42):
    """Inputs of the reference's flash test (gpu_test.py:770-774): Q, K, V in that order."""
    np.random.seed(seed)
    shape = (batch, seq_len, n_heads * head_dim)
    Q = np.random.randn(*shape).astype(np.float32)
    K = np.random.randn(*shape).astype(np.float32)
    V = np.random.randn(*shape).astype(np.float32)
    return Q, K, V


def qkv_project(x, wq, wk, wv):
    """The three projections of the attention block, C = A @ B per weight matrix
    (simple-llm/src/wgpu_backend.py:812-831, gpu_pass_forward.py:35-82), accumulated in float64 from
    the given (already storage-rounded) inputs.  Returns float32 arrays [rows, E]."""
    x64 = np.asarray(x, dtype=np.float64)
    return tuple((x64 @ np.asarray(w, dtype=np.float64)).astype(np.float32) for w in (wq, wk, wv))
