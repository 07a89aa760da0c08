"""The Q / K / V projection fused with the cache append against the oracle (three matmuls, then the
append indexing of the reference): Q and the new cache rows within two bf16 units in the last place
of the float64-accumulated product (rtol 2^-7, plus atol 1e-2 for values near zero), every other cache row
untouched bit for bit, and a decode over the updated cache equal to the oracle's."""
import numpy as np
import pytest
import torch

from oracle import c_oracle, kv_oracle
from tests import kv_util as U

pytestmark = pytest.mark.gpu
RTOL, ATOL = 2.0 ** -7, 1e-2


@pytest.fixture(scope="module")
def ctx(pkg):
    return U.make_ctx(pkg)


def _bf16(ctx, shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(torch.bfloat16).to(ctx.device)


@pytest.mark.parametrize("B,H,D,layout,ragged", [(3, 2, 64, "bthd", False), (17, 4, 64, "bhtd", True),
                                                  (64, 8, 128, "bhtd", True), (128, 2, 128, "bthd", True),
                                                  (1, 1, 128, "bhtd", False)])
def test_qkv_project_append_vs_oracle(pkg, ctx, B, H, D, layout, ragged):
    gpu = pkg.gpu
    E, T_max = H * D, 40
    x = _bf16(ctx, (B, E), 1)
    wq, wk, wv = (_bf16(ctx, (E, E), s, scale=E ** -0.5) for s in (2, 3, 4))
    cache = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=B, max_seq_len=T_max, n_layers=2, n_heads=H, head_dim=D,
                                                       dtype=torch.bfloat16, layout=layout, ragged=ragged))
    # pre-fill the layer with known rows, then pick where the step writes
    for layer in cache.layers:
        layer.k_cache.buffer.copy_(_bf16(ctx, tuple(layer.k_cache.buffer.shape), 5))
        layer.v_cache.buffer.copy_(_bf16(ctx, tuple(layer.v_cache.buffer.shape), 6))
    rng = np.random.default_rng(B)
    if ragged:
        lens = rng.integers(0, T_max - 1, size=B).astype(np.int32)
        gpu.kv_cache_set_lengths(cache, lens)
    else:
        lens = np.full(B, 7, dtype=np.int32)
        cache.current_len = 7
    before_k = U.logical_view(cache, cache.layers[1], "k").clone()
    before_v = U.logical_view(cache, cache.layers[1], "v").clone()
    other_k = cache.layers[0].k_cache.buffer.clone()
    q_out = torch.zeros((B, E), dtype=torch.bfloat16, device=ctx.device)
    gpu.batch_begin(ctx)
    gpu.qkv_project_append(ctx, cache, 1, U.buf2d(pkg, ctx, x), U.buf2d(pkg, ctx, wq), U.buf2d(pkg, ctx, wk),
                           U.buf2d(pkg, ctx, wv), U.buf2d(pkg, ctx, q_out))
    gpu.batch_commit(ctx)
    torch.cuda.synchronize()
    want_q, want_k, want_v = kv_oracle.qkv_project(U.to_f32(x), U.to_f32(wq), U.to_f32(wk), U.to_f32(wv))
    np.testing.assert_allclose(U.to_f32(q_out), want_q, rtol=RTOL, atol=ATOL)
    after_k = U.logical_view(cache, cache.layers[1], "k")
    after_v = U.logical_view(cache, cache.layers[1], "v")
    rows = torch.arange(B)
    pos = torch.from_numpy(lens.astype(np.int64))
    np.testing.assert_allclose(U.to_f32(after_k[rows, pos].reshape(B, E)), want_k, rtol=RTOL, atol=ATOL)
    np.testing.assert_allclose(U.to_f32(after_v[rows, pos].reshape(B, E)), want_v, rtol=RTOL, atol=ATOL)
    # nothing else moved: restore the written rows and compare bit for bit
    after_k[rows, pos] = before_k[rows, pos]
    after_v[rows, pos] = before_v[rows, pos]
    assert torch.equal(after_k, before_k) and torch.equal(after_v, before_v)
    assert torch.equal(cache.layers[0].k_cache.buffer, other_k)
    # lengths advanced like kv_cache_update
    assert cache.current_len == 8 if not ragged else True
    if ragged:
        assert np.array_equal(cache.seq_lens.cpu().numpy(), lens + 1)


def test_qkv_project_append_checks(pkg, ctx):
    gpu = pkg.gpu
    B, H, D = 2, 2, 64
    E = H * D
    cache = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=B, max_seq_len=4, n_layers=1, n_heads=H, head_dim=D,
                                                       dtype=torch.bfloat16, layout="bhtd"))
    mk = lambda r, c: U.buf2d(pkg, ctx, torch.zeros((r, c), dtype=torch.bfloat16, device=ctx.device))  # noqa: E731
    x, w, q = mk(B, E), mk(E, E), mk(B, E)
    gpu.batch_begin(ctx)
    with pytest.raises(ValueError, match="layer_idx 3 out of range"):
        gpu.qkv_project_append(ctx, cache, 3, x, w, w, w, q)
    with pytest.raises(ValueError, match="wk shape mismatch"):
        gpu.qkv_project_append(ctx, cache, 0, x, w, mk(E, 64), w, q)
    cache.current_len = 4
    with pytest.raises(ValueError, match="Cache is full"):
        gpu.qkv_project_append(ctx, cache, 0, x, w, w, w, q)
    gpu.batch_commit(ctx)


@pytest.mark.parametrize("M,K,N,with_residual", [(64, 1024, 512, False), (5, 128, 256, True), (128, 512, 128, True),
                                                 (1, 4096, 1024, False), (33, 256, 1280, True), (8, 512, 8192, True)])
def test_matmul_rows_vs_oracle(pkg, ctx, M, K, N, with_residual):
    gpu = pkg.gpu
    A = _bf16(ctx, (M, K), 11)
    W = _bf16(ctx, (K, N), 12, scale=K ** -0.5)
    R = _bf16(ctx, (M, N), 13) if with_residual else None
    C = torch.zeros((M, N), dtype=torch.bfloat16, device=ctx.device)
    gpu.batch_begin(ctx)
    gpu.matmul(ctx, U.buf2d(pkg, ctx, A), U.buf2d(pkg, ctx, W), U.buf2d(pkg, ctx, C),
               residual=None if R is None else U.buf2d(pkg, ctx, R))
    gpu.batch_commit(ctx)
    want = U.to_f32(A).astype(np.float64) @ U.to_f32(W).astype(np.float64)
    if R is not None:
        want = want + U.to_f32(R)
    np.testing.assert_allclose(U.to_f32(C), want.astype(np.float32), rtol=RTOL, atol=ATOL)


def test_matmul_with_bias_gelu_and_residual_like_the_mlp(pkg, ctx):
    """C = gelu(A @ W + b) + R, the reference's matmul -> bias_add -> gelu (-> residual_add) chain."""
    gpu = pkg.gpu
    M, K, N = 64, 512, 1024
    A, W = _bf16(ctx, (M, K), 21), _bf16(ctx, (K, N), 22, scale=K ** -0.5)
    bias, R = _bf16(ctx, (N,), 23), _bf16(ctx, (M, N), 24)
    C = torch.zeros((M, N), dtype=torch.bfloat16, device=ctx.device)
    gpu.batch_begin(ctx)
    gpu.matmul(ctx, U.buf2d(pkg, ctx, A), U.buf2d(pkg, ctx, W), U.buf2d(pkg, ctx, C), residual=U.buf2d(pkg, ctx, R),
               bias=gpu.GPUBuffer1D(buffer=bias, shape=(N,), size=N), activation="gelu")
    gpu.batch_commit(ctx)
    z = U.to_f32(A).astype(np.float64) @ U.to_f32(W).astype(np.float64) + U.to_f32(bias)
    want = z / (1.0 + np.exp(-1.702 * z)) + U.to_f32(R)
    np.testing.assert_allclose(U.to_f32(C), want.astype(np.float32), rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("splits", [1, 2, 3, 4, 8])
def test_matmul_rows_with_forced_input_ranges(pkg, ctx, splits):
    """Every way of cutting the input features over a thread-block cluster gives the same product (the number of
    ranges is a power of two: 3 is taken as 2, and 8 as 4 because there are only six tiles of input features)."""
    gpu = pkg.gpu
    M, K, N = 16, 768, 256
    A, W, R = _bf16(ctx, (M, K), 31), _bf16(ctx, (K, N), 32, scale=K ** -0.5), _bf16(ctx, (M, N), 33)
    C = torch.zeros((M, N), dtype=torch.bfloat16, device=ctx.device)
    try:
        pkg._native.tune("matmul_splits", splits)
        gpu.batch_begin(ctx)
        gpu.matmul(ctx, U.buf2d(pkg, ctx, A), U.buf2d(pkg, ctx, W), U.buf2d(pkg, ctx, C), residual=U.buf2d(pkg, ctx, R))
        gpu.batch_commit(ctx)
        torch.cuda.synchronize()
    finally:
        pkg._native.tune("matmul_splits", 0)
    want = U.to_f32(A).astype(np.float64) @ U.to_f32(W).astype(np.float64) + U.to_f32(R)
    np.testing.assert_allclose(U.to_f32(C), want.astype(np.float32), rtol=RTOL, atol=ATOL)


def test_matmul_checks(pkg, ctx):
    gpu = pkg.gpu
    mk = lambda r, c, dt=torch.bfloat16: U.buf2d(pkg, ctx, torch.zeros((r, c), dtype=dt, device=ctx.device))  # noqa: E731
    gpu.batch_begin(ctx)
    with pytest.raises(ValueError, match=r"matmul: Dimension mismatch A.shape\[1\]=128 != B.shape\[0\]=256"):
        gpu.matmul(ctx, mk(4, 128), mk(256, 128), mk(4, 128))
    with pytest.raises(ValueError, match="matmul: Output shape"):
        gpu.matmul(ctx, mk(4, 128), mk(128, 128), mk(4, 256))
    with pytest.raises(ValueError, match="bfloat16"):
        gpu.matmul(ctx, mk(4, 128, torch.float32), mk(128, 128), mk(4, 128))
    with pytest.raises(ValueError, match="multiples of 8"):
        gpu.matmul(ctx, mk(4, 60), mk(60, 128), mk(4, 128))
    gpu.batch_commit(ctx)


@pytest.mark.parametrize("M,K,N,epilogue", [
    (129, 128, 128, "none"),       # one row past a tile: the second row tile is almost empty
    (256, 64, 256, "none"),        # a single stage per tile
    (1000, 520, 776, "all"),       # ragged rows, input features and columns (zero-filled edges, masked stores)
    (64, 72, 40, "residual"),      # a decode-sized matrix whose dimensions the rows kernel does not take
    (4096, 1024, 1024, "all"),     # several tiles per CTA: both accumulators, ring wrap-around
    (2048, 512, 4096, "bias"),     # more column tiles than a band has row tiles
    (3000, 256, 264, "gelu"),      # a last column tile of 8 columns
])
@pytest.mark.parametrize("variant", [1, 2, 3])
def test_matmul_tiled_gemm_vs_oracle(pkg, ctx, M, K, N, epilogue, variant):
    """The tiled tensor-core GEMM behind ``matmul`` for more rows than a decode step has, in both forms
    (1: one CTA per 128 x 256 tile; 2, 3: a CTA pair per 256 x 256 tile with 64 or 128 input features per
    ring stage), with each epilogue, against a float64
    product."""
    gpu = pkg.gpu
    pkg._native.tune("gemm_variant", variant)
    try:
        _tiled_gemm_case(pkg, ctx, M, K, N, epilogue)
    finally:
        pkg._native.tune("gemm_variant", 0)


def _tiled_gemm_case(pkg, ctx, M, K, N, epilogue):
    gpu = pkg.gpu
    A, W = _bf16(ctx, (M, K), 41), _bf16(ctx, (K, N), 42, scale=K ** -0.5)
    bias = _bf16(ctx, (N,), 43) if epilogue in ("all", "bias") else None
    R = _bf16(ctx, (M, N), 44) if epilogue in ("all", "residual") else None
    act = "gelu" if epilogue in ("all", "gelu") else None
    C = torch.full((M + 1, N), 7.0, dtype=torch.bfloat16, device=ctx.device)  # one guard row behind the output
    Cb = U.buf2d(pkg, ctx, C[:M])
    gpu.batch_begin(ctx)
    gpu.matmul(ctx, U.buf2d(pkg, ctx, A), U.buf2d(pkg, ctx, W), Cb, residual=None if R is None else U.buf2d(pkg, ctx, R),
               bias=None if bias is None else gpu.GPUBuffer1D(buffer=bias, shape=(N,), size=N), activation=act)
    gpu.batch_commit(ctx)
    z = U.to_f32(A).astype(np.float64) @ U.to_f32(W).astype(np.float64)
    if bias is not None:
        z = z + U.to_f32(bias)
    if act:
        z = z / (1.0 + np.exp(-1.702 * z))
    if R is not None:
        z = z + U.to_f32(R)
    np.testing.assert_allclose(U.to_f32(C[:M]), z.astype(np.float32), rtol=RTOL, atol=ATOL)
    assert bool((C[M] == 7.0).all())  # nothing written past the last row
