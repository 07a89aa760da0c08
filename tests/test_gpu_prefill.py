"""GPU parity: causal flash-attention prefill against the fixtures made from the reference
test's own math (simple-llm/src/gpu_test.py:743-868) and against the oracle, plus the fused
cache write (bit-exact)."""
import numpy as np
import pytest
import torch

from oracle import c_oracle, kv_oracle
from tests import kv_util as U

pytestmark = pytest.mark.gpu

# fp32 prompts on the tensor cores (operands as two bfloat16 halves, 16 mantissa bits): see the tests that use it
SPLIT_TOL = dict(rtol=1e-4, atol=3e-5)


@pytest.fixture(scope="module")
def ctx(pkg):
    return U.make_ctx(pkg)


def _run_flash(pkg, ctx, Q, K, V, B, N, H, D, dtype, cache=None, stats=True):
    gpu = pkg.gpu
    ctx.config.flash_attn_max_head_dim = max(D, 128)
    mk = lambda a: U.buf2d(pkg, ctx, a.reshape(B * N, H * D).contiguous())  # noqa: E731
    Qb, Kb, Vb = mk(Q), mk(K), mk(V)
    Ob = U.buf2d(pkg, ctx, torch.empty((B * N, H * D), dtype=dtype, device=ctx.device))
    Lb = gpu.gpu_buffer_1d_create(ctx, B * N * H) if stats else None
    Mb = gpu.gpu_buffer_1d_create(ctx, B * N * H) if stats else None
    gpu.batch_begin(ctx)
    gpu.flash_attention(ctx, Qb, Kb, Vb, Ob, Lb, Mb, B, N, H, D, cache=cache, layer_idx=0)
    gpu.batch_commit(ctx)
    torch.cuda.synchronize()
    return Ob.buffer, (Lb.buffer if stats else None), (Mb.buffer if stats else None)


@pytest.mark.parametrize("case", range(len(kv_oracle.FLASH_RECIPE_SHAPES)))
def test_reference_flash_recipes(pkg, ctx, golden, case):
    B, N, H, D = kv_oracle.FLASH_RECIPE_SHAPES[case]
    Qn, Kn, Vn = kv_oracle.recipe_flash_inputs(B, N, H, D, seed=42)
    dev = lambda a: torch.from_numpy(a).to(ctx.device)  # noqa: E731
    O, L, M = _run_flash(pkg, ctx, dev(Qn), dev(Kn), dev(Vn), B, N, H, D, torch.float32)
    np.testing.assert_allclose(O.cpu().numpy().reshape(B, N, H * D), golden[f"flash_out_{case}"], rtol=1e-4, atol=1e-5)
    # L and M, which the reference writes but never checks: against the shader-order oracle
    _, Lw, Mw = kv_oracle.flash_attention_tiled(Qn, Kn, Vn, B, N, H, D, Br=8, Bc=8)
    np.testing.assert_allclose(L.cpu().numpy(), Lw, rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(M.cpu().numpy(), Mw, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,N,H,D", [(2, 1, 2, 64), (1, 33, 3, 128), (2, 200, 2, 64), (1, 77, 2, 256), (2, 95, 4, 32),
                                     (1, 129, 2, 16)])
def test_prefill_ragged_shapes_vs_oracle(pkg, ctx, dtype, B, N, H, D):
    Q = U.randn((B, N, H * D), dtype, ctx.device, 1)
    K = U.randn((B, N, H * D), dtype, ctx.device, 2)
    V = U.randn((B, N, H * D), dtype, ctx.device, 3)
    O, L, M = _run_flash(pkg, ctx, Q, K, V, B, N, H, D, dtype)
    Ow, Lw, Mw = c_oracle.prefill(U.to_oracle(Q.reshape(B * N, H * D)), U.to_oracle(K.reshape(B * N, H * D)),
                                  U.to_oracle(V.reshape(B * N, H * D)), B, N, H, D)
    np.testing.assert_allclose(U.to_f32(O), Ow, **U.TOL[dtype])
    np.testing.assert_allclose(L.cpu().numpy(), Lw, rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(M.cpu().numpy(), Mw, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("dtype,D", [(torch.float32, 64), (torch.bfloat16, 128), (torch.bfloat16, 64)])
@pytest.mark.parametrize("layout", ["bthd", "bhtd"])
def test_prefill_writes_cache_rows_bit_exact_then_decode_continues(pkg, ctx, dtype, D, layout):
    gpu = pkg.gpu
    B, N, H, T_max = 2, 150, 3, 256
    E = H * D
    Q = U.randn((B, N, E), dtype, ctx.device, 4)
    K = U.randn((B, N, E), dtype, ctx.device, 5)
    V = U.randn((B, N, E), dtype, ctx.device, 6)
    cache = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=B, max_seq_len=T_max, n_layers=1, n_heads=H,
                                                       head_dim=D, dtype=dtype, layout=layout))
    O, _, _ = _run_flash(pkg, ctx, Q, K, V, B, N, H, D, dtype, cache=cache, stats=False)
    assert cache.current_len == N
    kview = U.logical_view(cache, cache.layers[0], "k")
    vview = U.logical_view(cache, cache.layers[0], "v")
    assert torch.equal(kview[:, :N].reshape(B, N, E), K) and torch.equal(vview[:, :N].reshape(B, N, E), V)
    assert float(kview[:, N:].float().abs().sum()) == 0.0
    # decoding the last prompt token over the prefilled cache reproduces the prefill's last row
    q_last = Q[:, N - 1].contiguous()
    out = torch.empty_like(q_last)
    gpu.batch_begin(ctx)
    gpu.attention_with_kv_cache(ctx, cache, 0, U.buf2d(pkg, ctx, q_last), U.buf2d(pkg, ctx, out))
    gpu.batch_commit(ctx)
    tol = U.TOL[dtype]
    np.testing.assert_allclose(U.to_f32(out), U.to_f32(O.reshape(B, N, E)[:, N - 1]), rtol=max(tol["rtol"], 1e-4),
                               atol=tol["atol"])


@pytest.mark.parametrize("B,N,H,with_cache", [(1, 256, 1, False), (2, 512, 3, True), (1, 1280, 2, True), (2, 2048, 2, False)])
def test_prefill_cta_pair_kernel_vs_oracle_and_one_cta_kernel(pkg, ctx, B, N, H, with_cache):
    """The CTA-pair kernel (opt-in through the "prefill_variant" knob) against the oracle and against
    the default kernel: O within the bf16 tolerance, L / M as the shader defines them, cache rows bit-exact."""
    gpu = pkg.gpu
    D, dtype = 128, torch.bfloat16
    E = H * D
    Q = U.randn((B, N, E), dtype, ctx.device, 21)
    K = U.randn((B, N, E), dtype, ctx.device, 22)
    V = U.randn((B, N, E), dtype, ctx.device, 23)
    results = {}
    try:
        for variant in (0, 2):
            pkg._native.tune("prefill_variant", variant)
            cache = None
            if with_cache:
                cache = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=B, max_seq_len=N + 64, n_layers=1, n_heads=H,
                                                                   head_dim=D, dtype=dtype, layout="bhtd"))
            O, Lb, Mb = _run_flash(pkg, ctx, Q, K, V, B, N, H, D, dtype, cache=cache)
            results[variant] = (O.clone(), Lb.clone(), Mb.clone(), cache)
    finally:
        pkg._native.tune("prefill_variant", 0)
    flat = lambda a: U.to_oracle(a.reshape(B * N, E))  # noqa: E731
    Ow, Lw, Mw = c_oracle.prefill(flat(Q), flat(K), flat(V), B, N, H, D)
    O2, L2, M2, cache2 = results[2]
    np.testing.assert_allclose(U.to_f32(O2), Ow, **U.TOL[dtype])
    np.testing.assert_allclose(L2.cpu().numpy(), Lw, rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(M2.cpu().numpy(), Mw, rtol=1e-4, atol=1e-5)
    O0 = results[0][0]
    assert float((O2.float() - O0.float()).abs().max()) <= 2e-2
    if with_cache:
        kview = U.logical_view(cache2, cache2.layers[0], "k")
        vview = U.logical_view(cache2, cache2.layers[0], "v")
        assert torch.equal(kview[:, :N].reshape(B, N, E), K) and torch.equal(vview[:, :N].reshape(B, N, E), V)
        assert float(kview[:, N:].float().abs().sum()) == 0.0


@pytest.mark.parametrize("dtype,D,N,bs", [(torch.bfloat16, 128, 200, 16), (torch.float32, 64, 77, 16),
                                          (torch.bfloat16, 128, 256, 16), (torch.bfloat16, 128, 300, 8),
                                          (torch.bfloat16, 64, 200, 64), (torch.bfloat16, 128, 200, 128),
                                          (torch.bfloat16, 128, 300, 256), (torch.bfloat16, 128, 200, 24),
                                          (torch.bfloat16, 128, 260, 32)])
def test_prefill_into_a_paged_cache_bit_exact_then_decode_continues(pkg, ctx, dtype, D, N, bs):
    """flash_attention with a paged cache: the prompt's K / V rows land in the blocks that a permuted block
    table names (bit-exact, nothing else in the pool touched), and decoding the last prompt token over the
    pool reproduces the prefill's last row.  Block sizes that tile the kernel's 128-row K / V tiles are stored by
    the tensor-core kernel itself (whole blocks; a partly filled last block by the copy kernel), the others
    (24 here, and every fp32 case) by the copy kernel alone."""
    gpu = pkg.gpu
    B, H, T_max = 2, 3, 320
    E = H * D
    Q = U.randn((B, N, E), dtype, ctx.device, 31)
    K = U.randn((B, N, E), dtype, ctx.device, 32)
    V = U.randn((B, N, E), dtype, ctx.device, 33)
    n_blocks = max(64, B * ((T_max + bs - 1) // bs) + 7)
    cache = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=B, max_seq_len=T_max, n_layers=1, n_heads=H, head_dim=D,
                                                       dtype=dtype, block_size=bs, n_blocks=n_blocks))
    max_blocks = cache.block_table.shape[1]
    g = torch.Generator().manual_seed(5)
    perm = torch.randperm(n_blocks, generator=g)[: B * max_blocks].to(torch.int32)
    cache.block_table.copy_(perm.reshape(B, max_blocks).to(ctx.device))
    layer = cache.layers[0]
    layer.k_cache.buffer.fill_(3.0)  # a sentinel in every block
    layer.v_cache.buffer.fill_(3.0)
    O, _, _ = _run_flash(pkg, ctx, Q, K, V, B, N, H, D, dtype, cache=cache, stats=False)
    assert cache.current_len == N
    gpu.batch_begin(ctx)
    kview = gpu.kv_cache_gather(ctx, cache, 0, "k", length=N)
    vview = gpu.kv_cache_gather(ctx, cache, 0, "v", length=N)
    gpu.batch_commit(ctx)
    assert torch.equal(kview.reshape(B, N, E), K) and torch.equal(vview.reshape(B, N, E), V)
    # rows written: B * N * E elements per pool; every other element still holds the sentinel
    assert int((layer.k_cache.buffer != 3.0).sum()) <= B * N * E
    used_blocks = (N + bs - 1) // bs
    pool = layer.k_cache.buffer.reshape(n_blocks, -1)
    untouched = torch.ones(n_blocks, dtype=torch.bool)
    untouched[cache.block_table[:, :used_blocks].reshape(-1).cpu().long()] = False
    assert bool((pool[untouched.to(ctx.device)] == 3.0).all())
    q_last = Q[:, N - 1].contiguous()
    out = torch.empty_like(q_last)
    gpu.batch_begin(ctx)
    gpu.attention_with_kv_cache(ctx, cache, 0, U.buf2d(pkg, ctx, q_last), U.buf2d(pkg, ctx, out))
    gpu.batch_commit(ctx)
    tol = U.TOL[dtype]
    np.testing.assert_allclose(U.to_f32(out), U.to_f32(O.reshape(B, N, E)[:, N - 1]), rtol=max(tol["rtol"], 1e-4),
                               atol=tol["atol"])


def test_wait_that_runs_out_in_the_tensor_core_kernel_is_reported(pkg, ctx):
    """The softmax warps of one small launch (a single CTA) are told to behave as if their first
    barrier wait had run out.  The MMA-issuing thread and the copy thread then run out on their own
    bounded waits (about two seconds), every warp meets at the common exit, the tensor memory is
    released and the status word reads B2KV_DEV_WAIT_TIMEOUT, which batch_commit raises.  Nothing
    faults, and the next launch on the same context is correct."""
    gpu, native = pkg.gpu, pkg._native
    B, N, H, D = 1, 256, 1, 128
    dtype = torch.bfloat16
    Q = U.randn((B, N, H * D), dtype, ctx.device, 4)
    K = U.randn((B, N, H * D), dtype, ctx.device, 5)
    V = U.randn((B, N, H * D), dtype, ctx.device, 6)
    ctx.config.check_device_status = True
    native.tune("prefill_test_expire", 1)
    try:
        with pytest.raises(RuntimeError, match="bounded wait"):
            _run_flash(pkg, ctx, Q, K, V, B, N, H, D, dtype, stats=False)
    finally:
        native.tune("prefill_test_expire", 0)
    try:
        O, _, _ = _run_flash(pkg, ctx, Q, K, V, B, N, H, D, dtype, stats=False)
    finally:
        ctx.config.check_device_status = False
    Ow, _, _ = c_oracle.prefill(U.to_oracle(Q.reshape(B * N, H * D)), U.to_oracle(K.reshape(B * N, H * D)),
                                U.to_oracle(V.reshape(B * N, H * D)), B, N, H, D)
    np.testing.assert_allclose(U.to_f32(O), Ow, **U.TOL[dtype])


def test_profiled_batch_fills_the_perf_monitor(pkg, ctx):
    """batch_begin(enable_profiling=True): every operation is timed under the reference function's name
    (simple-llm/src/gpu/gpu_ops.py:245-250, gpu_device.py:569-608)."""
    gpu = pkg.gpu
    B, N, H, D = 1, 64, 2, 64
    Q = U.randn((B, N, H * D), torch.float32, ctx.device, 7)
    mk = lambda a: U.buf2d(pkg, ctx, a.reshape(B * N, H * D).contiguous())  # noqa: E731
    Qb, Ob = mk(Q), mk(torch.empty_like(Q))
    ctx.perf_monitor = None
    gpu.batch_begin(ctx, enable_profiling=True)
    gpu.flash_attention(ctx, Qb, Qb, Qb, Ob, None, None, B, N, H, D)
    gpu.flash_attention(ctx, Qb, Qb, Qb, Ob, None, None, B, N, H, D)
    gpu.batch_commit(ctx)
    stats = gpu.perf_monitor_stats_get(ctx.perf_monitor)
    assert stats.total_submissions == 1
    fa = stats.kernel_times["flash_attention"]
    assert fa.count == 2 and 0.0 < fa.min_ms <= fa.max_ms


@pytest.mark.parametrize("B,N,H,D", [(1, 128, 2, 128), (2, 300, 2, 64), (1, 1000, 3, 128), (2, 129, 1, 64),
                                     (1, 2048, 2, 128)])
def test_fp32_prompts_on_the_tensor_cores_keep_the_fp32_bar(pkg, ctx, B, N, H, D):
    """fp32 prompts of head_dim 128 / 64 and at least 128 tokens run on the tensor cores with every operand split into
    two bfloat16 halves (three MMAs per product), which keeps 16 of fp32's 24 mantissa bits per operand.  Bar: rtol
    1e-4 with atol 3e-5 against the oracle on outputs of order one (the SIMT kernel's atol is 1e-5; the worst element
    seen here is 1.3e-5 off), L and M at the SIMT kernel's tolerance; and the two kernels agree with each other."""
    dtype = torch.float32
    Q = U.randn((B, N, H * D), dtype, ctx.device, 41)
    K = U.randn((B, N, H * D), dtype, ctx.device, 42)
    V = U.randn((B, N, H * D), dtype, ctx.device, 43)
    assert pkg._native.lib.b2kv_prefill_workspace_bytes(B, N, H, D, pkg._native.DTYPE_F32) == 6 * B * N * H * D * 2
    O, L, M = _run_flash(pkg, ctx, Q, K, V, B, N, H, D, dtype)
    flat = lambda a: U.to_oracle(a.reshape(B * N, H * D))  # noqa: E731
    Ow, Lw, Mw = c_oracle.prefill(flat(Q), flat(K), flat(V), B, N, H, D)
    np.testing.assert_allclose(U.to_f32(O), Ow, **SPLIT_TOL)
    np.testing.assert_allclose(L.cpu().numpy(), Lw, rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(M.cpu().numpy(), Mw, rtol=1e-4, atol=1e-5)
    pkg._native.tune("prefill_f32_simt", 1)
    try:
        O_simt, _, _ = _run_flash(pkg, ctx, Q, K, V, B, N, H, D, dtype)
    finally:
        pkg._native.tune("prefill_f32_simt", 0)
    assert not torch.equal(O, O_simt)  # two different kernels ran
    np.testing.assert_allclose(U.to_f32(O), U.to_f32(O_simt), **SPLIT_TOL)


@pytest.mark.parametrize("layout", ["bthd", "bhtd"])
def test_fp32_tensor_core_prefill_fills_the_cache_bit_exact(pkg, ctx, layout):
    gpu = pkg.gpu
    B, N, H, D, dtype = 2, 200, 2, 64, torch.float32
    E = H * D
    Q = U.randn((B, N, E), dtype, ctx.device, 51)
    K = U.randn((B, N, E), dtype, ctx.device, 52)
    V = U.randn((B, N, E), dtype, ctx.device, 53)
    cache = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=B, max_seq_len=N + 24, n_layers=1, n_heads=H,
                                                       head_dim=D, dtype=dtype, layout=layout))
    O, _, _ = _run_flash(pkg, ctx, Q, K, V, B, N, H, D, dtype, cache=cache, stats=False)
    assert cache.current_len == N
    kview = U.logical_view(cache, cache.layers[0], "k")
    vview = U.logical_view(cache, cache.layers[0], "v")
    assert torch.equal(kview[:, :N].reshape(B, N, E), K) and torch.equal(vview[:, :N].reshape(B, N, E), V)
    assert float(kview[:, N:].abs().sum()) == 0.0
    flat = lambda a: U.to_oracle(a.reshape(B * N, E))  # noqa: E731
    Ow, _, _ = c_oracle.prefill(flat(Q), flat(K), flat(V), B, N, H, D, want_stats=False)
    np.testing.assert_allclose(U.to_f32(O), Ow, **SPLIT_TOL)
