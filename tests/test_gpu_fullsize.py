"""GPU parity at the full sizes of the named configurations: the decode microbenchmark
(B=64, H=32, D=128, bf16, lengths ~U[512,8192]), its paged variant (16-token blocks, 65536-block
pool), the prefill shape (B=8, H=32, D=128, N=4096) and the long-context decode (B=4, H=64,
T=131072).  Where the CPU oracle is fast enough it checks every output; elsewhere it checks a
sample of (sequence, head) pairs and size-independent properties cover the rest."""
import numpy as np
import pytest
import torch

from oracle import c_oracle
from tests import kv_util as U

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx(pkg):
    return U.make_ctx(pkg)


def _fill_random(buf, seed):
    flat = buf.view(-1)
    g = torch.Generator(device=buf.device).manual_seed(seed)
    slab = 1 << 27
    for off in range(0, flat.numel(), slab):
        n = min(slab, flat.numel() - off)
        flat[off:off + n] = torch.randn(n, generator=g, device=buf.device, dtype=torch.float32).to(buf.dtype)


def _decode(pkg, ctx, cache, q):
    gpu = pkg.gpu
    out = torch.empty_like(q)
    gpu.batch_begin(ctx)
    gpu.attention_with_kv_cache(ctx, cache, 0, U.buf2d(pkg, ctx, q), U.buf2d(pkg, ctx, out))
    gpu.batch_commit(ctx)
    torch.cuda.synchronize()
    return out


def test_decode_microbench_and_paged_variant_full_size(pkg, ctx):
    gpu = pkg.gpu
    B, H, D, T_max, bs = 64, 32, 128, 8192, 16
    lens = np.random.default_rng(0).integers(512, 8193, size=B)
    cache = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=B, max_seq_len=T_max, n_layers=1, n_heads=H,
                                                       head_dim=D, dtype=torch.bfloat16, layout="bhtd", ragged=True))
    kbuf, vbuf = cache.layers[0].k_cache.buffer, cache.layers[0].v_cache.buffer
    _fill_random(kbuf, 1)
    _fill_random(vbuf, 2)
    gpu.kv_cache_set_lengths(cache, lens)
    q = U.randn((B, H * D), torch.bfloat16, ctx.device, 3)
    out = _decode(pkg, ctx, cache, q)

    # every output against the CPU oracle (bf16 tolerance of the path: 2e-2 absolute)
    k_host = U.to_oracle(kbuf)
    v_host = U.to_oracle(vbuf)
    want = c_oracle.decode(U.to_oracle(q), k_host, v_host, lens.astype(np.int32), B, H, D,
                           (H * T_max * D, D, T_max * D))
    del k_host, v_host
    np.testing.assert_allclose(U.to_f32(out), want, rtol=0, atol=2e-2)

    # split invariance: another ring configuration and another grid (other cut points) give the same result
    pkg._native.tune("decode_variant", 9)
    pkg._native.tune("decode_grid_per_sm", 1)
    try:
        out2 = _decode(pkg, ctx, cache, q)
    finally:
        pkg._native.tune("decode_variant", 0)
        pkg._native.tune("decode_grid_per_sm", 0)
    assert float((out2.float() - out.float()).abs().max()) <= 4e-3

    # paged variant: the same logical content behind a seeded permutation of a 65536-block pool
    n_blocks = 65536
    max_blocks = T_max // bs
    paged = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=B, max_seq_len=T_max, n_layers=1, n_heads=H,
                                                       head_dim=D, dtype=torch.bfloat16, ragged=True, block_size=bs,
                                                       n_blocks=n_blocks))
    perm = np.random.default_rng(0).permutation(n_blocks)[: B * max_blocks].astype(np.int64)
    table = torch.from_numpy(perm).to(ctx.device)
    paged.block_table = table.to(torch.int32).reshape(B, max_blocks)
    for src, dst in ((kbuf, paged.layers[0].k_cache.buffer), (vbuf, paged.layers[0].v_cache.buffer)):
        blocks = src.reshape(B, H, max_blocks, bs, D).permute(0, 2, 1, 3, 4).reshape(B * max_blocks, H, bs, D)
        dst.reshape(n_blocks, H, bs, D)[table] = blocks
        del blocks
    gpu.kv_cache_set_lengths(paged, lens)
    out_paged = _decode(pkg, ctx, paged, q)
    # The same rows behind the table: the same result, bit for bit, from the same kernel (by default a contiguous
    # cache runs two CTAs of three stages per SM and a paged one three of two, which cut the sums elsewhere).
    pkg._native.tune("decode_variant", 17)
    try:
        out_same_kernel = _decode(pkg, ctx, cache, q)
        assert torch.equal(out_paged.view(torch.int16), _decode(pkg, ctx, paged, q).view(torch.int16))
    finally:
        pkg._native.tune("decode_variant", 0)
    assert torch.equal(out_paged.view(torch.int16), out_same_kernel.view(torch.int16))
    assert float((out_paged.float() - out.float()).abs().max()) <= 4e-3

    # one appended row per sequence through the block table, then attention over len + 1
    nk = U.randn((B, H * D), torch.bfloat16, ctx.device, 4)
    nv = U.randn((B, H * D), torch.bfloat16, ctx.device, 5)
    grow = lens < T_max  # a full sequence cannot take another row
    for c in (cache, paged):
        gpu.kv_cache_set_lengths(c, np.where(grow, lens, lens - 1))
        gpu.batch_begin(ctx)
        gpu.kv_cache_update(ctx, c, 0, U.buf2d(pkg, ctx, nk), U.buf2d(pkg, ctx, nv))
        gpu.batch_commit(ctx)
    pkg._native.tune("decode_variant", 17)
    try:
        a = _decode(pkg, ctx, cache, q)
        b = _decode(pkg, ctx, paged, q)
    finally:
        pkg._native.tune("decode_variant", 0)
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    assert cache.seq_lens.cpu().tolist() == np.where(grow, lens + 1, lens).tolist()


def test_prefill_full_size_sampled_oracle_and_properties(pkg, ctx):
    gpu = pkg.gpu
    B, N, H, D = 8, 4096, 32, 128
    E = H * D
    Q = U.randn((B * N, E), torch.bfloat16, ctx.device, 11)
    K = U.randn((B * N, E), torch.bfloat16, ctx.device, 12)
    V = U.randn((B * N, E), torch.bfloat16, ctx.device, 13)
    cache = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=B, max_seq_len=N, n_layers=1, n_heads=H, head_dim=D,
                                                       dtype=torch.bfloat16, layout="bhtd"))
    ctx.config.flash_attn_max_head_dim = 128
    O = torch.empty_like(Q)
    L = gpu.gpu_buffer_1d_create(ctx, B * N * H)
    M = gpu.gpu_buffer_1d_create(ctx, B * N * H)
    gpu.batch_begin(ctx)
    gpu.flash_attention(ctx, U.buf2d(pkg, ctx, Q), U.buf2d(pkg, ctx, K), U.buf2d(pkg, ctx, V), U.buf2d(pkg, ctx, O), L,
                        M, B, N, H, D, cache=cache, layer_idx=0)
    gpu.batch_commit(ctx)
    torch.cuda.synchronize()
    # fused cache write: bit-exact rows, every sequence and head
    kc = cache.layers[0].k_cache.buffer.reshape(B, H, N, D).permute(0, 2, 1, 3).reshape(B * N, E)
    vc = cache.layers[0].v_cache.buffer.reshape(B, H, N, D).permute(0, 2, 1, 3).reshape(B * N, E)
    assert torch.equal(kc, K) and torch.equal(vc, V)
    assert cache.current_len == N
    # sampled (sequence, head) pairs against the CPU oracle
    Lh = L.buffer.reshape(B, N, H)
    Mh = M.buffer.reshape(B, N, H)
    for b, h in [(0, 0), (3, 17), (7, 31)]:
        sl = lambda X: U.to_oracle(X.reshape(B, N, H, D)[b, :, h, :].contiguous())  # noqa: E731
        Ow, Lw, Mw = c_oracle.prefill(sl(Q), sl(K), sl(V), 1, N, 1, D)
        got = U.to_f32(O.reshape(B, N, H, D)[b, :, h, :])
        np.testing.assert_allclose(got, Ow, rtol=0, atol=2e-2)
        np.testing.assert_allclose(Lh[b, :, h].cpu().numpy(), Lw, rtol=2e-3, atol=1e-4)
        np.testing.assert_allclose(Mh[b, :, h].cpu().numpy(), Mw, rtol=1e-4, atol=1e-4)
    # the tensor-core kernel and the SIMT kernel agree everywhere
    pkg._native.tune("prefill_force_simt", 1)
    try:
        O2 = torch.empty_like(Q)
        gpu.batch_begin(ctx)
        gpu.flash_attention(ctx, U.buf2d(pkg, ctx, Q), U.buf2d(pkg, ctx, K), U.buf2d(pkg, ctx, V),
                            U.buf2d(pkg, ctx, O2), None, None, B, N, H, D)
        gpu.batch_commit(ctx)
        torch.cuda.synchronize()
    finally:
        pkg._native.tune("prefill_force_simt", 0)
    assert float((O.float() - O2.float()).abs().max()) <= 2e-2
    # row 0 of every sequence attends to itself only: O[0] == V[0] exactly
    assert torch.equal(O.reshape(B, N, E)[:, 0], V.reshape(B, N, E)[:, 0])
    # decode of the last token over the prefilled cache reproduces the prefill's last row
    q_last = Q.reshape(B, N, E)[:, N - 1].contiguous()
    out = _decode(pkg, ctx, cache, q_last)
    assert float((out.float() - O.reshape(B, N, E)[:, N - 1].float()).abs().max()) <= 2e-2


def test_long_context_decode_full_size_sampled_oracle(pkg, ctx):
    gpu = pkg.gpu
    B, H, D, T = 4, 64, 128, 131072
    cache = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=B, max_seq_len=T, n_layers=1, n_heads=H, head_dim=D,
                                                       dtype=torch.bfloat16, layout="bhtd"))
    kbuf, vbuf = cache.layers[0].k_cache.buffer, cache.layers[0].v_cache.buffer
    _fill_random(kbuf, 21)
    _fill_random(vbuf, 22)
    cache.current_len = T
    q = U.randn((B, H * D), torch.bfloat16, ctx.device, 23)
    out = _decode(pkg, ctx, cache, q)
    k4, v4 = kbuf.reshape(B, H, T, D), vbuf.reshape(B, H, T, D)
    for b, h in [(0, 0), (1, 33), (3, 63)]:
        want = c_oracle.decode(U.to_oracle(q.reshape(B, H, D)[b, h].reshape(1, D).contiguous()),
                               U.to_oracle(k4[b, h].contiguous()), U.to_oracle(v4[b, h].contiguous()), T, 1, 1, D,
                               (T * D, D, T * D))
        got = U.to_f32(out.reshape(B, H, D)[b, h])
        np.testing.assert_allclose(got, want[0], rtol=0, atol=2e-2)
    # softmax weights sum to one at any length: V == 1 gives 1
    vbuf.fill_(1.0)
    ones = _decode(pkg, ctx, cache, q)
    assert torch.allclose(ones.float(), torch.ones_like(ones, dtype=torch.float32), atol=1e-2)


def test_prefill_full_size_into_a_paged_cache_and_fp32_on_the_tensor_cores(pkg, ctx):
    """The prefill configuration (B=8, H=32, D=128, N=4096, bf16) into a paged cache of 16-token blocks: the tensor-core
    kernel stores the blocks itself, the output is bit-identical to the run into a contiguous cache and the pool
    gathers back to K and V bit-exactly.  Then the same shape cut to two sequences in fp32 (split-bfloat16 operands),
    sampled against the oracle."""
    gpu = pkg.gpu
    B, H, D, N, bs = 8, 32, 128, 4096, 16
    E = H * D
    dtype = torch.bfloat16
    Q = U.randn((B * N, E), dtype, ctx.device, 61)
    K = U.randn((B * N, E), dtype, ctx.device, 62)
    V = U.randn((B * N, E), dtype, ctx.device, 63)
    outs = []
    for paged in (False, True):
        cfg = dict(batch_size=B, max_seq_len=N, n_layers=1, n_heads=H, head_dim=D, dtype=dtype)
        cfg.update(dict(block_size=bs, n_blocks=B * N // bs + 11) if paged else dict(layout="bhtd"))
        cache = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(**cfg))
        if paged:
            perm = torch.randperm(cache.n_blocks, generator=torch.Generator().manual_seed(3))[: B * N // bs]
            cache.block_table.copy_(perm.to(torch.int32).reshape(B, N // bs).to(ctx.device))
        O = torch.empty_like(Q)
        gpu.batch_begin(ctx)
        gpu.flash_attention(ctx, U.buf2d(pkg, ctx, Q), U.buf2d(pkg, ctx, K), U.buf2d(pkg, ctx, V), U.buf2d(pkg, ctx, O),
                            None, None, B, N, H, D, cache=cache, layer_idx=0)
        gpu.batch_commit(ctx)
        outs.append(O)
        if paged:
            gpu.batch_begin(ctx)
            for which, src in (("k", K), ("v", V)):
                rows = gpu.kv_cache_gather(ctx, cache, 0, which, length=N)
                assert torch.equal(rows.reshape(B * N, E), src)
                del rows
            gpu.batch_commit(ctx)
        del cache
    assert torch.equal(outs[0], outs[1])
    del outs, Q, K, V
    torch.cuda.empty_cache()
    B2 = 2
    Qf = U.randn((B2 * N, E), torch.float32, ctx.device, 64)
    Kf = U.randn((B2 * N, E), torch.float32, ctx.device, 65)
    Vf = U.randn((B2 * N, E), torch.float32, ctx.device, 66)
    Of = torch.empty_like(Qf)
    gpu.batch_begin(ctx)
    gpu.flash_attention(ctx, U.buf2d(pkg, ctx, Qf), U.buf2d(pkg, ctx, Kf), U.buf2d(pkg, ctx, Vf), U.buf2d(pkg, ctx, Of),
                        None, None, B2, N, H, D)
    gpu.batch_commit(ctx)
    torch.cuda.synchronize()
    for b, h in [(0, 0), (1, 31)]:
        sl = lambda X: U.to_oracle(X.reshape(B2, N, H, D)[b, :, h].contiguous())  # noqa: E731
        Ow, _, _ = c_oracle.prefill(sl(Qf), sl(Kf), sl(Vf), 1, N, 1, D, want_stats=False)
        np.testing.assert_allclose(Of.reshape(B2, N, H, D)[b, :, h].cpu().numpy(), Ow, rtol=1e-4, atol=3e-5)
