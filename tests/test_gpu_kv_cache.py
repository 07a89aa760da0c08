"""GPU parity: cache append / gather (bit-exact) and decode attention against the oracle,
through the reference-shaped API (which calls the C-ABI library)."""
import numpy as np
import pytest
import torch

from oracle import kv_oracle
from tests import kv_util as U

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx(pkg):
    return U.make_ctx(pkg)


# ---------------------------------------------------------------------------------------
# the reference's own test recipe (simple-llm/src/gpu_test.py:2200-2406)
# ---------------------------------------------------------------------------------------

@pytest.mark.parametrize("layout,block_size", [("bthd", 0), ("bhtd", 0), ("bhtd", 16)])
def test_reference_kv_recipe(pkg, ctx, golden, layout, block_size):
    gpu = pkg.gpu
    B, T_max, L, H, D = 2, 128, 2, 4, 64
    E = H * D
    cache = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=B, max_seq_len=T_max, n_layers=L, n_heads=H,
                                                       head_dim=D, layout=layout, block_size=block_size))
    assert len(cache.layers) == L and cache.current_len == 0
    cache.current_len = 50
    gpu.kv_cache_reset(cache)
    assert cache.current_len == 0
    ks, vs, Q = kv_oracle.recipe_kv_cache_inputs(B, H, D, 5, seed=42)
    for step in range(1, 6):
        nk = gpu.gpu_buffer_2d_create(ctx, B, E, ks[step - 1].reshape(B, E))
        nv = gpu.gpu_buffer_2d_create(ctx, B, E, vs[step - 1].reshape(B, E))
        gpu.batch_begin(ctx)
        gpu.kv_cache_update(ctx, cache, 0, nk, nv)
        gpu.batch_commit(ctx)
        assert cache.current_len == step
    q = gpu.gpu_buffer_2d_create(ctx, B, E, Q.reshape(B, E))
    o = gpu.gpu_buffer_2d_create(ctx, B, E)
    gpu.batch_begin(ctx)
    gpu.attention_with_kv_cache(ctx, cache, 0, q, o)
    gpu.batch_commit(ctx)
    got = np.zeros((B, E), dtype=np.float32)
    gpu.gpu_buffer_2d_read(ctx, o, got)
    # the reference test's tolerance (gpu_test.py:2431) is rtol 1e-4, atol 1e-3; ours is tighter
    np.testing.assert_allclose(got, golden["kv_out"], rtol=1e-4, atol=1e-5)
    # the cache rows themselves, which the reference never reads back: bit-exact
    gpu.batch_begin(ctx)
    kg = gpu.kv_cache_gather(ctx, cache, 0, "k", length=8)
    vg = gpu.kv_cache_gather(ctx, cache, 0, "v", length=8)
    gpu.batch_commit(ctx)
    assert np.array_equal(kg[:, :5].cpu().numpy(), np.concatenate(ks, axis=1))
    assert np.array_equal(vg[:, :5].cpu().numpy(), np.concatenate(vs, axis=1))
    assert float(kg[:, 5:].abs().sum()) == 0.0
    # layer 1 was never written
    assert float(cache.layers[1].k_cache.buffer.abs().sum()) == 0.0


# ---------------------------------------------------------------------------------------
# append / gather, bit-exact, every layout and storage type, ragged positions
# ---------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("layout,block_size", [("bthd", 0), ("bhtd", 0), ("bhtd", 16), ("bhtd", 4)])
def test_append_gather_bit_exact_ragged(pkg, ctx, dtype, layout, block_size):
    gpu = pkg.gpu
    B, T_max, H, D = 5, 40, 3, 32
    E = H * D
    max_blocks = (T_max + max(block_size, 1) - 1) // max(block_size, 1)
    n_blocks = 3 * B * max_blocks if block_size else 0
    cache = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=B, max_seq_len=T_max, n_layers=1, n_heads=H,
                                                       head_dim=D, dtype=dtype, layout=layout, ragged=True,
                                                       block_size=block_size, n_blocks=n_blocks))
    if block_size:
        perm = torch.randperm(n_blocks, generator=torch.Generator().manual_seed(3))[: B * max_blocks]
        cache.block_table = perm.to(torch.int32).reshape(B, max_blocks).to(ctx.device)
    start = [0, 1, 7, 16, 33]
    gpu.kv_cache_set_lengths(cache, start)
    want_k = torch.zeros(B, T_max, H, D, dtype=dtype)
    want_v = torch.zeros(B, T_max, H, D, dtype=dtype)
    steps = 6
    for s in range(steps):
        nk = U.randn((B, E), dtype, ctx.device, 100 + s)
        nv = U.randn((B, E), dtype, ctx.device, 200 + s)
        for b in range(B):
            want_k[b, start[b] + s] = nk[b].cpu().reshape(H, D)
            want_v[b, start[b] + s] = nv[b].cpu().reshape(H, D)
        gpu.batch_begin(ctx)
        gpu.kv_cache_update(ctx, cache, 0, U.buf2d(pkg, ctx, nk), U.buf2d(pkg, ctx, nv))
        gpu.batch_commit(ctx)
    assert cache.seq_lens.cpu().tolist() == [x + steps for x in start]
    assert cache.current_len == max(start) + steps
    gpu.batch_begin(ctx)
    kg = gpu.kv_cache_gather(ctx, cache, 0, "k").cpu()
    vg = gpu.kv_cache_gather(ctx, cache, 0, "v").cpu()
    gpu.batch_commit(ctx)
    for b in range(B):
        lo, hi = start[b], start[b] + steps
        assert torch.equal(kg[b, lo:hi].view(torch.uint8), want_k[b, lo:hi].view(torch.uint8))
        assert torch.equal(vg[b, lo:hi].view(torch.uint8), want_v[b, lo:hi].view(torch.uint8))
        assert float(kg[b, hi:].float().abs().sum()) == 0.0  # gather zero-fills past the length
        assert float(kg[b, :lo].float().abs().sum()) == 0.0  # rows below the start were never written
    if not block_size:
        # nothing outside the appended rows was touched in the physical buffer either
        phys = U.logical_view(cache, cache.layers[0], "k").cpu()
        mask = torch.ones(B, T_max, dtype=torch.bool)
        for b in range(B):
            mask[b, start[b] : start[b] + steps] = False
        assert float(phys[mask].float().abs().sum()) == 0.0


def test_append_bad_block_sets_status_and_does_not_fault(pkg, ctx):
    gpu = pkg.gpu
    cache = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=2, max_seq_len=32, n_layers=1, n_heads=2,
                                                       head_dim=16, block_size=16, n_blocks=8))
    cache.block_table[1, 0] = 99  # outside the pool of 8 blocks
    nk = U.randn((2, 32), torch.float32, ctx.device, 1)
    ctx.dev_status = None
    gpu.batch_begin(ctx)
    gpu.kv_cache_update(ctx, cache, 0, U.buf2d(pkg, ctx, nk), U.buf2d(pkg, ctx, nk))
    gpu.batch_commit(ctx)
    torch.cuda.synchronize()
    assert int(ctx.dev_status.item()) == 1  # B2KV_DEV_BAD_BLOCK
    ctx.dev_status.zero_()
    # sequence 0 was written, sequence 1 skipped
    pool = cache.layers[0].k_cache.buffer.reshape(8, 2, 16, 16)
    assert torch.equal(pool[0, :, 0, :].reshape(-1), nk[0])
    assert float(pool[1:].abs().sum()) == 0.0


# ---------------------------------------------------------------------------------------
# decode attention against the oracle
# ---------------------------------------------------------------------------------------

def _decode_case(pkg, ctx, dtype, layout, block_size, B, H, D, T_max, lens, seed=0, poison=True):
    gpu = pkg.gpu
    E = H * D
    max_blocks = (T_max + max(block_size, 1) - 1) // max(block_size, 1)
    n_blocks = 2 * B * max_blocks if block_size else 0
    cache = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=B, max_seq_len=T_max, n_layers=1, n_heads=H,
                                                       head_dim=D, dtype=dtype, layout=layout, ragged=True,
                                                       block_size=block_size, n_blocks=n_blocks))
    if block_size:
        perm = torch.randperm(n_blocks, generator=torch.Generator().manual_seed(seed + 5))[: B * max_blocks]
        cache.block_table = perm.to(torch.int32).reshape(B, max_blocks).to(ctx.device)
    k_log = U.randn((B, T_max, H, D), dtype, ctx.device, seed + 1)
    v_log = U.randn((B, T_max, H, D), dtype, ctx.device, seed + 2)
    q = U.randn((B, E), dtype, ctx.device, seed + 3)
    if poison:
        # rows past each length hold NaN: an over-read would poison the output
        for b in range(B):
            k_log[b, lens[b]:] = float("nan")
            v_log[b, lens[b]:] = float("nan")
    U.fill_cache_logical(cache, 0, k_log, v_log)
    gpu.kv_cache_set_lengths(cache, lens)
    out = torch.empty((B, E), dtype=dtype, device=ctx.device)
    gpu.batch_begin(ctx)
    gpu.attention_with_kv_cache(ctx, cache, 0, U.buf2d(pkg, ctx, q), U.buf2d(pkg, ctx, out))
    gpu.batch_commit(ctx)
    torch.cuda.synchronize()
    want = U.oracle_decode(q, torch.nan_to_num(k_log), torch.nan_to_num(v_log), lens)
    return U.to_f32(out), want


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D", [16, 32, 64, 128, 256])
def test_decode_every_head_dim(pkg, ctx, dtype, D):
    lens = [1, 63, 64, 65, 300]
    got, want = _decode_case(pkg, ctx, dtype, "bhtd", 0, B=5, H=3, D=D, T_max=320, lens=lens, seed=D)
    assert np.isfinite(got).all()
    np.testing.assert_allclose(got, want, **U.TOL[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("layout,block_size", [("bthd", 0), ("bhtd", 0), ("bhtd", 16), ("bhtd", 64), ("bhtd", 128),
                                               ("bhtd", 48)])
def test_decode_layouts_ragged_with_empty_sequence(pkg, ctx, dtype, layout, block_size):
    D = 128 if dtype == torch.bfloat16 else 64
    lens = [0, 5, 129, 1000, 2048, 777]
    got, want = _decode_case(pkg, ctx, dtype, layout, block_size, B=6, H=4, D=D, T_max=2048, lens=lens, seed=11)
    assert np.all(got[0] == 0.0)  # an empty sequence gives zeros
    np.testing.assert_allclose(got, want, **U.TOL[dtype])


def test_decode_uniform_length_mode_matches_ragged_mode(pkg, ctx):
    gpu = pkg.gpu
    B, H, D, T_max, n = 3, 2, 64, 512, 300
    k_log = U.randn((B, T_max, H, D), torch.float32, ctx.device, 1)
    v_log = U.randn((B, T_max, H, D), torch.float32, ctx.device, 2)
    q = U.randn((B, H * D), torch.float32, ctx.device, 3)
    outs = []
    for ragged in (False, True):
        cache = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=B, max_seq_len=T_max, n_layers=1, n_heads=H,
                                                           head_dim=D, ragged=ragged))
        U.fill_cache_logical(cache, 0, k_log, v_log)
        if ragged:
            gpu.kv_cache_set_lengths(cache, [n] * B)
        else:
            cache.current_len = n
        out = torch.empty((B, H * D), dtype=torch.float32, device=ctx.device)
        gpu.batch_begin(ctx)
        gpu.attention_with_kv_cache(ctx, cache, 0, U.buf2d(pkg, ctx, q), U.buf2d(pkg, ctx, out))
        gpu.batch_commit(ctx)
        outs.append(out.cpu())
    assert torch.equal(outs[0], outs[1])
    want = U.oracle_decode(q, k_log, v_log, [n] * B)
    np.testing.assert_allclose(outs[0].numpy(), want, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("variant,per_sm", [(0, 0), (0, 1), (0, 2), (1, 0), (2, 0), (3, 0), (4, 1), (5, 3), (6, 0),
                                            (7, 4), (8, 0), (9, 0), (10, 0), (11, 0), (12, 0), (13, 0), (14, 0),
                                            (15, 0), (16, 0)])
def test_decode_kernel_variants_agree_with_oracle(pkg, ctx, variant, per_sm):
    pkg._native.tune("decode_variant", variant)
    pkg._native.tune("decode_grid_per_sm", per_sm)
    try:
        lens = [2048, 1, 1500, 31, 2000, 513]
        got, want = _decode_case(pkg, ctx, torch.bfloat16, "bhtd", 0, B=6, H=8, D=128, T_max=2048, lens=lens, seed=7)
        np.testing.assert_allclose(got, want, **U.TOL[torch.bfloat16])
        got, want = _decode_case(pkg, ctx, torch.bfloat16, "bhtd", 16, B=6, H=8, D=128, T_max=2048, lens=lens, seed=7)
        np.testing.assert_allclose(got, want, **U.TOL[torch.bfloat16])
    finally:
        pkg._native.tune("decode_variant", 0)
        pkg._native.tune("decode_grid_per_sm", 0)


def test_decode_softmax_weights_sum_to_one(pkg, ctx):
    """Size-independent property: with V == 1 everywhere the output is 1 whatever K and q are."""
    gpu = pkg.gpu
    B, H, D, T_max = 4, 8, 128, 8192
    lens = [8192, 4097, 512, 6000]
    cache = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=B, max_seq_len=T_max, n_layers=1, n_heads=H,
                                                       head_dim=D, dtype=torch.bfloat16, layout="bhtd", ragged=True))
    cache.layers[0].k_cache.buffer.copy_(U.randn(cache.layers[0].k_cache.shape, torch.bfloat16, ctx.device, 5))
    cache.layers[0].v_cache.buffer.fill_(1.0)
    gpu.kv_cache_set_lengths(cache, lens)
    q = U.randn((B, H * D), torch.bfloat16, ctx.device, 6)
    out = torch.empty_like(q)
    gpu.batch_begin(ctx)
    gpu.attention_with_kv_cache(ctx, cache, 0, U.buf2d(pkg, ctx, q), U.buf2d(pkg, ctx, out))
    gpu.batch_commit(ctx)
    assert torch.allclose(out.float(), torch.ones_like(out, dtype=torch.float32), atol=1e-2)


def test_decode_paged_equals_contiguous(pkg, ctx):
    lens = [1500, 16, 17, 4096]
    a, want = _decode_case(pkg, ctx, torch.bfloat16, "bhtd", 0, B=4, H=4, D=128, T_max=4096, lens=lens, seed=21)
    b, _ = _decode_case(pkg, ctx, torch.bfloat16, "bhtd", 16, B=4, H=4, D=128, T_max=4096, lens=lens, seed=21)
    np.testing.assert_allclose(a, want, **U.TOL[torch.bfloat16])
    assert np.array_equal(a, b)  # same tiles, same order of operations: identical bits


def test_decode_bad_block_reports_status(pkg, ctx):
    gpu = pkg.gpu
    cache = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=1, max_seq_len=64, n_layers=1, n_heads=2,
                                                       head_dim=64, block_size=16, n_blocks=4))
    cache.block_table[0, 1] = -7
    cache.current_len = 40
    q = U.randn((1, 128), torch.float32, ctx.device, 1)
    out = torch.empty_like(q)
    ctx.dev_status = None
    gpu.batch_begin(ctx)
    gpu.attention_with_kv_cache(ctx, cache, 0, U.buf2d(pkg, ctx, q), U.buf2d(pkg, ctx, out))
    gpu.batch_commit(ctx)
    torch.cuda.synchronize()
    assert int(ctx.dev_status.item()) == 1
    ctx.dev_status.zero_()
    ctx.config.check_device_status = False


def test_multi_layer_decode_loop_with_the_reference_quirk(pkg, ctx):
    """kv_cache_update advances current_len on every call (gpu_kv_cache.py:186); a two-layer
    loop sets it back before the second layer's update, or passes advance=False."""
    gpu = pkg.gpu
    B, H, D, T_max, L = 2, 2, 64, 64, 2
    E = H * D
    cache = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=B, max_seq_len=T_max, n_layers=L, n_heads=H,
                                                       head_dim=D))
    ks = [[U.randn((B, E), torch.float32, ctx.device, 10 * t + l) for l in range(L)] for t in range(3)]
    for t in range(3):
        for l in range(L):
            gpu.batch_begin(ctx)
            gpu.kv_cache_update(ctx, cache, l, U.buf2d(pkg, ctx, ks[t][l]), U.buf2d(pkg, ctx, ks[t][l]),
                                advance=(l == L - 1))
            gpu.batch_commit(ctx)
        assert cache.current_len == t + 1
    for l in range(L):
        view = U.logical_view(cache, cache.layers[l], "k")
        for t in range(3):
            assert torch.equal(view[:, t].reshape(B, E), ks[t][l])


def test_batch_commit_raises_on_device_status_when_asked(pkg, ctx):
    gpu = pkg.gpu
    cache = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=1, max_seq_len=32, n_layers=1, n_heads=2,
                                                       head_dim=16, block_size=16, n_blocks=2))
    cache.block_table[0, 0] = 5  # outside the pool
    nk = U.randn((1, 32), torch.float32, ctx.device, 1)
    ctx.dev_status = None
    ctx.config.check_device_status = True
    try:
        gpu.batch_begin(ctx)
        gpu.kv_cache_update(ctx, cache, 0, U.buf2d(pkg, ctx, nk), U.buf2d(pkg, ctx, nk))
        with pytest.raises(RuntimeError, match="block-table entry points outside the pool"):
            gpu.batch_commit(ctx)
        assert int(ctx.dev_status.item()) == 0  # cleared after it was reported
    finally:
        ctx.config.check_device_status = False


@pytest.mark.parametrize("seed", range(16))
def test_decode_random_shapes_against_oracle(pkg, ctx, seed):
    """Randomised shapes: batch, heads, head_dim, storage type, layout, block size and ragged
    lengths (with empty sequences) drawn from a seeded generator."""
    rng = np.random.default_rng(1000 + seed)
    dtype = [torch.float32, torch.bfloat16][int(rng.integers(0, 2))]
    D = int(rng.choice([16, 32, 64, 128, 256]))
    B = int(rng.integers(1, 71))
    H = int(rng.integers(1, 10))
    T_max = int(rng.choice([1, 7, 64, 65, 200, 1025, 3000]))
    if B * H * T_max * D > 60_000_000:  # keep the oracle quick
        B = max(1, 60_000_000 // (H * T_max * D))
    layout, block_size = [("bthd", 0), ("bhtd", 0), ("bhtd", 16), ("bhtd", 32), ("bhtd", 5)][int(rng.integers(0, 5))]
    lens = rng.integers(0, T_max + 1, size=B)
    if rng.random() < 0.3:
        lens[rng.integers(0, B)] = 0
    lens[rng.integers(0, B)] = T_max  # at least one full sequence
    got, want = _decode_case(pkg, ctx, dtype, layout, block_size, B=B, H=H, D=D, T_max=T_max, lens=lens.tolist(),
                             seed=seed)
    assert np.isfinite(got).all()
    for b in range(B):
        if lens[b] == 0:
            assert np.all(got[b] == 0.0)
    np.testing.assert_allclose(got, want, **U.TOL[dtype])


@pytest.mark.parametrize("B,H,T", [(1, 1, 60000), (2, 1, 40000), (1, 2, 50000), (3, 4, 9000)])
@pytest.mark.parametrize("merge_kernel", [0, 1])
def test_decode_one_pair_over_hundreds_of_ctas(pkg, ctx, B, H, T, merge_kernel):
    """Few (sequence, head) pairs and long sequences: a pair is cut into hundreds of pieces (more than 255 for one
    pair of 60000 tokens on 444 CTAs), each CTA holds one, and whoever finishes a pair's last piece merges them all.
    With the merge inside the split kernel and with the separate merge kernel; the two agree bit for bit."""
    D, dtype = 128, torch.bfloat16
    lens = [T] + [T // 3] * (B - 1)
    outs = []
    for which in (merge_kernel, 1 - merge_kernel):
        pkg._native.tune("decode_merge_kernel", which)
        try:
            got, want = _decode_case(pkg, ctx, dtype, "bhtd", 0, B=B, H=H, D=D, T_max=T, lens=lens, seed=77, poison=False)
        finally:
            pkg._native.tune("decode_merge_kernel", 0)
        np.testing.assert_allclose(got, want, **U.TOL[dtype])
        outs.append(got)
    assert np.array_equal(outs[0], outs[1])


def test_decode_replayed_from_a_cuda_graph(pkg, ctx):
    """A decode launch captured into a CUDA graph and replayed with new queries and new lengths (both on the device):
    every replay equals the eager call on the same inputs, bit for bit, although the replays carry the launch number
    they were captured with.  Few pairs and long sequences, so every pair is cut over many CTAs and merged through
    the tickets in the workspace."""
    gpu = pkg.gpu
    B, H, D, T, dtype = 2, 2, 128, 20000, torch.bfloat16
    E = H * D
    cache = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=B, max_seq_len=T, n_layers=1, n_heads=H, head_dim=D,
                                                       dtype=dtype, layout="bhtd", ragged=True))
    cache.layers[0].k_cache.buffer.copy_(U.randn((B * H * T, D), dtype, ctx.device, 1))
    cache.layers[0].v_cache.buffer.copy_(U.randn((B * H * T, D), dtype, ctx.device, 2))
    gpu.kv_cache_set_lengths(cache, [T, T // 2])
    cache.current_len = T  # the upper bound that sizes the launch stays fixed
    q, out = U.randn((B, E), dtype, ctx.device, 3), torch.empty((B, E), dtype=dtype, device=ctx.device)
    qb, ob = U.buf2d(pkg, ctx, q), U.buf2d(pkg, ctx, out)

    def launch():
        gpu.batch_begin(ctx)
        gpu.attention_with_kv_cache(ctx, cache, 0, qb, ob)
        gpu.batch_commit(ctx)

    side = torch.cuda.Stream(device=ctx.device)
    side.wait_stream(torch.cuda.current_stream(ctx.device))
    with torch.cuda.stream(side):
        launch()  # first-use set-up outside the capture
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            launch()
    torch.cuda.current_stream(ctx.device).wait_stream(side)
    for i, lens in enumerate([[T, T // 2], [777, T], [T - 1, 1], [12345, 6789]]):
        q.copy_(U.randn((B, E), dtype, ctx.device, 10 + i))
        cache.seq_lens.copy_(torch.tensor(lens, dtype=torch.int32))
        graph.replay()
        torch.cuda.synchronize()
        replayed = out.clone()
        launch()
        torch.cuda.synchronize()
        assert torch.equal(replayed.view(torch.int16), out.view(torch.int16)), f"replay {i}"
        k4 = cache.layers[0].k_cache.buffer.view(B, H, T, D).permute(0, 2, 1, 3)
        v4 = cache.layers[0].v_cache.buffer.view(B, H, T, D).permute(0, 2, 1, 3)
        want = U.oracle_decode(q, k4.contiguous(), v4.contiguous(), lens)
        np.testing.assert_allclose(U.to_f32(replayed), want, **U.TOL[dtype])


@pytest.mark.parametrize("dtype,layout,block_size,B,H,D,T,merge_kernel", [
    (torch.bfloat16, "bhtd", 0, 6, 8, 128, 9000, 0),    # several chunks per CTA, pairs cut into many pieces
    (torch.bfloat16, "bhtd", 0, 6, 8, 128, 9000, 1),    # the same through the separate merge kernel
    (torch.bfloat16, "bhtd", 16, 5, 4, 128, 7000, 0),   # paged
    (torch.float32, "bthd", 0, 3, 4, 64, 5000, 0),      # the reference's row layout and type
    (torch.bfloat16, "bhtd", 0, 40, 2, 128, 300, 0),    # short sequences: chunks hold many whole pairs
    (torch.bfloat16, "bhtd", 0, 300, 2, 64, 260, 0),    # more sequences than a warp scans at once, 128-byte rows
    (torch.float32, "bhtd", 0, 70, 1, 256, 900, 1),     # one head, 1 KB rows, through the merge kernel
])
def test_decode_with_small_chunks_handed_out_on_demand(pkg, ctx, dtype, layout, block_size, B, H, D, T, merge_kernel):
    """The launch of a long batch deals three quarters of the caches out in advance and the rest as small chunks
    that a CTA takes from a counter when it has finished what it had (knob ``decode_dynamic_chunks``: 1 forces
    that for any size, 2 forbids it).  Which CTA takes which chunk differs from run to run, the cuts do not: two
    runs agree bit for bit, both forms agree with the oracle, and with each other within the tolerance (they cut
    the sums in different places)."""
    rng = np.random.default_rng(B * 31 + T)
    lens = [int(x) for x in rng.integers(1, T + 1, size=B)]
    lens[0] = T
    if B > 2:
        lens[1] = 0
    outs = {}
    for mode in (1, 1, 2):
        pkg._native.tune("decode_dynamic_chunks", mode)
        pkg._native.tune("decode_merge_kernel", merge_kernel)
        try:
            got, want = _decode_case(pkg, ctx, dtype, layout, block_size, B=B, H=H, D=D, T_max=T, lens=lens, seed=5)
        finally:
            pkg._native.tune("decode_dynamic_chunks", 0)
            pkg._native.tune("decode_merge_kernel", 0)
        np.testing.assert_allclose(got, want, **U.TOL[dtype])
        outs.setdefault(mode, []).append(got)
    assert np.array_equal(outs[1][0], outs[1][1])
    np.testing.assert_allclose(outs[1][0], outs[2][0], **U.TOL[dtype])


def test_decode_with_chunks_on_demand_replayed_from_a_cuda_graph(pkg, ctx):
    """The chunk counter of a launch goes back to zero with the launch's last request, so a launch replayed from a
    CUDA graph (which carries the launch number it was captured with) hands its chunks out afresh every time."""
    gpu = pkg.gpu
    B, H, D, T, dtype = 3, 4, 128, 12000, torch.bfloat16
    E = H * D
    cache = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=B, max_seq_len=T, n_layers=1, n_heads=H, head_dim=D,
                                                       dtype=dtype, layout="bhtd", ragged=True))
    cache.layers[0].k_cache.buffer.copy_(U.randn((B * H * T, D), dtype, ctx.device, 1))
    cache.layers[0].v_cache.buffer.copy_(U.randn((B * H * T, D), dtype, ctx.device, 2))
    gpu.kv_cache_set_lengths(cache, [T, T // 2, 100])
    cache.current_len = T  # the upper bound that sizes the launch stays fixed
    q, out = U.randn((B, E), dtype, ctx.device, 3), torch.empty((B, E), dtype=dtype, device=ctx.device)
    qb, ob = U.buf2d(pkg, ctx, q), U.buf2d(pkg, ctx, out)

    def launch():
        gpu.batch_begin(ctx)
        gpu.attention_with_kv_cache(ctx, cache, 0, qb, ob)
        gpu.batch_commit(ctx)

    pkg._native.tune("decode_dynamic_chunks", 1)
    try:
        side = torch.cuda.Stream(device=ctx.device)
        side.wait_stream(torch.cuda.current_stream(ctx.device))
        with torch.cuda.stream(side):
            launch()  # first-use set-up outside the capture
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                launch()
        torch.cuda.current_stream(ctx.device).wait_stream(side)
        for i, lens in enumerate([[T, T // 2, 100], [5, T, T], [T - 1, 1, 0], [12345 % T, 6789, 4000]]):
            q.copy_(U.randn((B, E), dtype, ctx.device, 10 + i))
            cache.seq_lens.copy_(torch.tensor(lens, dtype=torch.int32))
            for _ in range(3):
                graph.replay()
            torch.cuda.synchronize()
            replayed = out.clone()
            launch()
            torch.cuda.synchronize()
            assert torch.equal(replayed.view(torch.int16), out.view(torch.int16)), f"replay {i}"
            k4 = cache.layers[0].k_cache.buffer.view(B, H, T, D).permute(0, 2, 1, 3)
            v4 = cache.layers[0].v_cache.buffer.view(B, H, T, D).permute(0, 2, 1, 3)
            want = U.oracle_decode(q, k4.contiguous(), v4.contiguous(), lens)
            np.testing.assert_allclose(U.to_f32(replayed), want, **U.TOL[dtype])
    finally:
        pkg._native.tune("decode_dynamic_chunks", 0)
    assert int(ctx.dev_status.item()) == 0


def test_advance_lengths_in_stream_order(pkg, ctx):
    """``b2kv_advance_lengths`` adds to the device-side lengths of a ragged cache, ordered with the kernels of its
    stream: an append that does not advance, the advance, then a decode over the lengths it left."""
    gpu = pkg.gpu
    B, H, D, T, dtype = 70, 2, 64, 40, torch.bfloat16
    E = H * D
    cache = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=B, max_seq_len=T, n_layers=1, n_heads=H, head_dim=D,
                                                       dtype=dtype, layout="bhtd", ragged=True))
    lens = [int(x) for x in np.random.default_rng(3).integers(0, T - 3, size=B)]
    gpu.kv_cache_set_lengths(cache, lens)
    stream = torch.cuda.current_stream().cuda_stream
    for delta in (1, 2):
        pkg._native.check(pkg._native.lib.b2kv_advance_lengths(cache.seq_lens.data_ptr(), B, delta, stream))
    torch.cuda.synchronize()
    assert cache.seq_lens.cpu().tolist() == [n + 3 for n in lens]
