"""The fused decode + all-gather epilogue (`b2kv_decode_allgather`) on ONE GPU: two head-split
"ranks" are emulated in one process with ordinary device buffers that both can see.  Their calls
are queued one after the other without the wait kernel (a kernel that waits for a flag written
by a kernel queued behind it on the same GPU would never see it), then the buffers and flags are
checked on the host.  A single real rank (world = 1) exercises the wait kernel."""
import numpy as np
import pytest
import torch

from tests import kv_util as U

pytestmark = pytest.mark.gpu


def _make_cache(pkg, ctx, B, H, D, T_max, dtype, k_log, v_log, lens):
    gpu = pkg.gpu
    cache = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=B, max_seq_len=T_max, n_layers=1, n_heads=H,
                                                       head_dim=D, dtype=dtype, layout="bhtd", ragged=True))
    U.fill_cache_logical(cache, 0, k_log, v_log)
    gpu.kv_cache_set_lengths(cache, lens)
    return cache


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_two_emulated_ranks_write_each_others_buffers(pkg, dtype):
    from llm_experiments_b200 import sharding

    ctx = U.make_ctx(pkg)
    gpu = pkg.gpu
    dev = ctx.device
    world, B, H, T_max = 2, 3, 8, 700
    D = 128 if dtype == torch.bfloat16 else 64
    Hl = H // world
    lens = [700, 1, 333]
    k_log = U.randn((B, T_max, H, D), dtype, dev, 1)
    v_log = U.randn((B, T_max, H, D), dtype, dev, 2)
    outs = [torch.full((2, B, H * D), float("nan"), dtype=dtype, device=dev) for _ in range(world)]
    flags = [torch.zeros(world, dtype=torch.int32, device=dev) for _ in range(world)]
    ranks, caches = [], []
    for r in range(world):
        ranks.append(sharding.FusedHeadGather.from_buffers(dev, r, world, B, H, D, dtype, outs, flags))
        caches.append(_make_cache(pkg, ctx, B, Hl, D, T_max, dtype, k_log[:, :, r * Hl:(r + 1) * Hl].contiguous(),
                                  v_log[:, :, r * Hl:(r + 1) * Hl].contiguous(), lens))
    for step in range(1, 4):  # three steps: both result buffers and the counting word of the workspace are reused
        q = U.randn((B, H * D), dtype, dev, 10 + step)
        results = []
        for r in range(world):
            q_local = sharding.slice_heads(q, H, D, r, world)
            gpu.batch_begin(ctx)
            results.append(ranks[r].decode(ctx, caches[r], 0, U.buf2d(pkg, ctx, q_local), wait=False))
            gpu.batch_commit(ctx)
        torch.cuda.synchronize()
        want = U.oracle_decode(q, k_log, v_log, lens)
        for r in range(world):
            assert flags[r].cpu().tolist() == [step] * world  # every rank raised its flag on every rank
            np.testing.assert_allclose(U.to_f32(results[r]), want, **U.TOL[dtype])
        assert torch.equal(results[0].view(torch.uint8), results[1].view(torch.uint8))


def test_single_rank_waits_on_its_own_flag(pkg):
    from llm_experiments_b200 import sharding

    ctx = U.make_ctx(pkg)
    gpu = pkg.gpu
    dev = ctx.device
    B, H, D, T_max, dtype = 2, 4, 128, 300, torch.bfloat16
    lens = [300, 77]
    k_log = U.randn((B, T_max, H, D), dtype, dev, 3)
    v_log = U.randn((B, T_max, H, D), dtype, dev, 4)
    out = torch.zeros((2, B, H * D), dtype=dtype, device=dev)
    flag = torch.zeros(1, dtype=torch.int32, device=dev)
    rank = sharding.FusedHeadGather.from_buffers(dev, 0, 1, B, H, D, dtype, [out], [flag])
    cache = _make_cache(pkg, ctx, B, H, D, T_max, dtype, k_log, v_log, lens)
    q = U.randn((B, H * D), dtype, dev, 5)
    ctx.dev_status = None
    gpu.batch_begin(ctx)
    res = rank.decode(ctx, cache, 0, U.buf2d(pkg, ctx, q))  # with the wait kernel
    gpu.batch_commit(ctx)
    torch.cuda.synchronize()
    assert int(ctx.dev_status.item()) == 0  # the wait found its flag, no timeout
    np.testing.assert_allclose(U.to_f32(res), U.oracle_decode(q, k_log, v_log, lens), **U.TOL[dtype])


def test_wait_that_nobody_answers_runs_out_and_reports(pkg):
    """Failure detection without a fault: rank 0 of two waits for a peer that never runs.  The
    bounded wait gives up after about two seconds, records B2KV_DEV_WAIT_TIMEOUT in the status word
    and returns; the context stays usable and the rank's own rows are in place."""
    import time

    from llm_experiments_b200 import sharding

    ctx = U.make_ctx(pkg)
    gpu = pkg.gpu
    dev = ctx.device
    world, B, H, D, T_max, dtype = 2, 2, 4, 128, 128, torch.bfloat16
    Hl = H // world
    k_log = U.randn((B, T_max, H, D), dtype, dev, 1)
    v_log = U.randn((B, T_max, H, D), dtype, dev, 2)
    outs = [torch.zeros((2, B, H * D), dtype=dtype, device=dev) for _ in range(world)]
    flags = [torch.zeros(world, dtype=torch.int32, device=dev) for _ in range(world)]
    rank0 = sharding.FusedHeadGather.from_buffers(dev, 0, world, B, H, D, dtype, outs, flags)
    cache = _make_cache(pkg, ctx, B, Hl, D, T_max, dtype, k_log[:, :, :Hl].contiguous(), v_log[:, :, :Hl].contiguous(),
                        [T_max, 5])
    q = U.randn((B, H * D), dtype, dev, 3)
    ctx.dev_status = None
    t0 = time.perf_counter()
    gpu.batch_begin(ctx)
    res = rank0.decode(ctx, cache, 0, U.buf2d(pkg, ctx, sharding.slice_heads(q, H, D, 0, world)))
    gpu.batch_commit(ctx)
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    assert int(ctx.dev_status.item()) == 3  # B2KV_DEV_WAIT_TIMEOUT: rank 1's flag never came
    assert 0.2 < waited < 30.0
    ctx.dev_status.zero_()
    assert flags[0].cpu().tolist() == [1, 0] and flags[1].cpu().tolist() == [1, 0]
    want = U.oracle_decode(q, k_log, v_log, [T_max, 5]).reshape(B, H, D)[:, :Hl].reshape(B, Hl * D)
    np.testing.assert_allclose(U.to_f32(res[:, : Hl * D]), want, **U.TOL[dtype])
    # the device still works
    assert float(torch.ones(4, device=dev).sum()) == 4.0
