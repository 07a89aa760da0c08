"""Sequence-split (context-parallel) decode on one GPU: the cache of every sequence is cut into R
token slices, each slice is attended with `b2kv_decode_partial` as if it lived on its own rank,
and `b2kv_merge_partials` must reproduce attention over the whole cache.  (The all-gather
between real ranks is covered by tests/test_gpu_multi.py when two GPUs are present.)"""
import numpy as np
import pytest
import torch

from tests import kv_util as U

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,D", [(torch.bfloat16, 128), (torch.float32, 64)])
@pytest.mark.parametrize("R", [1, 2, 5])
def test_slices_merge_to_full_attention(pkg, dtype, D, R):
    from llm_experiments_b200 import sharding

    ctx = U.make_ctx(pkg)
    gpu = pkg.gpu
    dev = ctx.device
    B, H, T = 4, 3, 1000
    lens = [1000, 0, 333, 7]
    k_log = U.randn((B, T, H, D), dtype, dev, 1)
    v_log = U.randn((B, T, H, D), dtype, dev, 2)
    q = U.randn((B, H * D), dtype, dev, 3)
    per = (T + R - 1) // R
    parts = []
    for r in range(R):
        lo = r * per
        local_lens = [max(0, min(n, lo + per) - lo) for n in lens]  # tokens of each sequence inside this slice
        cache = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=B, max_seq_len=per, n_layers=1, n_heads=H,
                                                           head_dim=D, dtype=dtype, layout="bhtd", ragged=True))
        hi = min(T, lo + per)
        k_slice = torch.full((B, per, H, D), float("nan"), dtype=dtype, device=dev)
        v_slice = torch.full((B, per, H, D), float("nan"), dtype=dtype, device=dev)
        k_slice[:, : hi - lo] = k_log[:, lo:hi]
        v_slice[:, : hi - lo] = v_log[:, lo:hi]
        for b in range(B):  # rows past the local length stay NaN: an over-read would poison the result
            k_slice[b, local_lens[b]:] = float("nan")
            v_slice[b, local_lens[b]:] = float("nan")
        U.fill_cache_logical(cache, 0, k_slice, v_slice)
        gpu.kv_cache_set_lengths(cache, local_lens)
        cache.current_len = max(1, cache.current_len)
        gpu.batch_begin(ctx)
        parts.append(sharding.decode_partial(ctx, cache, 0, U.buf2d(pkg, ctx, q)))
        gpu.batch_commit(ctx)
    gpu.batch_begin(ctx)
    out = sharding.merge_partials(ctx, torch.stack(parts), B, H, D, dtype)
    gpu.batch_commit(ctx)
    torch.cuda.synchronize()
    want = U.oracle_decode(q, k_log, v_log, lens)
    got = U.to_f32(out)
    assert np.isfinite(got).all() and np.all(got[1] == 0.0)
    np.testing.assert_allclose(got, want, **U.TOL[dtype])
