"""Two real GPUs (skipped on a single-GPU machine): the head-split decode with the NCCL
all-gather and with the all-gather fused into the merge kernel (peer stores into symmetric
memory) must both reproduce the oracle's full-head result on every rank."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    import __graft_entry__
    from tests import kv_util as U

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        pkg = __graft_entry__.import_package()
        from llm_experiments_b200 import sharding

        gpu = pkg.gpu
        ctx = gpu.context_create(rank)
        B, H, D, T_max, dtype = 3, 8, 128, 900, torch.bfloat16
        Hl = H // world
        lens = [900, 17, 512]
        # the same seeded problem on every rank (generated on the CPU so that devices agree)
        g = torch.Generator().manual_seed(7)
        k_log = torch.randn((B, T_max, H, D), generator=g).to(dtype).to(dev)
        v_log = torch.randn((B, T_max, H, D), generator=g).to(dtype).to(dev)
        cache = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=B, max_seq_len=T_max, n_layers=1, n_heads=Hl,
                                                           head_dim=D, dtype=dtype, layout="bhtd", ragged=True))
        h0, h1 = sharding.head_range(H, rank, world)
        U.fill_cache_logical(cache, 0, k_log[:, :, h0:h1].contiguous(), v_log[:, :, h0:h1].contiguous())
        gpu.kv_cache_set_lengths(cache, lens)
        fused = sharding.FusedHeadGather(dev, B, H, D, dtype)
        for step in range(3):
            q = torch.randn((B, H * D), generator=g).to(dtype).to(dev)
            want = U.oracle_decode(q, k_log, v_log, lens)
            q_local = sharding.slice_heads(q, H, D, rank, world)
            # NCCL all-gather
            out_local = torch.empty_like(q_local)
            gpu.batch_begin(ctx)
            gpu.attention_with_kv_cache(ctx, cache, 0, U.buf2d(pkg, ctx, q_local), U.buf2d(pkg, ctx, out_local))
            gpu.batch_commit(ctx)
            via_nccl = sharding.gather_heads(out_local)
            # fused peer-store gather
            gpu.batch_begin(ctx)
            via_fused = fused.decode(ctx, cache, 0, U.buf2d(pkg, ctx, q_local))
            gpu.batch_commit(ctx)
            torch.cuda.synchronize()
            np.testing.assert_allclose(U.to_f32(via_nccl), want, **U.TOL[dtype])
            assert torch.equal(via_fused.view(torch.uint8), via_nccl.view(torch.uint8))
            assert int(ctx.dev_status.item()) == 0
        # sequence split: rank r caches tokens [r*T/W, (r+1)*T/W) of every sequence, all heads
        per = T_max // world
        lo = rank * per
        local_lens = [max(0, min(n, lo + per) - lo) for n in lens]
        seq_cache = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=B, max_seq_len=per, n_layers=1, n_heads=H,
                                                               head_dim=D, dtype=dtype, layout="bhtd", ragged=True))
        U.fill_cache_logical(seq_cache, 0, k_log[:, lo:lo + per].contiguous(), v_log[:, lo:lo + per].contiguous())
        gpu.kv_cache_set_lengths(seq_cache, local_lens)
        seq_cache.current_len = max(1, seq_cache.current_len)
        q = torch.randn((B, H * D), generator=g).to(dtype).to(dev)
        gpu.batch_begin(ctx)
        via_seq = sharding.sequence_split_decode(ctx, seq_cache, 0, U.buf2d(pkg, ctx, q))
        gpu.batch_commit(ctx)
        torch.cuda.synchronize()
        np.testing.assert_allclose(U.to_f32(via_seq), U.oracle_decode(q, k_log, v_log, lens), **U.TOL[dtype])
        open(os.path.join(out_dir, f"ok_{rank}"), "w").write("ok")
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_head_split_gather_nccl_and_fused_on_two_gpus(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok_{r}").exists() for r in range(world))
