"""The N > 1 paths on CPU: two gloo ranks.  Batch sharding needs no exchange (the union of
the ranks' slices must equal the single-rank result); head splitting all-gathers the local
outputs.  The local attention is the CPU oracle here, so only the sharding logic is under test."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import kv_oracle


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _problem():
    rng = np.random.default_rng(0)
    B, T, H, D = 5, 24, 4, 16
    lens = np.array([24, 1, 7, 16, 9])
    q = rng.standard_normal((B, H, D)).astype(np.float32)
    k = rng.standard_normal((B, T, H, D)).astype(np.float32)
    v = rng.standard_normal((B, T, H, D)).astype(np.float32)
    return B, T, H, D, lens, q, k, v


def _worker(rank, world, port, out_dir):
    import __graft_entry__

    __graft_entry__.import_package()
    from llm_experiments_b200 import sharding
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, T, H, D, lens, q, k, v = _problem()
        # ---- batch sharding: no collective in the step ----
        b0, b1 = sharding.shard_range(B, rank, world)
        mine = kv_oracle.decode_attention(q[b0:b1], k[b0:b1], v[b0:b1], lens[b0:b1])
        np.save(os.path.join(out_dir, f"batch_{rank}.npy"), mine)
        # ---- head split + all-gather ----
        h0, h1 = sharding.head_range(H, rank, world)

        def local_attention(q_local):
            ql = q_local.numpy().reshape(B, h1 - h0, D)
            o = kv_oracle.decode_attention(ql, k[:, :, h0:h1], v[:, :, h0:h1], lens)
            return torch.from_numpy(o.reshape(B, (h1 - h0) * D))

        full = sharding.head_split_decode(local_attention, torch.from_numpy(q.reshape(B, H * D)), H, D)
        np.save(os.path.join(out_dir, f"heads_{rank}.npy"), full.numpy())
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_rank_batch_shard_and_head_split(tmp_path):
    world = 2
    port = _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    B, T, H, D, lens, q, k, v = _problem()
    want = kv_oracle.decode_attention(q, k, v, lens)
    got = np.concatenate([np.load(tmp_path / f"batch_{r}.npy") for r in range(world)], axis=0)
    np.testing.assert_array_equal(got, want)  # sharding by sequence changes nothing
    for r in range(world):
        np.testing.assert_allclose(np.load(tmp_path / f"heads_{r}.npy"), want.reshape(B, H * D), rtol=1e-6, atol=1e-7)


def test_shard_ranges_cover_everything(pkg):
    from llm_experiments_b200 import sharding

    for total in (0, 1, 4, 7, 64):
        for world in (1, 2, 3, 8):
            spans = [sharding.shard_range(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    assert sharding.head_range(64, 3, 8) == (24, 32)
    with pytest.raises(ValueError):
        sharding.head_range(6, 0, 4)
    with pytest.raises(ValueError):
        sharding.shard_range(4, 2, 2)


def _worker_missing_rank(rank, world, port, out_dir):
    import datetime
    import time

    import __graft_entry__

    __graft_entry__.import_package()
    from llm_experiments_b200 import sharding

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    if rank == 0:
        try:
            sharding.gather_heads(torch.zeros(2, 8))
            outcome = "completed"
        except Exception as exc:  # the collective gives up instead of waiting for ever
            outcome = "error: " + type(exc).__name__
        with open(os.path.join(out_dir, "rank0.txt"), "w") as f:
            f.write(outcome)
    else:
        time.sleep(8)  # this rank never joins the exchange
    os._exit(0)  # skip the group shutdown: it would wait for the rank that never joined


def test_rank_that_never_joins_ends_the_collective_with_an_error(tmp_path):
    world = 2
    mp.spawn(_worker_missing_rank, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert (tmp_path / "rank0.txt").read_text().startswith("error")
