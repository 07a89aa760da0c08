"""The N > 1 paths on CPU: two gloo ranks.  Batch sharding needs no exchange (the union of
the ranks' slices must equal the single-rank result); head splitting all-gathers the local
outputs; sequence splitting all-gathers unnormalised partials and merges them.  The local attention is
the CPU oracle here, so only the sharding logic is under test."""
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


def _partial(q, k, v, lens):
    """What b2kv_decode_partial leaves per (sequence, head) for a slice of the tokens: the unnormalised row,
    the maximum of the scaled scores in the log2 domain (-inf for an empty slice) and the sum of weights."""
    B, H, D = q.shape
    out = np.zeros((B * H, D + 2), dtype=np.float32)
    for b in range(B):
        for h in range(H):
            n = int(lens[b])
            row = out[b * H + h]
            row[D] = -np.inf
            if n == 0:
                continue
            s = (k[b, :n, h] @ q[b, h]) * np.float32(np.log2(np.e) / np.sqrt(D))
            row[D] = s.max()
            w = np.exp2(s - row[D])
            row[D + 1] = w.sum()
            row[:D] = w @ v[b, :n, h]
    return out


def _merge(parts, B, H, D):
    """The arithmetic of b2kv_merge_partials on the gathered [R, B*H, D + 2] partials."""
    m = parts[:, :, D].max(axis=0)
    w = np.where(np.isfinite(parts[:, :, D]), np.exp2(parts[:, :, D] - np.where(np.isfinite(m), m, 0.0)), 0.0)
    l = (w * parts[:, :, D + 1]).sum(axis=0)
    o = (w[:, :, None] * parts[:, :, :D]).sum(axis=0)
    return np.where(l[:, None] > 0, o / np.maximum(l, 1e-38)[:, None], 0.0).astype(np.float32).reshape(B, H * D)


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
        # ---- sequence split: every rank attends a slice of the tokens, partials are exchanged and merged ----
        per = T // world
        lo = rank * per
        part = _partial(q, k[:, lo:lo + per], v[:, lo:lo + per], np.clip(lens - lo, 0, per))
        merged = sharding.exchange_partials(torch.from_numpy(part), lambda parts: torch.from_numpy(_merge(parts.numpy(), B, H, D)))
        np.save(os.path.join(out_dir, f"seq_{rank}.npy"), merged.numpy())
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
        np.testing.assert_allclose(np.load(tmp_path / f"seq_{r}.npy"), want.reshape(B, H * D), rtol=1e-5, atol=1e-6)


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


def test_balanced_assignment_evens_out_a_ragged_batch(pkg):
    import numpy as np

    from llm_experiments_b200 import sharding

    lens = np.random.default_rng(0).integers(512, 8193, size=64)
    for world in (1, 2, 4, 8):
        parts = sharding.balanced_assignment(lens, world)
        assert sorted(i for part in parts for i in part) == list(range(64))
        assert all(len(part) == 64 // world for part in parts)
        loads = [int(lens[part].sum()) for part in parts]
        assert max(loads) <= 1.02 * lens.sum() / world
    # sizes that do not divide: the first ranks take one more
    parts = sharding.balanced_assignment([5, 1, 9, 3, 7], 2)
    assert [len(part) for part in parts] == [3, 2] and sorted(parts[0] + parts[1]) == [0, 1, 2, 3, 4]
