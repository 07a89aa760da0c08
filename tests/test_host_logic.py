"""Host-side behaviour of the reference API mirror, on CPU tensors: the same checks, texts
and state changes as simple-llm/src/gpu/gpu_kv_cache.py and gpu_ops.py, exercised up to (not
including) the kernel launch."""
import pytest
import torch


@pytest.fixture()
def ctx(pkg):
    gpu = pkg.gpu
    return gpu.GPUContext(device=torch.device("cpu"), config=gpu.GPUConfig(), batch_state=None)


def _cfg(gpu, **kw):
    base = dict(batch_size=2, max_seq_len=8, n_layers=2, n_heads=2, head_dim=16)
    base.update(kw)
    return gpu.KVCacheConfig(**base)


def test_create_validates_dimensions_like_the_reference(pkg, ctx):
    gpu = pkg.gpu
    for field in ["batch_size", "max_seq_len", "n_layers", "n_heads", "head_dim"]:
        with pytest.raises(ValueError, match=f"{field} must be > 0, got 0"):
            gpu.kv_cache_create(ctx, _cfg(gpu, **{field: 0}))
    with pytest.raises(ValueError, match="layout"):
        gpu.kv_cache_create(ctx, _cfg(gpu, layout="htbd"))


def test_create_shapes_and_zero_fill(pkg, ctx):
    gpu = pkg.gpu
    cache = gpu.kv_cache_create(ctx, _cfg(gpu))
    assert len(cache.layers) == 2 and cache.current_len == 0
    assert cache.layers[0].k_cache.shape == (2 * 8, 2 * 16)  # [B*T_max, H*D] as the reference
    assert float(cache.layers[1].v_cache.buffer.abs().sum()) == 0.0
    bhtd = gpu.kv_cache_create(ctx, _cfg(gpu, layout="bhtd", dtype=torch.bfloat16))
    assert bhtd.layers[0].k_cache.shape == (2 * 2 * 8, 16) and bhtd.layers[0].k_cache.buffer.dtype == torch.bfloat16
    paged = gpu.kv_cache_create(ctx, _cfg(gpu, block_size=4, n_blocks=10, ragged=True))
    assert paged.block_table.shape == (2, 2) and paged.layers[0].k_cache.shape == (10 * 2 * 4, 16)
    assert paged.seq_lens.tolist() == [0, 0]
    with pytest.raises(ValueError, match="n_blocks"):
        gpu.kv_cache_create(ctx, _cfg(gpu, block_size=4, n_blocks=3))


def test_reset_and_set_lengths(pkg, ctx):
    gpu = pkg.gpu
    cache = gpu.kv_cache_create(ctx, _cfg(gpu, ragged=True))
    cache.current_len = 5
    gpu.kv_cache_reset(cache)
    assert cache.current_len == 0
    gpu.kv_cache_set_lengths(cache, [3, 7])
    assert cache.current_len == 7 and cache.seq_lens.tolist() == [3, 7]
    with pytest.raises(ValueError):
        gpu.kv_cache_set_lengths(cache, [3, 9])


def test_update_checks_fire_before_the_launch(pkg, ctx):
    gpu = pkg.gpu
    cache = gpu.kv_cache_create(ctx, _cfg(gpu))
    good = gpu.gpu_buffer_2d_create(ctx, 2, 32)
    with pytest.raises(ValueError, match=r"layer_idx 2 out of range \[0, 2\)"):
        gpu.kv_cache_update(ctx, cache, 2, good, good)
    cache.current_len = 8
    with pytest.raises(ValueError, match="Cache is full: current_len=8, max_seq_len=8"):
        gpu.kv_cache_update(ctx, cache, 0, good, good)
    cache.current_len = 0
    bad = gpu.gpu_buffer_2d_create(ctx, 2, 16)
    with pytest.raises(ValueError, match="new_k shape mismatch"):
        gpu.kv_cache_update(ctx, cache, 0, bad, good)
    with pytest.raises(ValueError, match="new_v shape mismatch"):
        gpu.kv_cache_update(ctx, cache, 0, good, bad)
    # no open batch: the operation is refused on the host
    with pytest.raises(RuntimeError, match="batch_begin"):
        gpu.kv_cache_update(ctx, cache, 0, good, good)
    assert cache.current_len == 0


def test_attention_checks(pkg, ctx):
    gpu = pkg.gpu
    cache = gpu.kv_cache_create(ctx, _cfg(gpu, max_seq_len=512))
    q = gpu.gpu_buffer_2d_create(ctx, 2, 32)
    with pytest.raises(ValueError, match="Cache is empty: current_len=0"):
        gpu.attention_with_kv_cache(ctx, cache, 0, q, q)
    cache.current_len = 3
    with pytest.raises(ValueError, match="out of range"):
        gpu.attention_with_kv_cache(ctx, cache, -1, q, q)
    with pytest.raises(ValueError, match="q_new shape mismatch"):
        gpu.attention_with_kv_cache(ctx, cache, 0, gpu.gpu_buffer_2d_create(ctx, 2, 31), q)
    with pytest.raises(ValueError, match="output shape mismatch"):
        gpu.attention_with_kv_cache(ctx, cache, 0, q, gpu.gpu_buffer_2d_create(ctx, 1, 32))
    # the reference's 256-token limit is opt-in
    cache.current_len = 300
    ctx.config.enforce_reference_decode_limit = True
    with pytest.raises(ValueError, match=r"current_len \(300\) exceeds maximum supported"):
        gpu.attention_with_kv_cache(ctx, cache, 0, q, q)


def test_flash_attention_checks(pkg, ctx):
    gpu = pkg.gpu
    mk = lambda r, c: gpu.gpu_buffer_2d_create(ctx, r, c)  # noqa: E731
    Q = mk(8, 32)
    L = gpu.gpu_buffer_1d_create(ctx, 16)
    ctx.config.flash_attn_max_head_dim = 8
    with pytest.raises(ValueError, match="head_dim 16 exceeds maximum supported by config: 8"):
        gpu.flash_attention(ctx, Q, Q, Q, Q, L, L, 2, 4, 2, 16)
    ctx.config.flash_attn_max_head_dim = 128
    with pytest.raises(ValueError, match="Invalid dimensions"):
        gpu.flash_attention(ctx, Q, Q, Q, Q, L, L, 0, 4, 2, 16)
    with pytest.raises(ValueError, match="K shape mismatch"):
        gpu.flash_attention(ctx, Q, mk(8, 16), Q, Q, L, L, 2, 4, 2, 16)
    with pytest.raises(ValueError, match="L shape mismatch"):
        gpu.flash_attention(ctx, Q, Q, Q, Q, gpu.gpu_buffer_1d_create(ctx, 8), L, 2, 4, 2, 16)


def test_batch_rules(pkg, ctx):
    gpu = pkg.gpu
    with pytest.raises(RuntimeError, match="Batch already submitted or not initialized"):
        gpu.batch_commit(ctx)


def test_buffer_helpers(pkg, ctx):
    import numpy as np

    gpu = pkg.gpu
    with pytest.raises(ValueError, match="Buffer dimensions must be positive"):
        gpu.gpu_buffer_2d_create(ctx, 0, 4)
    with pytest.raises(ValueError, match="Buffer size must be positive"):
        gpu.gpu_buffer_1d_create(ctx, 0)
    with pytest.raises(ValueError, match="doesn't match buffer shape"):
        gpu.gpu_buffer_2d_create(ctx, 2, 2, np.zeros((2, 3), dtype=np.float32))
    with pytest.raises(ValueError, match="Unsupported dtype"):
        gpu.gpu_buffer_2d_create(ctx, 2, 2, np.zeros((2, 2), dtype=np.float64))
    buf = gpu.gpu_buffer_2d_create(ctx, 2, 2, np.arange(4, dtype=np.float32).reshape(2, 2))
    assert buf.shape == (2, 2) and buf.size == 4


def test_perf_monitor_mirrors_the_reference(pkg):
    """simple-llm/src/gpu/gpu_device.py:569-608: record, count, aggregate, reset."""
    gpu = pkg.gpu
    mon = gpu.perf_monitor_create()
    gpu.perf_monitor_kernel_time_record(mon, "kv_cache_update", 0.5)
    gpu.perf_monitor_kernel_time_record(mon, "kv_cache_update", 1.5)
    gpu.perf_monitor_kernel_time_record(mon, "flash_attention", 2.0)
    gpu.perf_monitor_submission_record(mon)
    stats = gpu.perf_monitor_stats_get(mon)
    assert stats.total_submissions == 1
    upd = stats.kernel_times["kv_cache_update"]
    assert (upd.count, upd.total_ms, upd.avg_ms, upd.min_ms, upd.max_ms) == (2, 2.0, 1.0, 0.5, 1.5)
    assert stats.kernel_times["flash_attention"].count == 1
    gpu.perf_monitor_reset(mon)
    assert gpu.perf_monitor_stats_get(mon).total_submissions == 0 and not mon.kernel_times


def test_embedding_checks_like_the_reference(pkg, ctx):
    """simple-llm/src/gpu/gpu_pass_forward.py:110-128."""
    gpu = pkg.gpu
    table = gpu.gpu_buffer_2d_create(ctx, 10, 16)
    pos = gpu.gpu_buffer_2d_create(ctx, 6, 16)
    ids = gpu.gpu_buffer_1d_create(ctx, 8, dtype=torch.int32)
    out = gpu.gpu_buffer_2d_create(ctx, 8, 16)
    with pytest.raises(ValueError, match="Invalid batch_size=0 or seq_len=4"):
        gpu.embedding(ctx, table, pos, ids, out, 0, 4)
    with pytest.raises(ValueError, match="Embedding dimension mismatch: table has 16, pos_encoding has 8"):
        gpu.embedding(ctx, table, gpu.gpu_buffer_2d_create(ctx, 6, 8), ids, out, 2, 4)
    with pytest.raises(ValueError, match="Sequence length 7 exceeds context size 6"):
        gpu.embedding(ctx, table, pos, ids, out, 2, 7)
    with pytest.raises(ValueError, match="input_ids shape mismatch"):
        gpu.embedding(ctx, table, pos, gpu.gpu_buffer_1d_create(ctx, 7, dtype=torch.int32), out, 2, 4)
    with pytest.raises(ValueError, match="output shape mismatch"):
        gpu.embedding(ctx, table, pos, ids, gpu.gpu_buffer_2d_create(ctx, 8, 8), 2, 4)
    with pytest.raises(RuntimeError, match="batch_begin"):
        gpu.embedding(ctx, table, pos, ids, out, 2, 4)


def test_decoder_state_and_graphed_step_checks(pkg, ctx):
    """model.py on CPU tensors: shapes of the state, and the checks that fire before anything is launched."""
    import numpy as np

    from llm_experiments_b200 import model

    cfg = model.DecoderConfig(vocab_size=64, context_size=32, embedding_dim=128, n_heads=1, n_layers=2)
    pe = model.positional_encoding(cfg.context_size, cfg.embedding_dim)
    assert pe.shape == (32, 128) and pe[0, 0] == 0.0 and pe[0, 1] == 1.0  # sin(0), cos(0) interleaved
    E, V = cfg.embedding_dim, cfg.vocab_size
    z = lambda *shape: np.zeros(shape, dtype=np.float32)  # noqa: E731
    layer = dict(ln1_gamma=z(E), ln1_beta=z(E), wq=z(E, E), wk=z(E, E), wv=z(E, E), wo=z(E, E), ln2_gamma=z(E),
                 ln2_beta=z(E), w1=z(E, 4 * E), b1=z(4 * E), w2=z(4 * E, E), b2=z(E))
    params = dict(embedding=z(V, E), pos_encoding=pe, layers=[layer, layer], lnf_gamma=z(E), lnf_beta=z(E),
                  out_proj=z(E, V))
    weights = model.weights_from_numpy(ctx, cfg, params)
    assert weights.out_proj.shape == (E, V) and weights.layers[1].w1.buffer.dtype == torch.bfloat16
    state = model.decoder_state_create(ctx, cfg, weights, batch_size=3)
    assert len(state.caches) == 2 and state.logits.shape == (3, V) and state.caches[0].layout == "bhtd"
    assert model.launches_per_decode_step(cfg) == 1 + 8 * 2 + 3
    with pytest.raises(ValueError, match="exceeds context size"):
        model.decoder_state_create(ctx, cfg, weights, batch_size=3, max_seq_len=33)
    with pytest.raises(ValueError, match="ragged=True"):
        model.GraphedDecodeStep(ctx, state)  # lengths must live on the device
    tok = pkg.gpu.gpu_buffer_1d_create(ctx, 3, dtype=torch.int32)
    with pytest.raises(RuntimeError, match="batch_begin"):
        model.decode_step(ctx, state, tok)
    for cache in state.caches:
        cache.current_len = 32
    with pytest.raises(ValueError, match="Cache is full"):
        model.decode_step(ctx, state, tok)
