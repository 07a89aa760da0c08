"""One decoder layer of a cached decode step (layernorm, fused Q/K/V projection + append, cached attention,
output projection + residual, layernorm, MLP with GELU + residual) against the numpy restatement of the
reference block that rounds to bf16 at the same places.  Tolerance: 2^-6 relative + 3e-2 absolute (seven
bf16-rounded stages; a single bf16 rounding is 2^-9 relative)."""
import numpy as np
import pytest
import torch

from oracle import decode_layer_oracle
from tests import kv_util as U

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,H,D,ragged", [(5, 2, 64, True), (16, 4, 128, False)])
def test_decoder_layer_step_vs_oracle(pkg, B, H, D, ragged):
    from llm_experiments_b200 import decode_layer

    gpu = pkg.gpu
    ctx = U.make_ctx(pkg)
    E, T_max = H * D, 48
    g = torch.Generator().manual_seed(B)
    rnd = lambda shape, scale=1.0: (torch.randn(shape, generator=g) * scale).to(torch.bfloat16).to(ctx.device)  # noqa: E731
    b2 = lambda t: gpu.GPUBuffer2D(buffer=t, shape=tuple(t.shape), size=t.numel())  # noqa: E731
    b1 = lambda t: gpu.GPUBuffer1D(buffer=t, shape=tuple(t.shape), size=t.numel())  # noqa: E731
    raw = dict(ln1_gamma=rnd((E,), 0.2) + 1, ln1_beta=rnd((E,), 0.1), wq=rnd((E, E), E ** -0.5), wk=rnd((E, E), E ** -0.5),
               wv=rnd((E, E), E ** -0.5), wo=rnd((E, E), E ** -0.5), ln2_gamma=rnd((E,), 0.2) + 1, ln2_beta=rnd((E,), 0.1),
               w1=rnd((E, 4 * E), E ** -0.5), b1=rnd((4 * E,), 0.1), w2=rnd((4 * E, E), (4 * E) ** -0.5), b2=rnd((E,), 0.1))
    w = decode_layer.DecoderLayerWeights(**{k: (b1(v) if v.dim() == 1 else b2(v)) for k, v in raw.items()})
    cache = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=B, max_seq_len=T_max, n_layers=1, n_heads=H, head_dim=D,
                                                       dtype=torch.bfloat16, layout="bhtd", ragged=ragged))
    layer = cache.layers[0]
    layer.k_cache.buffer.copy_(rnd(tuple(layer.k_cache.buffer.shape)))
    layer.v_cache.buffer.copy_(rnd(tuple(layer.v_cache.buffer.shape)))
    rng = np.random.default_rng(B)
    if ragged:
        lens = rng.integers(0, T_max - 1, size=B).astype(np.int32)
        gpu.kv_cache_set_lengths(cache, lens)
    else:
        lens = np.full(B, 11, dtype=np.int32)
        cache.current_len = 11
    k_before = U.to_f32(U.logical_view(cache, layer, "k")).reshape(B, T_max, E)
    v_before = U.to_f32(U.logical_view(cache, layer, "v")).reshape(B, T_max, E)
    x = rnd((B, E))
    y = torch.empty_like(x)
    scratch = decode_layer.decoder_layer_scratch(ctx, B, E)
    gpu.batch_begin(ctx)
    decode_layer.decoder_layer_step(ctx, cache, b2(x), w, scratch, b2(y))
    gpu.batch_commit(ctx)
    torch.cuda.synchronize()
    wf = {k: U.to_f32(v) for k, v in raw.items()}
    want_y, want_k, want_v = decode_layer_oracle.decoder_layer_step(U.to_f32(x), wf, list(k_before), list(v_before), lens, H)
    np.testing.assert_allclose(U.to_f32(y), want_y, rtol=2.0 ** -6, atol=3e-2)
    k_after = U.to_f32(U.logical_view(cache, layer, "k")).reshape(B, T_max, E)
    rows = np.arange(B)
    np.testing.assert_allclose(k_after[rows, lens], want_k, rtol=2.0 ** -7, atol=1e-2)
    if ragged:
        assert np.array_equal(cache.seq_lens.cpu().numpy(), lens + 1)
    else:
        assert cache.current_len == 12


def test_two_layers_over_several_steps_track_the_oracle(pkg):
    """Two stacked layers (one cache object each) over six decode steps: the caches grow by one row per step and
    layer, and every step's output stays within the layer tolerance of the oracle that is fed the GPU's own
    previous rows (so that rounding differences do not compound across steps)."""
    from llm_experiments_b200 import decode_layer

    gpu = pkg.gpu
    ctx = U.make_ctx(pkg)
    B, H, D, T_max, n_layers, n_steps = 4, 2, 64, 16, 2, 6
    E = H * D
    g = torch.Generator().manual_seed(7)
    rnd = lambda shape, scale=1.0: (torch.randn(shape, generator=g) * scale).to(torch.bfloat16).to(ctx.device)  # noqa: E731
    b2 = lambda t: gpu.GPUBuffer2D(buffer=t, shape=tuple(t.shape), size=t.numel())  # noqa: E731
    b1 = lambda t: gpu.GPUBuffer1D(buffer=t, shape=tuple(t.shape), size=t.numel())  # noqa: E731
    raws, weights, caches = [], [], []
    for _ in range(n_layers):
        raw = dict(ln1_gamma=rnd((E,), 0.2) + 1, ln1_beta=rnd((E,), 0.1), wq=rnd((E, E), E ** -0.5), wk=rnd((E, E), E ** -0.5),
                   wv=rnd((E, E), E ** -0.5), wo=rnd((E, E), E ** -0.5), ln2_gamma=rnd((E,), 0.2) + 1, ln2_beta=rnd((E,), 0.1),
                   w1=rnd((E, 4 * E), E ** -0.5), b1=rnd((4 * E,), 0.1), w2=rnd((4 * E, E), (4 * E) ** -0.5), b2=rnd((E,), 0.1))
        raws.append({k: U.to_f32(v) for k, v in raw.items()})
        weights.append(decode_layer.DecoderLayerWeights(**{k: (b1(v) if v.dim() == 1 else b2(v)) for k, v in raw.items()}))
        caches.append(gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=B, max_seq_len=T_max, n_layers=1, n_heads=H,
                                                                 head_dim=D, dtype=torch.bfloat16, layout="bhtd")))
    scratch = decode_layer.decoder_layer_scratch(ctx, B, E)
    bufs = [torch.empty((B, E), dtype=torch.bfloat16, device=ctx.device) for _ in range(n_layers + 1)]
    for step in range(n_steps):
        bufs[0].copy_(rnd((B, E)))
        before = [(U.to_f32(U.logical_view(c, c.layers[0], "k")).reshape(B, T_max, E),
                   U.to_f32(U.logical_view(c, c.layers[0], "v")).reshape(B, T_max, E)) for c in caches]
        gpu.batch_begin(ctx)
        for li in range(n_layers):
            decode_layer.decoder_layer_step(ctx, caches[li], b2(bufs[li]), weights[li], scratch, b2(bufs[li + 1]))
        gpu.batch_commit(ctx)
        torch.cuda.synchronize()
        lens = np.full(B, step, dtype=np.int32)
        for li in range(n_layers):
            assert caches[li].current_len == step + 1
            want_y, want_k, _ = decode_layer_oracle.decoder_layer_step(U.to_f32(bufs[li]), raws[li], list(before[li][0]),
                                                                        list(before[li][1]), lens, H)
            np.testing.assert_allclose(U.to_f32(bufs[li + 1]), want_y, rtol=2.0 ** -6, atol=3e-2)
            k_now = U.to_f32(U.logical_view(caches[li], caches[li].layers[0], "k")).reshape(B, T_max, E)
            np.testing.assert_allclose(k_now[:, step], want_k, rtol=2.0 ** -7, atol=1e-2)
            assert float(np.abs(k_now[:, step + 1:]).sum()) == 0.0  # rows after the new one are still untouched


@pytest.mark.parametrize("B,N,H,D", [(2, 256, 2, 128), (3, 160, 4, 64)])
def test_prompt_layer_step_vs_oracle_then_decode_continues(pkg, B, N, H, D):
    """The same layer over a whole prompt (projections on the tiled GEMM, causal attention fused with the
    cache write), then one cached decode step on top of the prefilled cache: both against the oracle."""
    from llm_experiments_b200 import decode_layer

    gpu = pkg.gpu
    ctx = U.make_ctx(pkg)
    ctx.config.flash_attn_max_head_dim = 128
    E, T_max = H * D, N + 16
    g = torch.Generator().manual_seed(100 + B)
    rnd = lambda shape, scale=1.0: (torch.randn(shape, generator=g) * scale).to(torch.bfloat16).to(ctx.device)  # noqa: E731
    b2 = lambda t: gpu.GPUBuffer2D(buffer=t, shape=tuple(t.shape), size=t.numel())  # noqa: E731
    b1 = lambda t: gpu.GPUBuffer1D(buffer=t, shape=tuple(t.shape), size=t.numel())  # noqa: E731
    raw = dict(ln1_gamma=rnd((E,), 0.2) + 1, ln1_beta=rnd((E,), 0.1), wq=rnd((E, E), E ** -0.5), wk=rnd((E, E), E ** -0.5),
               wv=rnd((E, E), E ** -0.5), wo=rnd((E, E), E ** -0.5), ln2_gamma=rnd((E,), 0.2) + 1, ln2_beta=rnd((E,), 0.1),
               w1=rnd((E, 4 * E), E ** -0.5), b1=rnd((4 * E,), 0.1), w2=rnd((4 * E, E), (4 * E) ** -0.5), b2=rnd((E,), 0.1))
    w = decode_layer.DecoderLayerWeights(**{k: (b1(v) if v.dim() == 1 else b2(v)) for k, v in raw.items()})
    wf = {k: U.to_f32(v) for k, v in raw.items()}
    cache = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=B, max_seq_len=T_max, n_layers=1, n_heads=H, head_dim=D,
                                                       dtype=torch.bfloat16, layout="bhtd"))
    x = rnd((B * N, E))
    y = torch.empty_like(x)
    scratch = decode_layer.prompt_layer_scratch(ctx, B * N, E)
    gpu.batch_begin(ctx)
    decode_layer.prompt_layer_step(ctx, cache, b2(x), w, scratch, b2(y), B, N)
    gpu.batch_commit(ctx)
    torch.cuda.synchronize()
    want_y, want_k, want_v = decode_layer_oracle.prompt_layer_step(U.to_f32(x), wf, B, N, H)
    np.testing.assert_allclose(U.to_f32(y), want_y, rtol=2.0 ** -6, atol=3e-2)
    assert cache.current_len == N
    layer = cache.layers[0]
    k_rows = U.logical_view(cache, layer, "k")[:, :N].reshape(B * N, E)
    v_rows = U.logical_view(cache, layer, "v")[:, :N].reshape(B * N, E)
    # the cache holds exactly the projected rows (bit-exact copy), which match the oracle's projection
    assert torch.equal(k_rows, scratch.k.buffer) and torch.equal(v_rows, scratch.v.buffer)
    np.testing.assert_allclose(U.to_f32(k_rows), want_k, rtol=2.0 ** -7, atol=1e-2)
    np.testing.assert_allclose(U.to_f32(v_rows), want_v, rtol=2.0 ** -7, atol=1e-2)
    # one decode step over the prefilled cache
    k_before = U.to_f32(U.logical_view(cache, layer, "k")).reshape(B, T_max, E)
    v_before = U.to_f32(U.logical_view(cache, layer, "v")).reshape(B, T_max, E)
    x1 = rnd((B, E))
    y1 = torch.empty_like(x1)
    dscratch = decode_layer.decoder_layer_scratch(ctx, B, E)
    gpu.batch_begin(ctx)
    decode_layer.decoder_layer_step(ctx, cache, b2(x1), w, dscratch, b2(y1))
    gpu.batch_commit(ctx)
    torch.cuda.synchronize()
    want_y1, _, _ = decode_layer_oracle.decoder_layer_step(U.to_f32(x1), wf, list(k_before), list(v_before),
                                                           np.full(B, N, dtype=np.int32), H)
    np.testing.assert_allclose(U.to_f32(y1), want_y1, rtol=2.0 ** -6, atol=3e-2)
    assert cache.current_len == N + 1


def test_overlapped_launches_give_the_results_of_plain_stream_order(pkg):
    """The kernels of a decode step are launched ahead of the end of the kernel before them and wait inside for
    it.  Three layers over eight steps, queued without a host synchronisation, must leave bit for bit the rows
    and caches that the same chain leaves when every launch is in plain stream order (knob ``serial_launches``)."""
    from llm_experiments_b200 import _native, decode_layer

    gpu = pkg.gpu
    B, H, D, T_max, n_layers, n_steps = 24, 8, 128, 2048, 3, 8
    E = H * D

    def run(serial):
        _native.tune("serial_launches", 1 if serial else 0)
        try:
            ctx = U.make_ctx(pkg)
            g = torch.Generator().manual_seed(11)
            rnd = lambda shape, scale=1.0: (torch.randn(shape, generator=g) * scale).to(torch.bfloat16).to(ctx.device)  # noqa: E731
            b2 = lambda t: gpu.GPUBuffer2D(buffer=t, shape=tuple(t.shape), size=t.numel())  # noqa: E731
            b1 = lambda t: gpu.GPUBuffer1D(buffer=t, shape=tuple(t.shape), size=t.numel())  # noqa: E731
            weights, caches = [], []
            lens = np.random.default_rng(5).integers(100, T_max - n_steps - 1, size=B).astype(np.int32)
            for _ in range(n_layers):
                raw = dict(ln1_gamma=rnd((E,), 0.2) + 1, ln1_beta=rnd((E,), 0.1), wq=rnd((E, E), E ** -0.5),
                           wk=rnd((E, E), E ** -0.5), wv=rnd((E, E), E ** -0.5), wo=rnd((E, E), E ** -0.5),
                           ln2_gamma=rnd((E,), 0.2) + 1, ln2_beta=rnd((E,), 0.1), w1=rnd((E, 4 * E), E ** -0.5),
                           b1=rnd((4 * E,), 0.1), w2=rnd((4 * E, E), (4 * E) ** -0.5), b2=rnd((E,), 0.1))
                weights.append(decode_layer.DecoderLayerWeights(**{k: (b1(v) if v.dim() == 1 else b2(v)) for k, v in raw.items()}))
                cache = gpu.kv_cache_create(ctx, gpu.KVCacheConfig(batch_size=B, max_seq_len=T_max, n_layers=1, n_heads=H,
                                                                   head_dim=D, dtype=torch.bfloat16, layout="bhtd",
                                                                   ragged=True))
                cache.layers[0].k_cache.buffer.copy_(rnd(tuple(cache.layers[0].k_cache.buffer.shape)))
                cache.layers[0].v_cache.buffer.copy_(rnd(tuple(cache.layers[0].v_cache.buffer.shape)))
                gpu.kv_cache_set_lengths(cache, lens)
                caches.append(cache)
            scratch = decode_layer.decoder_layer_scratch(ctx, B, E)
            bufs = [rnd((B, E))] + [torch.empty((B, E), dtype=torch.bfloat16, device=ctx.device) for _ in range(n_layers)]
            outs = []
            for _ in range(n_steps):
                gpu.batch_begin(ctx)
                for li in range(n_layers):
                    decode_layer.decoder_layer_step(ctx, caches[li], b2(bufs[li]), weights[li], scratch, b2(bufs[li + 1]))
                gpu.batch_commit(ctx)
                outs.append(bufs[n_layers].clone())
                bufs[0].copy_(bufs[n_layers])  # the next step's rows are this step's output
            torch.cuda.synchronize()
            assert int(ctx.dev_status.item()) == 0
            state = [t.view(torch.int16).cpu() for t in outs]
            for c in caches:
                state.append(c.layers[0].k_cache.buffer.view(torch.int16).cpu())
                state.append(c.layers[0].v_cache.buffer.view(torch.int16).cpu())
                state.append(c.seq_lens.cpu())
            return state
        finally:
            _native.tune("serial_launches", 0)

    overlapped, serial = run(False), run(True)
    assert len(overlapped) == len(serial)
    for a, b in zip(overlapped, serial):
        assert torch.equal(a, b)
    assert not torch.equal(overlapped[0], overlapped[n_steps - 1])  # the steps did something
