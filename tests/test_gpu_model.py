"""The whole bf16 decoder on the library's kernels against the stacked layer oracle: a prompt pass, then cached
decode steps driven by the greedy tokens; logits within the decoder-layer tolerance at every step, greedy tokens
equal wherever the oracle's two best logits are further apart than that tolerance, cache rows as the oracle's."""
import numpy as np
import pytest
import torch

from oracle import model_oracle
from oracle.decode_layer_oracle import bf16_round

pytestmark = pytest.mark.gpu

TOL = 6e-2  # absolute, on logits of order one: bf16 storage of every intermediate row over two layers


def _params(cfg, model, seed):
    rs = np.random.RandomState(seed)
    E, V = cfg.embedding_dim, cfg.vocab_size
    r = lambda shape, scale=1.0: bf16_round((rs.randn(*shape) * scale).astype(np.float32))  # noqa: E731

    def layer():
        return dict(ln1_gamma=r((E,), 0.1) + 1, ln1_beta=r((E,), 0.1), wq=r((E, E), E ** -0.5), wk=r((E, E), E ** -0.5),
                    wv=r((E, E), E ** -0.5), wo=r((E, E), E ** -0.5), ln2_gamma=r((E,), 0.1) + 1, ln2_beta=r((E,), 0.1),
                    w1=r((E, 4 * E), E ** -0.5), b1=r((4 * E,), 0.1), w2=r((4 * E, E), (4 * E) ** -0.5), b2=r((E,), 0.1))

    p = dict(embedding=r((V, E)), pos_encoding=bf16_round(model.positional_encoding(cfg.context_size, E)),
             layers=[layer() for _ in range(cfg.n_layers)], lnf_gamma=r((E,), 0.1) + 1, lnf_beta=r((E,), 0.1),
             out_proj=r((E, V), E ** -0.5))
    for lw in p["layers"]:
        for k in ("ln1_gamma", "ln2_gamma"):
            lw[k] = bf16_round(lw[k])
    p["lnf_gamma"] = bf16_round(p["lnf_gamma"])
    return p


def _check(got_logits, want_logits, got_next, what):
    got = got_logits.float().cpu().numpy()
    assert np.abs(got - want_logits).max() <= TOL, what
    top2 = np.sort(want_logits, axis=1)[:, -2:]
    clear = (top2[:, 1] - top2[:, 0]) > 2 * TOL
    want_next = want_logits.argmax(axis=1)
    assert np.array_equal(got_next[clear], want_next[clear]), what
    # the device's greedy choice is the argmax of the device's own logits (lowest index among equals)
    assert np.array_equal(got_next, got.argmax(axis=1)), what


def test_cached_decoder_matches_the_stacked_layer_oracle(pkg):
    from llm_experiments_b200 import model

    gpu = pkg.gpu
    ctx = gpu.context_create(0)
    cfg = model.DecoderConfig(vocab_size=512, context_size=96, embedding_dim=256, n_heads=2, n_layers=2)
    params = _params(cfg, model, seed=3)
    weights = model.weights_from_numpy(ctx, cfg, params)
    B, N, steps = 3, 48, 5
    state = model.decoder_state_create(ctx, cfg, weights, batch_size=B)
    prompt = np.random.default_rng(1).integers(0, cfg.vocab_size, size=B * N).astype(np.int32)
    ids = gpu.gpu_buffer_1d_create(ctx, B * N, torch.from_numpy(prompt), dtype=torch.int32)
    nxt = gpu.gpu_buffer_1d_create(ctx, B, dtype=torch.int32)
    ctx.config.check_device_status = True
    gpu.batch_begin(ctx)
    model.prefill(ctx, state, ids, N, nxt)
    gpu.batch_commit(ctx)
    want_logits, cache = model_oracle.prefill(params, prompt, B, N, cfg.n_heads)
    got_next = nxt.buffer.cpu().numpy()
    _check(state.logits.buffer, want_logits, got_next, "prompt")
    assert all(c.current_len == N for c in state.caches)
    for step in range(steps):
        # both sides continue from the DEVICE's tokens, so one near-tie does not fork the two histories
        tokens = got_next.copy()
        tok = gpu.gpu_buffer_1d_create(ctx, B, torch.from_numpy(tokens), dtype=torch.int32)
        gpu.batch_begin(ctx)
        model.decode_step(ctx, state, tok, nxt)
        gpu.batch_commit(ctx)
        want_logits = model_oracle.decode_step(params, tokens, cache, cfg.n_heads)
        got_next = nxt.buffer.cpu().numpy()
        _check(state.logits.buffer, want_logits, got_next, f"step {step}")
    assert all(c.current_len == N + steps for c in state.caches)
    # the last layer's cache rows of sequence 1 against the oracle's (projection outputs: bf16 rounding apart)
    k_dev = state.caches[-1].layers[0].k_cache.buffer.view(B, cfg.n_heads, cfg.context_size, cfg.head_dim)
    k_dev = k_dev[1, :, :N + steps].permute(1, 0, 2).reshape(N + steps, cfg.embedding_dim).float().cpu().numpy()
    assert np.abs(k_dev - cache[-1][0][1]).max() <= TOL


def test_generate_text_drives_the_cached_decoder(pkg):
    """generate_text (the reference's sampling rules) over the batch-of-one adapter: greedy generation equals
    stepping the decoder by hand, and the sampling path runs."""
    from llm_experiments_b200 import generate, model

    gpu = pkg.gpu
    ctx = gpu.context_create(0)
    cfg = model.DecoderConfig(vocab_size=512, context_size=64, embedding_dim=256, n_heads=2, n_layers=2)
    weights = model.weights_from_numpy(ctx, cfg, _params(cfg, model, seed=5))
    dec = model.CachedDecoder(ctx, cfg, weights)
    prompt = [int(t) for t in np.random.default_rng(2).integers(0, 512, size=9)]
    greedy = generate.generate_text(dec, prompt, max_tokens=6, temperature=0.0)
    assert greedy[:9] == prompt and len(greedy) == 15
    by_hand = list(prompt)
    gpu.kv_cache_reset(dec.cache)
    logits = dec.prefill(by_hand)
    for i in range(6):
        by_hand.append(int(torch.argmax(logits[0])))
        if i < 5:
            logits = dec.decode_step(by_hand[-1])
    assert greedy == by_hand
    sampled = generate.generate_text(dec, prompt, max_tokens=6, temperature=0.8, top_k=20, top_p=0.9, seed=42)
    assert len(sampled) == 15 and all(0 <= t < 512 for t in sampled)


def test_graphed_decode_step_equals_the_eager_step(pkg):
    """decode_step captured into a CUDA graph and replayed gives the same logits and cache rows as the eager step,
    step after step, on ragged lengths (same tokens fed to both); the host-side lengths advance alike.  The two are
    not bit-identical: the captured attention launch is sized for the cache's capacity, so its split-K cuts fall
    elsewhere and the fp32 partial sums are added in another order."""
    from llm_experiments_b200 import model

    gpu = pkg.gpu
    ctx = gpu.context_create(0)
    cfg = model.DecoderConfig(vocab_size=512, context_size=96, embedding_dim=256, n_heads=2, n_layers=2)
    weights = model.weights_from_numpy(ctx, cfg, _params(cfg, model, seed=9))
    B, N, steps = 3, 32, 6
    prompt = np.random.default_rng(4).integers(0, cfg.vocab_size, size=B * N).astype(np.int32)
    lens = [32, 7, 19]  # after the prompt pass the sequences are cut back to ragged lengths
    fed = [torch.from_numpy(np.random.default_rng(10 + i).integers(0, cfg.vocab_size, size=B).astype(np.int32))
           for i in range(steps)]
    runs = {}
    for mode in ("eager", "graph", "graph_feed_back"):
        state = model.decoder_state_create(ctx, cfg, weights, batch_size=B, ragged=True)
        ids = gpu.gpu_buffer_1d_create(ctx, B * N, torch.from_numpy(prompt), dtype=torch.int32)
        nxt = gpu.gpu_buffer_1d_create(ctx, B, dtype=torch.int32)
        gpu.batch_begin(ctx)
        model.prefill(ctx, state, ids, N, nxt)
        gpu.batch_commit(ctx)
        for c in state.caches:
            gpu.kv_cache_set_lengths(c, lens)
        tokens, logits = [], []
        if mode == "eager":
            tok = gpu.gpu_buffer_1d_create(ctx, B, dtype=torch.int32)
            for i in range(steps):
                tok.buffer.copy_(fed[i])
                gpu.batch_begin(ctx)
                model.decode_step(ctx, state, tok, nxt)
                gpu.batch_commit(ctx)
                tokens.append(nxt.buffer.cpu().clone())
                logits.append(state.logits.buffer.float().cpu().clone())
        else:
            graphed = model.GraphedDecodeStep(ctx, state, feed_back=(mode == "graph_feed_back"))
            graphed.token_ids.buffer.copy_(fed[0])
            graphed.capture()
            assert [c.current_len for c in state.caches] == [max(lens)] * cfg.n_layers
            assert state.caches[0].seq_lens.tolist() == lens  # the warm-up step was undone
            assert torch.equal(graphed.token_ids.buffer.cpu(), fed[0])
            for i in range(steps):
                if mode == "graph":
                    graphed.token_ids.buffer.copy_(fed[i])
                graphed.step()
                tokens.append(graphed.next_ids.buffer.cpu().clone())
                logits.append(state.logits.buffer.float().cpu().clone())
            if mode == "graph_feed_back":  # every step was fed the step before's choice, on the device
                assert torch.equal(graphed.token_ids.buffer.cpu(), tokens[-1])
        torch.cuda.synchronize()
        runs[mode] = (tokens, logits, [c.current_len for c in state.caches], state.caches[0].seq_lens.tolist(),
                      state.caches[-1].layers[0].k_cache.buffer.float().cpu().clone())
    for a, b in zip(runs["eager"][1], runs["graph"][1]):
        assert float((a - b).abs().max()) <= 2e-2
    assert torch.equal(runs["graph_feed_back"][0][0], runs["graph"][0][0])  # the first step saw the same tokens
    for mode in ("graph", "graph_feed_back"):
        assert runs["eager"][2] == runs[mode][2] == [max(lens) + steps] * cfg.n_layers
        assert runs["eager"][3] == runs[mode][3] == [n + steps for n in lens]
    # cache rows within each sequence's length agree (rows past it may differ: the warm-up step wrote one there)
    k_e = runs["eager"][4].view(B, cfg.n_heads, cfg.context_size, cfg.head_dim)
    k_g = runs["graph"][4].view(B, cfg.n_heads, cfg.context_size, cfg.head_dim)
    for b, n in enumerate(lens):
        assert float((k_e[b, :, : n + steps] - k_g[b, :, : n + steps]).abs().max()) <= 2e-2
