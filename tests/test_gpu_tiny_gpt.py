"""End-to-end correctness case: tiny GPT (4 layers, d_model 256, 4 heads x 64, byte vocabulary,
context 256, fp32, seed-0 weights), greedy decode of 128 new tokens from a seeded 32-byte prompt.
Cached decode on the GPU (prefill + KV cache) must produce the same tokens as the CPU oracle that
recomputes the whole context for every token, and logits within 1e-4 relative."""
import numpy as np
import pytest
import torch

from oracle import tiny_gpt_oracle

pytestmark = pytest.mark.gpu


def test_cached_greedy_decode_equals_uncached_recompute(pkg):
    from llm_experiments_b200 import tiny_gpt

    torch.backends.cuda.matmul.allow_tf32 = False
    ctx = pkg.gpu.context_create(0)
    vocab, E, n_layers, n_heads, context = 256, 256, 4, 4, 256
    params = tiny_gpt.init_params(vocab, E, n_layers, context, seed=0)
    ref_params = tiny_gpt_oracle.init_params(vocab, E, n_layers, context, seed=0)
    assert np.array_equal(params["layers"][3]["w2"], ref_params["layers"][3]["w2"])
    prompt = np.random.default_rng(0).integers(0, 256, size=32).tolist()
    n_new = 128
    model = tiny_gpt.TinyGPT(ctx, params, n_heads, context)
    tokens, logits = model.generate(prompt, n_new)
    want_tokens, want_logits = tiny_gpt_oracle.greedy_generate_uncached(ref_params, prompt, n_new, n_heads)
    assert model.cache.current_len == 32 + n_new - 1
    assert tokens == want_tokens
    got = logits.cpu().numpy()
    scale = np.abs(want_logits).max()
    assert np.abs(got - want_logits).max() <= 1e-4 * scale
