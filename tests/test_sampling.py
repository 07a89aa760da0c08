"""The sampling rules of the generation loop against the numpy oracle (CPU tensors: these are host
rules, not kernels) and the cached generation loop on the GPU."""
import numpy as np
import pytest
import torch

from oracle import sampling_oracle


@pytest.mark.parametrize("kw", [
    dict(),
    dict(temperature=0.7),
    dict(top_k=5),
    dict(top_p=0.9),
    dict(min_p=0.1),
    dict(repetition_penalty=1.2, recent_tokens=[3, 3, 7, 250]),
    dict(temperature=1.3, top_k=40, top_p=0.95, min_p=0.02, repetition_penalty=1.1, recent_tokens=list(range(64))),
    dict(top_k=1),
    dict(top_p=0.0),
])
def test_filtered_distribution_matches_oracle(pkg, kw):
    from llm_experiments_b200 import generate

    rng = np.random.default_rng(5)
    logits = (rng.standard_normal(256) * 3).astype(np.float32)
    got = generate.filtered_distribution(torch.from_numpy(logits), **kw).numpy()
    want = sampling_oracle.filtered_distribution(logits, **kw)
    assert abs(float(got.sum()) - 1.0) < 1e-5
    assert np.array_equal(got > 0, want > 0)  # the same tokens survive the filters
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-7)


def test_greedy_and_seeded_draws(pkg):
    from llm_experiments_b200 import generate

    logits = torch.tensor([0.1, 2.0, -1.0, 1.9])
    assert generate.sample_token(None, logits, temperature=0.0) == 1
    # the reference divides by the penalty whatever the sign: a positive logit shrinks
    assert generate.sample_token(None, logits, temperature=0.0, repetition_penalty=1.5, recent_tokens=[1]) == 3
    g1 = torch.Generator().manual_seed(42)
    g2 = torch.Generator().manual_seed(42)
    a = [generate.sample_token(g1, logits, temperature=1.0) for _ in range(20)]
    b = [generate.sample_token(g2, logits, temperature=1.0) for _ in range(20)]
    assert a == b and all(0 <= t < 4 for t in a)
    assert generate.sample_token(torch.Generator().manual_seed(0), logits, top_k=1) == 1


@pytest.mark.gpu
def test_cached_generate_text_on_gpu(pkg):
    from llm_experiments_b200 import generate, tiny_gpt

    torch.backends.cuda.matmul.allow_tf32 = False
    ctx = pkg.gpu.context_create(0)
    params = tiny_gpt.init_params(256, 256, 4, 256, seed=0)
    model = tiny_gpt.TinyGPT(ctx, params, 4, 256)
    prompt = np.random.default_rng(0).integers(0, 256, size=32).tolist()
    greedy, _ = model.generate(prompt, 24)
    assert generate.generate_text(model, prompt, max_tokens=24, temperature=0.0) == greedy
    a = generate.generate_text(model, prompt, max_tokens=40, temperature=0.9, top_k=50, top_p=0.95, min_p=0.01,
                               repetition_penalty=1.1)
    b = generate.generate_text(model, prompt, max_tokens=40, temperature=0.9, top_k=50, top_p=0.95, min_p=0.01,
                               repetition_penalty=1.1)
    assert a == b and len(a) == 72 and a[:32] == prompt and all(0 <= t < 256 for t in a)
    assert model.cache.current_len == 32 + 40 - 1
    with pytest.raises(ValueError, match="exceeds the context"):
        generate.generate_text(model, prompt, max_tokens=250)
