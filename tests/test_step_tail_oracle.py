"""The CPU restatement of layernorm / softmax / extract_last_tokens against the outputs of the
reference's own test math on its seeded recipes (tests/golden/reference_recipes.npz), and the host-side
checks of the operator mirrors (same conditions and texts as simple-llm/src/gpu/gpu_pass_forward.py)."""
import numpy as np
import pytest
import torch

from oracle import step_tail_oracle as T

ROWS = T.GOLDEN_ROWS


@pytest.mark.parametrize("case", range(len(T.LAYERNORM_RECIPE_SHAPES)))
def test_layernorm_oracle_matches_reference_recipe(golden, case):
    n, size = T.LAYERNORM_RECIPE_SHAPES[case]
    x, gamma, beta = T.recipe_layernorm_inputs(n, size)
    np.testing.assert_allclose(T.layernorm(x, gamma, beta)[:ROWS], golden[f"layernorm_out_{case}"], rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("case", range(len(T.SOFTMAX_RECIPES)))
def test_softmax_oracle_matches_reference_recipe(golden, case):
    b, v, transform = T.SOFTMAX_RECIPES[case]
    x = T.recipe_softmax_inputs(b, v, transform)
    out = T.softmax(x)
    np.testing.assert_allclose(out[:ROWS], golden[f"softmax_out_{case}"], rtol=1e-4, atol=1e-7)
    np.testing.assert_allclose(out.sum(axis=1), 1.0, atol=1e-5)  # the reference test's sum-to-one check


@pytest.mark.parametrize("case", range(len(T.EXTRACT_RECIPE_SHAPES)))
def test_extract_oracle_matches_reference_recipe(golden, case):
    b, s, e = T.EXTRACT_RECIPE_SHAPES[case]
    x = T.recipe_extract_inputs(b, s, e)
    assert np.array_equal(T.extract_last_tokens(x, b, s, e)[:ROWS], golden[f"extract_out_{case}"])


@pytest.fixture()
def ctx(pkg):
    gpu = pkg.gpu
    return gpu.GPUContext(device=torch.device("cpu"), config=gpu.GPUConfig(), batch_state=None)


def test_operator_checks_fire_before_the_launch(pkg, ctx):
    gpu = pkg.gpu
    mk = lambda r, c: gpu.gpu_buffer_2d_create(ctx, r, c)  # noqa: E731
    v = lambda n: gpu.gpu_buffer_1d_create(ctx, n)  # noqa: E731
    with pytest.raises(ValueError, match="gamma"):
        gpu.layernorm(ctx, mk(4, 16), v(8), v(16), mk(4, 16))
    with pytest.raises(ValueError, match="beta"):
        gpu.layernorm(ctx, mk(4, 16), v(16), v(8), mk(4, 16))
    with pytest.raises(ValueError, match="output"):
        gpu.layernorm(ctx, mk(4, 16), v(16), v(16), mk(4, 8))
    with pytest.raises(ValueError, match="Invalid dimensions: batch_size=0"):
        gpu.extract_last_tokens(ctx, mk(8, 16), mk(2, 16), 0, 4, 16)
    with pytest.raises(ValueError, match="input_buf"):
        gpu.extract_last_tokens(ctx, mk(6, 16), mk(2, 16), 2, 4, 16)
    with pytest.raises(ValueError, match="output"):
        gpu.extract_last_tokens(ctx, mk(8, 16), mk(3, 16), 2, 4, 16)
    with pytest.raises(ValueError, match="Softmax shape mismatch"):
        gpu.softmax(ctx, mk(2, 16), mk(2, 8))
    # all shapes right: the operation is refused only because no batch is open (as in the reference)
    with pytest.raises(RuntimeError, match="Must call batch_begin"):
        gpu.softmax(ctx, mk(2, 16), mk(2, 16))
    assert ctx.config.layernorm_epsilon == 1e-5
