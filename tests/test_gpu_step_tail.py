"""GPU parity of the generation-step tail (layernorm, softmax, extract_last_tokens, argmax): the
reference's seeded test recipes through the operator mirrors against the fixture and the oracle, plus
row lengths that take every code path of the kernels."""
import numpy as np
import pytest
import torch

from oracle import step_tail_oracle as T
from tests import kv_util as U

pytestmark = pytest.mark.gpu
ROWS = T.GOLDEN_ROWS


@pytest.fixture(scope="module")
def ctx(pkg):
    return U.make_ctx(pkg)


def _dev(ctx, a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(ctx.device)


def _layernorm(pkg, ctx, x, gamma, beta):
    gpu = pkg.gpu
    n, size = x.shape
    out = gpu.gpu_buffer_2d_create(ctx, n, size)
    gpu.batch_begin(ctx)
    gpu.layernorm(ctx, gpu.gpu_buffer_2d_create(ctx, n, size, _dev(ctx, x)), gpu.gpu_buffer_1d_create(ctx, size, _dev(ctx, gamma)),
                  gpu.gpu_buffer_1d_create(ctx, size, _dev(ctx, beta)), out)
    gpu.batch_commit(ctx)
    return out.buffer.cpu().numpy()


def _softmax(pkg, ctx, x):
    gpu = pkg.gpu
    b, v = x.shape
    out = gpu.gpu_buffer_2d_create(ctx, b, v)
    gpu.batch_begin(ctx)
    gpu.softmax(ctx, gpu.gpu_buffer_2d_create(ctx, b, v, _dev(ctx, x)), out)
    gpu.batch_commit(ctx)
    return out.buffer.cpu().numpy()


@pytest.mark.parametrize("case", range(len(T.LAYERNORM_RECIPE_SHAPES)))
def test_layernorm_reference_recipes(pkg, ctx, golden, case):
    n, size = T.LAYERNORM_RECIPE_SHAPES[case]
    x, gamma, beta = T.recipe_layernorm_inputs(n, size)
    out = _layernorm(pkg, ctx, x, gamma, beta)
    np.testing.assert_allclose(out[:ROWS], golden[f"layernorm_out_{case}"], rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(out, T.layernorm(x, gamma, beta), rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("case", range(len(T.SOFTMAX_RECIPES)))
def test_softmax_reference_recipes(pkg, ctx, golden, case):
    b, v, transform = T.SOFTMAX_RECIPES[case]
    x = T.recipe_softmax_inputs(b, v, transform)
    out = _softmax(pkg, ctx, x)
    np.testing.assert_allclose(out[:ROWS], golden[f"softmax_out_{case}"], rtol=1e-4, atol=1e-7)
    np.testing.assert_allclose(out.sum(axis=1), 1.0, atol=1e-5)


@pytest.mark.parametrize("case", range(len(T.EXTRACT_RECIPE_SHAPES)))
def test_extract_last_tokens_reference_recipes(pkg, ctx, golden, case):
    gpu = pkg.gpu
    b, s, e = T.EXTRACT_RECIPE_SHAPES[case]
    x = T.recipe_extract_inputs(b, s, e)
    out = gpu.gpu_buffer_2d_create(ctx, b, e)
    gpu.batch_begin(ctx)
    gpu.extract_last_tokens(ctx, gpu.gpu_buffer_2d_create(ctx, b * s, e, _dev(ctx, x)), out, b, s, e)
    gpu.batch_commit(ctx)
    got = out.buffer.cpu().numpy()
    assert np.array_equal(got[:ROWS], golden[f"extract_out_{case}"])
    assert np.array_equal(got, T.extract_last_tokens(x, b, s, e))


# row lengths: below one warp's vector width, not a multiple of 4 (scalar path), each threads-per-row
# class, the largest row kept in registers, and rows that are re-read instead
@pytest.mark.parametrize("n,size", [(3, 1), (5, 7), (9, 33), (4, 252), (6, 260), (7, 1028), (64, 4096), (3, 8192),
                                    (2, 8196), (2, 10001), (300, 64)])
def test_layernorm_and_softmax_row_lengths_vs_oracle(pkg, ctx, n, size):
    rng = np.random.default_rng(size)
    x = (rng.standard_normal((n, size)) * 3 + 1).astype(np.float32)
    gamma = rng.standard_normal(size).astype(np.float32)
    beta = rng.standard_normal(size).astype(np.float32)
    np.testing.assert_allclose(_layernorm(pkg, ctx, x, gamma, beta), T.layernorm(x, gamma, beta), rtol=1e-4, atol=2e-5)
    np.testing.assert_allclose(_softmax(pkg, ctx, x), T.softmax(x), rtol=1e-4, atol=1e-8)


@pytest.mark.parametrize("b,s,e", [(3, 5, 6), (2, 7, 1), (64, 1, 4096)])
def test_extract_last_tokens_odd_shapes(pkg, ctx, b, s, e):
    gpu = pkg.gpu
    x = np.random.default_rng(e).standard_normal((b * s, e)).astype(np.float32)
    out = gpu.gpu_buffer_2d_create(ctx, b, e)
    gpu.batch_begin(ctx)
    gpu.extract_last_tokens(ctx, gpu.gpu_buffer_2d_create(ctx, b * s, e, _dev(ctx, x)), out, b, s, e)
    gpu.batch_commit(ctx)
    assert np.array_equal(out.buffer.cpu().numpy(), T.extract_last_tokens(x, b, s, e))


def test_argmax_takes_the_lowest_index_among_equals(pkg, ctx):
    gpu = pkg.gpu
    rng = np.random.default_rng(3)
    x = rng.standard_normal((37, 50257)).astype(np.float32)
    x[1, 40000] = x[1, 123] = 9.0   # tie: the lower index wins
    x[2, :] = -2.0                  # all equal: index 0
    x[3, 50256] = 11.0              # last element
    idx = gpu.gpu_buffer_1d_create(ctx, 37, dtype=torch.int32)
    gpu.batch_begin(ctx)
    gpu.argmax(ctx, gpu.gpu_buffer_2d_create(ctx, 37, 50257, _dev(ctx, x)), idx)
    gpu.batch_commit(ctx)
    assert np.array_equal(idx.buffer.cpu().numpy(), T.argmax(x))


@pytest.mark.parametrize("n,size", [(64, 4096), (5, 100), (3, 8200), (9, 36)])
def test_layernorm_bf16_rows_vs_oracle(pkg, ctx, n, size):
    """bf16 rows and parameters, fp32 arithmetic: the oracle on the bf16-rounded inputs, output within one
    bf16 unit in the last place (rtol 2^-8) plus 1e-2 near zero."""
    gpu = pkg.gpu
    rng = np.random.default_rng(size)
    tb = lambda a: torch.from_numpy(a).to(torch.bfloat16).to(ctx.device)  # noqa: E731
    x, gamma, beta = tb(rng.standard_normal((n, size)).astype(np.float32) * 2 + 0.5), \
        tb(rng.standard_normal(size).astype(np.float32)), tb(rng.standard_normal(size).astype(np.float32))
    out = torch.empty_like(x)
    gpu.batch_begin(ctx)
    gpu.layernorm(ctx, U.buf2d(pkg, ctx, x), gpu.GPUBuffer1D(buffer=gamma, shape=(size,), size=size),
                  gpu.GPUBuffer1D(buffer=beta, shape=(size,), size=size), U.buf2d(pkg, ctx, out))
    gpu.batch_commit(ctx)
    want = T.layernorm(U.to_f32(x), U.to_f32(gamma), U.to_f32(beta))
    np.testing.assert_allclose(U.to_f32(out), want, rtol=2.0 ** -8, atol=1e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_lookup_with_positions(pkg, ctx, dtype):
    """Reference kernel simple-llm/src/gpu/gpu_kernels.py:384-449: table row + position row, positions restarting
    at 0 in every sequence; extension: per-sequence start positions.  One rounding of the fp32 sum."""
    gpu = pkg.gpu
    V, C, E, B, S = 50, 40, 72, 3, 11
    g = torch.Generator().manual_seed(0)
    table = torch.randn((V, E), generator=g).to(dtype)
    pos = torch.randn((C, E), generator=g).to(dtype)
    ids = torch.randint(0, V, (B * S,), generator=g, dtype=torch.int32)
    mk2 = lambda t: gpu.GPUBuffer2D(buffer=t.to(ctx.device), shape=tuple(t.shape), size=t.numel())  # noqa: E731
    mk1 = lambda t: gpu.GPUBuffer1D(buffer=t.to(ctx.device), shape=tuple(t.shape), size=t.numel())  # noqa: E731
    out = mk2(torch.empty((B * S, E), dtype=dtype))
    gpu.batch_begin(ctx)
    gpu.embedding(ctx, mk2(table), mk2(pos), mk1(ids), out, B, S)
    gpu.batch_commit(ctx)
    where = torch.arange(S).repeat(B)
    want = (table[ids.long()].float() + pos[where].float()).to(dtype)
    assert torch.equal(out.buffer.cpu(), want)
    # one new token per sequence at that sequence's own position
    starts = torch.tensor([0, 39, 17], dtype=torch.int32)
    out1 = mk2(torch.empty((B, E), dtype=dtype))
    gpu.batch_begin(ctx)
    gpu.embedding(ctx, mk2(table), mk2(pos), mk1(ids[:B].contiguous()), out1, B, 1, start_pos=starts.to(ctx.device))
    gpu.batch_commit(ctx)
    want1 = (table[ids[:B].long()].float() + pos[starts.long()].float()).to(dtype)
    assert torch.equal(out1.buffer.cpu(), want1)


def test_embedding_reports_ids_outside_the_table(pkg, ctx):
    gpu = pkg.gpu
    mk2 = lambda t: gpu.GPUBuffer2D(buffer=t.to(ctx.device), shape=tuple(t.shape), size=t.numel())  # noqa: E731
    mk1 = lambda t: gpu.GPUBuffer1D(buffer=t.to(ctx.device), shape=tuple(t.shape), size=t.numel())  # noqa: E731
    table, pos = torch.ones((4, 8)), torch.zeros((4, 8))
    out = mk2(torch.empty((2, 8)))
    ctx.config.check_device_status = True
    try:
        gpu.batch_begin(ctx)
        gpu.embedding(ctx, mk2(table), mk2(pos), mk1(torch.tensor([1, 9], dtype=torch.int32)), out, 2, 1)
        with pytest.raises(RuntimeError, match="embedding table"):
            gpu.batch_commit(ctx)
    finally:
        ctx.config.check_device_status = False
    assert torch.equal(out.buffer.cpu(), torch.ones((2, 8)))  # the bad id was clamped to row 0, nothing faulted
