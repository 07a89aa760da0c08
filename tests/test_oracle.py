"""The oracle against the fixtures made from the reference's own test code.

``tests/golden/reference_recipes.npz`` holds the outputs of the reference test's
reference math (simple-llm/src/gpu_test.py:2328-2367 and :776-810) on its seeded
recipes.  Both oracles (numpy and C) must reproduce them at the reference test's
own tolerance (rtol 1e-4, atol 1e-5: gpu_test.py:23-24), and agree with each other
on the extensions (bf16 storage, ragged lengths, paged tables).
"""
import numpy as np
import pytest

from oracle import c_oracle, kv_oracle

RTOL, ATOL = 1e-4, 1e-5


def _kv_recipe_cache(B=2, T_max=128, H=4, D=64, steps=5):
    ks, vs, Q = kv_oracle.recipe_kv_cache_inputs(B, H, D, steps, seed=42)
    E = H * D
    k_cache = np.zeros((B * T_max, E), dtype=np.float32)
    v_cache = np.zeros((B * T_max, E), dtype=np.float32)
    for step in range(steps):
        kv_oracle.kv_update(k_cache, v_cache, ks[step].reshape(B, E), vs[step].reshape(B, E), step, B, T_max)
    return k_cache, v_cache, Q, ks, vs


def test_recipe_inputs_match_fixture(golden):
    ks, vs, Q = kv_oracle.recipe_kv_cache_inputs()
    got = np.array([sum(float(k.sum()) for k in ks), sum(float(v.sum()) for v in vs), float(Q.sum())])
    np.testing.assert_allclose(got, golden["kv_in_checksum"], rtol=0, atol=0)


def test_numpy_decode_matches_reference_recipe(golden):
    B, T_max, H, D = 2, 128, 4, 64
    k_cache, v_cache, Q, _, _ = _kv_recipe_cache()
    out = kv_oracle.decode_attention(Q.reshape(B, H, D), k_cache.reshape(B, T_max, H, D),
                                     v_cache.reshape(B, T_max, H, D), 5)
    np.testing.assert_allclose(out.reshape(B, H * D), golden["kv_out"], rtol=RTOL, atol=ATOL)
    # the sanity values quoted for this recipe
    assert abs(float(out.sum()) - 8.565736) < 1e-4


def test_shader_order_agrees():
    B, T_max, H, D = 2, 128, 4, 64
    k_cache, v_cache, Q, _, _ = _kv_recipe_cache()
    a = kv_oracle.decode_attention(Q.reshape(B, H, D), k_cache.reshape(B, T_max, H, D),
                                   v_cache.reshape(B, T_max, H, D), 5)
    b = kv_oracle.decode_attention_shader_order(Q.reshape(B, H, D), k_cache.reshape(B, T_max, H, D),
                                                v_cache.reshape(B, T_max, H, D), 5)
    np.testing.assert_allclose(a, b, rtol=RTOL, atol=ATOL)


def test_c_decode_matches_reference_recipe(golden):
    B, T_max, H, D = 2, 128, 4, 64
    ks, vs, Q = kv_oracle.recipe_kv_cache_inputs()
    E = H * D
    k_cache = np.zeros((B * T_max, E), dtype=np.float32)
    v_cache = np.zeros((B * T_max, E), dtype=np.float32)
    strides = (T_max * E, E, D)
    for step in range(5):
        c_oracle.append(np.ascontiguousarray(ks[step].reshape(B, E)), np.ascontiguousarray(vs[step].reshape(B, E)),
                        k_cache, v_cache, step, B, H, D, strides)
    ref_k, ref_v, _, _, _ = _kv_recipe_cache()
    assert np.array_equal(k_cache, ref_k) and np.array_equal(v_cache, ref_v)  # append is bit-exact
    out = c_oracle.decode(np.ascontiguousarray(Q.reshape(B, E)), k_cache, v_cache, 5, B, H, D, strides)
    np.testing.assert_allclose(out, golden["kv_out"], rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("case", range(len(kv_oracle.FLASH_RECIPE_SHAPES)))
def test_flash_oracles_match_reference_recipe(golden, case):
    B, N, H, D = kv_oracle.FLASH_RECIPE_SHAPES[case]
    Q, K, V = kv_oracle.recipe_flash_inputs(B, N, H, D)
    chk = np.array([float(Q.sum()), float(K.sum()), float(V.sum())])
    np.testing.assert_allclose(chk, golden[f"flash_in_checksum_{case}"], rtol=0, atol=0)
    want = golden[f"flash_out_{case}"]
    dense = kv_oracle.flash_attention_dense(Q, K, V, B, N, H, D)
    np.testing.assert_allclose(dense, want, rtol=RTOL, atol=ATOL)
    # the reference test runs its kernel with 8x8 tiles (gpu_test.py:2427-2429)
    tiled, L, M = kv_oracle.flash_attention_tiled(Q, K, V, B, N, H, D, Br=8, Bc=8)
    np.testing.assert_allclose(tiled, want, rtol=RTOL, atol=ATOL)
    Oc, Lc, Mc = c_oracle.prefill(Q.reshape(B * N, H * D), K.reshape(B * N, H * D), V.reshape(B * N, H * D),
                                  B, N, H, D)
    np.testing.assert_allclose(Oc.reshape(B, N, H * D), want, rtol=RTOL, atol=ATOL)
    np.testing.assert_allclose(Lc, L, rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(Mc, M, rtol=1e-5, atol=1e-5)


def test_flash_tiled_default_tiles_agree():
    B, N, H, D = 2, 64, 2, 32
    Q, K, V = kv_oracle.recipe_flash_inputs(B, N, H, D)
    a, La, Ma = kv_oracle.flash_attention_tiled(Q, K, V, B, N, H, D, Br=32, Bc=32)
    b, Lb, Mb = kv_oracle.flash_attention_tiled(Q, K, V, B, N, H, D, Br=8, Bc=16)
    np.testing.assert_allclose(a, b, rtol=RTOL, atol=ATOL)
    np.testing.assert_allclose(La, Lb, rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(Ma, Mb, rtol=0, atol=1e-6)


def test_bf16_round_trip_and_rounding():
    rng = np.random.default_rng(0)
    x = rng.standard_normal(4096).astype(np.float32)
    bits = kv_oracle.f32_to_bf16_bits(x)
    back = kv_oracle.bf16_bits_to_f32(bits)
    assert np.all(np.abs(back - x) <= np.abs(x) * 2.0 ** -8)
    assert np.array_equal(kv_oracle.f32_to_bf16_bits(back), bits)  # idempotent
    # ties go to even: 1 + 2^-8 is exactly half way between 1 and 1 + 2^-7
    tie = np.array([1.0 + 2.0 ** -8, 1.0 + 3 * 2.0 ** -8], dtype=np.float32)
    assert kv_oracle.bf16_bits_to_f32(kv_oracle.f32_to_bf16_bits(tie)).tolist() == [1.0, 1.0 + 2.0 ** -6]


def test_c_and_numpy_agree_on_ragged_bf16_paged():
    rng = np.random.default_rng(1)
    B, H, D, bs, T_max = 3, 2, 32, 16, 96
    lens = np.array([1, 37, 96], dtype=np.int32)
    n_blocks = 64
    perm = rng.permutation(n_blocks).astype(np.int32)
    max_blocks = T_max // bs
    table = perm[: B * max_blocks].reshape(B, max_blocks)
    k_pool = np.zeros((n_blocks, H, bs, D), dtype=np.uint16)
    v_pool = np.zeros((n_blocks, H, bs, D), dtype=np.uint16)
    k_log = np.zeros((B, T_max, H, D), dtype=np.float32)
    v_log = np.zeros((B, T_max, H, D), dtype=np.float32)
    strides = (0, D, bs * D)
    for t in range(T_max):
        nk = kv_oracle.f32_to_bf16_bits(rng.standard_normal((B, H * D)).astype(np.float32))
        nv = kv_oracle.f32_to_bf16_bits(rng.standard_normal((B, H * D)).astype(np.float32))
        pos = np.minimum(t, lens - 1).astype(np.int32)  # sequences that are full rewrite their last row
        c_oracle.append(nk, nv, k_pool, v_pool, pos, B, H, D, strides, table, bs, H * bs * D)
        for b in range(B):
            k_log[b, pos[b]] = kv_oracle.bf16_bits_to_f32(nk[b]).reshape(H, D)
            v_log[b, pos[b]] = kv_oracle.bf16_bits_to_f32(nv[b]).reshape(H, D)
    # gather through the numpy oracle equals the logical copy, bit for bit
    g = kv_oracle.paged_gather(k_pool, table, lens, bs, T_max)
    for b in range(B):
        assert np.array_equal(kv_oracle.bf16_bits_to_f32(g[b, : lens[b]]), k_log[b, : lens[b]])
    q = kv_oracle.f32_to_bf16_bits(rng.standard_normal((B, H * D)).astype(np.float32))
    got = c_oracle.decode(q, k_pool, v_pool, lens, B, H, D, strides, table, bs, H * bs * D)
    want = kv_oracle.decode_attention(kv_oracle.bf16_bits_to_f32(q).reshape(B, H, D), k_log, v_log, lens)
    np.testing.assert_allclose(got, want.reshape(B, H * D), rtol=1e-4, atol=1e-5)


def test_decode_zero_length_sequence_is_zero():
    B, H, D, T = 2, 2, 16, 8
    rng = np.random.default_rng(2)
    k = rng.standard_normal((B * T, H * D)).astype(np.float32)
    v = rng.standard_normal((B * T, H * D)).astype(np.float32)
    q = rng.standard_normal((B, H * D)).astype(np.float32)
    out = c_oracle.decode(q, k, v, np.array([0, 3], dtype=np.int32), B, H, D, (T * H * D, H * D, D))
    assert np.all(out[0] == 0) and np.any(out[1] != 0)


def test_prompt_layer_oracle_agrees_with_the_decode_layer_oracle_on_the_last_token():
    """Two restatements of the reference block (whole prompt with a causal mask; one new token over cached
    rows) must give the same row for the last token of every sequence."""
    from oracle import decode_layer_oracle as o

    E, H, B, N = 64, 2, 2, 24
    rng = np.random.default_rng(0)
    r = lambda *s: o.bf16_round(rng.standard_normal(s).astype(np.float32) * 0.2)  # noqa: E731
    w = dict(ln1_gamma=r(E) + 1, ln1_beta=r(E), wq=r(E, E), wk=r(E, E), wv=r(E, E), wo=r(E, E), ln2_gamma=r(E) + 1,
             ln2_beta=r(E), w1=r(E, 4 * E), b1=r(4 * E), w2=r(4 * E, E), b2=r(E))
    x = r(B * N, E)
    y, k, v = o.prompt_layer_step(x, w, B, N, H)
    last = [N - 1, 2 * N - 1]
    ks = [k[b * N:(b + 1) * N] for b in range(B)]
    vs = [v[b * N:(b + 1) * N] for b in range(B)]
    y_last, k_new, _ = o.decoder_layer_step(x[last], w, ks, vs, np.full(B, N - 1), H)
    np.testing.assert_allclose(y_last, y[last], rtol=0, atol=1e-6)
    np.testing.assert_array_equal(k_new, k[last])


def test_model_oracle_cached_step_equals_longer_prompt():
    """The stacked-layer decoder oracle agrees with itself: a cached decode step after a prompt of N tokens gives
    the logits of the last position of the same N + 1 tokens run as one prompt (up to bf16 rounding of the
    intermediate rows, which the two paths round at the same places)."""
    from oracle import model_oracle
    from oracle.decode_layer_oracle import bf16_round

    rs = np.random.RandomState(0)
    E, V, H, L, N, B = 64, 96, 2, 2, 7, 2
    r = lambda shape, s=1.0: bf16_round((rs.randn(*shape) * s).astype(np.float32))  # noqa: E731
    layer = lambda: dict(ln1_gamma=r((E,), 0.1) + 1, ln1_beta=r((E,), 0.1), wq=r((E, E), E ** -0.5),  # noqa: E731
                         wk=r((E, E), E ** -0.5), wv=r((E, E), E ** -0.5), wo=r((E, E), E ** -0.5),
                         ln2_gamma=r((E,), 0.1) + 1, ln2_beta=r((E,), 0.1), w1=r((E, 4 * E), E ** -0.5),
                         b1=r((4 * E,), 0.1), w2=r((4 * E, E), (4 * E) ** -0.5), b2=r((E,), 0.1))
    params = dict(embedding=r((V, E)), pos_encoding=r((N + 1, E)), layers=[layer() for _ in range(L)],
                  lnf_gamma=r((E,), 0.1) + 1, lnf_beta=r((E,), 0.1), out_proj=r((E, V), E ** -0.5))
    ids = rs.randint(0, V, size=(B, N + 1))
    _, cache = model_oracle.prefill(params, ids[:, :N].reshape(-1), B, N, H)
    stepped = model_oracle.decode_step(params, ids[:, N], cache, H)
    whole, _ = model_oracle.prefill(params, ids.reshape(-1), B, N + 1, H)
    assert len(cache[0][0][0]) == N + 1
    np.testing.assert_allclose(stepped, whole, rtol=0, atol=4e-2)
