#!/usr/bin/env python3
"""Generate ``reference_recipes.npz`` from the reference's own test code.

The reference keeps no golden output files: its tests pin the KV-cache path with
seeded recipes and compare the kernels with reference math written inside the test
file (simple-llm/src/gpu_test.py).  That file cannot be imported here (it imports
jax and wgpu at the top), so this script reads it as text and executes only the
reference-math lines, straight from the reference tree, on the recipes' inputs:

* lines 2328-2367: the numpy loop that computes the expected decode-attention output;
* lines 543-552, 1681-1686, 2082-2083: the expected outputs of the layernorm, softmax and
  extract_last_tokens tests (the first GOLDEN_ROWS rows of each are stored);
* lines 776-810:   the dense causal attention of the flash test.  It is written with
  ``jax.numpy``; every call it makes (array, reshape, transpose, sqrt, einsum, tril,
  ones, where) exists in numpy with the same meaning, so ``jnp`` is bound to numpy
  and ``jax.nn.softmax`` to a max-subtracted numpy softmax.

No reference source is copied into this repository; only the numeric outputs are
stored.  Run from the repository root, in a container that has the reference tree:

    python tests/golden/make_golden.py /path/to/reference

The fixture travels with the repository; the reference tree is not needed to run
the tests.
"""

from __future__ import annotations

import pathlib
import sys
import textwrap
import types

import numpy as np

HERE = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

from oracle import kv_oracle, step_tail_oracle  # noqa: E402  (recipe inputs only)


def snippet(lines, first, last):
    """Source lines ``first..last`` (1-based, inclusive), dedented."""
    return textwrap.dedent("".join(lines[first - 1 : last]))


def softmax(x, axis=-1):
    x = np.asarray(x)
    e = np.exp(x - x.max(axis=axis, keepdims=True))
    return e / e.sum(axis=axis, keepdims=True)


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/reference")
    ref_root = pathlib.Path(sys.argv[1])
    test_file = ref_root / "simple-llm" / "src" / "gpu_test.py"
    lines = test_file.read_text().splitlines(keepends=True)
    # Guard against a different revision of the reference: anchor lines must match.
    assert "K_cached_4d = np.concatenate(" in lines[2328], lines[2328]
    assert "O_jax_flat = O_jax_4d.reshape" in lines[2366], lines[2366]
    assert "Q_jax = (" in lines[777], lines[777]
    assert "output_jax_np = np.array(output_jax)" in lines[809], lines[809]

    out = {}

    # ---- KV-cache recipe (gpu_test.py:2208-2212, 2267-2289, 2317) ----
    batch_size, n_heads, head_dim, num_tokens = 2, 4, 64, 5
    ks, vs, Q_4d = kv_oracle.recipe_kv_cache_inputs(batch_size, n_heads, head_dim, num_tokens, seed=42)
    ns = {
        "np": np,
        "reference_k_list": ks,
        "reference_v_list": vs,
        "Q_4d": Q_4d,
        "batch_size": batch_size,
        "n_heads": n_heads,
        "head_dim": head_dim,
        "current_len": num_tokens,
        "query_len": 1,
        "embedding_dim": n_heads * head_dim,
    }
    exec(compile(snippet(lines, 2328, 2367), str(test_file), "exec"), ns)
    out["kv_out"] = np.asarray(ns["O_jax_flat"], dtype=np.float32)
    out["kv_in_checksum"] = np.array(
        [sum(float(k.sum()) for k in ks), sum(float(v.sum()) for v in vs), float(Q_4d.sum())]
    )

    # ---- flash-attention recipes (gpu_test.py:747-756, 770-774) ----
    jax_shim = types.SimpleNamespace(nn=types.SimpleNamespace(softmax=softmax))
    for i, (batch, seq_len, nh, hd) in enumerate(kv_oracle.FLASH_RECIPE_SHAPES):
        Q_np, K_np, V_np = kv_oracle.recipe_flash_inputs(batch, seq_len, nh, hd, seed=42)
        ns = {
            "np": np,
            "jnp": np,
            "jax": jax_shim,
            "Q_np": Q_np,
            "K_np": K_np,
            "V_np": V_np,
            "batch": batch,
            "seq_len": seq_len,
            "n_heads": nh,
            "head_dim": hd,
        }
        exec(compile(snippet(lines, 776, 810), str(test_file), "exec"), ns)
        out[f"flash_out_{i}"] = np.asarray(ns["output_jax_np"], dtype=np.float32)
        out[f"flash_in_checksum_{i}"] = np.array([float(Q_np.sum()), float(K_np.sum()), float(V_np.sum())])

    # ---- tail of a generation step: layernorm, softmax, extract_last_tokens ----
    assert "x_jax = jnp.array(x_np)" in lines[542] and "y_jax_np = np.array(y_jax)" in lines[551], lines[542]
    assert "softmax_jax_list = []" in lines[1680] and "softmax_jax_np = np.array(softmax_jax_list)" in lines[1685]
    assert "input_reshaped = input_np.reshape" in lines[2081] and "expected_np = input_reshaped" in lines[2082]
    rows = step_tail_oracle.GOLDEN_ROWS
    for i, (n_elements, size) in enumerate(step_tail_oracle.LAYERNORM_RECIPE_SHAPES):
        x_np, gamma_np, beta_np = step_tail_oracle.recipe_layernorm_inputs(n_elements, size)
        ns = {"np": np, "jnp": np, "x_np": x_np, "gamma_np": gamma_np, "beta_np": beta_np}
        exec(compile(snippet(lines, 543, 552), str(test_file), "exec"), ns)
        out[f"layernorm_out_{i}"] = np.asarray(ns["y_jax_np"], dtype=np.float32)[:rows]
    for i, (batch_size, vocab_size, transform) in enumerate(step_tail_oracle.SOFTMAX_RECIPES):
        x_np = step_tail_oracle.recipe_softmax_inputs(batch_size, vocab_size, transform)
        ns = {"np": np, "jnp": np, "jax": jax_shim, "x_np": x_np, "batch_size": batch_size}
        exec(compile(snippet(lines, 1681, 1686), str(test_file), "exec"), ns)
        out[f"softmax_out_{i}"] = np.asarray(ns["softmax_jax_np"], dtype=np.float32)[:rows]
    for i, (batch_size, seq_len, emb_dim) in enumerate(step_tail_oracle.EXTRACT_RECIPE_SHAPES):
        input_np = step_tail_oracle.recipe_extract_inputs(batch_size, seq_len, emb_dim)
        ns = {"np": np, "input_np": input_np, "batch_size": batch_size, "seq_len": seq_len, "emb_dim": emb_dim}
        exec(compile(snippet(lines, 2082, 2083), str(test_file), "exec"), ns)
        out[f"extract_out_{i}"] = np.asarray(ns["expected_np"], dtype=np.float32)[:rows]

    np.savez_compressed(HERE / "reference_recipes.npz", **out)
    print("wrote", HERE / "reference_recipes.npz")
    print("kv_out sum", float(out["kv_out"].sum()), "first", out["kv_out"][0, :4])
    print("flash_out_0 sum", float(out["flash_out_0"].sum()))


if __name__ == "__main__":
    main()
