"""Cached text generation with the reference's sampling options.

The reference's ``generate_text`` (simple-llm/src/generate.py:8-72) re-runs the whole forward
pass over a left-padded context for every new token; ``sample_token``
(simple-llm/src/jax_backend.py:413-515) turns the last position's logits into a token.  Here the
loop is the one the KV-cache path exists for: one prefill of the prompt (``flash_attention`` fused
with the cache write), then one ``kv_cache_update`` + ``attention_with_kv_cache`` per layer per
new token.  The sampling rules are the reference's, in its order: repetition penalty (the logit is
DIVIDED by the penalty whatever its sign, as in the reference), greedy when ``temperature == 0``,
temperature, softmax, min-p, top-k, top-p (each followed by a renormalisation), then one draw.
Argument names and defaults follow the reference; the random stream is torch's, seeded with 42
like the reference's ``PRNGKey(42)``, so draws differ from JAX's while the distributions agree.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch


def filtered_distribution(logits: torch.Tensor, temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0,
                          min_p: float = 0.0, repetition_penalty: float = 1.0,
                          recent_tokens: Optional[Sequence[int]] = None) -> torch.Tensor:
    """The probability vector that the reference samples from (``temperature`` must be > 0)."""
    logits = logits.to(torch.float32).clone()
    if repetition_penalty != 1.0 and recent_tokens is not None and len(recent_tokens) > 0:
        idx = torch.tensor(sorted(set(int(t) for t in recent_tokens)), device=logits.device, dtype=torch.long)
        logits[idx] = logits[idx] / repetition_penalty
    probs = torch.softmax(logits / temperature, dim=-1)
    if min_p > 0.0:
        probs = torch.where(probs >= min_p * probs.max(), probs, torch.zeros_like(probs))
        probs = probs / probs.sum()
    if top_k > 0:
        keep = torch.argsort(probs, stable=True)[-top_k:]  # ascending order, last k: ties as in the reference
        mask = torch.zeros_like(probs, dtype=torch.bool)
        mask[keep] = True
        probs = torch.where(mask, probs, torch.zeros_like(probs))
        probs = probs / probs.sum()
    if top_p < 1.0:
        order = torch.argsort(probs, stable=True).flip(0)  # descending
        sorted_probs = probs[order]
        keep = torch.cumsum(sorted_probs, dim=0) <= top_p
        keep[0] = True  # always keep the most likely token
        filtered = torch.zeros_like(probs)
        filtered[order] = torch.where(keep, sorted_probs, torch.zeros_like(sorted_probs))
        probs = filtered / filtered.sum()
    return probs


def sample_token(generator: Optional[torch.Generator], logits: torch.Tensor, temperature: float = 1.0, top_k: int = 0,
                 top_p: float = 1.0, min_p: float = 0.0, repetition_penalty: float = 1.0,
                 recent_tokens: Optional[Sequence[int]] = None) -> int:
    """One token id from ``logits [vocab]`` under the reference's filtering rules."""
    if temperature == 0.0:
        logits = logits.to(torch.float32).clone()
        if repetition_penalty != 1.0 and recent_tokens is not None and len(recent_tokens) > 0:
            idx = torch.tensor(sorted(set(int(t) for t in recent_tokens)), device=logits.device, dtype=torch.long)
            logits[idx] = logits[idx] / repetition_penalty
        return int(torch.argmax(logits))
    probs = filtered_distribution(logits, temperature, top_k, top_p, min_p, repetition_penalty, recent_tokens)
    return int(torch.multinomial(probs, 1, generator=generator))


def generate_text(model, prompt_tokens: Sequence[int], max_tokens: int = 100, temperature: float = 1.0,
                  top_k: int = 0, top_p: float = 1.0, min_p: float = 0.0, repetition_penalty: float = 1.0,
                  repetition_window: int = 64, seed: int = 42) -> List[int]:
    """Generates ``max_tokens`` tokens after the prompt with a KV cache; ``model`` is a ``TinyGPT``
    (anything with ``cache``, ``prefill(tokens)`` and ``decode_step(token)`` returning logits).
    The prompt plus the new tokens must fit the model's context (the cache does not slide)."""
    from . import gpu

    tokens = [int(t) for t in prompt_tokens]
    if len(tokens) == 0:
        raise ValueError("prompt_tokens must not be empty")
    if len(tokens) + max_tokens > model.context:
        raise ValueError(f"prompt ({len(tokens)}) + max_tokens ({max_tokens}) exceeds the context ({model.context})")
    device = model.ctx.device
    generator = torch.Generator(device=device).manual_seed(seed)
    gpu.kv_cache_reset(model.cache)
    logits = model.prefill(tokens)
    for i in range(max_tokens):
        recent = tokens[max(0, len(tokens) - repetition_window):]
        tokens.append(sample_token(generator, logits[0], temperature, top_k, top_p, min_p, repetition_penalty, recent))
        if i + 1 < max_tokens:
            logits = model.decode_step(tokens[-1])
    return tokens
