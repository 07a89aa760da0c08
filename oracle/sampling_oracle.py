"""CPU oracle (numpy) of the reference's token sampling rules.  TEST INFRASTRUCTURE ONLY.

Restates simple-llm/src/jax_backend.py:461-510: repetition penalty (logit / penalty for every
distinct recent token), temperature, softmax, min-p, top-k (``argsort(probs)[-k:]``), top-p
(descending order = reversed ascending argsort, cumulative sum <= top_p, first token always
kept), each filter followed by a renormalisation.  Returns the distribution that the reference
hands to ``jax.random.choice``; the draw itself is not part of the oracle.
"""
from __future__ import annotations

import numpy as np


def filtered_distribution(logits, temperature=1.0, top_k=0, top_p=1.0, min_p=0.0, repetition_penalty=1.0,
                          recent_tokens=()):
    logits = np.array(logits, dtype=np.float32)
    if repetition_penalty != 1.0 and len(recent_tokens) > 0:
        for token_id in set(int(t) for t in recent_tokens):
            logits[token_id] = logits[token_id] / np.float32(repetition_penalty)
    logits = logits / np.float32(temperature)
    e = np.exp(logits - logits.max())
    probs = (e / e.sum()).astype(np.float32)
    if min_p > 0.0:
        probs = np.where(probs >= np.float32(min_p) * probs.max(), probs, np.float32(0.0))
        probs = probs / probs.sum()
    if top_k > 0:
        keep = np.argsort(probs, kind="stable")[-top_k:]
        mask = np.zeros_like(probs, dtype=bool)
        mask[keep] = True
        probs = np.where(mask, probs, np.float32(0.0))
        probs = probs / probs.sum()
    if top_p < 1.0:
        order = np.argsort(probs, kind="stable")[::-1]
        sorted_probs = probs[order]
        keep = np.cumsum(sorted_probs) <= top_p
        keep[0] = True
        filtered = np.zeros_like(probs)
        filtered[order] = np.where(keep, sorted_probs, np.float32(0.0))
        probs = filtered / filtered.sum()
    return probs.astype(np.float32)
