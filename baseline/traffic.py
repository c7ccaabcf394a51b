"""Synthetic RAG traffic, shared by both arms of the headline benchmark.

Plain Python with no import of either implementation, so the reference arm and this
framework's arm serve the very same requests: a 64-token system prefix, ``k`` chunks drawn
Zipf(s = 1.1) from a pool of lognormal-length chunks (median 300 tokens, sigma 0.6, clipped to
64..1024, padded with token 0 to whole blocks) and a 64-token query.
"""

from __future__ import annotations

import math
import random

# model shapes by name: what a Hugging Face ``config.json`` of the architecture needs
MODEL_SHAPES = {
    "llama3-70b": dict(vocab_size=128256, hidden_size=8192, num_hidden_layers=80, num_attention_heads=64,
                       num_key_value_heads=8, head_dim=128, intermediate_size=28672, rope_theta=500000.0,
                       rms_norm_eps=1e-5, llama3_scaling=True),
    "llama3-8b": dict(vocab_size=128256, hidden_size=4096, num_hidden_layers=32, num_attention_heads=32,
                      num_key_value_heads=8, head_dim=128, intermediate_size=14336, rope_theta=500000.0,
                      rms_norm_eps=1e-5, llama3_scaling=True),
    "tiny-gqa": dict(vocab_size=1024, hidden_size=512, num_hidden_layers=2, num_attention_heads=8,
                     num_key_value_heads=2, head_dim=128, intermediate_size=1024, rope_theta=500000.0,
                     rms_norm_eps=1e-5, llama3_scaling=False),
}


def make_traffic(vocab_size: int, block_tokens: int, pool_size: int, k_chunks: int, n_requests: int, seed: int = 0):
    """Returns ``(prefix, pool, requests)``; a request is ``([prefix, chunk, ...], query, picks)``."""
    rng = random.Random(seed)
    bt = block_tokens
    pad = 0

    def tokens(n):
        return [rng.randrange(1, vocab_size) for _ in range(n)]

    def padded(n):
        t = tokens(n)
        return t + [pad] * (-len(t) % bt)

    prefix = padded(64)
    pool = []
    for _ in range(pool_size):
        n = int(round(math.exp(math.log(300.0) + 0.6 * rng.gauss(0, 1))))
        pool.append(padded(max(64, min(1024, n))))
    weights = [1.0 / (r + 1) ** 1.1 for r in range(pool_size)]
    reqs = []
    for _ in range(n_requests):
        picks = rng.choices(range(pool_size), weights=weights, k=k_chunks)
        reqs.append(([prefix] + [pool[i] for i in picks], tokens(64), picks))
    return prefix, pool, reqs


def percentile(vals, q):
    v = sorted(vals)
    return v[max(0, min(len(v) - 1, int(round(q / 100.0 * (len(v) - 1)))))]
