"""Truncated sampling (top-k, top-p) as a threshold on logit values.

Both truncations keep a prefix of the vocabulary sorted by logit, so each reduces to one number per
row: the smallest logit that stays.  Masking everything below that number commutes with sharding
the vocabulary, which is what lets the tensor-parallel engine keep its sampling scheme (every rank
masks its own shard, then the Gumbel-max candidate exchange picks the token): only the threshold
needs the whole row, and it is computed here with plain PyTorch on whatever device holds the logits.
This runs outside the captured layer loop and only for requests that ask for it.

Order as in vLLM's sampler (``vllm/v1/sample/ops/topk_topp_sampler.py``): top-k first, then top-p over
what is left, probabilities taken at the request's temperature; the token that crosses ``top_p`` is
kept.  The reference has no sampler (``daser/service/vllm_client.py:62-126`` forwards the fields).
"""

from __future__ import annotations

import torch


def sampling_threshold(logits: torch.Tensor, inv_temp: torch.Tensor, top_k: torch.Tensor,
                       top_p: torch.Tensor) -> torch.Tensor:
    """``logits [n, V]`` (whole rows), ``inv_temp [n]`` (0 = greedy row: untouched), ``top_k [n]``
    (0 = off), ``top_p [n]`` (1 = off)  ->  ``tau [n]``: sample among ``logits >= tau`` only."""
    n, vocab = logits.shape
    dev = logits.device
    tau = torch.full((n,), float("-inf"), device=dev)
    k = top_k.to(dev).long().clamp(min=0, max=vocab)
    p = top_p.to(dev).float()
    active = (inv_temp.to(dev) > 0) & (((k > 0) & (k < vocab)) | (p < 1.0))
    if not bool(active.any()):
        return tau
    ordered = logits.float().sort(dim=-1, descending=True).values
    rank = torch.arange(vocab, device=dev)[None, :]
    k_eff = torch.where(k > 0, k, torch.full_like(k, vocab))
    scaled = ordered * inv_temp.to(dev).float().clamp(min=1e-6)[:, None]
    scaled = scaled.masked_fill(rank >= k_eff[:, None], float("-inf"))      # top-k first
    probs = torch.softmax(scaled, dim=-1)
    before = probs.cumsum(-1) - probs                                      # mass of the strictly larger logits
    keep = (before < p[:, None]) & (rank < k_eff[:, None])
    count = keep.sum(-1).clamp(min=1)                                      # the best token always stays
    chosen = ordered.gather(1, (count - 1)[:, None]).squeeze(1)
    return torch.where(active, chosen, tau)


def apply_truncation(logits: torch.Tensor, inv_temp: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
                     whole_rows: torch.Tensor | None = None) -> None:
    """Mask ``logits`` (a rank's shard, or whole rows) in place below the rows' thresholds.
    ``whole_rows``: the gathered rows when ``logits`` is only a shard of them."""
    tau = sampling_threshold(logits if whole_rows is None else whole_rows, inv_temp, top_k, top_p)
    logits.masked_fill_(logits < tau[:, None].to(logits.dtype), float("-inf"))
