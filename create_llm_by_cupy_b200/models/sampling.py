"""Token sampling helpers for generation (reference: model/model.py:611-637).

The reference's nucleus sampler picks *uniformly* among the nucleus candidates and prints the
candidate count; here the draw is weighted by the renormalised probabilities, which is what
top-p sampling means, and nothing is printed.
"""
from __future__ import annotations

import torch


def apply_repetition_penalty(logits: torch.Tensor, seen_tokens, penalty: float = 1.2) -> torch.Tensor:
    """score < 0 -> score * penalty, else score / penalty, for every token id already produced."""
    if penalty == 1.0 or not seen_tokens:
        return logits
    idx = torch.tensor(sorted(set(int(t) for t in seen_tokens)), dtype=torch.long, device=logits.device)
    idx = idx[(idx >= 0) & (idx < logits.numel())]
    vals = logits[idx]
    logits = logits.clone()
    logits[idx] = torch.where(vals < 0, vals * penalty, vals / penalty)
    return logits


def softmax_with_temperature(logits: torch.Tensor, temp: float = 1.0) -> torch.Tensor:
    return torch.softmax(logits.float() / max(float(temp), 1e-6), dim=-1)


def top_p_sampling(logits: torch.Tensor, temp: float = 0.7, top_p: float = 0.9, generator=None) -> int:
    """Temperature softmax, keep the smallest set of tokens whose mass reaches ``top_p``, draw one
    of them with probability proportional to its mass."""
    probs = softmax_with_temperature(logits, temp)
    sp, si = torch.sort(probs, descending=True)
    cum = torch.cumsum(sp, 0)
    keep = int(torch.searchsorted(cum, torch.tensor(top_p, device=cum.device)).item()) + 1
    keep = max(1, min(keep, sp.numel()))
    cand = sp[:keep]
    cand = cand / cand.sum()
    pick = torch.multinomial(cand, 1, generator=generator)
    return int(si[pick].item())
