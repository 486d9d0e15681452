"""Sampling parameters and the host-side reference sampler.

Defaults and the greedy rule follow the reference (reference: src/v2/config/OrchestrationConfig.h:364-366
CLI defaults T=0.8 / top-k 40 / top-p 0.9; src/v2/utils/Sampler.h ``is_greedy``: temperature == 0 or
(top_k == 1 and top_p >= 1); src/v2/models/qwen3/Qwen3Schema.h:44-51 model-recommended values).
The GPU path uses the kernels in ops/csrc/ops.cu; this module is the CPU path and the oracle.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch


@dataclass
class SamplingParams:
    temperature: float = 0.8
    top_k: int = 40
    top_p: float = 0.9
    seed: int | None = None
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    dry_multiplier: float = 0.0
    dry_base: float = 1.75
    dry_allowed_length: int = 2
    max_tokens: int = 128
    stop_token_ids: tuple[int, ...] = ()
    ignore_eos: bool = False
    logprobs: int = -1                  # -1 off; k >= 0: report the chosen token's log-probability and the k likeliest tokens

    @property
    def wants_logprobs(self) -> bool:
        return self.logprobs >= 0

    @property
    def is_greedy(self) -> bool:
        return self.temperature <= 0.0 or (self.top_k == 1 and self.top_p >= 1.0)

    @property
    def needs_penalties(self) -> bool:
        return self.presence_penalty != 0.0 or self.frequency_penalty != 0.0 or self.dry_multiplier > 0.0


MODEL_DEFAULTS = {
    # values a request inherits when it does not set the field itself
    "qwen3": dict(temperature=0.6, top_p=0.95, top_k=20, presence_penalty=1.5),
    "qwen3moe": dict(temperature=0.6, top_p=0.95, top_k=20, presence_penalty=1.5),
    "qwen2": dict(temperature=0.7, top_p=0.8, top_k=20, presence_penalty=0.0),
    # the hybrid families' recommended values (reference: src/v2/models/qwen35/Qwen35Schema.h:64-67)
    "qwen35": dict(temperature=0.6, top_p=0.95, top_k=20, presence_penalty=1.5),
    "qwen35moe": dict(temperature=0.6, top_p=0.95, top_k=20, presence_penalty=1.5),
}


def merge_with_model_defaults(arch: str, given: dict, cli: SamplingParams | None = None) -> SamplingParams:
    base = SamplingParams() if cli is None else SamplingParams(**{k: getattr(cli, k) for k in SamplingParams.__dataclass_fields__})
    for k, v in MODEL_DEFAULTS.get(arch, {}).items():
        setattr(base, k, v)
    for k, v in given.items():
        if v is not None and hasattr(base, k):
            setattr(base, k, v)
    return base


def apply_penalties(logits: torch.Tensor, history: list[int], p: SamplingParams) -> torch.Tensor:
    """Presence / frequency / DRY penalties on one row of logits (returns a new tensor)."""
    if not history or not p.needs_penalties:
        return logits
    out = logits.clone()
    if p.presence_penalty or p.frequency_penalty:
        toks, counts = torch.unique(torch.tensor(history, dtype=torch.long), return_counts=True)
        toks = toks.to(out.device)
        out[toks] -= p.presence_penalty + p.frequency_penalty * counts.to(out.device, out.dtype)
    if p.dry_multiplier > 0.0:
        for tok, length in dry_match_lengths(history).items():
            if length >= p.dry_allowed_length:
                out[tok] -= p.dry_multiplier * p.dry_base ** (length - p.dry_allowed_length)
    return out


def dry_match_lengths(history: list[int]) -> dict[int, int]:
    """For every token t: the longest suffix of ``history`` that, earlier in the history, was followed by t.

    Computed with the Z-algorithm on the reversed history (a repeat of length L ending right before an
    earlier occurrence of t means emitting t would extend a verbatim repetition by one more token).
    """
    n = len(history)
    if n < 2:
        return {}
    rev = history[::-1]
    z = [0] * n
    l = r = 0
    for i in range(1, n):
        if i < r:
            z[i] = min(r - i, z[i - l])
        while i + z[i] < n and rev[z[i]] == rev[i + z[i]]:
            z[i] += 1
        if i + z[i] > r:
            l, r = i, i + z[i]
    best: dict[int, int] = {}
    for i in range(1, n):
        if z[i] > 0:
            follower = rev[i - 1]           # token that came right after the earlier copy of the suffix
            if z[i] > best.get(follower, 0):
                best[follower] = z[i]
    return best


def sample_row(logits: torch.Tensor, p: SamplingParams, gen: torch.Generator | None = None) -> int:
    """Reference sampler: temperature -> top-k -> top-p -> multinomial."""
    if p.is_greedy:
        return int(torch.argmax(logits))
    x = logits.float() / max(p.temperature, 1e-6)
    k = p.top_k if 0 < p.top_k < x.numel() else min(x.numel(), 1024)
    vals, idx = torch.topk(x, k)
    probs = torch.softmax(vals, dim=-1)
    if p.top_p < 1.0:
        cum = torch.cumsum(probs, dim=-1)
        keep = (cum - probs) < p.top_p
        keep[0] = True
        probs = torch.where(keep, probs, torch.zeros_like(probs))
        probs = probs / probs.sum()
    choice = torch.multinomial(probs.cpu(), 1, generator=gen)
    return int(idx[choice])


def filtered_probs(logits: torch.Tensor, p: SamplingParams) -> torch.Tensor:
    """The distribution `sample_row` draws from, as a dense [vocab] vector (speculative-sampling verification)."""
    out = torch.zeros(logits.numel(), dtype=torch.float32, device=logits.device)
    if p.is_greedy:
        out[int(torch.argmax(logits))] = 1.0
        return out
    x = logits.float() / max(p.temperature, 1e-6)
    k = p.top_k if 0 < p.top_k < x.numel() else min(x.numel(), 1024)
    vals, idx = torch.topk(x, k)
    probs = torch.softmax(vals, dim=-1)
    if p.top_p < 1.0:
        cum = torch.cumsum(probs, dim=-1)
        keep = (cum - probs) < p.top_p
        keep[0] = True
        probs = torch.where(keep, probs, torch.zeros_like(probs))
        probs = probs / probs.sum()
    out[idx] = probs
    return out
