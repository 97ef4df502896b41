"""CPU restatement of the reference's token sampling (test infrastructure only).

``ref_sample`` / ``ref_top_p`` follow ``cwm/fastgen/utils/sampling.py:6-18`` and
``:21-45`` operation for operation in fp32; ``ref_sample_logits`` follows
``FastGen._sample`` (``cwm/fastgen/generate.py:996-1014``).  The one substitution:
where the reference calls ``torch.multinomial(weights, 1)``, whose random stream
cannot be reproduced outside torch, the draw is ``inverse_cdf(weights, u)`` with a
caller-supplied uniform number per row -- the first index whose inclusive running
sum exceeds ``u * total``.  ``tests/golden/make_sampling_golden.py`` runs the
reference's own functions with the same substitution and stores their outputs;
``tests/test_oracle_sampling.py`` pins this file to them.

``exact_top_p`` / ``exact_sample`` state the same operations in exact integer
arithmetic (probabilities as multiples of 2^-44): the specification the CUDA
kernel is held to bit for bit.  It differs from the fp32 restatement only where
the fp32 running sum's rounding decides (an entry whose exclusive running sum is
within rounding of ``p``, a uniform number within rounding of an interval end) and
in the order of entries of equal probability, which ``torch.sort`` leaves open
and which is ascending index here.
"""

from __future__ import annotations

import numpy as np
import torch

UNIT_SHIFT = 44


def inverse_cdf(weights: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
    """Stand-in for ``torch.multinomial(weights, num_samples=1)``: per row the
    first index whose inclusive running sum (fp32, like the weights) exceeds
    ``u * total``; shape ``(rows, 1)`` like multinomial's result."""
    csum = torch.cumsum(weights, dim=-1)
    target = u.to(weights.dtype)[:, None] * csum[:, -1:]
    idx = (csum > target).to(torch.int8).argmax(dim=-1, keepdim=True)
    return idx


def ref_sample(probs: torch.Tensor, u: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``sample`` of ``sampling.py:6-18``."""
    next_tokens = inverse_cdf(probs, u)
    next_tokens_prob = torch.gather(probs, -1, next_tokens)
    return next_tokens.squeeze(-1), next_tokens_prob.squeeze(-1)


def ref_top_p(probs: torch.Tensor, p: torch.Tensor, u: torch.Tensor, stable: bool = True
              ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``top_p`` of ``sampling.py:21-45``; additionally returns how many entries
    survive the mask.  ``p``: ``(rows, 1)``."""
    probs_sort, probs_idx = torch.sort(probs, dim=-1, descending=True, stable=stable)
    probs_sum = torch.cumsum(probs_sort, dim=-1)
    probs_sort[probs_sum - probs_sort > p] = 0.0
    kept = (probs_sort > 0).sum(-1)
    probs_sort /= probs_sort.sum(-1, keepdim=True)
    sample = inverse_cdf(probs_sort, u)
    next_tokens = torch.gather(probs_idx, -1, sample)
    next_tokens_prob = torch.gather(probs_sort, -1, sample)
    return next_tokens.squeeze(-1), next_tokens_prob.squeeze(-1), kept


def ref_sample_logits(logits: torch.Tensor, temps: torch.Tensor, top_ps: torch.Tensor | None,
                      use_sampling: bool, u: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``FastGen._sample`` of ``generate.py:996-1014`` (``top_ps`` None stands for
    an empty ``top_p_lanes`` set)."""
    if use_sampling:
        probs = torch.softmax(logits / temps[:, None], dim=-1)
        if top_ps is None:
            next_tokens, next_tokens_prob = ref_sample(probs, u)
        else:
            next_tokens, next_tokens_prob, _ = ref_top_p(probs, top_ps[:, None], u)
        return next_tokens, torch.log(next_tokens_prob)
    next_tokens = torch.argmax(logits, dim=-1)
    return next_tokens, torch.zeros_like(next_tokens, dtype=logits.dtype)


# ------------------------------------------------------- exact integer statement
def to_units(p: np.ndarray) -> np.ndarray:
    """fp32 probabilities -> integer multiples of 2^-44 (truncated; a positive
    probability is at least one unit; zero and negative values are zero)."""
    p = np.asarray(p, dtype=np.float32)
    bits = p.view(np.uint32).astype(np.uint64)
    e = (bits >> np.uint64(23)).astype(np.int64) & 0xFF
    m = (bits & np.uint64(0x7FFFFF)) | np.uint64(0x800000)
    shift = e - (127 + 23 - UNIT_SHIFT)
    left = np.clip(shift, 0, 39).astype(np.uint64)
    right = np.clip(-shift, 0, 63).astype(np.uint64)
    units = np.where(shift >= 0, m << left, np.where(shift < -24, np.uint64(0), m >> right))
    units = np.maximum(units, np.uint64(1))
    units = np.where(e == 0, np.uint64(1), units)
    dead = (bits == 0) | ((bits >> np.uint64(31)) != 0)
    return np.where(dead, np.uint64(0), units).astype(np.uint64)


def exact_sample(probs: np.ndarray, u: float) -> tuple[int, float]:
    """One row of ``sample`` in integer arithmetic: (index, probability / total)."""
    units = to_units(probs)
    csum = np.cumsum(units, dtype=np.uint64)
    total = int(csum[-1])
    if total == 0:
        return 0, 0.0
    target = min(int(np.float64(np.float32(u)) * np.float64(total)), total - 1)
    idx = int(np.searchsorted(csum, target, side="right"))
    return idx, float(np.float32(np.float64(probs[idx]) * 2.0**UNIT_SHIFT / np.float64(total)))


def exact_top_p(probs: np.ndarray, p: float, u: float) -> tuple[int, float, int]:
    """One row of ``top_p`` in integer arithmetic: (index, renormalised
    probability, surviving entries).  Descending order, equal values by ascending
    index; ``p >= 1`` keeps every positive entry."""
    probs = np.asarray(probs, dtype=np.float32)
    units = to_units(probs)
    order = np.lexsort((np.arange(len(probs)), -probs.astype(np.float64)))
    order = order[units[order] > 0]
    if len(order) == 0:
        return 0, 0.0, 0
    su = units[order]
    incl = np.cumsum(su, dtype=np.uint64)
    excl = incl - su
    p32 = np.float32(p)
    if p32 >= 1:
        keep = np.ones(len(order), dtype=bool)
    else:
        limit = 0 if p32 <= 0 else int(np.float64(p32) * 2.0**UNIT_SHIFT)
        keep = excl <= np.uint64(limit)
    n_keep = int(keep.sum())  # a prefix of the order
    kept_mass = int(incl[n_keep - 1])
    target = min(int(np.float64(np.float32(u)) * np.float64(kept_mass)), kept_mass - 1)
    pos = int(np.searchsorted(incl[:n_keep], target, side="right"))
    idx = int(order[pos])
    prob = float(np.float32(np.float64(probs[idx]) * 2.0**UNIT_SHIFT / np.float64(kept_mass)))
    return idx, prob, n_keep
