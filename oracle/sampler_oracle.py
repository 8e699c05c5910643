"""CPU restatement of the reference's token sampler. TEST INFRASTRUCTURE ONLY: imported by tests/
and nothing else; the product path is the CUDA kernel behind `pb_sample_top_p`.

Follows parrot/engine/builtin/models/sampler.py:19-66: logits = hidden @ embedding^T, divided by the
per-row temperature, nucleus (top-p) filtering over the row sorted by descending logit (a token is
dropped when the probability mass sorted BEFORE it exceeds top_p), softmax of what is left, one draw
per row. Pinned on the probability rows the reference's own code hands to `torch.multinomial`
(tests/golden/sampler_probs_ref.npz).

The reference draws with `torch.multinomial`; its stream of random numbers is a property of torch,
not of the algorithm, so the draw is restated as the inverse CDF over the row in INDEX order for a
given uniform number u: the smallest index whose cumulative probability exceeds u. Same distribution.
Ties in the sort are ordered by index (a stable sort), the order the CUDA kernel uses too.
"""
from __future__ import annotations

import numpy as np


def nucleus_probs_reference(logits: np.ndarray, temperature: np.ndarray, top_p: np.ndarray) -> np.ndarray:
    """[rows, vocab] probabilities the sampler draws from (sampler.py:31-63), float64."""
    x = np.asarray(logits, dtype=np.float64) / np.asarray(temperature, dtype=np.float64)[:, None]
    out = np.zeros_like(x)
    for r in range(x.shape[0]):
        row = x[r]
        order = np.argsort(-row, kind="stable")               # descending, ties by index
        srt = row[order]
        p = np.exp(srt - srt[0])
        p /= p.sum()
        before = np.cumsum(p) - p                             # mass sorted before each token
        keep = ~(before > float(top_p[r])) if top_p[r] < 1.0 else np.ones_like(p, dtype=bool)
        kept = np.where(keep, np.exp(srt - srt[0]), 0.0)
        kept /= kept.sum()
        out[r, order] = kept
    return out


def nucleus_margin(logits: np.ndarray, temperature: np.ndarray, top_p: np.ndarray) -> np.ndarray:
    """Per row: (distance of top_p from the nearest 'mass before' value, probability of that token,
    index of that token). A comparison with a float32 implementation is only meaningful for the
    tokens whose distance is well above float32 rounding; tests use this to know which token may
    fall either way."""
    x = np.asarray(logits, dtype=np.float64) / np.asarray(temperature, dtype=np.float64)[:, None]
    res = np.zeros((x.shape[0], 3))
    for r in range(x.shape[0]):
        order = np.argsort(-x[r], kind="stable")
        srt = x[r][order]
        p = np.exp(srt - srt[0])
        p /= p.sum()
        before = np.cumsum(p) - p
        i = int(np.argmin(np.abs(before - float(top_p[r]))))
        res[r] = (abs(before[i] - float(top_p[r])), p[i], order[i])
    return res


def sample_inverse_cdf(probs: np.ndarray, u: np.ndarray) -> np.ndarray:
    """ids[r] = smallest index i with sum(probs[r, :i+1]) > u[r]; the last token with non-zero
    probability if rounding leaves none."""
    ids = np.zeros(probs.shape[0], dtype=np.int64)
    for r in range(probs.shape[0]):
        c = np.cumsum(probs[r])
        hit = np.nonzero(c > float(u[r]))[0]
        ids[r] = hit[0] if len(hit) else np.nonzero(probs[r] > 0)[0][-1]
    return ids
