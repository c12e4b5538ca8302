"""CPU oracle for typical sampling.  TEST INFRASTRUCTURE ONLY.

Restates the reference's host-side sampler (rwkvstic ``src/rwkvstic/agnostic/samplers/typical.py``
lines 1-17) in numpy, split into the deterministic part (which tokens survive and with what
weight) and the draw.  Only the tests may import it; nothing in the product package does.

Parity status: PINNED for the deterministic part.  ``tests/golden/make_typical.py`` imports the
unmodified reference function, intercepts the tensor it hands to ``torch.multinomial`` and stores
which entries are non-zero plus their sum under ``tests/golden/typical.npz``;
``tests/test_typical.py`` checks this restatement against that file.  The kept set is decided by
comparing an fp32 running sum with tau, so the one entry at the cutoff depends on the summation
order (torch's blocked cumsum, a sequential sum and an exact sum can each place it one entry
apart): ``kept_sets_agree`` is the comparison every test uses - identical sets, or sets that
differ in exactly the last entry in order of ``shifted``.  The draw itself
(``torch.multinomial``) is a random stream no other implementation can reproduce; ``draw`` below
is the inverse-CDF rule the CUDA kernel documents, not something the reference defines.
"""
from __future__ import annotations

import numpy as np


def typical_shifted(logits: np.ndarray):
    """(probs, shifted): softmax and the distance of each token's surprise from the entropy."""
    l = np.asarray(logits, dtype=np.float32)
    e = np.exp(l - l.max(), dtype=np.float32)
    probs = (e / e.sum(dtype=np.float32)).astype(np.float32)                       # typical.py:5
    with np.errstate(divide="ignore", invalid="ignore"):
        nl = (-np.log(probs)).astype(np.float32)                                     # :6
        ent = np.float32(np.nansum((nl * probs).astype(np.float32), dtype=np.float32))   # :7
        shifted = np.abs(nl - ent).astype(np.float32)                               # :8
    return probs, shifted


def typical_weights(logits: np.ndarray, temp: float = 1.0, tau: float = 0.95) -> np.ndarray:
    """The unnormalised distribution the reference draws from: fp32 like typical.py:5-16."""
    probs, shifted = typical_shifted(logits)
    order = np.argsort(shifted, kind="stable")                                      # :9
    cum = np.cumsum(probs[order], dtype=np.float32)                                 # :12
    cutoff = int(np.sum(cum < np.float32(tau)))                                     # :13
    out = probs.copy()
    if cutoff < len(out):                       # the reference indexes past the end otherwise
        out[shifted > shifted[order][cutoff]] = 0                                   # :14
    if temp != 1.0:
        out = np.power(out, np.float32(1.0 / temp), dtype=np.float32)               # :15-16
    return out


def draw(weights: np.ndarray, u: float) -> int:
    """First index whose running sum (index order, fp64) reaches u * total, zero weights skipped."""
    w = np.asarray(weights, dtype=np.float64)
    cum = np.cumsum(w)
    target = float(u) * cum[-1]
    nz = np.nonzero(w > 0)[0]
    hit = nz[cum[nz] >= target]
    return int(hit[0] if len(hit) else nz[-1])


def draw_bracket(weights: np.ndarray, u: float, token: int, rel: float = 1e-5) -> bool:
    """True when ``token`` is a legitimate answer of ``draw`` up to fp32 rounding of the weights:
    its weight is non-zero and u * total lies in its interval widened by ``rel`` of the total."""
    w = np.asarray(weights, dtype=np.float64)
    cum = np.cumsum(w)
    target, eps = float(u) * cum[-1], rel * cum[-1]
    return bool(w[token] > 0 and cum[token] - w[token] - eps <= target <= cum[token] + eps)


def kept_sets_agree(a: np.ndarray, b: np.ndarray, shifted: np.ndarray) -> bool:
    """Boolean masks a, b are the same kept set up to the single entry at the cutoff: equal, or one
    holds exactly one entry more and that entry has the largest ``shifted`` value of its set."""
    a, b = np.asarray(a, dtype=bool), np.asarray(b, dtype=bool)
    diff = np.nonzero(a != b)[0]
    if len(diff) == 0:
        return True
    if len(diff) != 1:
        return False
    big = a if a.sum() > b.sum() else b
    return bool(shifted[diff[0]] >= shifted[big].max())
