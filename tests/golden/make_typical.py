"""Write tests/golden/typical.npz from the UNMODIFIED reference's typical sampler.

    python tests/golden/make_typical.py /path/to/rwkvstic-checkout

For every case the reference function ``typical(logits, temp, tau)``
(src/rwkvstic/agnostic/samplers/typical.py) runs on seeded synthetic logits with
``torch.multinomial`` replaced by a recorder, so that the tensor it would draw from is captured:
the file keeps, per case, which entries of that tensor are non-zero (bit-packed), their count and
their fp64 sum.  Logits are regenerated from the seed by ``case_logits`` below (the tests import
it); a fp64 checksum of the logits is stored so that a changed random stream is noticed.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

# (vocabulary, seed, scale of the normal logits, temperature, tau)
CASES = [
    (257, 1, 2.0, 1.0, 0.95),
    (257, 2, 5.0, 1.0, 0.5),
    (257, 3, 1.0, 0.7, 0.2),
    (1000, 4, 8.0, 1.3, 0.9),
    (50277, 5, 3.0, 1.0, 0.95),
    (50277, 6, 6.0, 0.8, 0.8),
    (50277, 7, 1.0, 1.0, 0.6),
    (65536, 8, 4.0, 1.0, 0.99),
]


def case_logits(vocab: int, seed: int, scale: float) -> np.ndarray:
    """Normal logits with a few strong peaks, the shape a language model's output has."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal(vocab).astype(np.float32) * np.float32(scale)
    peaks = rng.integers(0, vocab, size=8)
    x[peaks] += np.float32(2.0 * scale)
    return x


def main():
    sys.path.insert(0, HERE)
    from make_golden import import_reference
    import_reference(sys.argv[1])
    from rwkvstic.agnostic.samplers.typical import typical

    seen = {}
    real = torch.multinomial

    def recorder(probs, num_samples=1, *a, **k):
        seen["probs"] = probs.detach().clone()
        return real(probs, num_samples, *a, **k)

    out = {"cases": np.array(CASES, dtype=np.float64)}
    torch.multinomial = recorder
    try:
        for i, (vocab, seed, scale, temp, tau) in enumerate(CASES):
            x = case_logits(vocab, seed, scale)
            tok = typical(torch.from_numpy(x.copy()), temp=temp, tau=tau)
            p = seen["probs"].numpy()
            assert p[tok] > 0
            out[f"kept_{i}"] = np.packbits(p > 0)
            out[f"count_{i}"] = np.int64((p > 0).sum())
            out[f"sum_{i}"] = np.float64(p.astype(np.float64).sum())
            out[f"check_{i}"] = np.float64(x.astype(np.float64).sum())
            print(i, vocab, "kept", int((p > 0).sum()), "sum", float(p.sum()))
    finally:
        torch.multinomial = real
    path = os.path.join(HERE, "typical.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes; torch", torch.__version__)


if __name__ == "__main__":
    main()
