"""Generate ``torch_mode.npz`` by running the UNMODIFIED reference in its TORCH mode on CPU.

Usage (only where the reference checkout exists; the fixture is committed):

    python tests/golden/make_torch_mode.py /path/to/rwkvstic-checkout

What is run: ``helpers.loadWeights.loadWeights(TORCH, path, useGPU=False, dtype=T,
runtimedtype=torch.float32)`` followed by ``agnostic.agnosticRwkv.AgnosticRWKV(ops, w)`` for
T in {fp32, bf16, fp16}: matrices in T, vectors and state in fp32, the max-trick WKV.  With
``useGPU=False`` the ops object builds its ``emptyState`` in T (agnostic/backends/torch.py:115) while
the network writes fp32 rows into it, so the state handed in here is that tensor cast to fp32 - the
type the GPU branch of the same class gives it (torch.py:166).  The ``inquirer`` stand-in of
``make_golden.py`` is used; nothing of the reference is altered.

Two shapes: L=2 D=128 V=257 (9 tokens in one call, and token by token) and L=3 D=768 V=1000
(12 tokens token by token, rows long enough for the summation order to matter in bf16).
"""
from __future__ import annotations

import os
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, HERE)

from make_golden import import_reference  # noqa: E402
from rwkvstic_b200.synth import synth_checkpoint, synth_tokens  # noqa: E402

TYPES = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}
SHAPES = {"tiny": (2, 128, 257, 31, 9), "mid": (3, 768, 1000, 32, 12)}     # L, D, V, weight seed, tokens


def reference_model(ck, dtype):
    from rwkvstic.agnostic.agnosticRwkv import AgnosticRWKV
    from rwkvstic.agnostic.backends import TORCH
    from rwkvstic.helpers.loadWeights import loadWeights
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "synth.pth")
        torch.save(ck, path)
        ops, w = loadWeights(TORCH, path, useGPU=False, dtype=dtype, runtimedtype=torch.float32)
    return AgnosticRWKV(ops, w), ops.emptyState.float()


def main():
    out = {"torch_version": torch.__version__}
    for shape, (L, D, V, seed, n_tok) in SHAPES.items():
        ck = synth_checkpoint(L, D, vocab=V, seed=seed)
        toks = synth_tokens(n_tok, seed=5, vocab=V)
        out[f"{shape}_tokens"] = toks.numpy()
        for name, dt in TYPES.items():
            model, empty = reference_model(ck, dt)
            s = empty.clone()
            rows = []
            for t in toks:
                lg, s = model.forward(torch.LongTensor([int(t)]), s)
                rows.append(lg.clone())
            out[f"{shape}_{name}_logits_tok"] = torch.stack(rows).numpy()
            out[f"{shape}_{name}_state_tok"] = s.numpy()
            if shape == "tiny":
                s = empty.clone()
                lg, s = model.forward(toks, s)
                out[f"{shape}_{name}_logits_seq"] = lg.numpy()
                out[f"{shape}_{name}_state_seq"] = s.numpy()
            print(shape, name, "max |logit|", float(rows[-1].abs().max()))
    np.savez_compressed(os.path.join(HERE, "torch_mode.npz"), **out)
    print("torch_mode.npz written")


if __name__ == "__main__":
    import_reference(sys.argv[1])
    main()
