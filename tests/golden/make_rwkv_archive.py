"""Write tests/golden/model_tiny.rwkv with the UNMODIFIED reference's own exporter.

    python tests/golden/make_rwkv_archive.py /path/to/rwkvstic-checkout

``OptRWKV(path, jit=True, export=<prefix>, device="cpu", config=<cpu uint8>)`` scripts the
FASTQUANT model and calls ``torch.jit.save(model, prefix + ".rwkv")`` followed by ``exit()``
(agnostic/backends/opt.py:112-117); the SystemExit is caught here.  The checkpoint is the same
seeded L=2 D=128 V=257 model as model_tiny.npz, so the archive's logits are pinned by that file.
"""
from __future__ import annotations

import os
import sys
import tempfile

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from make_golden import CPU_CFG, import_reference  # noqa: E402
from rwkvstic_b200.synth import synth_checkpoint  # noqa: E402


def main():
    import_reference(sys.argv[1])
    from rwkvstic.agnostic.backends.opt import OptRWKV
    ck = synth_checkpoint(2, 128, vocab=257, seed=31)
    with tempfile.TemporaryDirectory() as d:
        pth = os.path.join(d, "synth.pth")
        torch.save(ck, pth)
        try:
            OptRWKV(pth, jit=True, export=os.path.join(HERE, "model_tiny"), device="cpu", config=CPU_CFG)
        except SystemExit:
            pass
    out = os.path.join(HERE, "model_tiny.rwkv")
    print(out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
    main()
