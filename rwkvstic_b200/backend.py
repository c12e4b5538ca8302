"""The ops-object boundary: selecting this backend through the reference's own loader.

``rwkvstic.load.RWKV(path, mode=...)`` instantiates ``Backends[mode](layers, embed, **kw)``
(helpers/loadWeights.py:31-32), pushes every checkpoint tensor through ``ops.initTensor``
(:70-83), builds ``AgnosticRWKV(ops, weights)`` (agnosticRwkv.py:12-63) and finally lets the
backend replace the whole model through ``ops.postProcessModule`` (agnosticRwkv.py:193).
``install()`` registers a backend under ``MODE`` whose op table keeps the tensors as they are
and whose ``postProcessModule`` returns a ``B200RWKV`` built from them, so

    import rwkvstic_b200.backend as b; b.install()
    model = rwkvstic.load.RWKV("model.pth", mode=b.MODE)       # -> RWKVMaster
    model.loadContext(newctx="..."); model.forward(number=32)

runs the reference's session code (rwkvMaster.py:28-105) on the sm_100a kernels.  Nothing
here imports the reference at module import time; ``install()`` needs it to be importable.

The reference's TORCH mode takes ``dtype=`` for the matrices (agnostic/backends/torch.py:8-22).  The
same keyword selects the model here: ``dtype=torch.bfloat16`` / ``float16`` / ``float32`` keeps the
weights unquantised (``B200DenseRWKV``, the arithmetic of torch.py:125-166), no ``dtype`` or
``torch.uint8`` gives the FASTQUANT model (``B200RWKV``).  With ``target=GB`` (and ``pinMem=``), the
keywords of the TORCH_STREAM mode the reference's README describes, only that many GB of the unquantised
model's matrices stay on the GPU and the other blocks are streamed from (pinned) host memory.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional

import torch

MODE = "b200-fastquant(gpu)"


def checkpoint_from_agnostic(model) -> Dict[str, torch.Tensor]:
    """Rebuild a checkpoint-shaped dict from the attributes AgnosticRWKV stores
    (agnosticRwkv.py:22-63).  ``time_decay`` is already ``-exp(raw)`` at that point
    (helpers/loadWeights.py:63-64); it is exported under ``att.time_decay_final``."""
    ck = {"emb.weight": model.emb, "blocks.0.ln0.weight": model.emb1, "blocks.0.ln0.bias": model.emb2,
          "ln_out.weight": model.postprocess0, "ln_out.bias": model.postprocess1, "head.weight": model.postprocess2}
    per_layer = {"ln1.weight": "ln1w", "ln1.bias": "ln1b", "ln2.weight": "ln2w", "ln2.bias": "ln2b",
                 "att.time_decay_final": "time_decay", "att.time_first": "time_first",
                 "att.time_mix_k": "kktk", "att.time_mix_v": "vvtv", "att.time_mix_r": "rrtr",
                 "att.key.weight": "key", "att.value.weight": "value", "att.receptance.weight": "receptance",
                 "att.output.weight": "outputvv", "ffn.time_mix_k": "time_mix_k_ffn", "ffn.time_mix_r": "time_mix_r_ffn",
                 "ffn.key.weight": "key_ffn", "ffn.receptance.weight": "receptance_ffn", "ffn.value.weight": "value_ffn"}
    for i in range(len(model.ln1w)):
        for name, attr in per_layer.items():
            ck[f"blocks.{i}.{name}"] = getattr(model, attr)[i]
    return ck


def make_ops_class(base_module, model_factory: Optional[Callable] = None, device="cuda:0", scheme="fastquant"):
    """Subclass of the reference's ``agnostic.backends.base.module`` for ``Backends[MODE]``."""

    class RWKVB200Ops(base_module):
        def __init__(self, layers, embed, *args, dtype=None, target=None, pinMem=True, **kwargs):
            super().__init__(layers, embed, *args, **kwargs)
            self.target, self.pinMem = target, pinMem        # TORCH_STREAM's keywords: GB of matrices kept on the GPU, pinned host copies
            if dtype not in (None, torch.uint8, torch.float32, torch.bfloat16, torch.float16):
                raise ValueError("dtype must be torch.uint8 (FASTQUANT), torch.float32, torch.bfloat16 or torch.float16")
            self.dtype = dtype
            self.initTensor = lambda x: x.detach().float() if x.is_floating_point() else x   # keep [out,in] fp32
            self.initCpuTensor = self.initTensor
            self.intTensor = lambda x: torch.tensor(x if isinstance(x, list) else [x], dtype=torch.int64)
            self.stack = torch.stack
            self.mnstack = lambda x: x
            self.module = torch.nn.Module
            self.stackEmb = False
            self.TensorType = self.MatrixType = self.VectorType = torch.Tensor
            self.emptyState = torch.zeros(layers, 5, embed)
            self.emptyState[:, 4] = -1e30
            factory = model_factory

            def post(model):
                ck = checkpoint_from_agnostic(model)
                if factory is not None:
                    new = factory(ck)
                elif self.dtype in (torch.float32, torch.bfloat16, torch.float16):
                    from .dense_model import B200DenseRWKV
                    new = B200DenseRWKV(ck.items(), dtype=self.dtype, device=device, target_gb=self.target, pin_memory=self.pinMem)
                else:
                    from .model import B200RWKV
                    new = B200RWKV.from_checkpoint(ck, device=device, scheme=scheme)
                self.emptyState = new.emptyState        # load.RWKV reads ops.emptyState afterwards (load.py:81)
                return new

            self.postProcessModule = post
            def sample(logits, temp=1.0, tau=0.95, **kw):
                # logits that are still on the GPU are sampled there (same arithmetic, 8 bytes come
                # back instead of the whole vector); anything else goes to the reference's sampler
                if torch.is_tensor(logits) and logits.device.type == "cuda":
                    from . import ops
                    return int(ops.sample_typical(logits.float().contiguous(), temp, tau)[0])
                from rwkvstic.agnostic.samplers.typical import typical
                return typical(logits, temp, tau, **kw)

            self.sample = sample

    return RWKVB200Ops


def install(model_factory: Optional[Callable] = None, device="cuda:0", scheme="fastquant") -> str:
    """Register the backend in the reference's ``Backends`` table; returns the mode string."""
    import rwkvstic.agnostic.backends as backends
    from rwkvstic.agnostic.backends.base import module as base_module
    backends.Backends[MODE] = make_ops_class(base_module, model_factory, device, scheme)
    return MODE
