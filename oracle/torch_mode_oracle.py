"""CPU oracle for the RWKV-4 TORCH-mode (unquantised weights) inference path.  TEST INFRASTRUCTURE ONLY.

Plain torch-on-CPU restatement of what the reference computes when it is loaded with
``mode=TORCH``: matrices kept in ``dtype`` (bf16 / fp16 / fp32), every vector, the state and all
element-wise work in ``runtimedtype`` (fp32 here), the network of ``agnostic/agnosticRwkv.py``
with the max-trick WKV.  Only the tests, the smoke check and the benchmark's CPU legs may import
it; nothing in the product package does.

Parity status: PINNED.  ``tests/golden/make_torch_mode.py`` imports the unmodified reference
(``helpers/loadWeights.py`` with ``useGPU=False`` + ``AgnosticRWKV``), runs it on seeded weights and
tokens for the three matrix types and stores logits and states in ``tests/golden/torch_mode.npz``;
``tests/test_oracle.py`` checks this restatement against that file (bit-identical: both run the
same torch CPU operators in the same order).

Every function names the reference lines it follows (paths inside rwkvstic's ``src/rwkvstic``).
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch


def layernorm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """agnostic/backends/torch.py:102-110: centre, biased variance over dim 1, eps inside the sqrt."""
    c = x - torch.mean(x, dim=1, keepdim=True)
    s = torch.sqrt(torch.mean(c * c, dim=1, keepdim=True) + 1e-5)
    return w * (c / s) + b


def matvec(w_t: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """agnostic/backends/torch.py:54-55: rows rounded to the matrix type, product in that type, result
    cast back.  ``w_t`` is the ``[in, out]`` transposed view ``initTensor`` makes (torch.py:24-28)."""
    return torch.matmul(x.to(w_t.dtype), w_t).to(x.dtype)


class OracleTorchMode:
    """``AgnosticRWKV(*loadWeights(TORCH, path, useGPU=False, dtype=..., runtimedtype=...))``.

    ``forward(tokens int64[T], state [L,5,D]) -> (logits fp32[V], state)``; state rows per block:
    0 = ln1 output of the last token, 1 = ln2 output, 2 / 3 = WKV numerator / denominator scaled by
    ``exp(-row 4)``, 4 = the running maximum exponent (``-1e30`` when empty)."""

    def __init__(self, ck: Dict[str, torch.Tensor], dtype: torch.dtype, runtimedtype: torch.dtype = torch.float32):
        self.dtype, self.rt = dtype, runtimedtype
        self.n_layer = 1 + max(int(k.split(".")[1]) for k in ck if k.startswith("blocks."))
        self.n_embd = ck["blocks.0.ffn.time_mix_k"].numel()
        w = {}
        for k, v in ck.items():                                   # helpers/loadWeights.py:57-83
            v = v.detach()
            if ".time_" in k:
                v = v.squeeze()
            if ".time_decay" in k:
                v = -torch.exp(v.double())
            if k == "emb.weight":
                w[k] = v.to(runtimedtype)                         # rows through initCpuTensor, then stacked
            elif v.squeeze().dim() == 2:
                w[k] = v.to(dtype).t()                            # torch.py:24-26
            else:
                w[k] = v.to(runtimedtype)                         # torch.py:27-28
        self.w = w
        state = torch.zeros(self.n_layer, 5, self.n_embd, dtype=runtimedtype)   # base.py:61-62 with useLogFix
        state[:, 4] = -1e30
        self.emptyState = state

    def _wkv(self, k, v, st, td, tf):
        """agnosticRwkv.py:68-103 (processLayerx), one row at a time (:116-121)."""
        out = []
        for i in range(k.shape[0]):
            ww = tf + k[i]
            p = torch.maximum(st[4], ww)
            e1, e2 = torch.exp(st[4] - p), torch.exp(ww - p)
            a = e1 * st[2] + e2 * v[i]
            b = e1 * st[3] + e2
            wwn = st[4] + td
            p1 = torch.maximum(wwn, k[i])
            e11, e21 = torch.exp(wwn - p1), torch.exp(k[i] - p1)
            nb, nc = e11 * st[2] + e21 * v[i], e11 * st[3] + e21
            st[2], st[3], st[4] = nb, nc, p1
            out.append(a / b)
        return torch.stack(out)

    def _layer(self, x, st, i):
        """agnosticRwkv.py:123-169 (doLayer)."""
        w, p = self.w, f"blocks.{i}."
        xy = layernorm(x, w[p + "ln1.weight"], w[p + "ln1.bias"])
        tc = torch.roll(xy, xy.shape[1])                          # rows move down by one (torch.py:50-51)
        tc[0] = st[0]                                             # base.py:86-89 (push)
        k = matvec(w[p + "att.key.weight"], torch.lerp(tc, xy, w[p + "att.time_mix_k"]))
        v = matvec(w[p + "att.value.weight"], torch.lerp(tc, xy, w[p + "att.time_mix_v"]))
        r = torch.sigmoid(matvec(w[p + "att.receptance.weight"], torch.lerp(tc, xy, w[p + "att.time_mix_r"])))
        rz = self._wkv(k, v, st, w[p + "att.time_decay"], w[p + "att.time_first"])
        mvv = x + matvec(w[p + "att.output.weight"], r * rz)
        ddd = layernorm(mvv, w[p + "ln2.weight"], w[p + "ln2.bias"])
        rc = torch.roll(ddd, ddd.shape[1])
        rc[0] = st[1]
        st[0], st[1] = xy[-1], ddd[-1]
        km = torch.relu(matvec(w[p + "ffn.key.weight"], torch.lerp(rc, ddd, w[p + "ffn.time_mix_k"])))
        rt = torch.sigmoid(matvec(w[p + "ffn.receptance.weight"], torch.lerp(rc, ddd, w[p + "ffn.time_mix_r"])))
        return mvv + matvec(w[p + "ffn.value.weight"], km * km) * rt

    def forward(self, tokens: torch.Tensor, state: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """agnosticRwkv.py:171-187.  The state is updated in place and returned."""
        w = self.w
        x = layernorm(w["emb.weight"][tokens.reshape(-1)], w["blocks.0.ln0.weight"], w["blocks.0.ln0.bias"])
        for i in range(self.n_layer):
            x = self._layer(x, state[i], i)
        x = matvec(w["head.weight"], layernorm(x[-1:], w["ln_out.weight"], w["ln_out.bias"])).squeeze()
        return x.float(), state
