"""CPU statement of the ARITHMETIC CONTRACT of the CUDA kernels (test infrastructure).

Not the oracle (that is ``oracle/fastquant_oracle.py``, the reference's algorithm) and not a
fallback (the product never imports this).  It predicts what the kernels compute so that

* the integer part of the GEMV can be checked bit-for-bit on the GPU (``fixed_point_gemv``
  reproduces the 24-bit fixed-point digits and the exact integer dot product), and
* the accuracy of the fp32 / fixed-point design against the reference (fp64 vectors, fp32
  matmul) can be measured on the CPU, where the GPU is not available.
"""
from __future__ import annotations

import numpy as np
import torch

from rwkvstic_b200.quant import QuantMatrix

QMAX = np.float32(8355000.0)


def fixed_point_gemv(x: torch.Tensor, m: QuantMatrix, with_affine: bool = True) -> torch.Tensor:
    """y[N] for one fp32 input vector, following stream_gemv.cuh step by step."""
    x = x.to(torch.float32)
    xs = x * m.ry                                            # fp32 product
    amax = xs.abs().max()
    if float(amax) == 0.0:
        main = torch.zeros(m.n_out, dtype=torch.float32)
    else:
        inv = (torch.tensor(QMAX) / amax).to(torch.float32)  # fp32 division
        X = torch.round(xs * inv).to(torch.float64)          # cvt.rni of the fp32 product (half to even)
        I = (m.qt.to(torch.float64) @ X).to(torch.int64)     # exact: |I| < 2^46
        sd = torch.tensor(1.0, dtype=torch.float32) / inv    # value of one fixed-point unit: IEEE fp32 division
        main = I.to(torch.float32) * sd                      # int64 -> fp32 (nearest even), fp32 product
    if not with_affine:
        return main
    y = main + np.float32(m.half) * xs.sum()
    if m.rx is not None:
        y = y * m.rx
    y = y + (x * m.my).sum()
    if m.mx is not None:
        y = y + m.mx * x.sum()
    return y


def layernorm32(x, w, b):
    mean = x.mean()
    xc = x - mean
    sd = torch.sqrt((xc * xc).mean() + np.float32(1e-5))
    return w * (xc / sd) + b


def wkv_step32(k, v, w, u, aa, bb, pp):
    ww = u + k
    p = torch.maximum(pp, ww)
    e1, e2 = torch.exp(pp - p), torch.exp(ww - p)
    y = (e1 * aa + e2 * v) / (e1 * bb + e2)
    ww2 = pp + w
    p2 = torch.maximum(ww2, k)
    f1, f2 = torch.exp(ww2 - p2), torch.exp(k - p2)
    return y, f1 * aa + f2 * v, f1 * bb + f2, p2


class ContractModel:
    """The decode-step sequence of b200rwkv_decode_step on CPU tensors (fp32 state [L,5,D])."""

    def __init__(self, weights):
        self.w = weights  # rwkvstic_b200.model.QuantizedWeights on the CPU
        self.emptyState = torch.zeros(weights.n_layer, 5, weights.n_embd, dtype=torch.float32)
        self.emptyState[:, 4] = -1e30

    def step(self, token: int, state: torch.Tensor, want_logits: bool = True):
        w = self.w
        xa = self.blocks(layernorm32(w.emb[token], *w.ln0), state)
        if not want_logits:
            return None, state
        return fixed_point_gemv(layernorm32(xa, *w.ln_out), w.head), state

    def blocks(self, xa: torch.Tensor, state: torch.Tensor) -> torch.Tensor:
        """All blocks this object holds applied to one residual-stream row; ``state`` in place."""
        w = self.w
        for i, ly in enumerate(w.layers):
            v, m, st = ly.vec, ly.mat, state[i]
            xy = layernorm32(xa, v["ln1.weight"], v["ln1.bias"])
            tc = st[0].clone()
            mix = lambda mu: xy * mu + tc * (1 - mu)
            k = fixed_point_gemv(mix(v["att.time_mix_k"]), m["att.key"])
            vv = fixed_point_gemv(mix(v["att.time_mix_v"]), m["att.value"])
            r = torch.sigmoid(fixed_point_gemv(mix(v["att.time_mix_r"]), m["att.receptance"]))
            y, st[2], st[3], st[4] = wkv_step32(k, vv, v["att.time_decay"], v["att.time_first"], st[2], st[3], st[4])
            st[0] = xy
            xb = xa + fixed_point_gemv(r * y, m["att.output"])
            dd = layernorm32(xb, v["ln2.weight"], v["ln2.bias"])
            rc = st[1].clone()
            fk = dd * v["ffn.time_mix_k"] + rc * (1 - v["ffn.time_mix_k"])
            fr = dd * v["ffn.time_mix_r"] + rc * (1 - v["ffn.time_mix_r"])
            kk = torch.relu(fixed_point_gemv(fk, m["ffn.key"])) ** 2
            rf = torch.sigmoid(fixed_point_gemv(fr, m["ffn.receptance"]))
            st[1] = dd
            xa = xb + rf * fixed_point_gemv(kk, m["ffn.value"])
        return xa

    def stage(self, tokens, x: torch.Tensor, state: torch.Tensor, want_logits: bool):
        """CPU stand-in for B200RWKV.forward_rows_stage: ``tokens [B,T]`` or None, ``x [B*T, D]`` in
        place, ``state [B, L_stage, 5, D]``; logits ``[B,V]`` of each stream's last row when asked."""
        w = self.w
        B = state.shape[0]
        T = x.shape[0] // B
        out = torch.empty(B, w.n_vocab) if want_logits else None
        for b in range(B):
            for t in range(T):
                row = b * T + t
                xin = layernorm32(w.emb[int(tokens[b, t])], *w.ln0) if tokens is not None else x[row]
                x[row] = self.blocks(xin, state[b])
            if want_logits:
                out[b] = fixed_point_gemv(layernorm32(x[b * T + T - 1], *w.ln_out), w.head)
        return out

    def forward(self, tokens, state):
        logits = None
        toks = [int(t) for t in tokens]
        for i, t in enumerate(toks):
            logits, state = self.step(t, state, want_logits=(i == len(toks) - 1))
        return logits, state
