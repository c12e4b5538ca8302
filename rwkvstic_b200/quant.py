"""uint8 weight quantisation for the two affine schemes the GEMV/GEMM kernels accept.

Both schemes are instances of one kernel contract.  For a matrix used as
``y = x @ W`` with ``W[K_in, N_out]`` and quantised bytes ``Q``:

    y[n] = rx[n] * ( sum_k (x[k]*ry[k]) * Q[k,n]  +  h * sum_k x[k]*ry[k] )
           + sum_k x[k]*my[k]  +  mx[n] * sum_k x[k]

* FASTQUANT (rwkvstic agnostic/backends/modules/matmul.py:26-40): one scale and one
  offset per input feature k: ``ry = range, my = offset, rx = 1, mx = 0, h = 0``.
* two-axis "fp32i8" scheme: ``W ~ (Q + 0.5) * ry[k] * rx[n] + my[k] + mx[n]``, ``h = 0.5``.

The kernels want the bytes output-major (``Qt[N_out, K_in]``, K contiguous) so that
every output row is one sequential byte stream; the reference keeps them
``[K_in, N_out]``.  ``QuantMatrix`` stores the kernel layout and can give back the
reference layout for export.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class QuantMatrix:
    """One quantised matrix in kernel layout."""
    qt: torch.Tensor                 # uint8 [N_out, K_in], K contiguous
    ry: torch.Tensor                 # f32 [K]  per-input scale
    my: torch.Tensor                 # f32 [K]  per-input offset
    rx: Optional[torch.Tensor] = None  # f32 [N] per-output scale (None = 1)
    mx: Optional[torch.Tensor] = None  # f32 [N] per-output offset (None = 0)
    half: float = 0.0                # h in the contract above
    my64: Optional[torch.Tensor] = None  # f64 [K] offset as the reference stores it

    @property
    def n_out(self) -> int:
        return self.qt.shape[0]

    @property
    def k_in(self) -> int:
        return self.qt.shape[1]

    def to(self, device) -> "QuantMatrix":
        mv = lambda t: None if t is None else t.to(device)
        return QuantMatrix(mv(self.qt), mv(self.ry), mv(self.my), mv(self.rx), mv(self.mx),
                           self.half, mv(self.my64))

    def reference_layout(self) -> torch.Tensor:
        """uint8 [K_in, N_out] as MM8.weight holds it (matmul.py:15-21)."""
        return self.qt.t().contiguous()

    def dequant(self) -> torch.Tensor:
        """fp64 W_hat[N_out, K_in] implied by the contract (test helper)."""
        q = self.qt.double() + self.half
        w = q * self.ry.double()[None, :]
        if self.rx is not None:
            w = w * self.rx.double()[:, None]
        w = w + (self.my64 if self.my64 is not None else self.my.double())[None, :]
        if self.mx is not None:
            w = w + self.mx.double()[:, None]
        return w


def quantize_fastquant(w: torch.Tensor) -> QuantMatrix:
    """FASTQUANT quantisation of ``w[N_out, K_in]`` (a checkpoint ``*.weight``).

    Same arithmetic, in the same order and precision, as MM8.QuantizeMatrix
    (matmul.py:26-40) so that the bytes, ranges and offsets are identical to the
    reference's: statistics are taken per input feature over all outputs; the
    lower bound and the span/255 are fp64; the byte is the truncated quotient;
    the offset is moved up by the mean truncation loss so the rounding error has
    zero mean.  Runs on whatever device ``w`` lives on.
    """
    assert w.dim() == 2
    lo = w.min(dim=0).values.double()                 # [K]
    shifted = w - lo                                  # fp64 [N,K] (fp32 - fp64 promotes)
    step = shifted.max(dim=0).values.double() / 255   # [K]
    scaled = shifted / step
    loss = scaled.frac().double().mean(dim=0)         # mean truncation loss per k
    offset = lo + loss * step
    qt = scaled.to(torch.uint8).contiguous()          # truncation; [N,K] is already kernel layout
    return QuantMatrix(qt=qt, ry=step.float(), my=offset.float(), half=0.0, my64=offset)


def quantize_two_axis(w: torch.Tensor) -> QuantMatrix:
    """Two-axis uint8 quantisation of ``w[N_out, K_in]``: subtract the per-input minimum
    then the per-output minimum, divide by the per-output maximum then the per-input
    maximum, take ``floor(256*x)`` clipped to 0..255, and dequantise as
    ``(q + 0.5) * ry * rx + my + mx``.  The 1/256 of the byte scale is folded into ry.
    """
    assert w.dim() == 2
    x = w.double()
    my = x.min(dim=0).values                          # [K] per input feature
    x = x - my[None, :]
    mx = x.min(dim=1).values                          # [N] per output
    x = x - mx[:, None]
    rx = x.max(dim=1).values.clamp_min(1e-30)         # [N]
    x = x / rx[:, None]
    ry = x.max(dim=0).values.clamp_min(1e-30)         # [K]
    x = x / ry[None, :]
    qt = torch.floor(x * 256).clamp(0, 255).to(torch.uint8).contiguous()
    return QuantMatrix(qt=qt, ry=(ry / 256).float(), my=my.float(), rx=rx.float(),
                       mx=mx.float(), half=0.5, my64=my)
