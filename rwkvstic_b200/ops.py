"""Operator-level entry points over the C ABI, taking torch CUDA tensors.

These mirror the reference's three custom ops (cuda/wrapper.cpp:45-129, called from
modules/matmul.py:42-49, :70-80 and modules/wkv.py:18): a one- or three-matrix uint8
GEMV and the WKV recurrence.  They validate, pass raw device pointers to the library and
launch on torch's current stream.  No CPU path.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import torch

from . import _lib
from .quant import QuantMatrix


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _cmatrix(m: QuantMatrix) -> _lib.Matrix:
    return _lib.Matrix(_lib.ptr(m.qt), _lib.ptr(m.ry), _lib.ptr(m.my), _lib.ptr(m.rx), _lib.ptr(m.mx),
                       float(m.half), m.n_out, m.k_in)


_workspaces = {}


def gemv_workspace(device, k_in: int, nmat: int) -> torch.Tensor:
    """Zeroed scratch for ``gemv_u8``, cached per device, size AND current CUDA stream: calls that share
    a workspace must be ordered on one stream, so every stream gets its own.  Its first int32 is the
    kernels' status word."""
    n = int(_lib.lib().b200rwkv_gemv_workspace_bytes(k_in, nmat))
    key = (str(device), n, _stream(device))
    if key not in _workspaces:
        _workspaces[key] = torch.zeros(n, dtype=torch.uint8, device=device)
    return _workspaces[key]


def gemv_u8(mats: Sequence[QuantMatrix], xs: Sequence[torch.Tensor], ys: Optional[Sequence[torch.Tensor]] = None,
            accumulate: bool = False, workspace: Optional[torch.Tensor] = None,
            trace: Optional[torch.Tensor] = None) -> List[torch.Tensor]:
    """``ys[i] = xs[i] @ W_i`` for 1..3 quantised matrices of equal k_in, one launch.

    ``xs[i]`` fp32 ``[k_in]`` on the matrices' CUDA device; ``ys[i]`` fp32 ``[n_out_i]``
    (allocated when omitted; with ``accumulate`` the result is added onto them, which is
    what the reference ops do with their zero-filled ``y``).  ``trace``: optional int64
    ``[1024, 8]`` CUDA tensor that receives the per-CTA phase timeline (profiling).
    ``workspace``: scratch from ``gemv_workspace`` (a cached one is used when omitted)."""
    n = len(mats)
    if n < 1 or n > 3 or len(xs) != n:
        raise ValueError("gemv_u8 takes 1..3 matrices and as many input vectors")
    dev = mats[0].qt.device
    if dev.type != "cuda":
        raise RuntimeError("gemv_u8 needs CUDA tensors (no CPU path)")
    if ys is None:
        if accumulate:
            raise ValueError("accumulate needs caller-provided outputs")
        ys = [torch.empty(m.n_out, dtype=torch.float32, device=dev) for m in mats]
    for m, x, y in zip(mats, xs, ys):
        if x.dtype != torch.float32 or y.dtype != torch.float32 or not x.is_contiguous() or not y.is_contiguous():
            raise ValueError("gemv_u8 needs contiguous fp32 vectors")
        if x.numel() != m.k_in or y.numel() != m.n_out or x.device != dev or y.device != dev:
            raise ValueError("gemv_u8 vector shape/device does not match its matrix")
    cm = (_lib.Matrix * n)(*[_cmatrix(m) for m in mats])
    cx = (C.c_void_p * n)(*[x.data_ptr() for x in xs])
    cy = (C.c_void_p * n)(*[y.data_ptr() for y in ys])
    if workspace is None:
        workspace = gemv_workspace(dev, mats[0].k_in, n)
    with torch.cuda.device(dev):
        if trace is None:
            _lib.check(_lib.lib().b200rwkv_gemv_u8(n, cm, cx, cy, int(accumulate), workspace.data_ptr(),
                                                   workspace.numel(), _stream(dev)))
        else:
            _lib.check(_lib.lib().b200rwkv_gemv_u8_traced(n, cm, cx, cy, int(accumulate), workspace.data_ptr(),
                                                          workspace.numel(), trace.data_ptr(), _stream(dev)))
    return list(ys)


def gemm_u8(mats: Sequence[QuantMatrix], xs: Sequence[torch.Tensor],
            ys: Optional[Sequence[torch.Tensor]] = None) -> List[torch.Tensor]:
    """``ys[i] = xs[i] @ W_i`` for 1..3 quantised matrices of equal k_in and ``xs[i]`` fp32
    ``[rows, k_in]``: the many-rows (tensor-core) form of ``gemv_u8``, which the reference serves by
    dequantising the matrix (modules/matmul.py:64-68).  Returns fp32 ``[rows, n_out_i]``."""
    n = len(mats)
    if n < 1 or n > 3 or len(xs) != n:
        raise ValueError("gemm_u8 takes 1..3 matrices and as many input matrices")
    dev = mats[0].qt.device
    if dev.type != "cuda":
        raise RuntimeError("gemm_u8 needs CUDA tensors (no CPU path)")
    rows = xs[0].shape[0]
    if ys is None:
        ys = [torch.empty(rows, m.n_out, dtype=torch.float32, device=dev) for m in mats]
    for m, x, y in zip(mats, xs, ys):
        if x.dtype != torch.float32 or y.dtype != torch.float32 or not x.is_contiguous() or not y.is_contiguous():
            raise ValueError("gemm_u8 needs contiguous fp32 matrices")
        if tuple(x.shape) != (rows, m.k_in) or tuple(y.shape) != (rows, m.n_out) or x.device != dev or y.device != dev:
            raise ValueError("gemm_u8 operand shape/device does not match its matrix")
    cm = (_lib.Matrix * n)(*[_cmatrix(m) for m in mats])
    cx = (C.c_void_p * n)(*[x.data_ptr() for x in xs])
    cy = (C.c_void_p * n)(*[y.data_ptr() for y in ys])
    nbytes = int(_lib.lib().b200rwkv_gemm_workspace_bytes(mats[0].k_in, n, rows))
    key = (str(dev), "gemm", nbytes)
    if key not in _workspaces:
        _workspaces[key] = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
    ws = _workspaces[key]
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().b200rwkv_gemm_u8(n, cm, cx, cy, rows, ws.data_ptr(), ws.numel(), _stream(dev)))
    status = int(ws[:4].view(torch.int32).item())
    if status:
        ws[:4].zero_()
        raise _lib.B200RWKVError(_lib.ETIMEOUT, f"gemm_u8: a bounded device-side wait expired (status bits {status})")
    return list(ys)


def wkv_scan(w: torch.Tensor, u: torch.Tensor, k: torch.Tensor, v: torch.Tensor, aa: torch.Tensor,
             bb: torch.Tensor, pp: torch.Tensor, convention: int = 0) -> torch.Tensor:
    """WKV-4 over ``k, v [B,T,C]`` (or ``[T,C]``); ``aa, bb, pp [B,C]`` (or ``[C]``) updated in
    place.  ``convention`` 0 = max-trick state, 1 = the reference FASTQUANT state."""
    if k.dim() == 2:
        k, v = k.unsqueeze(0), v.unsqueeze(0)
    B, T, Cc = k.shape
    for t in (w, u, k, v, aa, bb, pp):
        if t.dtype != torch.float32 or not t.is_contiguous() or t.device.type != "cuda":
            raise ValueError("wkv_scan needs contiguous fp32 CUDA tensors")
    if aa.numel() != B * Cc or bb.numel() != B * Cc or pp.numel() != B * Cc or w.numel() != Cc or u.numel() != Cc:
        raise ValueError("wkv_scan state/parameter shapes do not match k")
    y = torch.empty_like(k)
    with torch.cuda.device(k.device):
        _lib.check(_lib.lib().b200rwkv_wkv_scan(B, T, Cc, w.data_ptr(), u.data_ptr(), k.data_ptr(), v.data_ptr(),
                                                y.data_ptr(), aa.data_ptr(), bb.data_ptr(), pp.data_ptr(),
                                                convention, _stream(k.device)))
    return y


def sample_typical(logits: torch.Tensor, temp: float = 1.0, tau: float = 0.95, u: Optional[torch.Tensor] = None,
                   generator: Optional[torch.Generator] = None, return_probs: bool = False):
    """Typical sampling of one token per row of ``logits [rows,V]`` (or ``[V]``) on the device:
    the arithmetic of the reference's ``typical(logits, temp, tau)`` (samplers/typical.py:1-17)
    with the draw made by inverse CDF from ``u`` (device f32 [rows] uniform in [0,1); drawn from
    ``generator`` when absent).  Returns device int64 [rows], and with ``return_probs`` also the
    masked, tempered, unnormalised probabilities [rows,V] the draw was made from."""
    x = logits if logits.dim() == 2 else logits.reshape(1, -1)
    if x.dtype != torch.float32 or x.device.type != "cuda" or x.stride(1) != 1:
        raise ValueError("sample_typical needs fp32 CUDA logits with contiguous rows")
    rows, n = x.shape
    if u is None:
        u = torch.rand(rows, device=x.device, dtype=torch.float32, generator=generator)
    if u.dtype != torch.float32 or u.device != x.device or u.numel() != rows or not u.is_contiguous():
        raise ValueError("u must be a contiguous fp32 tensor of one number per row on the logits' device")
    out = torch.empty(rows, dtype=torch.int64, device=x.device)
    probs = torch.empty(rows, n, dtype=torch.float32, device=x.device) if return_probs else None
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().b200rwkv_sample_typical(x.data_ptr(), rows, n, x.stride(0), float(temp), float(tau),
                                                      u.data_ptr(), out.data_ptr(),
                                                      probs.data_ptr() if return_probs else None, None, None, 0,
                                                      _stream(x.device)))
    return (out, probs) if return_probs else out


def argmax_rows(logits: torch.Tensor) -> torch.Tensor:
    """Index of the largest value of every row of ``logits [rows,V]`` (fp32, CUDA, contiguous rows), on the
    device: int64 [rows]; ties go to the lowest index like ``torch.argmax`` on a CPU tensor."""
    x = logits if logits.dim() == 2 else logits.reshape(1, -1)
    if x.dtype != torch.float32 or x.device.type != "cuda" or x.stride(1) != 1:
        raise ValueError("argmax_rows needs fp32 CUDA logits with contiguous rows")
    rows, n = x.shape
    out = torch.empty(rows, dtype=torch.int64, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().b200rwkv_argmax(x.data_ptr(), rows, n, x.stride(0), out.data_ptr(), None, None, 0, _stream(x.device)))
    return out


_DENSE_DTYPES = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


def gemv_dense(w: torch.Tensor, x: torch.Tensor, y: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Unquantised matrix-vector product ``y[o] = sum_j x[j] * w[o,j]`` for ``w [out,in]`` of bf16,
    fp16 or fp32 with contiguous rows (a row stride >= in is allowed) and fp32 ``x [in]``:
    x is rounded to the weights' type, products are summed in fp32, the result is rounded to the
    weights' type and returned as fp32 - what the reference's TORCH-mode ``matvec`` computes
    (agnostic/backends/torch.py:162-164)."""
    if w.dim() != 2 or w.dtype not in _DENSE_DTYPES or w.device.type != "cuda" or w.stride(1) != 1:
        raise ValueError("gemv_dense needs a CUDA [out,in] matrix of bf16/fp16/fp32 with contiguous rows")
    n_out, k_in = w.shape
    if x.dtype != torch.float32 or x.device != w.device or x.numel() != k_in or not x.is_contiguous():
        raise ValueError(f"x must be a contiguous fp32 vector of {k_in} values on the weights' device")
    if y is None:
        y = torch.empty(n_out, dtype=torch.float32, device=w.device)
    elif y.dtype != torch.float32 or y.device != w.device or y.numel() != n_out or not y.is_contiguous():
        raise ValueError(f"y must be a contiguous fp32 vector of {n_out} values on the weights' device")
    with torch.cuda.device(w.device):
        _lib.check(_lib.lib().b200rwkv_gemv_dense(w.data_ptr(), _DENSE_DTYPES[w.dtype], k_in, n_out, w.stride(0),
                                                  x.data_ptr(), y.data_ptr(), _stream(w.device)))
    return y


def matvec(W: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """The reference's TORCH-mode op table entry ``matvec(W, x)`` (agnostic/backends/torch.py:162-164)
    for one vector: ``W`` is the ``[in,out]`` transposed view the reference's ``initTensor`` makes of
    the checkpoint's ``[out,in]`` tensor; the result has ``x``'s dtype.  A matrix that is not such a
    view (its transpose does not have contiguous rows) is refused rather than copied."""
    if W.dim() != 2 or W.stride(0) != 1:
        raise ValueError("matvec expects the transposed view of an [out,in] matrix (stride 1 along the input index)")
    xv = x.reshape(-1)
    if xv.numel() != W.shape[0]:
        raise ValueError("matvec handles one vector per call")
    y = gemv_dense(W.t(), xv.float().contiguous())
    return y.to(x.dtype).reshape(*x.shape[:-1], W.shape[1])
