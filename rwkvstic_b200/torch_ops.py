"""Drop-in replacement for the reference's custom op library (``torch.ops.rwkv.*``).

The reference registers three ops from a JIT-built C++/CUDA extension
(cuda/wrapper.cpp:131-141, loaded by cuda/load.py:1-13) and calls them from
modules/matmul.py:45, :78 and modules/wkv.py:18 - also from inside TorchScript ``.rwkv``
archives exported on CUDA.  ``register()`` defines the same three names with the same
argument order in the same ``rwkv`` namespace, backed by this package's kernels, so that code
keeps running unchanged.  Call it INSTEAD of the reference's ``loadCustomCudaModule()``: a
second definition of the same op names in one process raises.

Semantics kept from the reference kernels (cuda/operators32.cu:18-115, cuda/operators.cu:6-44):
* ``mm8_one(N, M, x, w, y, r)``: ``y[k] += sum_j x[j] * r[j] * w[j, k]`` with ``w`` uint8
  ``[N, M]`` (input-major, as ``MM8.weight``), ``y`` accumulated in place.  The offset term is
  NOT part of the op; the caller adds it (modules/matmul.py:58-62).
* ``mm8_three``: the same for three (x, w, y, r) groups.
* ``wkv_forward(B, T, C, w, u, k, v, y, aa, bb, pp)``: the plain recurrence of
  cuda/operators.cu:24-33 on fp64 tensors; ``y, aa, bb`` written in place, ``pp`` untouched.

Cost of the compatibility layer: the kernels stream weights output-major, so each ``w`` is
transposed once and cached - twice the weight memory while ``w`` is alive.  The cache entry is
tied to the tensor object by a weak reference and checked against its version counter: when
``w`` is freed the transposed copy goes with it, and an address reused by another matrix (or
bytes modified in place) never gets stale data.  New code should use
``rwkvstic_b200.model.B200RWKV`` instead, which keeps one copy.
"""
from __future__ import annotations

import weakref
from typing import Dict, Tuple

import torch

from . import ops
from .quant import QuantMatrix

_lib_handle = None
_cache: Dict[int, Tuple[weakref.ref, int, QuantMatrix]] = {}     # id(w) -> (weak reference to w, its version, transposed copy)


def _matrix(w: torch.Tensor, r: torch.Tensor) -> QuantMatrix:
    if w.dtype != torch.uint8 or w.dim() != 2 or w.stride(1) != 1:
        raise RuntimeError("rwkv::mm8: w must be a uint8 [N, M] matrix with unit inner stride")
    key = id(w)
    hit = _cache.get(key)
    if hit is not None and hit[0]() is w and hit[1] == w._version:
        m = hit[2]
        m.ry = r.to(torch.float32).contiguous()
        return m
    zeros = torch.zeros(w.shape[0], dtype=torch.float32, device=w.device)
    m = QuantMatrix(qt=w.t().contiguous(), ry=r.to(torch.float32).contiguous(), my=zeros)
    _cache[key] = (weakref.ref(w, lambda _ref, k=key: _cache.pop(k, None)), w._version, m)
    return m


def _check_vec(name, t, n):
    if t.dim() != 1 or t.numel() != n or t.stride(0) != 1:
        raise RuntimeError(f"rwkv::mm8: {name} must be a contiguous vector of {n} elements")


def mm8_three(N: int, M: int, x, x1, x2, w, w1, w2, y, y1, y2, r, r1, r2) -> None:
    xs, ws, ys, rs = (x, x1, x2), (w, w1, w2), (y, y1, y2), (r, r1, r2)
    for a, b, c in zip(xs, ys, rs):
        _check_vec("x", a, N), _check_vec("y", b, M), _check_vec("r", c, N)
    mats = [_matrix(wi, ri) for wi, ri in zip(ws, rs)]
    if all(t.dtype == torch.float32 for t in ys):
        ops.gemv_u8(mats, [a.to(torch.float32).contiguous() for a in xs], list(ys), accumulate=True)
    else:   # fp64 callers (cuda/wrapper.cpp:98-112): compute in fp32, accumulate in the caller's dtype
        out = ops.gemv_u8(mats, [a.to(torch.float32).contiguous() for a in xs])
        for b, o in zip(ys, out):
            b += o.to(b.dtype)


def mm8_one(N: int, M: int, x, w, y, r) -> None:
    _check_vec("x", x, N), _check_vec("y", y, M), _check_vec("r", r, N)
    m = _matrix(w, r)
    if y.dtype == torch.float32:
        ops.gemv_u8([m], [x.to(torch.float32).contiguous()], [y], accumulate=True)
    else:
        y += ops.gemv_u8([m], [x.to(torch.float32).contiguous()])[0].to(y.dtype)


def wkv_forward(B: int, T: int, C: int, w, u, k, v, y, aa, bb, pp) -> None:
    f = lambda t: t.to(torch.float32).contiguous()
    a32, b32 = f(aa).reshape(B, C), f(bb).reshape(B, C)
    p32 = f(pp).reshape(B, C)
    out = ops.wkv_scan(f(w), f(u), f(k).reshape(B, T, C), f(v).reshape(B, T, C), a32, b32, p32, convention=1)
    y.copy_(out.reshape(y.shape).to(y.dtype))
    aa.copy_(a32.reshape(aa.shape).to(aa.dtype))
    bb.copy_(b32.reshape(bb.shape).to(bb.dtype))


def register() -> None:
    """Define ``rwkv::mm8_one``, ``rwkv::mm8_three`` and ``rwkv::wkv_forward`` (CUDA only)."""
    global _lib_handle
    if _lib_handle is not None:
        return
    lib = torch.library.Library("rwkv", "DEF")
    # The written-to tensors carry alias annotations: a schema parsed from text is otherwise taken
    # to be pure, and TorchScript would drop a call that returns nothing.  (The reference's ops get
    # their schema inferred from C++ and are treated as side-effecting wholesale.)
    lib.define("wkv_forward(int B, int T, int C, Tensor w, Tensor u, Tensor k, Tensor v, Tensor(a!) y, "
               "Tensor(b!) aa, Tensor(c!) bb, Tensor(d!) pp) -> ()")
    lib.define("mm8_one(int N, int M, Tensor x, Tensor w, Tensor(a!) y, Tensor r) -> ()")
    lib.define("mm8_three(int N, int M, Tensor x, Tensor x1, Tensor x2, Tensor w, Tensor w1, Tensor w2, "
               "Tensor(a!) y, Tensor(b!) y1, Tensor(c!) y2, Tensor r, Tensor r1, Tensor r2) -> ()")
    lib.impl("wkv_forward", wkv_forward, "CUDA")
    lib.impl("mm8_one", mm8_one, "CUDA")
    lib.impl("mm8_three", mm8_three, "CUDA")
    _lib_handle = lib
