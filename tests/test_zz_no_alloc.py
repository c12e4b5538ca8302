"""The allocation-free GEMV entry point, called through the C ABI.

Some callers of the library may not allocate device memory (a plugin host that owns the pool, code
that runs during a stream capture, a bare C program).  ``b200rwkv_gemv_u8_static`` serves them from
a scratch array built into the library.  It must give exactly what ``b200rwkv_gemv_u8`` gives with
a caller-provided workspace, call after call (the array keeps the previous call's contents), and it
must refuse sizes beyond its fixed scratch.  Collected last on purpose.
"""
import ctypes as C

import pytest
import torch

from rwkvstic_b200 import _lib, ops
from rwkvstic_b200.quant import QuantMatrix

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _matrix(n, k, seed):
    g = torch.Generator().manual_seed(seed)
    return QuantMatrix(qt=torch.randint(0, 256, (n, k), generator=g, dtype=torch.uint8),
                       ry=torch.rand(k, generator=g) * 1e-3 + 1e-4, my=torch.randn(k, generator=g) * 0.05).to(DEV)


def _static_call(mats, xs, ys, status, accumulate=0):
    n = len(mats)
    cm = (_lib.Matrix * n)(*[_lib.Matrix(m.qt.data_ptr(), m.ry.data_ptr(), m.my.data_ptr(), None, None, 0.0,
                                         m.n_out, m.k_in) for m in mats])
    cx = (C.c_void_p * n)(*[x.data_ptr() for x in xs])
    cy = (C.c_void_p * n)(*[y.data_ptr() for y in ys])
    stream = torch.cuda.current_stream(torch.device(DEV)).cuda_stream
    return _lib.lib().b200rwkv_gemv_u8_static(n, cm, cx, cy, accumulate, None if status is None else status.data_ptr(), stream)


def test_static_scratch_variant_matches_workspace_variant_twice_in_a_row():
    torch.cuda.set_device(0)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    # call 1: three [768,768] matrices; call 2: one long-K matrix that overwrites the same scratch
    cases = [([_matrix(768, 768, s) for s in (1, 2, 3)], 768), ([_matrix(1031, 16384, 4)], 16384)]
    for mats, k in cases + cases[:1]:
        g = torch.Generator().manual_seed(k)
        xs = [torch.randn(k, generator=g).to(DEV) for _ in mats]
        want = ops.gemv_u8(mats, xs)                               # existing entry point, own workspace
        got = [torch.full((m.n_out,), -7.0, device=DEV) for m in mats]
        assert _static_call(mats, xs, got, status) == _lib.OK, _lib.lib().b200rwkv_last_error()
        torch.cuda.synchronize()
        for a, b in zip(got, want):
            assert torch.equal(a, b)                               # same kernels, same bits
    assert int(status.item()) == 0


def test_static_scratch_variant_without_status_word_and_with_accumulate():
    """The two documented options: no status word (NULL), and adding onto the caller's outputs."""
    torch.cuda.set_device(0)
    mats = [_matrix(515, 1024, s) for s in (7, 8)]
    g = torch.Generator().manual_seed(3)
    xs = [torch.randn(1024, generator=g).to(DEV) for _ in mats]
    want = ops.gemv_u8(mats, xs)
    got = [torch.full((m.n_out,), 5.0, device=DEV) for m in mats]
    assert _static_call(mats, xs, got, None) == _lib.OK, _lib.lib().b200rwkv_last_error()
    torch.cuda.synchronize()
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    base = [torch.randn(m.n_out, generator=g).to(DEV) for m in mats]
    acc_want = [b.clone() for b in base]
    ops.gemv_u8(mats, xs, acc_want, accumulate=True)
    acc_got = [b.clone() for b in base]
    assert _static_call(mats, xs, acc_got, None, accumulate=1) == _lib.OK, _lib.lib().b200rwkv_last_error()
    torch.cuda.synchronize()
    for a, b in zip(acc_got, acc_want):
        assert torch.equal(a, b)


def test_static_scratch_variant_rejects_oversize_requests():
    torch.cuda.set_device(0)
    mats = [_matrix(8, 32768, s) for s in (5, 6)]                  # 2 * 4 * 32768 bytes > 192 KB
    xs = [torch.zeros(32768, device=DEV) for _ in mats]
    ys = [torch.zeros(8, device=DEV) for _ in mats]
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert _static_call(mats, xs, ys, status) == _lib.EINVAL
    assert b"exceeds the built-in scratch" in _lib.lib().b200rwkv_last_error()
