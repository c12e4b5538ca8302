"""GPU parity of the unquantised matrix-vector product against the reference's TORCH-mode
``matvec`` expression evaluated on the CPU (agnostic/backends/torch.py:162-164)."""
import numpy as np
import pytest
import torch

from rwkvstic_b200 import ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def reference_matvec(W, x):
    """torch.py:162-164 verbatim in meaning: W is the [in,out] transposed view, x the fp32 vector."""
    return x.to(dtype=W.dtype).matmul(W).to(dtype=x.dtype)


def steps_apart(a, b, dtype):
    """Largest distance between a and b counted in representable values of ``dtype``."""
    if dtype == torch.float32:
        return float(((a - b).abs() / b.abs().clamp_min(1e-30)).max()) / 2.0 ** -23
    ia = a.to(dtype).view(torch.int16).to(torch.int32)
    ib = b.to(dtype).view(torch.int16).to(torch.int32)
    same_sign = (ia < 0) == (ib < 0)
    d = (ia - ib).abs()
    small = (a.abs() < 1e-3) & (b.abs() < 1e-3)         # across zero: compare magnitudes instead
    return int(d[same_sign & ~small].max()) if bool((same_sign & ~small).any()) else 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("n,k", [(768, 768), (3072, 768), (768, 3072), (4096, 4096), (257, 1000), (50277, 1024), (33, 72)])
def test_matvec_matches_the_reference_expression(dtype, n, k):
    g = torch.Generator().manual_seed(n + k)
    w_oi = (torch.randn(n, k, generator=g) * 0.02).to(dtype)            # the checkpoint's [out,in] tensor
    x = torch.randn(k, generator=g)
    want = reference_matvec(w_oi.t(), x)                                # CPU, the reference's own expression
    W = w_oi.to(DEV).t()                                                # what initTensor keeps on the device
    got = ops.matvec(W, x.to(DEV)).cpu()
    assert got.dtype == x.dtype and got.shape == want.shape
    if dtype == torch.float32:
        # fp32 sums in another order: error relative to the size of the terms, not of the result
        assert float((got - want).abs().max()) <= 2e-6 * float(x.norm()) * float(w_oi.float().norm(dim=1).max())
    else:
        # both are values of the weights' type; fp32 summation order may move a sum across one
        # rounding boundary, never further
        assert torch.equal(got.to(dtype).float(), got)
        assert steps_apart(got, want, dtype) <= 1
        assert float((got == want).float().mean()) > 0.95
    assert torch.equal(ops.matvec(W, x.to(DEV)).cpu(), got)             # deterministic


def test_gemv_dense_padded_rows_odd_sizes_and_bad_arguments():
    g = torch.Generator().manual_seed(9)
    n, k = 1001, 1003                                   # rows do not start on 16-byte boundaries: element path
    w = (torch.randn(n, k, generator=g) * 0.05).bfloat16()
    x = torch.randn(k, generator=g)
    want = reference_matvec(w.t(), x)
    got = ops.gemv_dense(w.to(DEV), x.to(DEV)).cpu()
    assert steps_apart(got, want, torch.bfloat16) <= 1
    # the same matrix inside a buffer with a padded row stride (vector path plus a tail of 3 inputs)
    buf = torch.zeros(n, 1008, dtype=torch.bfloat16, device=DEV)
    buf[:, :k] = w.to(DEV)
    assert torch.equal(ops.gemv_dense(buf[:, :k], x.to(DEV)).cpu(), got)
    canary = torch.full((n + 2,), 7.5, device=DEV)
    ops.gemv_dense(buf[:, :k], x.to(DEV), y=canary[1:n + 1])
    assert float(canary[0]) == 7.5 and float(canary[-1]) == 7.5 and torch.equal(canary[1:n + 1].cpu(), got)
    with pytest.raises(ValueError):
        ops.gemv_dense(w.to(DEV).t(), x.to(DEV))                         # columns, not rows, contiguous
    with pytest.raises(ValueError):
        ops.gemv_dense(w.to(DEV), x[:10].to(DEV))
    with pytest.raises(ValueError):
        ops.matvec(w.to(DEV), x.to(DEV))                                 # not a transposed view
