"""GPU parity tests of the individual kernels, called through the C ABI."""
import numpy as np
import pytest
import torch

from oracle import fastquant_oracle as O
from rwkvstic_b200 import ops
from rwkvstic_b200.quant import QuantMatrix, quantize_fastquant, quantize_two_axis

from kernel_contract import fixed_point_gemv

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
CANARY = 12345.678


def random_matrix(n, k, seed, zero_offset=False):
    g = torch.Generator().manual_seed(seed)
    qt = torch.randint(0, 256, (n, k), generator=g, dtype=torch.uint8)
    ry = (torch.rand(k, generator=g) + 0.5) * 1e-3
    my = torch.zeros(k) if zero_offset else torch.randn(k, generator=g) * 0.05
    return QuantMatrix(qt=qt, ry=ry, my=my, my64=my.double())


def run_gemv(mats, xs, accumulate=False, ys=None):
    """Outputs live inside canary-padded buffers so that a write outside [0, n_out) is seen."""
    bufs, views = [], []
    for i, m in enumerate(mats):
        b = torch.full((m.n_out + 64,), CANARY, dtype=torch.float32, device=DEV)
        if ys is not None:
            b[32:32 + m.n_out] = ys[i].to(DEV)
        bufs.append(b)
        views.append(b[32:32 + m.n_out])
    ws = ops.gemv_workspace(DEV, mats[0].k_in, len(mats))
    ops.gemv_u8([m.to(DEV) for m in mats], [x.to(DEV) for x in xs], views, accumulate=accumulate, workspace=ws)
    torch.cuda.synchronize()
    assert int(ws[:4].view(torch.int32).item()) == 0        # no device-side wait expired
    for b in bufs:
        assert bool((b[:32] == CANARY).all()) and bool((b[-32:] == CANARY).all())
    return [v.cpu() for v in views]


# (n_out, k_in): ragged small shapes, every RWKV-4 family shape incl. the 7B/14B full sizes
SHAPES = [(80, 128), (1, 128), (19, 384), (257, 768), (3072, 768), (768, 3072), (2048, 2048), (2560, 2560), (521, 10240),
          (4096, 4096), (16384, 4096), (4096, 16384), (5120, 5120), (1031, 20480), (50277, 4096)]


@pytest.mark.parametrize("n,k", SHAPES)
def test_gemv_integer_part_is_bit_exact(n, k):
    m = random_matrix(n, k, seed=n + k, zero_offset=True)
    x = torch.randn(k, generator=torch.Generator().manual_seed(k)) * 3
    got = run_gemv([m], [x])[0]
    want = fixed_point_gemv(x, m, with_affine=False)
    assert torch.equal(got, want)


@pytest.mark.parametrize("n,k", [(80, 128), (3072, 768), (4096, 4096), (4096, 16384), (50277, 768)])
def test_gemv_fastquant_vs_oracle(n, k):
    g = torch.Generator().manual_seed(n * 7 + k)
    w = torch.randn(n, k, generator=g) * 0.02
    m = quantize_fastquant(w)
    weight, rng, off = O.quantize_matrix(w)
    x = torch.randn(1, k, generator=g, dtype=torch.float64)
    want = O.mm8(x, weight, rng, off)[0]
    got = run_gemv([m], [x[0].float()])[0]
    # fp32 input rounding + 24-bit fixed point vs the oracle's fp32 matmul: well inside 2e-3
    assert float((got.double() - want).abs().max()) < 1e-4 * max(1.0, float(want.abs().max()))


def test_gemv_three_matrices_one_launch_and_accumulate():
    g = torch.Generator().manual_seed(5)
    mats = [quantize_fastquant(torch.randn(n, 768, generator=g) * 0.02) for n in (768, 768, 768)]
    xs = [torch.randn(768, generator=g) for _ in range(3)]
    one_by_one = [run_gemv([m], [x])[0] for m, x in zip(mats, xs)]
    together = run_gemv(mats, xs)
    for a, b in zip(one_by_one, together):
        assert torch.equal(a, b)                       # partitioning never changes the arithmetic
    base = [torch.randn(768, generator=g) for _ in range(3)]
    acc = run_gemv(mats, xs, accumulate=True, ys=base)
    for a, b, c in zip(acc, together, base):
        assert torch.equal(a, b + c)
    # ragged: different n_out per matrix (the ffn key + receptance launch)
    mats2 = [quantize_fastquant(torch.randn(n, 768, generator=g) * 0.02) for n in (3072, 768)]
    xs2 = [torch.randn(768, generator=g) for _ in range(2)]
    both = run_gemv(mats2, xs2)
    for m, x, y in zip(mats2, xs2, both):
        assert torch.equal(run_gemv([m], [x])[0], y)


def test_gemv_two_axis_scheme():
    g = torch.Generator().manual_seed(6)
    w = torch.randn(1000, 512, generator=g) * 0.02
    m = quantize_two_axis(w)
    x = torch.randn(512, generator=g)
    want = x.double() @ m.dequant().t()
    got = run_gemv([m], [x])[0]
    assert float((got.double() - want).abs().max()) < 1e-4
    assert torch.allclose(got, fixed_point_gemv(x, m), rtol=1e-5, atol=1e-5)


def test_gemv_zero_and_tiny_inputs():
    m = random_matrix(300, 256, seed=1)
    assert torch.equal(run_gemv([m], [torch.zeros(256)])[0], torch.zeros(300))
    x = torch.zeros(256)
    x[7] = 1e-30
    got = run_gemv([m], [x])[0]
    assert torch.isfinite(got).all()


def test_gemv_deterministic():
    m = random_matrix(4096, 4096, seed=2)
    x = torch.randn(4096, generator=torch.Generator().manual_seed(1))
    a = run_gemv([m], [x])[0]
    for _ in range(3):
        assert torch.equal(run_gemv([m], [x])[0], a)


def test_gemv_rejects_bad_shapes():
    m = random_matrix(8, 128, seed=1).to(DEV)
    bad = QuantMatrix(qt=torch.zeros(8, 96, dtype=torch.uint8, device=DEV), ry=torch.zeros(96, device=DEV),
                      my=torch.zeros(96, device=DEV))
    with pytest.raises(Exception):
        ops.gemv_u8([bad], [torch.zeros(96, device=DEV)])
    with pytest.raises(ValueError):
        ops.gemv_u8([m], [torch.zeros(8, device=DEV)])


def test_wkv_scan_against_reference_vectors(golden):
    g = golden("ops_small.npz")
    f = lambda n: torch.from_numpy(g[n]).float().to(DEV).contiguous()
    # reference state convention in and out
    aa, bb, pp = f("wkv_aa"), f("wkv_bb"), f("wkv_pp")
    y = ops.wkv_scan(f("wkv_w"), f("wkv_u"), f("wkv_k"), f("wkv_v"), aa, bb, pp, convention=1)
    torch.cuda.synchronize()
    assert torch.allclose(y[0].cpu().double(), torch.from_numpy(g["wkv_y"]), rtol=1e-5, atol=1e-5)
    assert torch.allclose(aa.cpu().double(), torch.from_numpy(g["wkv_aa2"]), rtol=1e-5, atol=1e-5)
    assert torch.allclose(bb.cpu().double(), torch.from_numpy(g["wkv_bb2"]), rtol=1e-5, atol=1e-5)
    assert torch.equal(pp.cpu(), f("wkv_pp").cpu())
    # max-trick convention: start from the converted state, compare in canonical form
    w = f("wkv_w")
    aa, bb, pp = f("wkv_aa"), f("wkv_bb"), (-w).clone()
    y2 = ops.wkv_scan(w, f("wkv_u"), f("wkv_k"), f("wkv_v"), aa, bb, pp, convention=0)
    torch.cuda.synchronize()
    assert torch.allclose(y2, y, rtol=1e-6, atol=1e-6)
    e = torch.exp(w + pp)
    assert torch.allclose((aa * e).cpu().double(), torch.from_numpy(g["wkv_aa2"]), rtol=1e-5, atol=1e-5)


def test_wkv_scan_batched_streams_and_large_k():
    """B streams are independent; exp(k) beyond fp32 range must not overflow (max-trick)."""
    g = torch.Generator().manual_seed(9)
    B, T, C = 3, 17, 96
    w = -torch.exp(torch.rand(C, generator=g) * 8 - 5)
    u = torch.rand(C, generator=g) * 2 - 1
    k = torch.randn(B, T, C, generator=g) * 3
    k[1, 5] += 100.0                                    # exp(100) overflows fp32
    v = torch.randn(B, T, C, generator=g)
    aa, bb, pp = torch.zeros(B, C), torch.zeros(B, C), torch.full((B, C), -1e30)
    dev = lambda t: t.to(DEV).contiguous()
    a, b, p = dev(aa), dev(bb), dev(pp)
    y = ops.wkv_scan(dev(w), dev(u), dev(k), dev(v), a, b, p).cpu()
    assert torch.isfinite(y).all()
    for s in range(B):
        yo, ao, bo, _ = O.wkv(T, C, w.double(), u.double(), k[s].double(), v[s].double(),
                              torch.zeros(C, dtype=torch.float64), torch.zeros(C, dtype=torch.float64), None)
        assert torch.allclose(y[s].double(), yo, rtol=2e-5, atol=2e-5)
        a1, b1, p1 = dev(aa[s]), dev(bb[s]), dev(pp[s])
        y1 = ops.wkv_scan(dev(w), dev(u), dev(k[s]), dev(v[s]), a1, b1, p1).cpu()
        assert torch.equal(y1[0], y[s]) and torch.equal(a1.cpu(), a[s].cpu())


def test_reference_op_library_names_and_semantics(golden):
    """torch.ops.rwkv.{mm8_one,mm8_three,wkv_forward} as the reference modules call them
    (modules/matmul.py:42-49, :70-80; modules/wkv.py:8-19), including from TorchScript."""
    from rwkvstic_b200 import torch_ops
    torch_ops.register()
    g = torch.Generator().manual_seed(12)
    N, M = 256, 320                                        # in, out
    wq = [torch.randint(0, 256, (N, M), generator=g, dtype=torch.uint8).to(DEV) for _ in range(3)]
    r = [(torch.rand(N, generator=g) * 1e-3 + 1e-4).to(DEV) for _ in range(3)]
    x = [torch.randn(N, generator=g).to(DEV) for _ in range(3)]
    want = [(xi.double() * ri.double()) @ wi.double() for xi, ri, wi in zip(x, r, wq)]
    y = torch.zeros(M, device=DEV)
    torch.ops.rwkv.mm8_one(N, M, x[0], wq[0], y, r[0])
    assert torch.allclose(y.double(), want[0], rtol=1e-5, atol=1e-5)
    torch.ops.rwkv.mm8_one(N, M, x[0], wq[0], y, r[0])     # accumulates onto y, like the atomicAdd kernels
    assert torch.allclose(y.double(), 2 * want[0], rtol=1e-5, atol=1e-5)
    ys = [torch.zeros(M, device=DEV) for _ in range(3)]
    torch.ops.rwkv.mm8_three(N, M, *x, *wq, *ys, *r)
    for a, b in zip(ys, want):
        assert torch.allclose(a.double(), b, rtol=1e-5, atol=1e-5)

    @torch.jit.script
    def scripted(N: int, M: int, x, w, y, r):
        torch.ops.rwkv.mm8_one(N, M, x, w, y, r)
        return y
    y2 = scripted(N, M, x[1], wq[1], torch.zeros(M, device=DEV), r[1])
    assert torch.allclose(y2.double(), want[1], rtol=1e-5, atol=1e-5)

    gg = golden("ops_small.npz")
    d = lambda n: torch.from_numpy(gg[n]).to(DEV)
    yk = torch.empty(7, 32, dtype=torch.float64, device=DEV)
    aa, bb, pp = d("wkv_aa").clone(), d("wkv_bb").clone(), d("wkv_pp").clone()
    torch.ops.rwkv.wkv_forward(1, 7, 32, d("wkv_w"), d("wkv_u"), d("wkv_k"), d("wkv_v"), yk, aa, bb, pp)
    assert torch.allclose(yk.cpu(), torch.from_numpy(gg["wkv_y"]), rtol=1e-5, atol=1e-5)
    assert torch.allclose(aa.cpu(), torch.from_numpy(gg["wkv_aa2"]), rtol=1e-5, atol=1e-5)
    assert torch.allclose(bb.cpu(), torch.from_numpy(gg["wkv_bb2"]), rtol=1e-5, atol=1e-5)
    assert torch.equal(pp.cpu(), torch.from_numpy(gg["wkv_pp"]))
