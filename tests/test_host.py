"""CPU-side checks: the C-ABI library loads and exports what the header declares, the product
quantiser is bit-identical to the reference's, launch geometry invariants, and the accuracy of
the kernels' arithmetic contract (tests/kernel_contract.py) against the reference goldens."""
import os
import re

import numpy as np
import pytest
import torch

from oracle import fastquant_oracle as O
from rwkvstic_b200 import _lib
from rwkvstic_b200.model import quantize_tensors, state_from_reference, state_to_reference
from rwkvstic_b200.quant import quantize_fastquant, quantize_two_axis
from rwkvstic_b200.synth import SHAPES, VOCAB, synth_checkpoint

from kernel_contract import ContractModel, fixed_point_gemv

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "b200rwkv.h")).read()
    declared = set(re.findall(r"\b(b200rwkv_[a-z0-9_]+)\s*\(", header))
    assert declared == set(_lib.EXPORTS)
    L = _lib.lib()
    for name in declared:
        assert hasattr(L, name), name
    assert L.b200rwkv_version() >= 100


def test_bad_arguments_return_codes_not_aborts():
    L = _lib.lib()
    assert L.b200rwkv_gemv_u8(0, None, None, None, 0, None, 0, None) == _lib.EINVAL
    assert b"gemv_u8" in L.b200rwkv_last_error()
    assert L.b200rwkv_wkv_scan(1, 1, 0, *([None] * 8), 0, None) == _lib.EINVAL
    assert L.b200rwkv_decode_step(None, None, None, None, None, 0, None) == _lib.EINVAL
    # the many-rows entry points validate before any CUDA call as well
    assert L.b200rwkv_gemm_u8(1, None, None, None, 4, None, 0, None) == _lib.EINVAL
    assert L.b200rwkv_gemm_u8(4, None, None, None, 4, None, 0, None) == _lib.EINVAL
    assert b"gemm_u8" in L.b200rwkv_last_error()
    assert L.b200rwkv_forward_rows(None, None, 1, 1, None, 0, None, None, 0, None) == _lib.EINVAL
    assert L.b200rwkv_forward_rows_stage(None, None, None, 1, 1, None, 0, None, None, 0, None) == _lib.EINVAL
    assert L.b200rwkv_argmax(None, 1, 8, 8, None, None, None, 0, None) == _lib.EINVAL
    assert L.b200rwkv_sample_typical(None, 1, 8, 8, 1.0, 0.9, None, None, None, None, None, 0, None) == _lib.EINVAL
    assert L.b200rwkv_sample_typical(1, 1, 8, 8, 0.0, 0.9, 1, 1, None, None, None, 0, None) == _lib.EINVAL   # temp must be > 0
    assert L.b200rwkv_sample_typical(1, 2, 8, 8, 1.0, 0.9, 1, 1, None, 1, 1, 4, None) == _lib.EINVAL    # history needs rows == 1
    assert b"sample_typical" in L.b200rwkv_last_error()
    assert L.b200rwkv_gemv_dense(None, 1, 8, 8, 8, None, None, None) == _lib.EINVAL
    assert L.b200rwkv_gemv_dense(1, 7, 8, 8, 8, 1, 1, None) == _lib.EINVAL          # unknown dtype
    assert L.b200rwkv_gemv_dense(1, 1, 8, 8, 4, 1, 1, None) == _lib.EINVAL          # row stride below k_in
    assert L.b200rwkv_gemm_workspace_bytes(4096, 3, 100) > 3 * 3 * 112 * 4096   # digit rows padded to 16
    assert L.b200rwkv_gemm_workspace_bytes(4096, 4, 100) == 0 and L.b200rwkv_rows_workspace_bytes(None, 1, 1) == 0
    with pytest.raises(_lib.B200RWKVError):
        _lib.gemv_plan(96, 1, 8)            # k_in not a multiple of 128
    with pytest.raises(_lib.B200RWKVError):
        _lib.gemv_plan(128 * 1024, 1, 8)    # beyond the supported reduction length


def test_quantiser_is_bit_identical_to_reference(golden):
    g = golden("ops_small.npz")
    w = torch.from_numpy(g["q_w"])
    m = quantize_fastquant(w)
    assert torch.equal(m.reference_layout(), torch.from_numpy(g["q_weight"]))
    assert torch.equal(m.ry, torch.from_numpy(g["q_range"]))
    assert torch.equal(m.my64, torch.from_numpy(g["q_offset"]))
    gen = torch.Generator().manual_seed(3)
    for shape in ((96, 64), (257, 48), (64, 256)):
        w = torch.randn(*shape, generator=gen) * 0.02
        weight, rng, off = O.quantize_matrix(w)
        m = quantize_fastquant(w)
        assert torch.equal(m.qt, weight.t()) and torch.equal(m.ry, rng) and torch.equal(m.my64, off)


def test_two_axis_quantiser_matches_oracle_restatement():
    gen = torch.Generator().manual_seed(4)
    w = torch.randn(40, 32, generator=gen) * 0.02
    q, my, ry, mx, rx = O.two_axis_quantize(w)
    m = quantize_two_axis(w)
    assert torch.equal(m.qt, q.t())
    assert torch.allclose(m.dequant(), ((q.double() + 0.5) * ry[:, None] * rx[None, :] + my[:, None] + mx[None, :]).t(),
                          rtol=1e-6, atol=5e-8)   # ry, rx, mx are stored as fp32


@pytest.mark.parametrize("name", list(SHAPES))
def test_gemv_geometry_invariants(name):
    L, D = SHAPES[name]
    F = 4 * D
    for K, nmat, N in ((D, 3, D), (D, 1, D), (D, 2, F), (F, 1, D), (D, 1, VOCAB)):
        p = _lib.gemv_plan(K, nmat, N)
        kc, n = p["chunk_bytes"], p["chunks_per_row"]
        assert kc % 128 == 0 and kc <= 2048 and kc * n >= K > kc * (n - 1)  # chunks tile a row, last one non-empty
        assert p["swizzle_bytes"] == 128 and p["rows_per_stage"] == 16
        assert p["stage_bytes"] == 16 * kc and p["stage_bytes"] % 1024 == 0
        assert p["ring_stages"] >= 3 and p["shared_memory_bytes"] <= 227 * 1024
        assert p["grid"] * p["max_rows_per_cta"] >= N and p["max_rows_per_cta"] % 16 == 0
        # at least 2.5 us of weight stream fits the ring at 6.5 TB/s over 148 SMs (44 KB/us per SM)
        assert p["ring_stages"] * 16 * kc >= 2.5 * 44e3


def test_fixed_point_contract_accuracy_single_matrix():
    gen = torch.Generator().manual_seed(8)
    w = torch.randn(320, 256, generator=gen) * 0.02
    m = quantize_fastquant(w)
    weight, rng, off = O.quantize_matrix(w)
    x = torch.randn(1, 256, generator=gen, dtype=torch.float64)
    want = O.mm8(x, weight, rng, off)[0]
    got = fixed_point_gemv(x[0].float(), m)
    assert float((got.double() - want).abs().max()) < 2e-5
    m2 = quantize_two_axis(w)
    q, my, ry, mx, rx = O.two_axis_quantize(w)
    want2 = O.two_axis_mm8(x, q, my, ry, mx, rx)[0]
    assert float((fixed_point_gemv(x[0].float(), m2).double() - want2).abs().max()) < 2e-5


def test_state_convention_round_trip():
    gen = torch.Generator().manual_seed(2)
    st = torch.randn(3, 5, 16, generator=gen).abs()
    st[:, 4] = torch.randn(3, 16, generator=gen)
    w = [-torch.rand(16, generator=gen) for _ in range(3)]
    ref = state_to_reference(st, w)
    back = state_from_reference(ref, w)
    again = state_to_reference(back, w)
    assert torch.allclose(ref[:, :4], again[:, :4], rtol=1e-5, atol=1e-6)
    empty = torch.zeros(3, 5, 16)
    empty[:, 4] = -1e30
    assert torch.equal(state_from_reference(state_to_reference(empty, w), w), empty)


def test_contract_model_meets_tolerance_on_tiny_golden(golden):
    g = golden("model_tiny.npz")
    wts = quantize_tensors(synth_checkpoint(2, 128, vocab=257, seed=31).items(), "cpu")
    m = ContractModel(wts)
    lg, st = m.forward(g["tokens"], m.emptyState.clone())
    assert float((lg.double() - torch.from_numpy(g["logits_seq"])).abs().max()) < 2e-3
    ref = torch.from_numpy(g["state_seq"])
    mine = state_to_reference(st, [ly.vec["att.time_decay"] for ly in wts.layers])
    assert torch.allclose(mine[:, :4], ref[:, :4], rtol=1e-3, atol=1e-4)


def test_contract_model_greedy_stream_169m(golden):
    """The fp32 + 24-bit fixed-point design reproduces the reference's 64 greedy tokens and stays
    far inside the 2e-3 logit tolerance (measured 2e-5) - checked here without a GPU."""
    g = golden("model_169m.npz")
    wts = quantize_tensors(synth_checkpoint(12, 768, seed=int(g["seed"])).items(), "cpu")
    m = ContractModel(wts)
    logits, st = m.forward(g["prompt"], m.emptyState.clone())
    probe = torch.from_numpy(g["probe_idx"])
    worst = 0.0
    for i in range(64):
        t = int(torch.argmax(logits))
        assert t == int(g["tokens"][i])
        worst = max(worst, float((logits[probe].double() - torch.from_numpy(g["probe_logits"][i])).abs().max()))
        logits, st = m.forward([t], st)
    assert worst < 2e-4
    assert float(g["margin"].min()) > 2 * 2e-3   # the golden's greedy choices are tolerance-proof
