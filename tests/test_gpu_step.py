"""GPU tests of the persistent decode step (one resident kernel per token) and of the network at
the large RWKV-4 widths: against the chained per-matrix path, and against the CPU oracle on models
truncated to two blocks and a small vocabulary so that the oracle finishes in seconds."""
import ctypes as C

import pytest
import torch

from oracle.fastquant_oracle import OracleRWKV
from rwkvstic_b200 import _lib
from rwkvstic_b200.model import B200RWKV
from rwkvstic_b200.synth import synth_checkpoint, synth_tokens

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 2e-3   # max |dlogit| against the reference's fp64-vector / fp32-matmul CPU path


def states_agree(mine, ref, rtol=2e-3, atol=2e-4, row_rel=2e-5):
    """Rows 0..3 of two reference-convention states.  The WKV sums (rows 2, 3) add terms of either sign
    whose size can exceed the sum by orders of magnitude, so their rounding scales with the largest
    entry of the row, not with the entry itself."""
    a, b = mine[:, :4].double().cpu(), ref[:, :4].double().cpu()
    excess = (a - b).abs() - (atol + rtol * b.abs() + row_rel * b.abs().amax(dim=2, keepdim=True))
    worst = int(excess.argmax())
    return float(excess.max()) <= 0, (worst, float(a.flatten()[worst]), float(b.flatten()[worst]))


@pytest.mark.parametrize("layers,embed,vocab", [(2, 128, 257), (3, 768, 1000), (2, 2048, 4096), (2, 2560, 50277),
                                                (2, 4096, 50277), (1, 5120, 3000)])
def test_persistent_step_equals_chained_step(layers, embed, vocab):
    """Same weights, same tokens: the one-kernel step and the launch-per-matrix step give the same
    logits and state up to the fp32 rounding of the offset sums (the integer parts are exact in both)."""
    one = B200RWKV.synthetic(layers, embed, vocab=vocab, seed=5, device=DEV, use_graph=False, decode_mode="persistent")
    assert one.decode_mode == "persistent"
    many = B200RWKV(one.w, use_graph=False, decode_mode="chained")
    toks = synth_tokens(7, seed=9, vocab=vocab)
    s1, s2 = one.emptyState.clone(), many.emptyState.clone()
    for i, t in enumerate(toks):
        l1, _ = one.forward(t.reshape(1), s1)
        l2, _ = many.forward(t.reshape(1), s2)
        scale = float(l2.abs().max()) + 1.0
        assert float((l1 - l2).abs().max()) <= 2e-5 * scale, (i, float((l1 - l2).abs().max()))
    ok, where = states_agree(one.to_reference_state(s1), many.to_reference_state(s2), rtol=1e-3, atol=1e-4, row_rel=1e-5)
    assert ok, where
    one.check_status()
    many.check_status()


def test_persistent_step_is_deterministic_and_graph_safe():
    m = B200RWKV.synthetic(2, 768, vocab=1000, seed=6, device=DEV, decode_mode="persistent")   # graph path after the second call
    eager = B200RWKV(m.w, use_graph=False, decode_mode="persistent")
    toks = synth_tokens(10, seed=2, vocab=1000)
    sg, se = m.emptyState.clone(), eager.emptyState.clone()
    for t in toks:
        lg, _ = m.forward(t.reshape(1), sg)
        le, _ = eager.forward(t.reshape(1), se)
        assert torch.equal(lg, le)
    assert torch.equal(sg, se) and len(m._graphs) >= 1
    again = m.emptyState.clone()
    for t in toks:
        l2, _ = m.forward(t.reshape(1), again)
    assert torch.equal(l2, lg) and torch.equal(again, sg)
    m.check_status()


def test_persistent_step_without_logits_leaves_the_same_state():
    m = B200RWKV.synthetic(2, 256, vocab=300, seed=8, device=DEV, use_graph=False, decode_mode="persistent")
    toks = synth_tokens(4, seed=3, vocab=300)
    a, b = m.emptyState.clone(), m.emptyState.clone()
    for t in toks:
        m._tok.copy_(t.reshape(1))
        m._step(a, want_logits=True)
        m._step(b, want_logits=False)
    assert torch.equal(a, b)


def test_step_geometry_and_plan_validation():
    m = B200RWKV.synthetic(1, 128, vocab=300, seed=1, device=DEV, use_graph=False, decode_mode="persistent")
    geo = (C.c_int64 * 8)()
    _lib.check(m._L.b200rwkv_step_geometry(C.byref(m._cmodel), 148, geo))
    grid, stages, slot, smem = (int(geo[i]) for i in range(4))
    assert grid == 128 and stages >= 2 and slot % 2048 == 0 and smem <= 227 * 1024
    need = int(m._L.b200rwkv_step_plan_bytes(C.byref(m._cmodel)))
    assert need == m._plan.numel()
    rc = m._L.b200rwkv_step_plan_init(C.byref(m._cmodel), m._plan.data_ptr(), need - 1)
    assert rc == _lib.EINVAL
    rc = m._L.b200rwkv_decode_step_persistent(C.byref(m._cmodel), m._plan.data_ptr() + 8, need, m._tok.data_ptr(),
                                              m.emptyState.data_ptr(), None, None, None, None)
    assert rc == _lib.EINVAL


@pytest.mark.parametrize("embed", [2048, 2560, 4096, 5120])
def test_two_block_model_against_the_oracle_at_the_large_widths(embed):
    """L = 2, V = 1024 at the widths of the 1.5B, 3B, 7B and 14B models: 32 tokens one at a time through
    both one-row paths (chained launches, persistent kernel), and 8 streams x 64 tokens through the
    tensor-core rows path, all against the oracle's sequence mode (final logits and state)."""
    vocab = 1024
    ck = synth_checkpoint(2, embed, vocab=vocab, seed=40 + embed % 7)
    ref = OracleRWKV(ck)
    model = B200RWKV.from_checkpoint(ck, device=DEV, use_graph=False)
    toks = synth_tokens(32, seed=embed, vocab=vocab)
    want, wstate = ref.forward(toks, ref.emptyState.clone())
    errs = {}
    for mode in ("chained", "persistent"):          # both one-row paths, token by token
        m1 = model if mode == "chained" else B200RWKV(model.w, use_graph=False, decode_mode=mode)
        state = m1.emptyState.clone()
        for t in toks:
            got, state = m1.forward(t.reshape(1), state)
        errs[mode] = float((got.cpu().double() - want).abs().max())
        assert errs[mode] < TOL, f"D={embed} one-row path ({mode}): max |dlogit| {errs[mode]}"
        ok, where = states_agree(m1.to_reference_state(state), wstate)
        assert ok, (mode, where)
        m1.check_status()
    err = max(errs.values())

    B, T = 8, 64
    btoks = synth_tokens(B * T, seed=embed + 1, vocab=vocab).reshape(B, T)
    bstate = model.empty_batch_state(B)
    out = model.forward_rows(btoks.to(DEV), bstate)
    worst = 0.0
    for b in range(B):
        w, ws = ref.forward(btoks[b], ref.emptyState.clone())
        worst = max(worst, float((out[b].cpu().double() - w).abs().max()))
        if b == 0:
            ok, where = states_agree(model.to_reference_state(bstate[b]), ws)
            assert ok, where
    assert worst < TOL, f"D={embed} rows path: max |dlogit| {worst}"
    print(f"D={embed}: max |dlogit| one-row chained {errs['chained']:.2e}, persistent {errs['persistent']:.2e}, rows {worst:.2e}")
