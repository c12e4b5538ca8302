"""The CPU oracle against fixtures produced by the unmodified reference (tests/golden/make_golden.py)."""
import pytest
import numpy as np
import torch

from oracle import fastquant_oracle as O
from rwkvstic_b200.synth import synth_checkpoint


def t(a):
    return torch.from_numpy(np.asarray(a))


def test_quantiser_bit_exact(golden):
    g = golden("ops_small.npz")
    weight, rng, off = O.quantize_matrix(t(g["q_w"]))
    assert weight.dtype == torch.uint8 and tuple(weight.shape) == (48, 80)
    assert torch.equal(weight, t(g["q_weight"]))
    assert torch.equal(rng, t(g["q_range"]))
    assert torch.equal(off, t(g["q_offset"]))


def test_mm8(golden):
    g = golden("ops_small.npz")
    weight, rng, off = O.quantize_matrix(t(g["q_w"]))
    for n in ("1", "5"):
        y = O.mm8(t(g["mm_x" + n]), weight, rng, off)
        assert torch.equal(y, t(g["mm_y" + n]))


def test_layernorm(golden):
    g = golden("ops_small.npz")
    y = O.layernorm(t(g["ln_x"]), t(g["ln_w"]).double(), t(g["ln_b"]).double())
    assert torch.equal(y, t(g["ln_y"]))


def test_wkv_and_maxtrick_form(golden):
    g = golden("ops_small.npz")
    w, u, k, v = (t(g["wkv_" + n]) for n in "wukv")
    y, aa, bb, pp = O.wkv(7, 32, w, u, k, v, t(g["wkv_aa"]), t(g["wkv_bb"]), t(g["wkv_pp"]))
    assert torch.equal(y, t(g["wkv_y"]))
    assert torch.equal(aa, t(g["wkv_aa2"])) and torch.equal(bb, t(g["wkv_bb2"]))
    assert torch.equal(pp, t(g["wkv_pp2"]))
    # the max-trick form reaches the same outputs; its state maps as aa_plain = exp(w)*aa*exp(pp)
    a, b, p = t(g["wkv_aa"]).clone(), t(g["wkv_bb"]).clone(), -w      # plain -> max-trick: pp = -w
    ys = []
    for i in range(7):
        yi, a, b, p = O.wkv_maxtrick_step(w, u, k[i], v[i], a, b, p)
        ys.append(yi)
    assert torch.allclose(torch.stack(ys), y, rtol=1e-12, atol=1e-12)
    assert torch.allclose(torch.exp(w + p) * a, aa, rtol=1e-12, atol=1e-12)
    assert torch.allclose(torch.exp(w + p) * b, bb, rtol=1e-12, atol=1e-12)


def test_block(golden):
    g = golden("ops_small.npz")
    blk = O.Block(synth_checkpoint(1, 64, vocab=97, seed=21), 0)
    for T in (1, 4):
        s = t(g["blk_state"]).clone()
        y, s2 = blk.forward(t(g[f"blk_x{T}"]).clone(), s)
        assert torch.equal(y, t(g[f"blk_y{T}"]))
        assert torch.equal(s2, t(g[f"blk_s{T}"]))


def test_tiny_model_sequence_chunk_token(golden):
    g = golden("model_tiny.npz")
    m = O.OracleRWKV(synth_checkpoint(2, 128, vocab=257, seed=31))
    toks = t(g["tokens"])
    lg, s = m.forward(toks, m.emptyState.clone())
    assert torch.equal(lg, t(g["logits_seq"])) and torch.equal(s, t(g["state_seq"]))
    _, s = m.forward(toks[:5], m.emptyState.clone())
    lg, s = m.forward(toks[5:], s)
    assert torch.equal(lg, t(g["logits_chunk"])) and torch.equal(s, t(g["state_chunk"]))
    s = m.emptyState.clone()
    for i, tok in enumerate(toks):
        lg, s = m.forward(tok.reshape(1), s)
        assert torch.equal(lg, t(g["logits_tok"][i]))
    assert torch.equal(s, t(g["state_tok"]))
    # sequence mode and token-by-token agree to rounding (the RNN identity the CUDA path relies on)
    assert float((t(g["logits_seq"]) - t(g["logits_tok"][-1])).abs().max()) < 1e-5


def test_169m_greedy_stream(golden):
    g = golden("model_169m.npz")
    m = O.OracleRWKV(synth_checkpoint(12, 768, seed=int(g["seed"])))
    toks, rows, state = m.greedy(t(g["prompt"]), 64)
    assert toks.tolist() == g["tokens"].tolist()
    assert torch.allclose(rows[:, t(g["probe_idx"])], t(g["probe_logits"]), rtol=0, atol=1e-9)
    assert torch.allclose(rows[-1].float(), t(g["logits_last"]), rtol=0, atol=1e-6)
    assert torch.allclose(state, t(g["state"]), rtol=1e-9, atol=1e-9)


def test_two_axis_scheme_self_consistent():
    gen = torch.Generator().manual_seed(5)
    w = torch.randn(40, 24, generator=gen) * 0.02
    q, my, ry, mx, rx = O.two_axis_quantize(w)
    w_hat = (q.double() + 0.5) * ry[:, None] * rx[None, :] + my[:, None] + mx[None, :]
    # reconstruction error is bounded by half a quantisation step of the local scale
    step = (ry[:, None] * rx[None, :])
    assert float(((w_hat - w.double().t()).abs() / step).max()) <= 0.5 + 1e-6
    x = torch.randn(3, 24, generator=gen, dtype=torch.float64)
    assert torch.allclose(O.two_axis_mm8(x, q, my, ry, mx, rx), x @ w_hat)


@pytest.mark.parametrize("name,dtype", [("f32", torch.float32), ("bf16", torch.bfloat16), ("f16", torch.float16)])
def test_torch_mode_oracle_reproduces_the_reference(golden, name, dtype):
    """The unquantised (TORCH-mode) restatement against logits and states the reference's own
    loadWeights + AgnosticRWKV produced on CPU: same torch operators in the same order, so identical."""
    from oracle.torch_mode_oracle import OracleTorchMode
    from rwkvstic_b200.synth import synth_tokens
    g = golden("torch_mode.npz")
    for shape, (L, D, V, seed, n_tok) in {"tiny": (2, 128, 257, 31, 9), "mid": (3, 768, 1000, 32, 12)}.items():
        m = OracleTorchMode(synth_checkpoint(L, D, vocab=V, seed=seed), dtype)
        toks = synth_tokens(n_tok, seed=5, vocab=V)
        assert toks.tolist() == g[f"{shape}_tokens"].tolist()
        s = m.emptyState.clone()
        for i, tok in enumerate(toks):
            lg, s = m.forward(tok.reshape(1), s)
            assert torch.equal(lg, t(g[f"{shape}_{name}_logits_tok"][i])), (shape, i)
        assert torch.equal(s, t(g[f"{shape}_{name}_state_tok"]))
        if shape == "tiny":
            lg, s = m.forward(toks, m.emptyState.clone())
            assert torch.equal(lg, t(g[f"{shape}_{name}_logits_seq"])) and torch.equal(s, t(g[f"{shape}_{name}_state_seq"]))
