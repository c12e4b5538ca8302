"""Typical sampling: the CPU restatement against what the unmodified reference sampler draws from
(tests/golden/typical.npz), and on the GPU the sampling kernel against both."""
import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
from make_typical import CASES, case_logits  # noqa: E402

from oracle import typical_oracle as TO  # noqa: E402

DEV = "cuda:0"


def cases(golden):
    g = golden("typical.npz")
    assert np.array_equal(g["cases"], np.array(CASES, dtype=np.float64))
    for i, (vocab, seed, scale, temp, tau) in enumerate(CASES):
        x = case_logits(int(vocab), int(seed), scale)
        assert float(x.astype(np.float64).sum()) == float(g[f"check_{i}"]), "the seeded logits changed"
        kept = np.unpackbits(g[f"kept_{i}"])[:int(vocab)].astype(bool)
        assert int(kept.sum()) == int(g[f"count_{i}"])
        yield i, x, temp, tau, kept, float(g[f"sum_{i}"])


def test_oracle_keeps_what_the_reference_keeps(golden):
    exact = 0
    for i, x, temp, tau, kept, total in cases(golden):
        w = TO.typical_weights(x, temp, tau)
        _, shifted = TO.typical_shifted(x)
        assert TO.kept_sets_agree(kept, w > 0, shifted), f"case {i}"
        exact += int(np.array_equal(kept, w > 0))
        both = kept & (w > 0)
        assert abs(float(w[both].astype(np.float64).sum()) - total) <= 1e-4 * total + float(w[(w > 0) != kept].sum()) + 1e-4
    assert exact >= len(CASES) - 1


def test_oracle_draw_rule():
    w = np.array([0, 0.2, 0, 0.3, 0.5, 0], dtype=np.float32)
    assert [TO.draw(w, u) for u in (0.0, 0.19, 0.21, 0.5, 0.51, 0.999)] == [1, 1, 3, 3, 4, 4]
    assert TO.draw_bracket(w, 0.21, 3) and not TO.draw_bracket(w, 0.21, 2) and not TO.draw_bracket(w, 0.21, 4)


@pytest.mark.gpu
def test_kernel_keeps_what_the_reference_keeps_and_draws_by_inverse_cdf(golden):
    from rwkvstic_b200 import ops
    rng = np.random.default_rng(77)
    for i, x, temp, tau, kept, total in cases(golden):
        xs = torch.from_numpy(x).to(DEV)
        for u in [0.0, 0.5, float(rng.random()), float(rng.random()), 0.999999]:
            ut = torch.tensor([u], dtype=torch.float32, device=DEV)
            tok, probs = ops.sample_typical(xs, temp, tau, u=ut, return_probs=True)
            w = probs[0].cpu().numpy()
            _, shifted = TO.typical_shifted(x)
            assert TO.kept_sets_agree(kept, w > 0, shifted), f"case {i}"
            want = TO.typical_weights(x, temp, tau)
            both = (w > 0) & (want > 0)
            assert np.allclose(w[both], want[both], rtol=2e-5, atol=1e-12)
            t = int(tok[0])
            assert TO.draw_bracket(w, float(ut.item()), t), f"case {i} u={u} token {t}"


@pytest.mark.gpu
def test_kernel_rows_are_independent_deterministic_and_follow_the_distribution():
    from rwkvstic_b200 import ops
    V, rows = 50277, 64
    x = torch.from_numpy(case_logits(V, 21, 4.0)).to(DEV)
    big = torch.full((rows, V + 3), -7.0, device=DEV)           # padded row stride
    xs = big[:, :V]
    xs.copy_(x.expand(rows, V))
    xs[5] = torch.from_numpy(case_logits(V, 22, 2.0)).to(DEV)
    u = torch.rand(rows, device=DEV, generator=torch.Generator(device=DEV).manual_seed(3))
    a = ops.sample_typical(xs, 0.9, 0.9, u=u)
    assert torch.equal(a, ops.sample_typical(xs, 0.9, 0.9, u=u))
    for r in (0, 5, 63):
        assert int(ops.sample_typical(xs[r].contiguous(), 0.9, 0.9, u=u[r:r + 1])[0]) == int(a[r])
    # many draws from one row follow the weights the kernel reports
    n = 4096
    xr = x.expand(n, V).contiguous()
    un = torch.rand(n, device=DEV, generator=torch.Generator(device=DEV).manual_seed(4))
    toks, probs = ops.sample_typical(xr, 1.0, 0.9, u=un, return_probs=True)
    w = probs[0].double()
    w = (w / w.sum()).cpu().numpy()
    top = np.argsort(-w)[:5]
    freq = np.bincount(toks.cpu().numpy(), minlength=V) / n
    assert bool((w[toks.cpu().numpy()] > 0).all())
    for t in top:
        assert abs(freq[t] - w[t]) < 5 * np.sqrt(w[t] * (1 - w[t]) / n) + 1e-3
    # tau >= 1 keeps every token with a non-zero probability; a tiny tau keeps the most typical one
    _, p_all = ops.sample_typical(x, 1.0, 1.5, u=un[:1], return_probs=True)
    assert int((p_all > 0).sum()) == int((torch.softmax(x, 0) > 0).sum())
    _, p_one = ops.sample_typical(x, 1.0, 1e-6, u=un[:1], return_probs=True)
    assert int((p_one > 0).sum()) == 1


@pytest.mark.gpu
def test_generate_typical_is_reproducible_and_low_temperature_tau_follows_greedy():
    from rwkvstic_b200.model import B200RWKV
    from rwkvstic_b200.synth import synth_checkpoint
    m = B200RWKV.from_checkpoint(synth_checkpoint(2, 128, vocab=257, seed=31), device=DEV)
    runs = []
    for _ in range(2):
        st = m.empty_batch_state(1)[0]
        runs.append(m.generate_typical(7, st, 24, temp=1.0, tau=0.9, seed=11).cpu())
    assert torch.equal(runs[0], runs[1]) and int(runs[0].min()) >= 0 and int(runs[0].max()) < 257
    st = m.empty_batch_state(1)[0]
    other = m.generate_typical(7, st, 24, temp=1.0, tau=0.9, seed=12).cpu()
    assert not torch.equal(other, runs[0])
    # the host-driven loop with the same uniform numbers gives the same tokens as the graph loop
    st = m.empty_batch_state(1)[0]
    gen = torch.Generator(device=DEV)
    gen.manual_seed(11)
    u = torch.rand(24, device=DEV, generator=gen)
    tok, host = 7, []
    for i in range(24):
        logits, st = m.forward(torch.tensor([tok]), st)
        tok = int(ops_sample(logits, 1.0, 0.9, u[i:i + 1]))
        host.append(tok)
    assert host == runs[0].tolist()


def ops_sample(logits, temp, tau, u):
    from rwkvstic_b200 import ops
    return ops.sample_typical(logits.to(DEV).float().contiguous(), temp, tau, u=u)[0]


@pytest.mark.gpu
def test_backend_sample_hook_samples_gpu_logits_on_the_device():
    """The ops object registered in the reference's backend table carries ``sample``; what
    ``RWKVMaster.sample`` passes it (logits, temp, top_p_usual) must give a kept token."""
    from rwkvstic_b200.backend import make_ops_class

    class Base:                                    # stands in for agnostic.backends.base.module
        def __init__(self, layers, embed, *a, **k):
            pass

    ops_obj = make_ops_class(Base)(2, 128)
    x = case_logits(50277, 5, 3.0)
    want = TO.typical_weights(x, 1.0, 0.8) > 0
    seen = {ops_obj.sample(torch.from_numpy(x).to(DEV), 1.0, 0.8) for _ in range(16)}
    assert all(isinstance(t, int) and want[t] for t in seen) and len(seen) > 1
