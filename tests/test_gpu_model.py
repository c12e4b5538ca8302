"""GPU parity tests of the whole decode path against the reference goldens."""
import numpy as np
import pytest
import torch

from rwkvstic_b200.model import B200RWKV
from rwkvstic_b200.synth import synth_checkpoint, synth_tokens

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 2e-3   # max |dlogit| against the reference's fp64-vector / fp32-matmul CPU path


def t64(a):
    return torch.from_numpy(np.asarray(a)).double()


@pytest.fixture(scope="module")
def tiny():
    return B200RWKV.from_checkpoint(synth_checkpoint(2, 128, vocab=257, seed=31), device=DEV)


@pytest.fixture(scope="module")
def m169():
    return B200RWKV.from_checkpoint(synth_checkpoint(12, 768, seed=1234), device=DEV)


def state_close(model, state, ref, rtol=1e-3, atol=1e-4):
    mine = model.to_reference_state(state).cpu()
    assert torch.allclose(mine[:, :4], t64(ref)[:, :4], rtol=rtol, atol=atol)


def test_tiny_sequence_chunk_and_token_modes(tiny, golden):
    g = golden("model_tiny.npz")
    toks = torch.from_numpy(g["tokens"])
    lg, st = tiny.forward(toks, tiny.emptyState.clone())
    assert float((lg.cpu().double() - t64(g["logits_seq"])).abs().max()) < TOL
    state_close(tiny, st, g["state_seq"])
    _, st = tiny.forward(toks[:5], tiny.emptyState.clone())
    lg, st = tiny.forward(toks[5:], st)
    assert float((lg.cpu().double() - t64(g["logits_chunk"])).abs().max()) < TOL
    st = tiny.emptyState.clone()
    for i, tok in enumerate(toks):
        lg, st2 = tiny.forward(tok.reshape(1), st)
        assert st2 is st                                   # updated in place like the reference
        assert float((lg.cpu().double() - t64(g["logits_tok"][i])).abs().max()) < TOL
    state_close(tiny, st, g["state_tok"])
    tiny.check_status()


def test_empty_state_matches_reference_layout(tiny):
    e = tiny.emptyState.cpu()
    assert tuple(e.shape) == (2, 5, 128) and bool((e[:, :4] == 0).all())
    assert bool((e[:, 4] == torch.tensor(-1e30, dtype=torch.float32)).all())


def test_graph_replay_equals_eager_and_is_deterministic(tiny):
    toks = synth_tokens(12, seed=3, vocab=257)
    eager = B200RWKV(tiny.w, use_graph=False)
    st_e, st_g = eager.emptyState.clone(), tiny.emptyState.clone()
    for tok in toks:                                       # same state buffer every step -> graph path
        le, _ = eager.forward(tok.reshape(1), st_e)
        lg, _ = tiny.forward(tok.reshape(1), st_g)
        assert torch.equal(le, lg)
    assert torch.equal(st_e, st_g)
    assert len(tiny._graphs) >= 1
    again = tiny.emptyState.clone()
    for tok in toks:
        l2, _ = tiny.forward(tok.reshape(1), again)
    assert torch.equal(l2, lg) and torch.equal(again, st_g)


def test_state_accepts_reference_dtype_and_device(tiny, golden):
    g = golden("model_tiny.npz")
    toks = torch.from_numpy(g["tokens"])
    st = tiny.emptyState.cpu().double()                    # what a reference user would hold
    lg, st2 = tiny.forward(toks, st)
    assert st2.dtype == torch.float32 and st2.device.type == "cuda"
    assert float((lg.cpu().double() - t64(g["logits_seq"])).abs().max()) < TOL


def test_batched_streams_equal_single_streams(tiny):
    toks = synth_tokens(3 * 4, seed=11, vocab=257).reshape(3, 4)
    stb = tiny.empty_batch_state(3)
    out, stb = tiny.forward_batch(toks.to(DEV), stb)
    for b in range(3):
        lg, st = tiny.forward(toks[b], tiny.emptyState.clone())
        assert torch.equal(lg, out[b]) and torch.equal(st, stb[b])


def test_169m_prompt_then_64_greedy_tokens(m169, golden):
    """The 169M shape (L=12, D=768, V=50277): 32 prompt tokens in sequence mode, 64 greedy steps, batch 1."""
    g = golden("model_169m.npz")
    probe = torch.from_numpy(g["probe_idx"]).to(DEV)
    state = m169.emptyState.clone()
    logits, state = m169.forward(torch.from_numpy(g["prompt"]), state)
    worst, toks = 0.0, []
    for i in range(64):
        tok = int(torch.argmax(logits))
        toks.append(tok)
        worst = max(worst, float((logits[probe].cpu().double() - t64(g["probe_logits"][i])).abs().max()))
        top = torch.from_numpy(g["top16_idx"][i]).to(DEV)
        worst = max(worst, float((logits[top].cpu().double() - t64(g["top16_val"][i])).abs().max()))
        logits, state = m169.forward(torch.tensor([tok]), state)
    assert toks == g["tokens"].tolist()
    assert worst < TOL, worst
    state_close(m169, state, g["state"], rtol=2e-3, atol=2e-4)
    m169.check_status()


def test_rejects_wrong_state_shape(tiny):
    with pytest.raises(ValueError):
        tiny.forward([1], torch.zeros(3, 5, 128))


def test_greedy_on_device_equals_host_argmax_loop(m169, golden):
    """The device-side arg-max feedback loop generates the reference's greedy tokens."""
    g = golden("model_169m.npz")
    state = m169.emptyState.clone()
    logits, state = m169.forward(torch.from_numpy(g["prompt"]), state)
    first = m169.argmax_token()
    assert int(first) == int(torch.argmax(logits)) == int(g["tokens"][0])
    st_graph, st_eager = state.clone(), state.clone()
    ids = m169.generate_greedy(int(first), st_graph, 63)
    assert [int(first)] + ids.cpu().tolist() == g["tokens"].tolist()
    eager = B200RWKV(m169.w, use_graph=False)
    ids2 = eager.generate_greedy(int(first), st_eager, 63)
    assert torch.equal(ids, ids2) and torch.equal(st_graph, st_eager)
    # host-driven loop with the arg-max on the device: same ids
    st_host = state.clone()
    tok, nxt = torch.tensor([int(first)]).pin_memory(), torch.zeros(1, dtype=torch.int64).pin_memory()
    host_ids = []
    for _ in range(6):
        m169.step_greedy(tok, st_host, nxt)
        torch.cuda.synchronize()
        host_ids.append(int(nxt[0]))
        tok[0] = int(nxt[0])
    assert host_ids == ids[:6].cpu().tolist()
    ties = torch.tensor([1.0, 5.0, 5.0, -2.0, 5.0], device=DEV)
    assert int(m169.argmax_token(ties)) == 1
    m169.check_status()
