"""Host logic of the session batcher on CPU: slot bookkeeping (packing, moves on close, capacity), state
hand-over, with a stand-in model whose rows are independent by construction."""
import pytest
import torch

from rwkvstic_b200 import ops
from rwkvstic_b200.sessions import SessionBatch


class FakeModel:
    """forward_rows on CPU: state row 0 accumulates the tokens seen, the logits put their peak at
    (sum of tokens + count) mod V, so every stream's continuation depends only on its own history."""
    n_vocab = 17

    def __init__(self):
        self.emptyState = torch.zeros(2, 5, 4)
        self.calls = []

    def forward_rows(self, tokens, state):
        B, T = tokens.shape
        self.calls.append((B, T))
        out = torch.zeros(B, self.n_vocab)
        for b in range(B):
            for t in range(T):
                state[b, 0, 0, 0] += float(tokens[b, t])
                state[b, 0, 0, 1] += 1.0
            out[b, int(state[b, 0, 0, 0] + state[b, 0, 0, 1]) % self.n_vocab] = 1.0
        return out


@pytest.fixture(autouse=True)
def cpu_argmax(monkeypatch):
    monkeypatch.setattr(ops, "argmax_rows", lambda lg: torch.argmax(lg, dim=1))


def alone(prompt, steps):
    b = SessionBatch(FakeModel(), capacity=1)
    s = b.open()
    b.feed(s, prompt)
    return [b.step(greedy=True)[s] for _ in range(steps)]


def test_slots_stay_packed_and_streams_independent():
    model = FakeModel()
    batch = SessionBatch(model, capacity=3)
    assert batch.step() == {}
    a, b = batch.open(), batch.open()
    with pytest.raises(RuntimeError):
        batch.step(greedy=True)                       # nothing fed yet
    batch.feed(a, [3, 4]); batch.feed(b, [5])
    got = {a: [], b: []}
    for _ in range(2):
        out = batch.step(greedy=True)
        for k, v in out.items():
            got[k].append(v)
    assert model.calls[-1] == (2, 1)                  # one rows call for both sessions
    c = batch.open(); batch.feed(c, [1, 1, 1]); got[c] = []
    with pytest.raises(RuntimeError):
        batch.open()
    batch.close(a)                                    # c (last slot) moves into a's slot
    assert batch.n == 2 and batch.slot_of == {b: 1, c: 0} and batch.sid_at[:3] == [c, b, None]
    for _ in range(3):
        out = batch.step(greedy=True)
        assert set(out) == {b, c}
        for k, v in out.items():
            got[k].append(v)
    assert got[a] == alone([3, 4], 2) and got[b] == alone([5], 5) and got[c] == alone([1, 1, 1], 3)
    d = batch.open(state=batch.state_lists(b))        # a copy of b's state as lists: same continuation once fed alike
    assert torch.equal(batch.state_tensor(d), batch.state_tensor(b))
    batch.close(b); batch.close(c); batch.close(d)
    assert batch.n == 0 and not batch.slot_of
    with pytest.raises(ValueError):
        batch.open(state=[[0.0]])
    with pytest.raises(ValueError):
        SessionBatch(model, capacity=0)
