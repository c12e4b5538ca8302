"""Independent sessions decoded together on the batched-stream kernels.

The reference's server answers one request at a time: the body carries a state as nested JSON lists
(or none), optionally an ``input`` text that goes through ``loadContext``, then ``forward`` samples a
few tokens, and state and logits go back as lists (server.py:59-86; the session calls are
rwkvMaster.py:28-125).  Requests of different clients are independent streams, which is exactly what
``forward_rows`` takes: B states, one token each per step.  ``SessionBatch`` keeps the states of all
open sessions in one device buffer ``[capacity, L, 5, D]`` with the open ones packed at the front (a
closed session's slot is refilled by moving the last open one into it), so that every decode step is
ONE rows call over ``pool[:n]`` without gathering or scattering states:

    batch = SessionBatch(model, capacity=256)
    a = batch.open()                        # fresh state;  batch.open(state=body["state"]) resumes one
    batch.feed(a, tokens)                   # prompt (loadContext): this session's rows through the model
    out = batch.step(temp=1.0, tau=0.8)     # every open session samples its next token and advances: {sid: token}
    body = batch.state_lists(a)             # what the server writes back: state as lists
    batch.close(a)

Works with ``B200RWKV`` (FASTQUANT) and ``B200DenseRWKV`` (unquantised, bf16 / fp16) alike: both offer
``forward_rows(tokens [B,T], state [B,L,5,D]) -> logits [B,V]`` and ``emptyState``.  A row's result does
not depend on which other rows share the call (the quantised path's dot products are exact integer
sums), so a session's token stream is the same whether it runs alone or packed with others.
No network code lives here; an HTTP handler only has to map requests onto these calls.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch


class SessionBatch:
    def __init__(self, model, capacity: int = 256):
        if capacity < 1:
            raise ValueError("capacity must be at least 1")
        self.model = model
        self.capacity = capacity
        empty = model.emptyState
        self.device = empty.device
        self.pool = empty.unsqueeze(0).repeat(capacity, 1, 1, 1).contiguous()      # [capacity, L, 5, D]
        self.logits = torch.zeros(capacity, model.n_vocab, dtype=torch.float32, device=self.device)
        self.has_logits: List[bool] = [False] * capacity
        self.slot_of: Dict[int, int] = {}          # session id -> slot
        self.sid_at: List[Optional[int]] = [None] * capacity
        self.n = 0                                 # open sessions = slots [0, n)
        self._next_sid = 1

    # ------------------------------------------------------------------ state in and out
    def _to_model_state(self, state) -> torch.Tensor:
        """A state as the reference's clients hold it (nested lists or a tensor ``[L,5,D]`` in the reference's
        convention, server.py:66-67) -> this model's own layout."""
        t = torch.as_tensor(state, dtype=torch.float32)
        if tuple(t.shape) != tuple(self.model.emptyState.shape):
            raise ValueError(f"state must have shape {tuple(self.model.emptyState.shape)}, got {tuple(t.shape)}")
        conv = getattr(self.model, "from_reference_state", None)
        return conv(t) if conv is not None else t.to(self.device)

    def state_tensor(self, sid: int) -> torch.Tensor:
        """The session's state in the reference's convention (a copy)."""
        s = self.pool[self.slot_of[sid]]
        conv = getattr(self.model, "to_reference_state", None)
        return conv(s) if conv is not None else s.clone()

    def state_lists(self, sid: int) -> list:
        """The state as the server sends it: one list per block (server.py:75-76)."""
        return [x.cpu().float().numpy().tolist() for x in self.state_tensor(sid)]

    # ------------------------------------------------------------------ sessions
    def open(self, state=None) -> int:
        if self.n == self.capacity:
            raise RuntimeError(f"all {self.capacity} session slots are in use")
        slot, sid = self.n, self._next_sid
        self._next_sid += 1
        self.pool[slot].copy_(self.model.emptyState if state is None else self._to_model_state(state))
        self.has_logits[slot] = False
        self.slot_of[sid], self.sid_at[slot] = slot, sid
        self.n += 1
        return sid

    def close(self, sid: int) -> None:
        slot = self.slot_of.pop(sid)
        last = self.n - 1
        if slot != last:                           # keep the open sessions packed: the last one moves into the hole
            self.pool[slot].copy_(self.pool[last])
            self.logits[slot].copy_(self.logits[last])
            self.has_logits[slot] = self.has_logits[last]
            moved = self.sid_at[last]
            self.sid_at[slot], self.slot_of[moved] = moved, slot
        self.sid_at[last], self.has_logits[last] = None, False
        self.n = last

    def feed(self, sid: int, tokens: Sequence[int]) -> None:
        """Run ``tokens`` through the model on this session's state (rwkvMaster.py:58-105, loadContext);
        the logits after the last one are kept for the next ``step``."""
        toks = torch.as_tensor(tokens, dtype=torch.int64).reshape(1, -1)
        if toks.numel() == 0:
            raise ValueError("feed needs at least one token")
        slot = self.slot_of[sid]
        out = self.model.forward_rows(toks.to(self.device), self.pool[slot:slot + 1])
        self.logits[slot].copy_(out[0])
        self.has_logits[slot] = True

    def step(self, temp: float = 1.0, tau: float = 0.8, greedy: bool = False, generator: Optional[torch.Generator] = None) -> Dict[int, int]:
        """Every open session draws its next token from its pending logits (typical sampling on the
        device, samplers/typical.py:1-17, or arg-max) and takes one decode step; all of them in one rows
        call.  Returns ``{session id: sampled token}``."""
        n = self.n
        if n == 0:
            return {}
        missing = [self.sid_at[i] for i in range(n) if not self.has_logits[i]]
        if missing:
            raise RuntimeError(f"sessions {missing} have no logits yet: feed them at least one token first")
        lg = self.logits[:n]
        from . import ops
        toks = ops.argmax_rows(lg) if greedy else ops.sample_typical(lg, temp, tau, generator=generator)
        out = self.model.forward_rows(toks.reshape(n, 1), self.pool[:n])
        self.logits[:n].copy_(out)
        host = toks.cpu().tolist()                  # the only device -> host transfer of the step: n ids
        return {self.sid_at[i]: int(host[i]) for i in range(n)}
