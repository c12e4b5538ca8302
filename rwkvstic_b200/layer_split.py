"""Layer split: the blocks of one model partitioned contiguously over several GPUs.

One process per GPU (``torch.distributed``).  Rank r holds blocks ``split_layers(L, world)[r]``
and the recurrent state of those blocks only; rank 0 also holds the embedding and ln0, the last
rank ln_out and the head.  This is the placement the reference's TORCH_SPLIT strategy describes
(whole layers live on a device and the ``1 x D`` activation moves between devices) and what its
in-tree multi-device code does with tensors (``.to(device)`` hops on the default stream,
modules/matmul.py:154-163); here the hop is a point-to-point send of the residual stream
``x [rows, D]`` over NCCL (NVLink), and nothing else crosses GPUs: no collective, no state traffic.

With a single work item only one GPU would be busy at a time, so a call is cut into work items
that flow through the stages as a pipeline: the streams are cut into ``microbatches`` groups and
long prompts into token pieces.  Every stage handles the items in the same order
(receive -> compute -> send); the sends and receives are asynchronous on the CUDA stream, so stage
r works on item i+1 while stage r+1 works on item i.  Items of one stream group are dependent
through the state and stay in order on every stage.

Decode steps are bound by streaming the stage's weights, and every stream group streams them
again, so ``microbatches=1`` is the fastest setting for decode (measured at the 14B shape, 64
streams, 2 GPUs: 8.8 / 11.7 / 19.0 ms per step with 1 / 2 / 4 groups); prompts are compute-bound
and their token pieces do overlap across the stages.  The split buys capacity, not decode speed: a
decode step is a chain through all stages, and a model that fits one GPU decodes as fast there.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def split_layers(n_layer: int, world: int) -> List[Tuple[int, int]]:
    """Contiguous block ranges per rank; sizes differ by at most one (earlier ranks get the extra)."""
    if world < 1 or n_layer < world:
        raise ValueError(f"cannot split {n_layer} layers over {world} ranks")
    base, extra = divmod(n_layer, world)
    out, l0 = [], 0
    for r in range(world):
        n = base + (1 if r < extra else 0)
        out.append((l0, l0 + n))
        l0 += n
    return out


def work_items(B: int, T: int, microbatches: int, tokens_per_piece: int) -> List[Tuple[int, int, int, int]]:
    """(b0, b1, t0, t1) in processing order: token pieces outermost, stream groups inside."""
    microbatches = max(1, min(microbatches, B))
    bounds = [B * i // microbatches for i in range(microbatches + 1)]
    items = []
    for t0 in range(0, T, tokens_per_piece):
        t1 = min(T, t0 + tokens_per_piece)
        for i in range(microbatches):
            if bounds[i + 1] > bounds[i]:
                items.append((bounds[i], bounds[i + 1], t0, t1))
    return items


StageFn = Callable[[Optional[torch.Tensor], torch.Tensor, torch.Tensor, bool], Optional[torch.Tensor]]


class LayerSplitPipeline:
    """The host-side schedule of one rank.  ``stage_fn(tokens | None, x, state, want_logits)`` runs
    this rank's blocks on ``x [rows, D]`` in place and returns logits ``[streams, V]`` when asked
    (``B200RWKV.forward_rows_stage`` on the GPU; the CPU tests pass a stand-in)."""

    def __init__(self, stage_fn: StageFn, n_embd: int, n_vocab: int, rank: int, world: int, device,
                 group=None, rows_per_item: int = 4096):
        self.stage_fn, self.n_embd, self.n_vocab = stage_fn, n_embd, n_vocab
        self.rank, self.world, self.device, self.group = rank, world, torch.device(device), group
        self.rows_per_item = rows_per_item
        self.first, self.last = rank == 0, rank == world - 1

    def forward_rows(self, tokens: torch.Tensor, state: torch.Tensor, microbatches: int = 1) -> Optional[torch.Tensor]:
        """``tokens [B,T]`` (read on rank 0 only, but every rank must pass the same shape),
        ``state [B, L_stage, 5, D]`` of this rank's blocks, updated in place.  Returns the logits
        ``[B,V]`` after each stream's last token on the last rank, None elsewhere."""
        B, T = tokens.shape
        mb = max(1, min(microbatches, B))
        per_group = -(-B // mb)
        piece = max(1, self.rows_per_item // per_group)
        items = work_items(B, T, mb, piece)
        logits = torch.empty(B, self.n_vocab, dtype=torch.float32, device=self.device) if self.last else None
        keep = []   # sends in flight: (request, buffer) stay referenced until the call returns
        for (b0, b1, t0, t1) in items:
            rows = (b1 - b0) * (t1 - t0)
            x = torch.empty(rows, self.n_embd, dtype=torch.float32, device=self.device)
            if not self.first:
                # batched point-to-point ops: NCCL runs them on their own channel instead of
                # serialising them with the group's collectives; wait() orders the stream, not the host
                for req in dist.batch_isend_irecv([dist.P2POp(dist.irecv, x, self.rank - 1, group=self.group)]):
                    req.wait()
            toks = tokens[b0:b1, t0:t1] if self.first else None
            want = self.last and t1 == T
            out = self.stage_fn(toks, x, state[b0:b1], want)
            if want:
                logits[b0:b1] = out
            if not self.last:
                keep.append((dist.batch_isend_irecv([dist.P2POp(dist.isend, x, self.rank + 1, group=self.group)]), x))
        for reqs, _ in keep:
            for req in reqs:
                req.wait()
        return logits

    def decode_greedy(self, tokens: torch.Tensor, state: torch.Tensor, steps: int, microbatches: int = 1) -> Optional[torch.Tensor]:
        """``steps`` greedy decode steps for B streams starting from ``tokens [B,1]``.  The sampled ids
        travel from the last rank straight to the first one (the only rank that reads token ids) as a
        point-to-point message of B integers per step, stream-ordered like the hand-off of the residual:
        no collective, and the ranks in between never wait for them.  Returns the generated ids
        ``[B, steps]`` on the first and the last rank, None on the others."""
        B = tokens.shape[0]
        tok = tokens.to(self.device).reshape(B, 1).clone()
        out = torch.empty(B, steps, dtype=torch.int64, device=self.device) if (self.first or self.last) else None
        keep = []
        for i in range(steps):
            lg = self.forward_rows(tok, state, microbatches)
            if self.last:
                tok = lg.argmax(dim=1, keepdim=True)
                out[:, i] = tok[:, 0]
                if not self.first:
                    keep.append((dist.batch_isend_irecv([dist.P2POp(dist.isend, tok, 0, group=self.group)]), tok))
            elif self.first:
                tok = torch.empty(B, 1, dtype=torch.int64, device=self.device)
                for req in dist.batch_isend_irecv([dist.P2POp(dist.irecv, tok, self.world - 1, group=self.group)]):
                    req.wait()
                out[:, i] = tok[:, 0]
        for reqs, _ in keep:
            for req in reqs:
                req.wait()
        return out


def build_stage(tensors, rank: int, world: int, n_layer: int, device, scheme: str = "fastquant"):
    """This rank's ``B200RWKV`` (its blocks only) from an iterable of (name, tensor) pairs of the
    whole checkpoint; tensors of other stages are skipped as they stream by."""
    from .model import B200RWKV, quantize_tensors
    l0, l1 = split_layers(n_layer, world)[rank]
    w = quantize_tensors(tensors, device, scheme, layer_range=(l0, l1), keep_emb=rank == 0, keep_head=rank == world - 1)
    return B200RWKV(w, use_graph=False)


def make_pipeline(model, rank: int, world: int, group=None, rows_per_item: int = 4096) -> LayerSplitPipeline:
    return LayerSplitPipeline(model.forward_rows_stage, model.n_embd, model.n_vocab, rank, world, model.device,
                              group=group, rows_per_item=rows_per_item)


def empty_stage_state(model, B: int) -> torch.Tensor:
    """``[B, L_stage, 5, D]`` empty state of the blocks this rank holds."""
    return model.empty_batch_state(B)
