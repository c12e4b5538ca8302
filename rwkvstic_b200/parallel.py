"""Data-parallel decode of independent streams: one process per GPU, no collective on the data path.

RWKV streams never interact (each has its own ``[L,5,D]`` state), so B streams are split into
contiguous shards, every rank decodes its shard on a full replica of the weights, and only
bookkeeping (timing, gathering results) crosses ranks.  Works with the ``nccl`` backend on GPUs
and ``gloo`` on CPUs (tests).
"""
from __future__ import annotations

import os
from typing import List, Sequence

import torch
import torch.distributed as dist


def stream_shard(n_streams: int, world: int, rank: int) -> range:
    """Contiguous, balanced shard of ``range(n_streams)`` for ``rank`` (sizes differ by at most 1)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    return range(n_streams * rank // world, n_streams * (rank + 1) // world)


def env_rank_world() -> tuple:
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))


def reduce_scalar(value: float, op: str = "max", device="cpu") -> float:
    """max / sum of a python float over all ranks (identity when not initialised)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX if op == "max" else dist.ReduceOp.SUM)
    return float(t[0])


def decode_sharded(model, tokens: torch.Tensor, state: torch.Tensor, steps_fn=None):
    """Run ``model.forward`` on this rank's shard of ``tokens [B,T]`` / ``state [B,L,5,D]``.

    Returns ``(shard_range, logits [b,V], state_shard)``.  ``state`` is updated in place for the
    shard rows only; other rows are left untouched (they belong to other ranks)."""
    rank, world = (dist.get_rank(), dist.get_world_size()) if dist.is_initialized() else (0, 1)
    shard = stream_shard(tokens.shape[0], world, rank)
    if hasattr(model, "forward_batch") and len(shard) > 0:
        # the GPU model applies every matrix to all rows of the shard at once (tensor-core rows path)
        view = state[shard.start:shard.stop]
        lg, _ = model.forward_batch(tokens[shard.start:shard.stop], view)
        return shard, lg, view
    outs = []
    for b in shard:
        lg, _ = model.forward(tokens[b], state[b])
        outs.append(lg.clone() if torch.is_tensor(lg) else lg)
    return shard, (torch.stack(outs) if outs else torch.empty(0)), state[shard.start:shard.stop]


def gather_streams(shard: range, values: torch.Tensor, n_streams: int) -> List[torch.Tensor]:
    """All ranks contribute their shard's rows; every rank gets the full list in stream order."""
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return list(values)
    parts: List = [None] * dist.get_world_size()
    dist.all_gather_object(parts, (shard.start, values.cpu()))
    out: List = [None] * n_streams
    for start, vals in parts:
        for i, v in enumerate(vals):
            out[start + i] = v
    return out
