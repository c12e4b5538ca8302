"""World-size-2 gloo run (CPU) of the data-parallel stream sharding: the shards tile the streams
exactly once and every stream's logits and state are bit-identical to the single-process run."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from rwkvstic_b200 import parallel
from rwkvstic_b200.model import quantize_tensors
from rwkvstic_b200.synth import synth_checkpoint, synth_tokens

from kernel_contract import ContractModel

B, T = 5, 3


def _build():
    wts = quantize_tensors(synth_checkpoint(2, 128, vocab=257, seed=31).items(), "cpu")
    model = ContractModel(wts)
    toks = synth_tokens(B * T, seed=9, vocab=257).reshape(B, T)
    state = model.emptyState.unsqueeze(0).repeat(B, 1, 1, 1).contiguous()
    return model, toks, state


def _worker(rank, world, port, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    model, toks, state = _build()
    shard, logits, st = parallel.decode_sharded(model, toks, state)
    full = parallel.gather_streams(shard, logits, B)
    states = parallel.gather_streams(shard, st, B)
    slowest = parallel.reduce_scalar(float(rank + 1), "max")
    total = parallel.reduce_scalar(float(len(shard)), "sum")
    if rank == 0:
        torch.save({"logits": torch.stack(full), "state": torch.stack(states), "slowest": slowest, "total": total}, out_path)
    dist.destroy_process_group()


def test_shards_tile_the_streams():
    for n in (1, 5, 256):
        for world in (1, 2, 3, 8):
            seen = [i for r in range(world) for i in parallel.stream_shard(n, world, r)]
            assert seen == list(range(n))
            sizes = [len(parallel.stream_shard(n, world, r)) for r in range(world)]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        parallel.stream_shard(4, 2, 2)


def test_two_rank_gloo_run_equals_single_process(tmp_path):
    out = str(tmp_path / "out.pt")
    mp.spawn(_worker, args=(2, 29611, out), nprocs=2, join=True)
    got = torch.load(out)
    model, toks, state = _build()
    for b in range(B):
        lg, st = model.forward(toks[b], state[b])
        assert torch.equal(got["logits"][b], lg) and torch.equal(got["state"][b], st)
    assert got["slowest"] == 2.0 and got["total"] == float(B)
