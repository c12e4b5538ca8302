"""Two-GPU layer split (one process per GPU, NCCL point-to-point handoff of the residual stream):
logits, generated ids and per-stage states must be bit-identical to the unsplit model on one GPU.
Skipped on a box with a single GPU."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from rwkvstic_b200 import layer_split as LS
from rwkvstic_b200.synth import synth_checkpoint, synth_tokens

pytestmark = pytest.mark.gpu
B, T, L = 6, 40, 4


def _checkpoint():
    return synth_checkpoint(L, 128, vocab=257, seed=31)


def _worker(rank, world, port, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    model = LS.build_stage(_checkpoint().items(), rank, world, L, dev)
    model.stage_stream_rows = 0                                        # first part: every item through the rows path
    pipe = LS.make_pipeline(model, rank, world, rows_per_item=64)      # 40 tokens x 3 streams -> pieces of 21 tokens
    toks = synth_tokens(B * T, seed=9, vocab=257).reshape(B, T)
    state = LS.empty_stage_state(model, B)
    logits = pipe.forward_rows(toks.to(dev), state, microbatches=2)
    ids = pipe.decode_greedy(torch.full((B, 1), 7), state, steps=3, microbatches=3)
    # second part: one stream, one token per step: every stage runs the one-row streaming step
    model.stage_stream_rows = 2
    state1 = LS.empty_stage_state(model, 1)
    before = model.launch_count
    ids1 = pipe.decode_greedy(torch.full((1, 1), 11), state1, steps=5)
    assert model.launch_count - before >= 5 * (model.launches_per_step - 2)      # the one-row launches, not the tile GEMM's
    torch.cuda.synchronize(dev)
    model.check_rows_status()
    model.check_status()
    torch.save({"logits": None if logits is None else logits.cpu(), "state": state.cpu(), "ids": ids.cpu(),
                "ids1": ids1.cpu(), "state1": state1.cpu()}, f"{out_path}.{rank}")
    dist.destroy_process_group()


def test_two_gpu_layer_split_equals_one_gpu(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from rwkvstic_b200.model import B200RWKV
    out = str(tmp_path / "out.pt")
    mp.spawn(_worker, args=(2, 29631, out), nprocs=2, join=True)
    r0, r1 = torch.load(out + ".0"), torch.load(out + ".1")
    full = B200RWKV.from_checkpoint(_checkpoint(), device="cuda:0")
    toks = synth_tokens(B * T, seed=9, vocab=257).reshape(B, T)
    state = full.empty_batch_state(B)
    want = full.forward_rows(toks, state)
    assert r0["logits"] is None and torch.equal(r1["logits"], want.cpu())
    tok = torch.full((B, 1), 7)
    ids = []
    for _ in range(3):
        tok = full.forward_rows(tok, state).argmax(dim=1, keepdim=True).cpu()
        ids.append(tok[:, 0])
    ids = torch.stack(ids, dim=1)
    assert torch.equal(r0["ids"], ids) and torch.equal(r1["ids"], ids)
    assert torch.equal(r0["state"], state[:, 0:2].cpu()) and torch.equal(r1["state"], state[:, 2:4].cpu())
    # one stream through the one-row stages against the unsplit one-row step
    st = full.emptyState.clone()
    tok, ids1 = torch.tensor([11]), []
    for _ in range(5):
        lg, st = full.forward(tok, st)
        tok = lg.argmax().reshape(1).cpu()
        ids1.append(int(tok))
    assert r0["ids1"].flatten().tolist() == ids1 and r1["ids1"].flatten().tolist() == ids1
    assert torch.equal(r0["state1"][0], st[0:2].cpu()) and torch.equal(r1["state1"][0], st[2:4].cpu())
