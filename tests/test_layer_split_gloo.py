"""Layer split on CPU: block partition, work-item schedule, and a world-size-2 gloo pipeline whose
stages run the CPU statement of the kernels' arithmetic; the result must be bit-identical to the
unsplit model for every micro-batch count and token-piece size."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from rwkvstic_b200 import layer_split as LS
from rwkvstic_b200.model import quantize_tensors
from rwkvstic_b200.synth import synth_checkpoint, synth_tokens

from kernel_contract import ContractModel

B, T, L = 4, 6, 4


def _checkpoint():
    return synth_checkpoint(L, 128, vocab=257, seed=31)


def test_split_layers_is_contiguous_and_balanced():
    for n, world in ((40, 8), (40, 3), (32, 2), (5, 5), (12, 1)):
        parts = LS.split_layers(n, world)
        assert parts[0][0] == 0 and parts[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(parts, parts[1:]))
        sizes = [b - a for a, b in parts]
        assert max(sizes) - min(sizes) <= 1 and min(sizes) >= 1
    with pytest.raises(ValueError):
        LS.split_layers(3, 4)


def test_work_items_cover_every_row_once_in_state_order():
    for Bn, Tn, mb, piece in ((4, 6, 2, 4), (5, 1, 3, 1), (1, 10, 4, 3), (64, 1, 4, 64)):
        items = LS.work_items(Bn, Tn, mb, piece)
        seen = torch.zeros(Bn, Tn, dtype=torch.int32)
        last_t = {}
        for (b0, b1, t0, t1) in items:
            seen[b0:b1, t0:t1] += 1
            for b in range(b0, b1):
                assert last_t.get(b, 0) == t0          # a stream's pieces arrive in time order
                last_t[b] = t1
        assert bool((seen == 1).all())


def test_stage_weights_hold_only_their_blocks():
    ck = _checkpoint()
    parts = LS.split_layers(L, 2)
    w0 = quantize_tensors(ck.items(), "cpu", layer_range=parts[0], keep_emb=True, keep_head=False)
    w1 = quantize_tensors(ck.items(), "cpu", layer_range=parts[1], keep_emb=False, keep_head=True)
    full = quantize_tensors(ck.items(), "cpu")
    assert (w0.n_layer, w0.first_layer, w1.n_layer, w1.first_layer) == (2, 0, 2, 2)
    assert w0.head is None and w1.emb is None and w0.n_vocab == w1.n_vocab == 257
    assert torch.equal(w1.layers[0].mat["ffn.key"].qt, full.layers[2].mat["ffn.key"].qt)
    assert torch.equal(w0.layers[1].vec["att.time_decay"], full.layers[1].vec["att.time_decay"])


def _worker(rank, world, port, out_path, microbatches, rows_per_item):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    l0, l1 = LS.split_layers(L, world)[rank]
    w = quantize_tensors(_checkpoint().items(), "cpu", layer_range=(l0, l1), keep_emb=rank == 0, keep_head=rank == world - 1)
    model = ContractModel(w)
    pipe = LS.LayerSplitPipeline(model.stage, w.n_embd, w.n_vocab, rank, world, "cpu", rows_per_item=rows_per_item)
    toks = synth_tokens(B * T, seed=9, vocab=257).reshape(B, T)
    state = model.emptyState.unsqueeze(0).repeat(B, 1, 1, 1).contiguous()
    logits = pipe.forward_rows(toks, state, microbatches)
    ids = pipe.decode_greedy(torch.full((B, 1), 7), state, steps=2, microbatches=microbatches)
    torch.save({"logits": logits, "state": state, "ids": ids, "range": (l0, l1)}, f"{out_path}.{rank}")
    dist.destroy_process_group()


@pytest.mark.parametrize("microbatches,rows_per_item,port", [(1, 4096, 29621), (2, 4, 29623)])
def test_two_rank_pipeline_equals_unsplit_model(tmp_path, microbatches, rows_per_item, port):
    out = str(tmp_path / "out.pt")
    mp.spawn(_worker, args=(2, port, out, microbatches, rows_per_item), nprocs=2, join=True)
    r0, r1 = torch.load(out + ".0"), torch.load(out + ".1")
    full = ContractModel(quantize_tensors(_checkpoint().items(), "cpu"))
    toks = synth_tokens(B * T, seed=9, vocab=257).reshape(B, T)
    state = full.emptyState.unsqueeze(0).repeat(B, 1, 1, 1).contiguous()
    want = torch.stack([full.forward(toks[b], state[b])[0] for b in range(B)])
    assert r0["logits"] is None and torch.equal(r1["logits"], want)
    ids = torch.empty(B, 2, dtype=torch.int64)
    tok = torch.full((B,), 7)
    for i in range(2):
        lg = torch.stack([full.forward(tok[b:b + 1], state[b])[0] for b in range(B)])
        tok = lg.argmax(dim=1)
        ids[:, i] = tok
    assert torch.equal(r0["ids"], ids) and torch.equal(r1["ids"], ids)
    # each rank carried the state of its own blocks only
    assert torch.equal(r0["state"], state[:, 0:2]) and torch.equal(r1["state"], state[:, 2:4])
