"""The .rwkv harvester against an archive written by the reference's own exporter
(tests/golden/model_tiny.rwkv, made by tests/golden/make_rwkv_archive.py)."""
import os

import numpy as np
import pytest
import torch

from rwkvstic_b200 import rwkv_archive
from rwkvstic_b200.model import quantize_tensors
from rwkvstic_b200.synth import synth_checkpoint

from kernel_contract import ContractModel

ARCHIVE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "model_tiny.rwkv")


def test_harvested_tensors_equal_own_quantisation_of_the_checkpoint():
    got = rwkv_archive.harvest(ARCHIVE, "cpu")
    want = quantize_tensors(synth_checkpoint(2, 128, vocab=257, seed=31).items(), "cpu")
    assert (got.n_layer, got.n_embd, got.n_ffn, got.n_vocab) == (2, 128, 512, 257)
    assert torch.equal(got.emb, want.emb) and torch.equal(got.head.qt, want.head.qt)
    assert torch.equal(got.head.ry, want.head.ry) and torch.equal(got.head.my64, want.head.my64)
    for a, b in zip(got.layers, want.layers):
        for k in b.mat:
            assert torch.equal(a.mat[k].qt, b.mat[k].qt), k
            assert torch.equal(a.mat[k].ry, b.mat[k].ry) and torch.equal(a.mat[k].my64, b.mat[k].my64), k
        for k in b.vec:
            assert torch.equal(a.vec[k], b.vec[k]), k
    for a, b in zip(got.ln0 + got.ln_out, want.ln0 + want.ln_out):
        assert torch.equal(a, b)


def test_harvested_model_reproduces_reference_logits_on_cpu_contract(golden):
    g = golden("model_tiny.npz")
    model = ContractModel(rwkv_archive.harvest(ARCHIVE, "cpu"))
    lg, _ = model.forward(torch.from_numpy(g["tokens"]), model.emptyState.clone())
    assert float((lg.double() - torch.from_numpy(g["logits_tok"][-1])).abs().max()) < 2e-3


def test_archive_runs_as_written_and_shards_concatenate():
    m = torch.jit.load(ARCHIVE, map_location="cpu")
    # the archive is self-contained TorchScript: it runs here without the reference installed
    lg, _ = m.forward(torch.tensor([3, 4], dtype=torch.int64), m.emptyState.clone())
    assert tuple(lg.shape) == (257,)

    class Shard:                      # two input-dimension shards of one matrix, as a 2-device export holds them
        def __init__(self, w, r, o):
            self.weight, self.range, self.offset = w, r, o
    full = rwkv_archive.harvest(m, "cpu").head
    kin = full.k_in // 2
    w = full.qt.t().contiguous()
    parts = [Shard(w[:kin], full.ry[:kin], full.my64[:kin]), Shard(w[kin:], full.ry[kin:], full.my64[kin:])]
    again = rwkv_archive._matrix(parts, "", torch.device("cpu"))
    assert torch.equal(again.qt, full.qt) and torch.equal(again.ry, full.ry) and torch.equal(again.my64, full.my64)
    with pytest.raises(ValueError):
        rwkv_archive._matrix([Shard(w.float(), full.ry, full.my64)], "", torch.device("cpu"))


@pytest.mark.gpu
def test_archive_on_the_gpu_matches_reference_goldens(golden):
    g = golden("model_tiny.npz")
    model = rwkv_archive.load(ARCHIVE, "cuda:0")
    toks = torch.from_numpy(g["tokens"])
    st = model.emptyState.clone()
    for i, tok in enumerate(toks):
        lg, st = model.forward(tok.reshape(1), st)
        assert float((lg.cpu().double() - torch.from_numpy(np.asarray(g["logits_tok"][i]))).abs().max()) < 2e-3
    model.check_status()


def test_export_round_trip_and_scripted_forward(tmp_path, golden):
    g = golden("model_tiny.npz")
    w = quantize_tensors(synth_checkpoint(2, 128, vocab=257, seed=31).items(), "cpu")
    path = rwkv_archive.export(w, str(tmp_path / "tiny"))
    assert path.endswith(".rwkv")
    m = torch.jit.load(path, map_location="cpu")
    # the archive runs by itself (what stock rwkvstic does with it) and reproduces the reference's numbers
    toks = torch.from_numpy(g["tokens"])
    lg, st = m.forward(toks, m.emptyState.clone())
    assert float((lg - torch.from_numpy(g["logits_seq"])).abs().max()) < 1e-5
    assert torch.allclose(st[:, :4], torch.from_numpy(g["state_seq"])[:, :4], rtol=1e-4, atol=1e-6)
    st = m.emptyState.clone()
    for i, tok in enumerate(toks):
        lg, st = m.forward(tok.reshape(1), st)
        assert float((lg - torch.from_numpy(np.asarray(g["logits_tok"][i]))).abs().max()) < 1e-5
    # and the harvester reads it back bit-identically
    back = rwkv_archive.harvest(path, "cpu")
    assert torch.equal(back.emb, w.emb) and torch.equal(back.head.qt, w.head.qt) and torch.equal(back.head.my64, w.head.my64)
    for a, b in zip(back.layers, w.layers):
        for k in b.mat:
            assert torch.equal(a.mat[k].qt, b.mat[k].qt) and torch.equal(a.mat[k].ry, b.mat[k].ry), k
        for k in b.vec:
            assert torch.equal(a.vec[k], b.vec[k]), k
    with pytest.raises(ValueError):
        from rwkvstic_b200.quant import quantize_two_axis
        w.layers[0].mat["att.key"] = quantize_two_axis(torch.randn(128, 128))
        rwkv_archive.export(w, str(tmp_path / "bad"))
