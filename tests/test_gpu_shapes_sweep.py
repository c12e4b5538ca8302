"""Seeded sweep over small shapes: layers, width, vocabulary, streams and tokens per stream drawn from lists
that include the edges (one stream, one token, odd vocabularies, the WKV scan's chunk boundary at 128 / 129
tokens); both models, the rows path and the one-row path, against their CPU oracles."""
import random

import pytest
import torch

from oracle.fastquant_oracle import OracleRWKV
from oracle.torch_mode_oracle import OracleTorchMode
from rwkvstic_b200.dense_model import B200DenseRWKV
from rwkvstic_b200.model import B200RWKV
from rwkvstic_b200.synth import synth_checkpoint, synth_tokens

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("case", range(10))
def test_random_shape_against_the_oracles(case):
    rng = random.Random(1000 + case)
    L, D, V = rng.choice([1, 2, 3]), rng.choice([128, 256, 384, 512, 768]), rng.choice([97, 257, 300, 1000])
    B, T = rng.choice([1, 2, 3, 5, 8, 17]), rng.choice([1, 2, 3, 7, 16, 33, 64, 127, 128, 129, 200])
    T = min(T, max(1, 1500 // B))
    dt = rng.choice([torch.bfloat16, torch.float16])
    tol = 4 * 2.0 ** -8 if dt == torch.bfloat16 else 4 * 2.0 ** -11
    ck = synth_checkpoint(L, D, vocab=V, seed=100 + case)
    toks = synth_tokens(B * T, seed=case, vocab=V).reshape(B, T)
    ref, dref = OracleRWKV(ck), OracleTorchMode(ck, dt)
    quant = B200RWKV.from_checkpoint(ck, device=DEV, use_graph=False)
    dense = B200DenseRWKV.from_checkpoint(ck, dtype=dt, device=DEV, use_graph=False)
    qout = quant.forward_rows(toks.to(DEV), quant.empty_batch_state(B))
    dout = dense.forward_rows(toks.to(DEV), dense.empty_batch_state(B))
    quant.check_rows_status()
    dense.check_status()
    for b in range(min(B, 3)):
        want, _ = ref.forward(toks[b], ref.emptyState.clone())
        assert float((qout[b].cpu().double() - want).abs().max()) < 2e-3, (L, D, V, B, T, b)
        dwant, _ = dref.forward(toks[b], dref.emptyState.clone())
        assert float((dout[b].cpu() - dwant).abs().max()) <= tol * float(dwant.abs().max()), (L, D, V, B, T, b, dt)
    head = toks[0][:3]
    qs, ds = quant.emptyState.clone(), dense.emptyState.clone()
    for t in head:
        q1, _ = quant.forward(t.reshape(1), qs)
        d1, _ = dense.forward(t.reshape(1), ds)
    want, _ = ref.forward(head, ref.emptyState.clone())
    dwant, _ = dref.forward(head, dref.emptyState.clone())
    assert float((q1.cpu().double() - want).abs().max()) < 2e-3
    assert float((d1.cpu() - dwant).abs().max()) <= tol * float(dwant.abs().max())
