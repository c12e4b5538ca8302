"""The ops-object boundary driven by the REFERENCE's own loader and session code.

Needs the reference checkout (only present where the goldens were generated); skipped elsewhere.
The GPU model is replaced by the CPU contract model through ``install(model_factory=...)``, so the
whole plumbing - Backends table, loadWeights, AgnosticRWKV, postProcessModule, RWKVMaster - is
exercised without a GPU and compared with the reference's FASTQUANT CPU model on the same file.
"""
import os
import sys
import tempfile

import pytest
import torch

# the reference checkout: $RWKVSTIC_REFERENCE, else a folder named "reference" beside this repository
REF = os.environ.get("RWKVSTIC_REFERENCE",
                     os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference"))
pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "src", "rwkvstic")),
                                reason="reference checkout not available")


@pytest.fixture(scope="module")
def reference():
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
    import make_golden
    make_golden.import_reference(REF)
    import rwkvstic.load as load
    return load


def test_load_through_reference_loader_and_master(reference):
    import rwkvstic_b200.backend as backend
    from rwkvstic_b200.model import quantize_tensors, state_to_reference
    from rwkvstic_b200.synth import synth_checkpoint
    from kernel_contract import ContractModel

    ck = synth_checkpoint(2, 128, seed=41)          # full 50277 vocabulary: the tokenizer emits real ids
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "tiny.pth")
        torch.save(ck, path)
        mode = backend.install(model_factory=lambda c: ContractModel(quantize_tensors(c.items(), "cpu")))
        ours = reference.RWKV(path, mode=mode)
        ref = reference.RWKV(path, device="cpu", jit=False,
                             config={"devices": [{"device": "cpu", "dtype": torch.uint8}], "custom": False})
    assert type(ours).__name__ == "RWKVMaster" and isinstance(ours.model, ContractModel)
    assert tuple(ours.emptyState.shape) == tuple(ref.emptyState.shape) == (2, 5, 128)
    text = "The quick brown fox jumps over the lazy dog, twenty tokens or more to cross one chunk boundary."
    ours.loadContext(newctx=text)
    ref.loadContext(newctx=text)
    assert ours.lastToken == ref.lastToken
    tok = torch.LongTensor([1234])
    lo, so = ours.model.forward(tok, ours.myState.clone())
    lr, sr = ref.model.forward(tok, ref.myState.clone())
    assert float((lo.double() - lr.double()).abs().max()) < 2e-3
    decay = [ly.vec["att.time_decay"] for ly in ours.model.w.layers]
    assert torch.allclose(state_to_reference(so, decay)[:, :4], sr[:, :4].double(), rtol=1e-3, atol=1e-4)
    out = ours.forward(number=2)                    # the reference's sampling loop runs on our logits
    assert out["logits"].shape[0] == 50277 and len(ours.getState()) == 2


def test_exported_archive_opens_in_the_reference(reference, tmp_path):
    """An archive written by rwkvstic_b200.rwkv_archive.export goes through the reference's own
    OptRWKV(path) branch for ``.rwkv`` files and RWKVMaster, and gives the logits of the
    reference's FASTQUANT CPU model built from the same checkpoint."""
    from rwkvstic.agnostic.backends.opt import OptRWKV
    from rwkvstic_b200 import rwkv_archive
    from rwkvstic_b200.model import quantize_tensors
    from rwkvstic_b200.synth import synth_checkpoint, synth_tokens
    import make_golden
    ck = synth_checkpoint(2, 128, vocab=257, seed=31)
    path = rwkv_archive.export(quantize_tensors(ck.items(), "cpu"), str(tmp_path / "exported"))
    theirs = OptRWKV(path, device="cpu", config=make_golden.CPU_CFG)       # torch.jit.load inside
    ref = make_golden.load_reference_model(ck)
    toks = synth_tokens(7, seed=2, vocab=257)
    a, sa = theirs.forward(toks, theirs.emptyState.clone())
    b, sb = ref.forward(toks, ref.emptyState.clone())
    assert float((a - b).abs().max()) < 1e-5
    assert torch.allclose(sa[:, :4], sb[:, :4], rtol=1e-3, atol=1e-5) and torch.equal(sa[:, 4], sb[:, 4])
