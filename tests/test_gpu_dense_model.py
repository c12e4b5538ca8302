"""GPU tests of the unquantised (TORCH-mode) model: against logits and states the reference itself
produced on CPU (tests/golden/torch_mode.npz), and against the CPU oracle at the large widths."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle.torch_mode_oracle import OracleTorchMode
from rwkvstic_b200 import _lib
from rwkvstic_b200.dense_model import B200DenseRWKV
from rwkvstic_b200.synth import synth_checkpoint, synth_tokens

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TYPES = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}
# Largest |dlogit| allowed, as a fraction of the largest |logit|.  Every product is rounded to the
# matrices' type (8 / 11 / 24 significant bits); a sum formed in another order can land on the other
# side of a rounding boundary, so the bound is a few units in the last place of that type.
REL_TOL = {"f32": 2e-5, "bf16": 4 * 2.0 ** -8, "f16": 4 * 2.0 ** -11}
SHAPES = {"tiny": (2, 128, 257, 31, 9), "mid": (3, 768, 1000, 32, 12)}


def state_excess(mine, ref, rel):
    """Worst violation of |mine - ref| <= rel * (|ref| + row max) over the rows of a state (row 4, the
    running exponent, holds -1e30 only before the first token)."""
    a, b = mine.double().cpu(), ref.double().cpu()
    bound = rel * (b.abs() + b.abs().amax(dim=2, keepdim=True)) + 1e-6
    return float(((a - b).abs() - bound).max())


@pytest.mark.parametrize("name", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("shape", ["tiny", "mid"])
def test_dense_model_against_the_reference_outputs(golden, shape, name):
    L, D, V, seed, n_tok = SHAPES[shape]
    g = golden("torch_mode.npz")
    model = B200DenseRWKV.from_checkpoint(synth_checkpoint(L, D, vocab=V, seed=seed), dtype=TYPES[name], device=DEV,
                                          use_graph=False)
    toks = torch.from_numpy(g[f"{shape}_tokens"])
    want = torch.from_numpy(g[f"{shape}_{name}_logits_tok"])
    state = model.emptyState.clone()
    worst = 0.0
    for i, tok in enumerate(toks):
        got, state = model.forward(tok.reshape(1), state)
        worst = max(worst, float((got.cpu() - want[i]).abs().max()) / float(want[i].abs().max()))
    print(f"{shape} {name}: worst |dlogit| / max |logit| over {n_tok} tokens = {worst:.2e}")
    assert worst <= REL_TOL[name], worst
    assert state_excess(state, torch.from_numpy(g[f"{shape}_{name}_state_tok"]), REL_TOL[name]) <= 0
    # Several tokens in one call.  fp32: fed one after another, the same result bit for bit.  bf16 / fp16: all rows
    # at once on the tensor cores (another summation order), against the reference's own sequence-mode outputs.
    again = model.emptyState.clone()
    got2, _ = model.forward(toks, again)
    if name == "f32":
        assert torch.equal(got2, got) and torch.equal(again, state)
    else:
        assert model.launch_count > 0 and len(model._rows_ws) == 1
        seq = torch.from_numpy(g[f"{shape}_{name}_logits_seq"]) if shape == "tiny" else want[-1]
        err = float((got2.cpu() - seq).abs().max()) / float(seq.abs().max())
        print(f"{shape} {name}: rows path |dlogit| / max |logit| = {err:.2e}")
        assert err <= REL_TOL[name], err
        ref_state = torch.from_numpy(g[f"{shape}_{name}_state_seq"]) if shape == "tiny" else torch.from_numpy(g[f"{shape}_{name}_state_tok"])
        assert state_excess(again, ref_state, REL_TOL[name]) <= 0
    model.check_status()


@pytest.mark.parametrize("embed,name", [(2048, "bf16"), (2560, "f16"), (4096, "bf16"), (5120, "bf16"), (4096, "f32")])
def test_dense_model_against_the_oracle_at_the_large_widths(embed, name):
    """Two blocks and a 1024-token vocabulary at the widths of the 1.5B ... 14B models, 12 tokens."""
    V = 1024
    ck = synth_checkpoint(2, embed, vocab=V, seed=60 + embed % 11)
    ref = OracleTorchMode(ck, TYPES[name])
    toks = synth_tokens(12, seed=embed, vocab=V)
    want, wstate = ref.forward(toks, ref.emptyState.clone())
    model = B200DenseRWKV.from_checkpoint(ck, dtype=TYPES[name], device=DEV, use_graph=False)
    got, state = model.forward(toks, model.emptyState.clone())
    err = float((got.cpu() - want).abs().max()) / float(want.abs().max())
    print(f"D={embed} {name}: |dlogit| / max |logit| = {err:.2e}")
    assert err <= REL_TOL[name], err
    assert state_excess(state, wstate, REL_TOL[name]) <= 0
    model.check_status()


def test_dense_step_graph_replay_is_bit_identical_and_deterministic():
    m = B200DenseRWKV.synthetic(2, 768, vocab=1000, seed=6, dtype=torch.bfloat16, device=DEV)     # graph from the second call on
    eager = B200DenseRWKV(m.t.items(), dtype=torch.bfloat16, device=DEV, use_graph=False, decay_is_final=True)
    toks = synth_tokens(10, seed=2, vocab=1000)
    sg, se = m.emptyState.clone(), eager.emptyState.clone()
    for t in toks:
        lg, _ = m.forward(t.reshape(1), sg)
        le, _ = eager.forward(t.reshape(1), se)
        assert torch.equal(lg, le)
    assert torch.equal(sg, se) and len(m._graphs) >= 1
    again = m.emptyState.clone()
    for t in toks:
        l2, _ = m.forward(t.reshape(1), again)
    assert torch.equal(l2, lg) and torch.equal(again, sg)
    m.check_status()


def test_dense_step_without_logits_and_bad_arguments():
    m = B200DenseRWKV.synthetic(1, 128, vocab=300, seed=1, dtype=torch.float16, device=DEV, use_graph=False)
    a, b = m.emptyState.clone(), m.emptyState.clone()
    for t in synth_tokens(3, seed=3, vocab=300):
        m._tok.copy_(t.reshape(1))
        m._step(a, want_logits=True)
        m._step(b, want_logits=False)
    assert torch.equal(a, b)
    # a token outside the table is clamped into it (as the quantised step does), not read out of bounds
    for bad, same_as in ((300 + 5, 299), (-3, 0)):
        x, y = m.emptyState.clone(), m.emptyState.clone()
        lx, _ = m.forward(torch.tensor([bad]), x)
        ly, _ = m.forward(torch.tensor([same_as]), y)
        assert torch.equal(lx, ly) and torch.equal(x, y)
    L = m._L
    args = (m._tok.data_ptr(), a.data_ptr(), None, m._ws.data_ptr(), m._ws.numel(), None)
    assert L.b200rwkv_dense_step(None, *args) == _lib.EINVAL
    assert L.b200rwkv_dense_step(C.byref(m._cmodel), m._tok.data_ptr(), a.data_ptr(), None, m._ws.data_ptr(),
                                 m._ws.numel() - 1, None) == _lib.EINVAL
    bad = _lib.DenseModel.from_buffer_copy(m._cmodel)
    bad.n_embd = 132                                               # not a multiple of 8
    assert L.b200rwkv_dense_step(C.byref(bad), *args) == _lib.EINVAL
    bad = _lib.DenseModel.from_buffer_copy(m._cmodel)
    bad.dtype = 7
    assert L.b200rwkv_dense_step(C.byref(bad), *args) == _lib.EINVAL


def test_loader_hook_with_dtype_builds_the_unquantised_model():
    """``dtype=`` on the registered ops class (the keyword of the reference's TORCH mode,
    agnostic/backends/torch.py:8-22) makes postProcessModule hand back the unquantised model, built from
    the attributes AgnosticRWKV holds (agnosticRwkv.py:22-63; time_decay already -exp(raw))."""
    from rwkvstic_b200.backend import make_ops_class
    L, D, V = 2, 256, 300
    ck = synth_checkpoint(L, D, vocab=V, seed=9)

    class Agnostic:
        pass

    a = Agnostic()
    a.emb, a.emb1, a.emb2 = ck["emb.weight"], ck["blocks.0.ln0.weight"], ck["blocks.0.ln0.bias"]
    a.postprocess0, a.postprocess1, a.postprocess2 = ck["ln_out.weight"], ck["ln_out.bias"], ck["head.weight"]
    per_layer = {"ln1w": "ln1.weight", "ln1b": "ln1.bias", "ln2w": "ln2.weight", "ln2b": "ln2.bias",
                 "time_first": "att.time_first", "kktk": "att.time_mix_k", "vvtv": "att.time_mix_v", "rrtr": "att.time_mix_r",
                 "key": "att.key.weight", "value": "att.value.weight", "receptance": "att.receptance.weight",
                 "outputvv": "att.output.weight", "time_mix_k_ffn": "ffn.time_mix_k", "time_mix_r_ffn": "ffn.time_mix_r",
                 "key_ffn": "ffn.key.weight", "receptance_ffn": "ffn.receptance.weight", "value_ffn": "ffn.value.weight"}
    for attr, name in per_layer.items():
        setattr(a, attr, [ck[f"blocks.{i}.{name}"].squeeze() if "time_" in name else ck[f"blocks.{i}.{name}"] for i in range(L)])
    a.time_decay = [-torch.exp(ck[f"blocks.{i}.att.time_decay"].double()) for i in range(L)]

    class Base:            # stands in for agnostic.backends.base.module
        def __init__(self, layers, embed, *args, **kwargs):
            pass

    ops_cls = make_ops_class(Base, device=DEV)
    with pytest.raises(ValueError):
        ops_cls(L, D, dtype=torch.int8)
    ops_obj = ops_cls(L, D, dtype=torch.bfloat16)
    model = ops_obj.postProcessModule(a)
    assert isinstance(model, B200DenseRWKV) and model.dtype == torch.bfloat16 and ops_obj.emptyState is model.emptyState
    ref = OracleTorchMode(ck, torch.bfloat16)
    toks = synth_tokens(6, seed=4, vocab=V)
    want, _ = ref.forward(toks, ref.emptyState.clone())
    got, _ = model.forward(toks, model.emptyState.clone())
    assert float((got.cpu() - want).abs().max()) <= REL_TOL["bf16"] * float(want.abs().max())


@pytest.mark.parametrize("embed,name,B,T", [(2048, "bf16", 3, 40), (2560, "f16", 2, 17), (4096, "bf16", 2, 300), (5120, "f16", 1, 130),
                                            (2048, "f16", 3, 129), (2048, "bf16", 5, 128), (512, "bf16", 6, 280)])
def test_dense_rows_path_against_the_oracle(embed, name, B, T):
    """B sequences of T tokens in one call through the tensor-core rows path (T = 300, 280 and 130 take the
    chunk-parallel WKV scan; 6 x 280 = 1680 rows are more than the GPU holds preparation CTAs, so each CTA
    walks three consecutive rows across the sequence boundaries) against the oracle's sequence mode, one sequence at a time: logits after the
    last token and the final state; then one more token through the one-row step from that state."""
    V = 1024
    ck = synth_checkpoint(2, embed, vocab=V, seed=70 + embed % 13)
    ref = OracleTorchMode(ck, TYPES[name])
    model = B200DenseRWKV.from_checkpoint(ck, dtype=TYPES[name], device=DEV, use_graph=False)
    toks = synth_tokens(B * T, seed=embed + 3, vocab=V).reshape(B, T)
    state = model.empty_batch_state(B)
    out = model.forward_rows(toks.to(DEV), state)
    model.check_status()
    worst = 0.0
    for b in range(B):
        want, wstate = ref.forward(toks[b], ref.emptyState.clone())
        worst = max(worst, float((out[b].cpu() - want).abs().max()) / float(want.abs().max()))
        assert state_excess(state[b], wstate, REL_TOL[name]) <= 0, b
        if b == 0:
            nxt = torch.tensor([5])
            w2, _ = ref.forward(nxt, wstate)
            g2, _ = model.forward(nxt, state[0].clone())
            assert float((g2.cpu() - w2).abs().max()) / float(w2.abs().max()) <= REL_TOL[name]
    print(f"D={embed} {name} rows path {B}x{T}: |dlogit| / max |logit| = {worst:.2e}")
    assert worst <= REL_TOL[name], worst


def test_dense_rows_path_arguments():
    m = B200DenseRWKV.synthetic(1, 128, vocab=300, seed=1, dtype=torch.float32, device=DEV, use_graph=False)
    with pytest.raises(ValueError):
        m.forward_rows(torch.zeros(1, 4, dtype=torch.int64), m.empty_batch_state(1))        # fp32 matrices
    h = B200DenseRWKV.synthetic(1, 128, vocab=300, seed=1, dtype=torch.float16, device=DEV, use_graph=False)
    with pytest.raises(ValueError):
        h.forward_rows(torch.zeros(2, 4, dtype=torch.int64), h.empty_batch_state(1))        # state of another batch size
    L = h._L
    st = h.empty_batch_state(1)
    tok = torch.zeros(1, 4, dtype=torch.int64, device=DEV)
    need = int(L.b200rwkv_dense_rows_workspace_bytes(C.byref(h._cmodel), 1, 4))
    ws = torch.zeros(need, dtype=torch.uint8, device=DEV)
    assert L.b200rwkv_dense_forward_rows(C.byref(h._cmodel), tok.data_ptr(), 1, 4, st.data_ptr(), st.stride(0), None,
                                         ws.data_ptr(), need - 1, None) == _lib.EINVAL
    assert L.b200rwkv_dense_forward_rows(C.byref(m._cmodel), tok.data_ptr(), 1, 4, st.data_ptr(), st.stride(0), None,
                                         ws.data_ptr(), need, None) == _lib.EINVAL
    assert int(L.b200rwkv_dense_rows_workspace_bytes(C.byref(h._cmodel), 300, 300)) == 0


@pytest.mark.parametrize("target_blocks", [0, 2])
def test_blocks_streamed_from_pinned_host_memory_give_the_same_bits(target_blocks):
    """``target_gb`` keeps only the first blocks' matrices on the device; the others are copied from pinned
    host memory into two staging buffers one block ahead of their kernels.  Same kernels on the same
    bytes: logits and states must equal the resident model's bit for bit, one token at a time (7 tokens:
    the three streamed blocks take the two buffers in turn across tokens) and through the rows path."""
    L, D, V = 5, 256, 300
    ck = synth_checkpoint(L, D, vocab=V, seed=12)
    block_bytes = (5 * D * D + 2 * D * 4 * D) * 2
    resident = B200DenseRWKV.from_checkpoint(ck, dtype=torch.float16, device=DEV, use_graph=False)
    streamed = B200DenseRWKV.from_checkpoint(ck, dtype=torch.float16, device=DEV, target_gb=(target_blocks + 0.5) * block_bytes / 1e9)
    assert streamed.n_res == target_blocks and len(streamed._blob) == L - target_blocks
    assert streamed.weight_bytes() == resident.weight_bytes()
    toks = synth_tokens(7, seed=8, vocab=V)
    sr, ss = resident.emptyState.clone(), streamed.emptyState.clone()
    for t in toks:
        lr, _ = resident.forward(t.reshape(1), sr)
        ls, _ = streamed.forward(t.reshape(1), ss)
        assert torch.equal(lr, ls)
    assert torch.equal(sr, ss)
    assert streamed.h2d_bytes >= 7 * (L - target_blocks) * streamed._blob[L - 1].numel()
    rows = synth_tokens(2 * 9, seed=9, vocab=V).reshape(2, 9)
    br, bs = resident.empty_batch_state(2), streamed.empty_batch_state(2)
    assert torch.equal(resident.forward_rows(rows.to(DEV), br), streamed.forward_rows(rows.to(DEV), bs))
    assert torch.equal(br, bs)
    streamed.check_status()
    full = B200DenseRWKV.from_checkpoint(ck, dtype=torch.float16, device=DEV, target_gb=1.0)      # everything fits: nothing streamed
    assert full.n_res is None and not full._blob


def test_few_rows_split_k_and_stay_deterministic():
    """With few rows a launch has few tiles and cuts K into slices whose partial sums are added in slice
    order: two runs agree bit for bit (whichever CTA finished last), and the result matches the oracle."""
    V, Dm = 1024, 4096
    ck = synth_checkpoint(1, Dm, vocab=V, seed=91)
    model = B200DenseRWKV.from_checkpoint(ck, dtype=torch.bfloat16, device=DEV, use_graph=False)
    toks = synth_tokens(24, seed=5, vocab=V).reshape(24, 1)           # 24 sequences, one token each: 32 weight tiles per matrix
    outs = []
    for _ in range(3):
        st = model.empty_batch_state(24)
        outs.append((model.forward_rows(toks.to(DEV), st).clone(), st.clone()))
    assert all(torch.equal(outs[0][0], o[0]) and torch.equal(outs[0][1], o[1]) for o in outs[1:])
    ref = OracleTorchMode(ck, torch.bfloat16)
    for b in (0, 23):
        want, _ = ref.forward(toks[b], ref.emptyState.clone())
        assert float((outs[0][0][b].cpu() - want).abs().max()) / float(want.abs().max()) <= REL_TOL["bf16"]
    model.check_status()
