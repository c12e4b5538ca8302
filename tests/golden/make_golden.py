"""Generate the golden fixtures in this folder by running the UNMODIFIED reference.

Usage (only where the reference checkout exists; the fixtures are committed so the
tests never need it):

    python tests/golden/make_golden.py /path/to/rwkvstic-checkout

The reference is imported from ``<checkout>/src``.  It imports the ``inquirer`` package
at module level (for interactive prompts that this script never triggers); that
package is not installed, so a three-line stand-in is written to a temp folder and put
on ``sys.path``.  Nothing else about the reference is altered.

What is run: ``rwkvstic.agnostic.backends.opt.OptRWKV(path, jit=False, device="cpu",
config={"devices":[{"device":"cpu","dtype":torch.uint8}],"custom":False})`` - the
FASTQUANT CPU path (uint8 weights, fp32 matmul, fp64 vectors, TorchWKV) - plus its
building blocks on small seeded inputs.

Outputs:
  ops_small.npz     per-op vectors (quantiser, mm8, layernorm, wkv, one Block)
  model_tiny.npz    L=2 D=128 V=257 model: sequence mode and token-by-token
  model_169m.npz    the 169M shape: L=12 D=768 V=50277, 32 prompt + 64 greedy tokens
"""
from __future__ import annotations

import os
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from rwkvstic_b200.synth import synth_checkpoint, synth_tokens  # noqa: E402

CPU_CFG = {"devices": [{"device": "cpu", "dtype": torch.uint8}], "custom": False}


def import_reference(checkout: str):
    stub = tempfile.mkdtemp(prefix="inquirer_stub_")
    os.makedirs(os.path.join(stub, "inquirer"))
    with open(os.path.join(stub, "inquirer", "__init__.py"), "w") as f:
        f.write("class List:\n    def __init__(self, *a, **k): pass\n"
                "def prompt(*a, **k): raise RuntimeError('interactive prompt')\n"
                "confirm = checkbox = prompt\n")
    sys.path.insert(0, stub)
    sys.path.insert(0, os.path.join(checkout, "src"))


def load_reference_model(ck):
    from rwkvstic.agnostic.backends.opt import OptRWKV
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "synth.pth")
        torch.save(ck, path)
        return OptRWKV(path, jit=False, device="cpu", config=CPU_CFG)


def greedy_run(model, prompt, steps):
    state = model.emptyState.clone()
    logits, state = model.forward(prompt, state)
    toks, rows = [], []
    for _ in range(steps):
        t = int(torch.argmax(logits))
        toks.append(t)
        rows.append(logits.clone())
        logits, state = model.forward(torch.LongTensor([t]), state)
    return np.array(toks), torch.stack(rows), state


def ops_small():
    from rwkvstic.agnostic.backends.modules.matmul import mm8Naive
    from rwkvstic.agnostic.backends.modules.layernorm import LayerNorm
    from rwkvstic.agnostic.backends.modules.wkv import TorchWKV
    from rwkvstic.agnostic.backends.modules.block import Block

    g = torch.Generator().manual_seed(11)
    out = {}
    # quantiser + mm8 on a ragged matrix [out=80, in=48]
    w = torch.randn(80, 48, generator=g) * 0.02
    m = mm8Naive(w, "cpu", torch.float32, False)
    x1 = torch.randn(1, 48, generator=g, dtype=torch.float64)
    x5 = torch.randn(5, 48, generator=g, dtype=torch.float64)
    out.update(q_w=w.numpy(), q_weight=m.weight.numpy(), q_range=m.range.numpy(), q_offset=m.offset.numpy(),
               mm_x1=x1.numpy(), mm_y1=m.forward(x1).numpy(), mm_x5=x5.numpy(), mm_y5=m.forward(x5).numpy())
    # layernorm
    lw, lb = torch.randn(48, generator=g), torch.randn(48, generator=g)
    ln = LayerNorm(lw, lb)
    out.update(ln_w=lw.numpy(), ln_b=lb.numpy(), ln_x=x5.numpy(), ln_y=ln.forward(x5).numpy())
    # wkv over T=7, C=32, from a non-empty state
    C, T = 32, 7
    wd = -torch.exp(torch.rand(C, generator=g, dtype=torch.float64) * 8 - 5)
    u = torch.rand(C, generator=g, dtype=torch.float64) * 2 - 1
    k = torch.randn(T, C, generator=g, dtype=torch.float64)
    v = torch.randn(T, C, generator=g, dtype=torch.float64)
    aa = torch.randn(C, generator=g, dtype=torch.float64)
    bb = torch.rand(C, generator=g, dtype=torch.float64) + 0.5
    pp = torch.full((C,), -1e30, dtype=torch.float64)
    y, aa2, bb2, pp2 = TorchWKV("cpu", torch.float64).forward(T, C, wd, u, k, v, aa.clone(), bb.clone(), pp.clone())
    out.update(wkv_w=wd.numpy(), wkv_u=u.numpy(), wkv_k=k.numpy(), wkv_v=v.numpy(), wkv_aa=aa.numpy(),
               wkv_bb=bb.numpy(), wkv_pp=pp.numpy(), wkv_y=y.numpy(), wkv_aa2=aa2.numpy(), wkv_bb2=bb2.numpy(),
               wkv_pp2=pp2.numpy())
    # one Block at D=64 for T=1 and T=4, non-empty state
    ck = synth_checkpoint(1, 64, vocab=97, seed=21)
    blk = Block(ck, 0)
    blk.config(0, **CPU_CFG)
    st = torch.randn(5, 64, generator=g, dtype=torch.float64) * 0.3
    st[3] = st[3].abs() + 0.5
    st[4] = -1e30
    for T in (1, 4):
        x = torch.randn(T, 64, generator=g, dtype=torch.float64)
        s = st.clone()
        yb, s2 = blk.forward(x.clone(), s)
        out[f"blk_x{T}"] = x.numpy()
        out[f"blk_y{T}"] = yb.detach().numpy()
        out[f"blk_s{T}"] = s2.numpy()
    out["blk_state"] = st.numpy()
    np.savez_compressed(os.path.join(HERE, "ops_small.npz"), **out)
    print("ops_small.npz written")


def model_tiny():
    ck = synth_checkpoint(2, 128, vocab=257, seed=31)
    model = load_reference_model(ck)
    toks = synth_tokens(9, seed=5, vocab=257)
    # sequence mode in one call
    s = model.emptyState.clone()
    lg_seq, s_seq = model.forward(toks, s)
    # two chunks (5 + 4), the way loadContext feeds chunks (rwkvMaster.py:58-77)
    s = model.emptyState.clone()
    _, s = model.forward(toks[:5], s)
    lg_chunk, s_chunk = model.forward(toks[5:], s)
    # token by token
    s = model.emptyState.clone()
    per_tok = []
    for t in toks:
        lg, s = model.forward(torch.LongTensor([int(t)]), s)
        per_tok.append(lg.clone())
    np.savez_compressed(os.path.join(HERE, "model_tiny.npz"), tokens=toks.numpy(),
                        logits_seq=lg_seq.detach().numpy(), state_seq=s_seq.numpy(),
                        logits_chunk=lg_chunk.detach().numpy(), state_chunk=s_chunk.numpy(),
                        logits_tok=torch.stack(per_tok).detach().numpy(), state_tok=s.numpy())
    print("model_tiny.npz written; seq vs token max |dlogit| =",
          float((lg_seq - per_tok[-1]).abs().max()))


def model_169m(seed=1234, prompt_seed=38):
    # Prompt seed 38 was picked from a scan of seeds 7..69: with random weights the top-1/top-2
    # logit gap over 64 greedy steps is often ~1e-3 (seed 7: 1.07e-3), below the 2e-3 logit
    # tolerance, which would make "identical greedy stream" untestable.  Seed 38 has a
    # minimum gap of 1.16e-2 (median 9.5e-2).
    ck = synth_checkpoint(12, 768, seed=seed)
    model = load_reference_model(ck)
    prompt = synth_tokens(32, seed=prompt_seed)
    toks, rows, state = greedy_run(model, prompt, 64)
    top = torch.topk(rows, 2, dim=1).values
    margin = (top[:, 0] - top[:, 1]).numpy()
    print("169m: min / median top1-top2 margin over 64 steps:", margin.min(), np.median(margin))
    probe = torch.from_numpy(np.random.RandomState(3).choice(50277, 256, replace=False))
    top16 = torch.topk(rows, 16, dim=1)
    np.savez_compressed(os.path.join(HERE, "model_169m.npz"), seed=seed, prompt=prompt.numpy(), tokens=toks,
                        margin=margin, prompt_seed=prompt_seed, probe_idx=probe.numpy(), probe_logits=rows[:, probe].detach().numpy(),
                        top16_val=top16.values.detach().numpy(), top16_idx=top16.indices.numpy(),
                        logits_first=rows[0].detach().numpy().astype(np.float32),
                        logits_last=rows[-1].detach().numpy().astype(np.float32),
                        state=state.numpy(), torch_version=torch.__version__)
    print("model_169m.npz written")


if __name__ == "__main__":
    import_reference(sys.argv[1])
    torch.manual_seed(0)
    ops_small()
    model_tiny()
    model_169m()
