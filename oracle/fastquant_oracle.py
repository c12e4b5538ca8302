"""CPU oracle for the RWKV-4 FASTQUANT inference path.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain torch-on-CPU code, the arithmetic of the reference's
FASTQUANT CPU path so that the CUDA kernels can be checked against it on a box that
does not have the reference.  Only the tests, the smoke check and the benchmark's
``cpu_baseline`` / ``--impl reference`` legs may import it; nothing in the product
package does.

Parity status: PINNED.  ``tests/golden/make_golden.py`` imports the unmodified
reference, runs it on seeded weights and tokens, and stores its outputs under
``tests/golden/``; ``tests/test_oracle.py`` checks this restatement against those
files (quantised bytes bit-exact, logits/state to 1e-9 relative in fp64 terms, the
greedy token stream identical).

Every function names the reference lines it follows (paths inside rwkvstic's
``src/rwkvstic/agnostic/backends``).

The second scheme at the bottom (``two_axis_*``) follows only the one-line formula
"(q+0.5)*ry*rx+my+mx with per-row/per-column offsets and scales"; its source is the
third-party ``rwkv`` pip package (unpinned dependency of the reference, not vendored,
not installed).  Parity for that scheme is UNPINNED: self-consistency only.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch


# ----------------------------------------------------------------------------- quantisation
def quantize_matrix(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """modules/matmul.py:18-40 (MM8.chunkQuantizeMatrix + QuantizeMatrix).

    ``w`` is the checkpoint matrix ``[out, in]``.  Returns ``(weight u8[in,out],
    range f32[in], offset f64[in])`` exactly as the MM8 module stores them.
    """
    x = w                                   # QuantizeMatrix sees xx = w.t(); x = xx.t() = w
    mini = x.min(0)[0].double()
    out = x - mini
    ran = out.max(0)[0].double() / 255
    out = out / ran
    fract = out.frac().double().mean(0)
    mini = mini.double() + fract * ran.double()
    weight = out.t().to(dtype=torch.uint8, memory_format=torch.contiguous_format)
    return weight, ran.to(torch.float32).clone(), mini.to(torch.float64).clone()


def mm8(x: torch.Tensor, weight: torch.Tensor, rng: torch.Tensor, offset: torch.Tensor) -> torch.Tensor:
    """modules/matmul.py:130-131 (mm8Naive.forward, naivedtype fp32 on cpu, :184).

    ``x`` is fp64 ``[T, in]``; the product is an fp32 matmul against the bytes cast
    to fp32, the offset term an fp64 mat-vec; the sum is fp64 ``[T, out]``.
    """
    main = (x * rng).to(dtype=torch.float32) @ weight.to(dtype=torch.float32)
    return main + x.mv(offset).reshape(-1, 1)


# ----------------------------------------------------------------------------- vector ops
def layernorm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """modules/layernorm.py:11-20: biased variance over dim 1, eps 1e-5 inside the sqrt, fp64."""
    x = x.to(torch.float64)
    xc = x - torch.mean(x, dim=1, keepdim=True)
    sd = torch.sqrt(torch.mean(xc * xc, dim=1, keepdim=True) + 1e-5)
    return weight * (xc / sd) + bias


def wkv(T: int, C: int, w, u, k, v, aa, bb, pp):
    """modules/wkv.py:23-40 (TorchWKV.forward): plain (no max-trick) fp64 recurrence.

    State convention: aa/bb hold the running sums already multiplied by exp(w)
    (the decay is applied at the end of each step); pp is passed through.
    """
    y = torch.empty((T, C), dtype=torch.float64)
    for i in range(T):
        kk = torch.exp(k[i])
        vv = v[i]
        e = torch.exp(u + w + k[i])
        y[i] = (aa + e * vv) / (bb + e)
        aa = (aa + kk * vv) * torch.exp(w)
        bb = (bb + kk) * torch.exp(w)
    return y, aa, bb, pp


def wkv_maxtrick_step(w, u, k, v, aa, bb, pp):
    """agnosticRwkv.py:68-103 (processLayerx): one step of the max-trick form.

    Here aa/bb are scaled by exp(-pp) and the decay is applied at the START of the
    next step (``pp + w``), so ``aa_plain = exp(w) * aa * exp(pp)`` links it to ``wkv``.
    """
    ww = u + k
    p = torch.maximum(pp, ww)
    e1 = torch.exp(pp - p)
    e2 = torch.exp(ww - p)
    a = e1 * aa + e2 * v
    b = e1 * bb + e2
    wwn = pp + w
    p1 = torch.maximum(wwn, k)
    e11 = torch.exp(wwn - p1)
    e21 = torch.exp(k - p1)
    return a / b, e11 * aa + e21 * v, e11 * bb + e21, p1


# ----------------------------------------------------------------------------- model
class Matrix:
    """One quantised Linear with a single cpu/uint8 shard (matmul.py:177-201)."""

    def __init__(self, w: torch.Tensor):
        self.weight, self.range, self.offset = quantize_matrix(w)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        # Linear.newfunc / forward (matmul.py:154-167): one shard, summed onto zeros, fp64.
        return mm8(x.to(torch.float64), self.weight, self.range, self.offset).to(torch.float64)


class Block:
    """modules/block.py:7-50 (parameters) and :56-102 (forward)."""

    def __init__(self, ck: Dict[str, torch.Tensor], i: int):
        p = f"blocks.{i}."
        d = lambda name: ck[p + name].squeeze().to(torch.float64).clone()
        self.ln1 = (d("ln1.weight"), d("ln1.bias"))
        self.ln2 = (d("ln2.weight"), d("ln2.bias"))
        self.key, self.value, self.receptance = (Matrix(ck[p + f"att.{n}.weight"])
                                                 for n in ("key", "value", "receptance"))
        self.attout = Matrix(ck[p + "att.output.weight"])
        self.ffnkey = Matrix(ck[p + "ffn.key.weight"])
        self.ffnvalue = Matrix(ck[p + "ffn.value.weight"])
        self.ffnreceptance = Matrix(ck[p + "ffn.receptance.weight"])
        self.attmix = torch.stack((d("att.time_mix_k"), d("att.time_mix_v"), d("att.time_mix_r"))).unsqueeze(1)
        self.ffnmix = torch.stack((d("ffn.time_mix_k"), d("ffn.time_mix_r"))).unsqueeze(1)
        self.time_first = d("att.time_first")
        self.time_decay = ck[p + "att.time_decay"].squeeze().double().exp().neg().clone()

    def forward(self, x: torch.Tensor, state: torch.Tensor):
        """``x`` fp64 [T,D]; ``state`` fp64 [5,D] updated in place (block.py:56-102)."""
        T = x.shape[0]
        xy = layernorm(x, *self.ln1)
        tc = xy[torch.arange(T) - 1]                 # row t-1, row 0 wraps to the last row ...
        last = tc[0].clone()
        tc[0] = state[0]                             # ... which is swapped with the carried row
        state[0] = last
        mix = xy.unsqueeze(0) * self.attmix + tc.unsqueeze(0) * (1 - self.attmix)
        k, v, r = self.key(mix[0]), self.value(mix[1]), self.receptance(mix[2])
        r = r.sigmoid()
        y, state[2], state[3], state[4] = wkv(T, k.shape[1], self.time_decay, self.time_first,
                                              k, v, state[2], state[3], state[4])
        y = y * r
        rz = x + self.attout(y)
        ddd = layernorm(rz, *self.ln2)
        rc = ddd[torch.arange(T) - 1]
        last = rc[0].clone()
        rc[0] = state[1]
        state[1] = last
        fmix = ddd * self.ffnmix + rc * (1 - self.ffnmix)
        rf = self.ffnreceptance(fmix[1]).sigmoid()
        kf = self.ffnkey(fmix[0]).relu()
        rvm = self.ffnvalue(torch.square(kf))
        return rvm * rf + rz, state


class OracleRWKV:
    """agnostic/backends/opt.py:25-76 (myRWKV)."""

    def __init__(self, ck: Dict[str, torch.Tensor]):
        self.embed = len(ck["blocks.0.att.key.weight"])
        self.layers = len([k for k in ck if "blocks" in k and "ln1.bias" in k])
        self.emb = ck["emb.weight"].clone()
        d = lambda name: ck[name].clone().to(torch.float64)
        self.ln_in = (d("blocks.0.ln0.weight"), d("blocks.0.ln0.bias"))
        self.ln_out = (d("ln_out.weight"), d("ln_out.bias"))
        self.head = Matrix(ck["head.weight"])
        self.blocks: List[Block] = [Block(ck, i) for i in range(self.layers)]
        # opt.py:31-32 builds [L,5,D] (rows 0..3 zero, row 4 = -1e30) as an fp32 tensor and
        # opt.py:80 widens it, so the stored value is fp32(-1e30) = -1.0000000150474662e30.
        self.emptyState = torch.zeros(self.layers, 5, self.embed, dtype=torch.float32)
        self.emptyState[:, 4] = -1e30
        self.emptyState = self.emptyState.to(torch.float64)

    def forward(self, tokens: torch.Tensor, state: torch.Tensor):
        """opt.py:61-76: tokens int64 [T]; state fp64 [L,5,D] (mutated); logits fp64 [V]."""
        x = self.emb[tokens.cpu()].to(torch.float64)            # emb.py:8-9
        x = layernorm(x, *self.ln_in)
        for i, blk in enumerate(self.blocks):
            x, st = blk.forward(x, state[i])
            state[i] = st
        x = layernorm(x, *self.ln_out)
        return self.head(x[-1:]).squeeze(), state

    def greedy(self, prompt: torch.Tensor, steps: int, chunk: int = 0):
        """Prompt in sequence mode (optionally in chunks), then ``steps`` greedy tokens.

        Returns (tokens [steps], logits of every step [steps,V] fp64, final state)."""
        state = self.emptyState.clone()
        chunk = chunk or len(prompt)
        logits = None
        for s in range(0, len(prompt), chunk):
            logits, state = self.forward(prompt[s:s + chunk], state)
        toks, all_logits = [], []
        for _ in range(steps):
            t = int(torch.argmax(logits))
            toks.append(t)
            all_logits.append(logits.clone())
            logits, state = self.forward(torch.tensor([t]), state)
        return torch.tensor(toks), torch.stack(all_logits), state


# ----------------------------------------------------------------------------- scheme 2 (unpinned)
def two_axis_quantize(w: torch.Tensor):
    """Two-axis uint8 scheme, restated from its one-line description (parity UNPINNED).

    ``w`` is ``[out, in]``.  Returns ``(q u8[in,out], my f64[in], ry f64[in], mx f64[out], rx f64[out])``
    with ``w_hat[o,k] = (q[k,o] + 0.5) * ry[k] * rx[o] + my[k] + mx[o]``.
    """
    x = w.double().t().clone()                      # [in, out] as used in x @ W
    my = x.min(dim=1, keepdim=True)[0]
    x = x - my
    mx = x.min(dim=0, keepdim=True)[0]
    x = x - mx
    rx = x.max(dim=0, keepdim=True)[0].clamp_min(1e-30)
    x = x / rx
    ry = x.max(dim=1, keepdim=True)[0].clamp_min(1e-30)
    x = x / ry
    q = torch.floor(x * 256).clamp(0, 255).to(torch.uint8)
    return q, my.squeeze(1), ry.squeeze(1) / 256, mx.squeeze(0), rx.squeeze(0)


def two_axis_mm8(x: torch.Tensor, q, my, ry, mx, rx) -> torch.Tensor:
    """y = x @ w_hat with w_hat as defined in ``two_axis_quantize``; fp64 throughout."""
    x = x.double()
    w_hat = (q.double() + 0.5) * ry[:, None] * rx[None, :] + my[:, None] + mx[None, :]
    return x @ w_hat
