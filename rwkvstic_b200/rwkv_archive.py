"""Reading the reference's FASTQUANT ``.rwkv`` archives straight into the fused backend.

A ``.rwkv`` file is what ``OptRWKV(..., export=...)`` writes (agnostic/backends/opt.py:112-117): the
TorchScript archive of the quantised model.  Its tensors are already in the kernels' number
format - uint8 bytes ``[in, out]`` per device shard with an fp32 range and an fp64 offset per
input feature (modules/matmul.py:15-21, :40) - so nothing is re-quantised: the bytes are
transposed to the output-major layout and uploaded.  Module layout read here (attribute names
of the reference's classes): ``emb.w``; ``ln_in`` / ``ln_out`` / ``blocks.i.ln1`` / ``ln2``
``.weight .bias``; ``blocks.i.attmix [3,1,D]`` (k, v, r), ``ffnmix [2,1,D]`` (k, r),
``time_first``, ``time_decay`` (already ``-exp(raw)``, modules/block.py:41);
``blocks.i.att.weights.<shard>.{weight,weight1,weight2,range*,offset*}`` (key, value,
receptance); ``blocks.i.{attout,ffnkey,ffnreceptance,ffnvalue}.weights.<shard>`` and
``head.weights.<shard>`` ``.{weight,range,offset}``.  Several shards (the reference's split of a
matrix along its input dimension over devices, modules/matmul.py:177-201) are concatenated
back along the input dimension.  Archives whose matrices are not uint8 hold no such attributes
and are refused.
"""
from __future__ import annotations

from typing import List, Union

import torch

from .model import B200RWKV, LayerWeights, QuantizedWeights
from .quant import QuantMatrix


def _shards(linear) -> list:
    shards = list(linear.weights.children())
    if not shards:
        raise ValueError("archive matrix has no shards (was the model configured before export?)")
    return shards


def _matrix(shards, suffix: str, dev) -> QuantMatrix:
    """One matrix from its input-dimension shards: bytes u8[in_i, out], range f32[in_i], offset f64[in_i]."""
    for s in shards:
        if not hasattr(s, "weight" + suffix) or getattr(s, "weight" + suffix).dtype != torch.uint8:
            raise ValueError("archive matrix is not uint8 FASTQUANT (float shards cannot be harvested)")
    w = torch.cat([getattr(s, "weight" + suffix).cpu() for s in shards], dim=0)          # [in, out]
    rng = torch.cat([getattr(s, "range" + suffix).cpu().reshape(-1) for s in shards]).to(torch.float32)
    off = torch.cat([getattr(s, "offset" + suffix).cpu().reshape(-1) for s in shards]).to(torch.float64)
    qt = w.t().contiguous()                                                              # [out, in], k contiguous
    return QuantMatrix(qt=qt.to(dev), ry=rng.contiguous().to(dev), my=off.float().contiguous().to(dev),
                       half=0.0, my64=off.to(dev))


def harvest(archive: Union[str, torch.jit.ScriptModule], device="cuda:0") -> QuantizedWeights:
    """``QuantizedWeights`` on ``device`` from a ``.rwkv`` path or an already loaded archive."""
    m = torch.jit.load(archive, map_location="cpu") if isinstance(archive, str) else archive
    dev = torch.device(device)
    f32 = lambda t: t.detach().cpu().reshape(-1).to(torch.float32).contiguous().to(dev)
    layers: List[LayerWeights] = []
    for blk in m.blocks.children():
        ly = LayerWeights()
        ly.vec["ln1.weight"], ly.vec["ln1.bias"] = f32(blk.ln1.weight), f32(blk.ln1.bias)
        ly.vec["ln2.weight"], ly.vec["ln2.bias"] = f32(blk.ln2.weight), f32(blk.ln2.bias)
        att, ffn = blk.attmix.detach().cpu(), blk.ffnmix.detach().cpu()
        for i, k in enumerate(("att.time_mix_k", "att.time_mix_v", "att.time_mix_r")):
            ly.vec[k] = f32(att[i])
        for i, k in enumerate(("ffn.time_mix_k", "ffn.time_mix_r")):
            ly.vec[k] = f32(ffn[i])
        ly.vec["att.time_decay"] = f32(blk.time_decay)       # stored as w = -exp(raw)
        ly.vec["att.time_first"] = f32(blk.time_first)
        sh = _shards(blk.att)
        ly.mat["att.key"], ly.mat["att.value"], ly.mat["att.receptance"] = (_matrix(sh, s, dev) for s in ("", "1", "2"))
        ly.mat["att.output"] = _matrix(_shards(blk.attout), "", dev)
        ly.mat["ffn.key"] = _matrix(_shards(blk.ffnkey), "", dev)
        ly.mat["ffn.receptance"] = _matrix(_shards(blk.ffnreceptance), "", dev)
        ly.mat["ffn.value"] = _matrix(_shards(blk.ffnvalue), "", dev)
        layers.append(ly)
    if not layers:
        raise ValueError("archive has no blocks")
    emb = m.emb.w.detach().cpu().to(torch.float32).contiguous().to(dev)
    head = _matrix(_shards(m.head), "", dev)
    D, F = layers[0].mat["att.key"].k_in, layers[0].mat["ffn.key"].n_out
    return QuantizedWeights(n_layer=len(layers), n_embd=D, n_ffn=F, n_vocab=emb.shape[0], emb=emb,
                            ln0=(f32(m.ln_in.weight), f32(m.ln_in.bias)),
                            ln_out=(f32(m.ln_out.weight), f32(m.ln_out.bias)), head=head, layers=layers)


def load(archive: Union[str, torch.jit.ScriptModule], device="cuda:0", **kw) -> B200RWKV:
    """The fused model for a ``.rwkv`` archive (the counterpart of ``OptRWKV(path)`` for a path
    ending in ``.rwkv``, agnostic/backends/opt.py:89-92)."""
    return B200RWKV(harvest(archive, device), **kw)


# ---------------------------------------------------------------------------------------- export
# Writing an archive that stock rwkvstic opens with ``OptRWKV(path)`` (a bare ``torch.jit.load``,
# agnostic/backends/opt.py:89-92) and drives through ``forward(tokens, state) -> (logits, state)``
# and ``emptyState``.  The module below is scripted from this file's own classes; it keeps the
# reference's attribute names and tensor layouts (so ``harvest`` reads it back unchanged) and
# evaluates the FASTQUANT network with plain torch ops on the CPU: uint8 bytes cast to fp32 for
# the product, fp64 vectors, the reference's state convention (aa, bb already multiplied by
# exp(w); pp untouched).  It is a portable container, not a fast path.
class _Emb(torch.nn.Module):
    def __init__(self, w: torch.Tensor):
        super().__init__()
        self.w = w.detach().cpu().to(torch.float32).contiguous()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.w[x.cpu()].to(torch.float64)


class _Norm(torch.nn.Module):
    def __init__(self, weight: torch.Tensor, bias: torch.Tensor):
        super().__init__()
        self.weight = weight.detach().cpu().to(torch.float64)
        self.bias = bias.detach().cpu().to(torch.float64)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        c = x - x.mean(dim=1, keepdim=True)
        return self.weight * (c / torch.sqrt((c * c).mean(dim=1, keepdim=True) + 1e-5)) + self.bias


def _bytes_in_out(m: QuantMatrix) -> torch.Tensor:
    return m.qt.detach().cpu().t().contiguous()                       # u8 [in, out] as the reference stores it


def _offset64(m: QuantMatrix) -> torch.Tensor:
    return (m.my64 if m.my64 is not None else m.my.double()).detach().cpu().to(torch.float64)


class _Shard(torch.nn.Module):
    def __init__(self, m: QuantMatrix):
        super().__init__()
        self.weight, self.range, self.offset = _bytes_in_out(m), m.ry.detach().cpu().float(), _offset64(m)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        main = (x * self.range).to(torch.float32) @ self.weight.to(torch.float32)
        return main.to(torch.float64) + (x @ self.offset).unsqueeze(1)


class _Shard3(torch.nn.Module):
    def __init__(self, k: QuantMatrix, v: QuantMatrix, r: QuantMatrix):
        super().__init__()
        self.weight, self.range, self.offset = _bytes_in_out(k), k.ry.detach().cpu().float(), _offset64(k)
        self.weight1, self.range1, self.offset1 = _bytes_in_out(v), v.ry.detach().cpu().float(), _offset64(v)
        self.weight2, self.range2, self.offset2 = _bytes_in_out(r), r.ry.detach().cpu().float(), _offset64(r)

    def forward(self, x: torch.Tensor):
        a = ((x[0] * self.range).to(torch.float32) @ self.weight.to(torch.float32)).to(torch.float64) + (x[0] @ self.offset).unsqueeze(1)
        b = ((x[1] * self.range1).to(torch.float32) @ self.weight1.to(torch.float32)).to(torch.float64) + (x[1] @ self.offset1).unsqueeze(1)
        c = ((x[2] * self.range2).to(torch.float32) @ self.weight2.to(torch.float32)).to(torch.float64) + (x[2] @ self.offset2).unsqueeze(1)
        return a, b, c


class _Linear(torch.nn.Module):
    def __init__(self, m: QuantMatrix):
        super().__init__()
        self.weights = torch.nn.ModuleList([_Shard(m)])

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        out = torch.zeros(1, 1, dtype=torch.float64)
        for shard in self.weights:       # one shard: the whole input dimension
            out = shard(x)
        return out


class _Linear3(torch.nn.Module):
    def __init__(self, k: QuantMatrix, v: QuantMatrix, r: QuantMatrix):
        super().__init__()
        self.weights = torch.nn.ModuleList([_Shard3(k, v, r)])

    def forward(self, x: torch.Tensor):
        a = torch.zeros(1, 1, dtype=torch.float64)
        b, c = a, a
        for shard in self.weights:
            a, b, c = shard(x)
        return a, b, c


class _Block(torch.nn.Module):
    def __init__(self, ly: LayerWeights):
        super().__init__()
        v, m = ly.vec, ly.mat
        f64 = lambda t: t.detach().cpu().to(torch.float64)
        self.ln1, self.ln2 = _Norm(v["ln1.weight"], v["ln1.bias"]), _Norm(v["ln2.weight"], v["ln2.bias"])
        self.att = _Linear3(m["att.key"], m["att.value"], m["att.receptance"])
        self.attout, self.ffnkey = _Linear(m["att.output"]), _Linear(m["ffn.key"])
        self.ffnreceptance, self.ffnvalue = _Linear(m["ffn.receptance"]), _Linear(m["ffn.value"])
        self.attmix = torch.stack([f64(v["att.time_mix_k"]), f64(v["att.time_mix_v"]), f64(v["att.time_mix_r"])]).unsqueeze(1)
        self.ffnmix = torch.stack([f64(v["ffn.time_mix_k"]), f64(v["ffn.time_mix_r"])]).unsqueeze(1)
        self.time_first, self.time_decay = f64(v["att.time_first"]), f64(v["att.time_decay"])   # decay stored as -exp(raw)

    def forward(self, x: torch.Tensor, state: torch.Tensor):
        T = x.shape[0]
        xy = self.ln1(x)
        prev = torch.cat([state[0:1], xy[:-1]], dim=0)          # token shift: row t sees row t-1, row 0 the carry
        state[0] = xy[T - 1]
        mix = xy.unsqueeze(0) * self.attmix + prev.unsqueeze(0) * (1 - self.attmix)
        k, v, r = self.att(mix)
        r = torch.sigmoid(r)
        w, u = self.time_decay, self.time_first
        aa, bb = state[2], state[3]
        y = torch.empty_like(k)
        for t in range(T):
            e = torch.exp(u + w + k[t])
            y[t] = (aa + e * v[t]) / (bb + e)
            ek = torch.exp(k[t])
            aa = (aa + ek * v[t]) * torch.exp(w)
            bb = (bb + ek) * torch.exp(w)
        state[2] = aa
        state[3] = bb
        xb = x + self.attout(y * r)
        dd = self.ln2(xb)
        prev2 = torch.cat([state[1:2], dd[:-1]], dim=0)
        state[1] = dd[T - 1]
        fmix = dd.unsqueeze(0) * self.ffnmix + prev2.unsqueeze(0) * (1 - self.ffnmix)
        rf = torch.sigmoid(self.ffnreceptance(fmix[1]))
        kf = torch.relu(self.ffnkey(fmix[0]))
        return xb + rf * self.ffnvalue(kf * kf), state


class _Archive(torch.nn.Module):
    def __init__(self, w: QuantizedWeights):
        super().__init__()
        if w.emb is None or w.head is None:
            raise ValueError("export needs the whole model (embedding and head), not a pipeline stage")
        self.emb = _Emb(w.emb)
        self.ln_in, self.ln_out = _Norm(*w.ln0), _Norm(*w.ln_out)
        self.head = _Linear(w.head)
        self.blocks = torch.nn.ModuleList([_Block(ly) for ly in w.layers])
        empty = torch.zeros(w.n_layer, 5, w.n_embd, dtype=torch.float32)
        empty[:, 4] = -1e30
        self.emptyState = empty.to(torch.float64)     # built in fp32, then widened, as the reference does

    def forward(self, x: torch.Tensor, state: torch.Tensor):
        h = self.ln_in(self.emb(x))
        i = 0
        for blk in self.blocks:
            h, s = blk(h, state[i])
            state[i] = s
            i += 1
        h = self.ln_out(h)
        return self.head(h[-1:]).squeeze(), state


def export(weights: QuantizedWeights, path: str) -> str:
    """Write ``weights`` (FASTQUANT scheme) as a ``.rwkv`` TorchScript archive that stock rwkvstic
    loads with ``OptRWKV(path)`` and that ``harvest`` reads back bit-identically.  Returns the path."""
    for ly in weights.layers:
        for m in ly.mat.values():
            if m.rx is not None or m.mx is not None or m.half != 0.0:
                raise ValueError("only the FASTQUANT scheme (per-input range and offset) has an archive format")
    if not path.endswith(".rwkv"):
        path += ".rwkv"
    module = torch.jit.script(_Archive(weights).eval())
    torch.jit.save(module, path)
    return path
