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
