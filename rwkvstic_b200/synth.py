"""Seeded synthetic RWKV-4 checkpoints and token schedules.

There is no network for real checkpoints, so every test and benchmark uses
random-init weights of the RWKV-4 architecture drawn from a fixed seed.  The
key names and tensor shapes are the ones the reference reads from a ``.pth``
file (rwkvstic agnostic/backends/opt.py:34-48, modules/block.py:13-47):

    emb.weight [V,D]; blocks.0.ln0.{weight,bias}; blocks.i.{ln1,ln2}.{weight,bias};
    blocks.i.att.{time_mix_k,time_mix_v,time_mix_r} [1,1,D];
    blocks.i.att.{time_decay,time_first} [D];
    blocks.i.att.{key,value,receptance,output}.weight [D,D];
    blocks.i.ffn.{time_mix_k,time_mix_r} [1,1,D];
    blocks.i.ffn.key.weight [F,D]; ffn.receptance.weight [D,D]; ffn.value.weight [D,F];
    ln_out.{weight,bias}; head.weight [V,D].

Distributions: matrices N(0, 0.02); emb N(0, 1e-4) scaled by ``emb_scale``;
layer-norm weight 1 / bias 0; time_mix_* U[0,1]; time_decay U[-5,3] (the
runtime uses w = -exp(time_decay)); time_first U[-1,1].
"""
from __future__ import annotations

from typing import Dict, Iterator, Tuple

import torch

VOCAB = 50277

# (layers, embed) of the RWKV-4 family members used as workloads.
SHAPES = {
    "169m": (12, 768),
    "1b5": (24, 2048),
    "3b": (32, 2560),
    "7b": (32, 4096),
    "14b": (40, 5120),
}


def matrix_names(layer: int) -> Tuple[str, ...]:
    p = f"blocks.{layer}."
    return (p + "att.key.weight", p + "att.value.weight", p + "att.receptance.weight",
            p + "att.output.weight", p + "ffn.key.weight", p + "ffn.receptance.weight",
            p + "ffn.value.weight")


def iter_synth_tensors(layers: int, embed: int, vocab: int = VOCAB, seed: int = 1234,
                       ffn: int | None = None, emb_scale: float = 1.0,
                       device: str = "cpu") -> Iterator[Tuple[str, torch.Tensor]]:
    """Yield (name, tensor) in a fixed order from one seeded generator.

    A generator so that 7B/14B shapes can be quantised matrix by matrix
    without ever holding the fp32 checkpoint (28 GB at 7B)."""
    ffn = 4 * embed if ffn is None else ffn
    g = torch.Generator(device=device)
    g.manual_seed(seed)

    def normal(*shape, std):
        return torch.randn(*shape, generator=g, device=device, dtype=torch.float32) * std

    def uniform(*shape, lo, hi):
        return torch.rand(*shape, generator=g, device=device, dtype=torch.float32) * (hi - lo) + lo

    ones = lambda n: torch.ones(n, device=device, dtype=torch.float32)
    zeros = lambda n: torch.zeros(n, device=device, dtype=torch.float32)

    yield "emb.weight", normal(vocab, embed, std=1e-4) * emb_scale
    yield "blocks.0.ln0.weight", ones(embed)
    yield "blocks.0.ln0.bias", zeros(embed)
    for i in range(layers):
        p = f"blocks.{i}."
        yield p + "ln1.weight", ones(embed)
        yield p + "ln1.bias", zeros(embed)
        yield p + "ln2.weight", ones(embed)
        yield p + "ln2.bias", zeros(embed)
        yield p + "att.time_mix_k", uniform(1, 1, embed, lo=0.0, hi=1.0)
        yield p + "att.time_mix_v", uniform(1, 1, embed, lo=0.0, hi=1.0)
        yield p + "att.time_mix_r", uniform(1, 1, embed, lo=0.0, hi=1.0)
        yield p + "att.time_decay", uniform(embed, lo=-5.0, hi=3.0)
        yield p + "att.time_first", uniform(embed, lo=-1.0, hi=1.0)
        yield p + "att.key.weight", normal(embed, embed, std=0.02)
        yield p + "att.value.weight", normal(embed, embed, std=0.02)
        yield p + "att.receptance.weight", normal(embed, embed, std=0.02)
        yield p + "att.output.weight", normal(embed, embed, std=0.02)
        yield p + "ffn.time_mix_k", uniform(1, 1, embed, lo=0.0, hi=1.0)
        yield p + "ffn.time_mix_r", uniform(1, 1, embed, lo=0.0, hi=1.0)
        yield p + "ffn.key.weight", normal(ffn, embed, std=0.02)
        yield p + "ffn.receptance.weight", normal(embed, embed, std=0.02)
        yield p + "ffn.value.weight", normal(embed, ffn, std=0.02)
    yield "ln_out.weight", ones(embed)
    yield "ln_out.bias", zeros(embed)
    yield "head.weight", normal(vocab, embed, std=0.02)


def synth_checkpoint(layers: int, embed: int, vocab: int = VOCAB, seed: int = 1234,
                     ffn: int | None = None, emb_scale: float = 1.0) -> Dict[str, torch.Tensor]:
    """Whole fp32 checkpoint on the CPU (small shapes only)."""
    return dict(iter_synth_tensors(layers, embed, vocab, seed, ffn, emb_scale, "cpu"))


def synth_tokens(n: int, seed: int = 7, vocab: int = VOCAB) -> torch.Tensor:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g, dtype=torch.int64)
