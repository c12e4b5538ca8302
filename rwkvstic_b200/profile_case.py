"""Small, self-contained GEMV / GEMM workloads for profilers: ``python -m rwkvstic_b200.profile_case``.

Launches the streaming uint8 GEMV (one activation-preparation CTA + one streaming grid per
launch) on a few DISTINCT random matrices of one RWKV-4 shape, so that every launch reads
bytes that are not in L2 while the whole run holds well under 1 GB on the device.  Meant for
``ncu -k regex:stream_gemv -c 3`` style captures; prints the CUDA-event time per launch.

With ``--rows R`` (R > 1) the same matrices are applied to R activation rows through the
tensor-core path instead (row preparation + ``tile_gemm_kernel``): ``ncu -k regex:tile_gemm``.

With ``--dense bf16|fp16|fp32`` the first matrix of the shape is streamed unquantised
(``dense_gemv_kernel``), and with ``--sampler`` one row of V logits goes through the typical
sampling kernel (``sample_typical_kernel``).  ``--dense-step bf16|fp16|fp32`` runs --launches
tokens through the unquantised model of --shape (``dense_rows_kernel``, ``dense_vec_kernel``;
``--network LAYERS`` truncates it), graph-replayed, and prints the time per token; with
``--dense-rows`` it makes --launches calls of --streams x --tokens rows through the unquantised
tensor-core rows path instead (``dense_tile_gemm_kernel``, ``dense_rows_prep_kernel``).
"""
from __future__ import annotations

import argparse

import torch

from . import ops
from .quant import QuantMatrix
from .synth import SHAPES, VOCAB


def matrices(kind: str, D: int, device, copies: int):
    F = 4 * D
    shapes = {"att_kvr": [(D, D)] * 3, "att_out": [(D, D)], "ffn_kr": [(F, D), (D, D)], "ffn_value": [(D, F)],
              "head": [(VOCAB, D)]}[kind]
    g = torch.Generator(device=device).manual_seed(1)
    out = []
    for _ in range(copies):
        out.append([QuantMatrix(qt=torch.randint(0, 256, (n, k), generator=g, dtype=torch.uint8, device=device),
                                ry=torch.rand(k, generator=g, device=device) * 1e-3 + 1e-4,
                                my=torch.randn(k, generator=g, device=device) * 0.05) for n, k in shapes])
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="7b", choices=list(SHAPES))
    ap.add_argument("--matrix", default="ffn_kr", choices=["att_kvr", "att_out", "ffn_kr", "ffn_value", "head"])
    ap.add_argument("--copies", type=int, default=4, help="distinct matrix sets (4 x 84 MB > the 126 MB L2)")
    ap.add_argument("--launches", type=int, default=8)
    ap.add_argument("--rows", type=int, default=1, help="activation rows; > 1 selects the tile GEMM")
    ap.add_argument("--network", type=int, default=0, metavar="LAYERS",
                    help="instead of single matrices: a LAYERS-block model of --shape, one forward_rows call of "
                         "--streams x --tokens rows (every kernel of the rows path, for a launch list)")
    ap.add_argument("--dense", default=None, choices=["bf16", "fp16", "fp32"],
                    help="stream the first matrix of --matrix unquantised in this type (dense_gemv_kernel)")
    ap.add_argument("--dense-step", default=None, choices=["bf16", "fp16", "fp32"],
                    help="decode --launches tokens with the unquantised model of --shape in this type")
    ap.add_argument("--dense-rows", action="store_true", help="with --dense-step: --streams x --tokens rows per call through the rows path")
    ap.add_argument("--sampler", action="store_true", help="typical sampling of one row of V logits")
    ap.add_argument("--trace", default=None, choices=["chained", "persistent"],
                    help="print the %%globaltimer timeline of one block of a graph-replayed decode step of --shape "
                         "(--network LAYERS blocks, default 4) in this decode mode")
    ap.add_argument("--streams", type=int, default=8)
    ap.add_argument("--tokens", type=int, default=512)
    args = ap.parse_args()
    if args.dense_step:
        from .dense_model import B200DenseRWKV
        dt = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[args.dense_step]
        L, D = SHAPES[args.shape]
        model = B200DenseRWKV.synthetic(args.network or L, D, dtype=dt, device="cuda:0")
        if args.dense_rows:
            toks = torch.randint(0, VOCAB, (args.streams, args.tokens), generator=torch.Generator().manual_seed(3)).to("cuda:0")
            bstate = model.empty_batch_state(args.streams)
            model.forward_rows(toks, bstate)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.launches):
                model.forward_rows(toks, bstate)
            e1.record()
            torch.cuda.synchronize()
            model.check_status()
            ms = e0.elapsed_time(e1) / args.launches
            print(f"unquantised {args.dense_step} rows path, {args.shape} width, {model.n_layer} blocks, {args.streams} x {args.tokens} rows: "
                  f"{ms:.3f} ms per call, {args.streams * args.tokens / ms * 1e3:.0f} tokens/s")
            return
        state = model.emptyState.clone()
        tok = torch.tensor([17])
        for _ in range(3):                                   # the third call replays the graph
            model.forward(tok, state)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.launches):
            model._step(state, True)
        e1.record()
        torch.cuda.synchronize()
        model.check_status()
        ms = e0.elapsed_time(e1) / args.launches
        print(f"unquantised {args.dense_step} decode, {args.shape} width, {model.n_layer} blocks: {ms:.4f} ms per token, "
              f"{model.weight_bytes() / 1e9:.2f} GB of weights -> {model.weight_bytes() / ms / 1e6:.0f} GB/s; "
              f"{model.launches_per_step} launches per token")
        return
    if args.trace:
        from .model import B200RWKV
        L, D = args.network or 4, SHAPES[args.shape][1]
        model = B200RWKV.synthetic(L, D, seed=1234, device="cuda:0", decode_mode=args.trace)
        state = model.emptyState.clone()
        names = ["key/value/receptance", "attention output", "ffn key + receptance", "ffn value"]
        if args.trace == "chained":
            tr = model.trace_step(17, state, graph=True).double() / 1e3        # [4L+1, 1024, 8] us
            grid = int((tr[0, :1023, 0] > 0).sum())
            t0 = float(tr[4, 1023, 0])
            print(f"chained decode step, {args.shape} width, block 1 of {L}; us since the block's first preparation kernel started")
            print("launch | prep: entry dep stats done | gemv: dep(med) planes(med) rows(med) rows(max) epilogue(max)")
            for j in range(4):
                g, pr = tr[4 + j, :grid], tr[4 + j, 1023]
                print(f"{names[j]:22s} | {float(pr[0]) - t0:7.2f} {float(pr[1]) - t0:7.2f} {float(pr[2]) - t0:7.2f} {float(pr[3]) - t0:7.2f} | "
                      f"{float(g[:, 1].median()) - t0:7.2f} {float(g[:, 4].median()) - t0:7.2f} {float(g[:, 5].median()) - t0:7.2f} "
                      f"{float(g[:, 5].max()) - t0:7.2f} {float(g[:, 6].max()) - t0:7.2f}")
            print(f"block time: {float(tr[8, 1023, 0] - tr[4, 1023, 0]):.2f} us; whole step {float(tr[-1, :grid, 6].max() - tr[0, 1023, 0]):.1f} us")
        else:
            tr = model.trace_persistent_step(17, state).double() / 1e3        # [4L+1, grid, 8] us
            t0 = float(tr[4, :, 5].median())
            print(f"persistent decode step, {args.shape} width, block 1 of {L}; us since the block's ln1 slices were published (medians over CTAs)")
            print("launch | statistics gathered, slice published | exchange read + planes, rows summed, epilogue done")
            for j in range(4):
                g = tr[4 + j]
                st = f"{float(g[:, 4].median()) - t0:7.2f} {float(g[:, 5].median()) - t0:7.2f}" if j in (0, 2) else "      -       -"
                print(f"{names[j]:22s} | {st} | {float(g[:, 1].median()) - t0:7.2f} {float(g[:, 2].median()) - t0:7.2f} {float(g[:, 3].median()) - t0:7.2f}")
            print(f"block time: {float(tr[8, :, 5].median() - tr[4, :, 5].median()):.2f} us")
        return
    if args.network > 0:
        from .model import B200RWKV
        _, D = SHAPES[args.shape]
        model = B200RWKV.synthetic(args.network, D, seed=1234, device="cuda:0")
        toks = torch.randint(0, VOCAB, (args.streams, args.tokens), generator=torch.Generator().manual_seed(3))
        for i in range(2):
            state = model.empty_batch_state(args.streams)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            model.forward_rows(toks, state)
            e1.record()
            e1.synchronize()
            print(f"{args.network} blocks of {args.shape}, {args.streams} x {args.tokens} rows: {e0.elapsed_time(e1):.2f} ms")
        return
    dev = torch.device("cuda", 0)
    _, D = SHAPES[args.shape]
    if args.sampler:
        g = torch.Generator(device=dev).manual_seed(2)
        logits = torch.randn(VOCAB, generator=g, device=dev) * 4.0
        u = torch.rand(args.launches, generator=g, device=dev)
        times = []
        for i in range(args.launches):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            ops.sample_typical(logits, 1.0, 0.95, u=u[i:i + 1])
            e1.record()
            e1.synchronize()
            times.append(e0.elapsed_time(e1) * 1e3)
        print(f"typical sampling of {VOCAB} logits, event time per launch (us): " + " ".join(f"{t:.1f}" for t in times))
        return
    if args.dense:
        dt = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[args.dense]
        F = 4 * D
        n, k = {"att_kvr": (D, D), "att_out": (D, D), "ffn_kr": (F, D), "ffn_value": (D, F), "head": (VOCAB, D)}[args.matrix]
        g = torch.Generator(device=dev).manual_seed(1)
        ws = [(torch.randn(n, k, generator=g, device=dev) * 0.02).to(dt) for _ in range(args.copies)]
        x, y = torch.randn(k, generator=g, device=dev), torch.empty(n, device=dev)
        times = []
        for i in range(args.launches):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            ops.gemv_dense(ws[i % len(ws)], x, y)
            e1.record()
            e1.synchronize()
            times.append(e0.elapsed_time(e1) * 1e3)
        nb = n * k * ws[0].element_size()
        print(f"dense {args.dense} [{n},{k}]: {nb / 1e6:.1f} MB of weights per launch, event time per launch (us): "
              + " ".join(f"{t:.1f}" for t in times))
        return
    sets = matrices(args.matrix, D, dev, args.copies)
    R = args.rows
    if R > 1:
        xs = {D: torch.randn(R, D, device=dev), 4 * D: torch.randn(R, 4 * D, device=dev)}
    else:
        xs = {D: torch.randn(D, device=dev), 4 * D: torch.randn(4 * D, device=dev)}
    nbytes = sum(m.qt.numel() for m in sets[0])
    times = []
    for i in range(args.launches):
        mats = sets[i % len(sets)]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        if R > 1:
            ops.gemm_u8(mats, [xs[m.k_in] for m in mats])
        else:
            ops.gemv_u8(mats, [xs[m.k_in] for m in mats])
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3)
    print(f"{args.matrix} {args.shape} rows={R}: {nbytes / 1e6:.1f} MB of weights per launch, event time per launch (us): "
          + " ".join(f"{t:.1f}" for t in times))
    if R > 1:
        print(f"multiply-adds per launch: {R * nbytes / 1e9:.2f} G (x3 activation digits on the tensor cores)")


if __name__ == "__main__":
    main()
