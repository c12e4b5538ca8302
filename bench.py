#!/usr/bin/env python
"""Benchmark of the hot path: RWKV-4 7B-shape uint8 batch-1 decode, tokens/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--shape 7b]

One "step" is one decode step (one token through 32 layers + head) of one stream per GPU.
With N > 1 (launched by torchrun, one rank per GPU) every rank holds a replica of the
weights and decodes its own stream: data-parallel replicas, no collective on the data path
(weak scaling).  Rank 0 prints ONE JSON line.

Keys beyond the basic contract:
  e2e        tokens/s through the public API with HOST tokens: per step an H2D copy of the
             token from pinned memory, the forward, a D2H copy of the logits, host argmax.
  roofline   HBM roofline of the streaming GEMV kernel (4L+1 = 129 launches per step; the one-CTA
             activation-preparation kernels run beside them on the SM the GEMV grid leaves
             free): algorithmic bytes per launch / average launch duration vs the measured
             copy bandwidth of this pool's B200s.
  kernels    the same kernel timed alone (CUDA events around single launches), per matrix shape.
  decode_1b5 the same batch-1 decode at the 1.5B shape (the configuration whose purpose is the GEMV's
             HBM bandwidth when the launch chain, not the stream, dominates).
  batched_decode, prefill
             256 streams per GPU / the 3B 8 x 1024 prompt through the tensor-core rows path; each with
             library_baseline = the reference's own GPU formulation of the same matrices (cast the
             uint8 weights to bf16, cuBLAS GEMM: modules/matmul.py:57, :87-89) timed with stock torch on
             the same box - a comparison only, never on the product path.
  split_decode, layer_split (N > 1), config4_one_gpu (N = 1)
             256 streams SPLIT over the ranks (strong scaling, no collective); the 14B shape with its
             blocks partitioned over the ranks (NCCL point-to-point hand-off), and the same model on one GPU.
  cpu_baseline / --impl reference
             the CPU oracle (a port of the reference's FASTQUANT CPU path) timed on the host cores:
             the whole 169M-shape schedule (32 prompt + 64 greedy tokens), and a bounded sample at
             the 7B shape (one block + the head, extrapolated to 32 blocks; "extrapolated": true).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

from rwkvstic_b200.synth import SHAPES, VOCAB  # noqa: E402

METRIC = "rwkv4_7b_int8_decode_tokens_per_s_b1"
UNIT = "tokens/s"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (earlier measurement on this pool)"


def measured_traffic_ratio():
    """DRAM (read + write) bytes of one stream_gemv_kernel launch over its algorithmic bytes, as the
    committed ncu summary of the current build states it (line `traffic_ratio = X`)."""
    import re
    path = os.path.join(ROOT, "profiles", "stream_gemv_kernel_7b_ffn_key_rec_ncu.md")
    try:
        with open(path) as f:
            m = re.search(r"traffic_ratio\s*=\s*([0-9.]+)", f.read())
        return (float(m.group(1)), os.path.relpath(path, ROOT)) if m else (None, None)
    except OSError:
        return None, None


def decode_bytes_per_token(L, D, V=VOCAB, F=None):
    """Algorithmic HBM bytes of one decode step: uint8 weights + fp32 scale/offset per input
    feature of every matrix + fp32 vector parameters + state read and write + embedding row."""
    F = 4 * D if F is None else F
    w8 = L * (5 * D * D + 2 * D * F) + V * D
    quant_vec = L * 8 * (6 * D + F) + 8 * D
    vec = L * 44 * D + 16 * D
    state = 40 * D * L
    return w8, w8 + quant_vec + vec + state + 4 * D


# ----------------------------------------------------------------------------------- clocks
class ClockSampler:
    FIELDS = ("timestamp,index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.path = tempfile.mktemp(prefix="clocks_", suffix=".csv")
        self.proc = None
        self.windows = []   # (start, end) wall-clock seconds of the timed regions

    def window(self, start, end):
        self.windows.append((start, end))

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self, gpu_indices):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        import datetime
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        rows = []
        with open(self.path) as f:
            for line in f:
                p = [c.strip() for c in line.split(",")]
                if len(p) < 10 or not p[1].isdigit() or int(p[1]) not in gpu_indices:
                    continue
                try:
                    ts = datetime.datetime.strptime(p[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                    rows.append((ts, float(p[2]), float(p[3]), [n for n, v in zip(names, p[6:10]) if v.lower().startswith("active")]))
                except ValueError:
                    continue
        os.unlink(self.path)
        inside = [r for r in rows if any(a <= r[0] <= b for a, b in self.windows)]
        scope = "inside the timed regions"
        if not inside and self.windows:   # regions shorter than the sampling period: take the span around them
            lo, hi = min(a for a, _ in self.windows) - 0.3, max(b for _, b in self.windows) + 0.3
            inside = [r for r in rows if lo <= r[0] <= hi]
            scope = "within 0.3 s of the timed regions (regions shorter than the sampling period)"
        if not inside:
            inside, scope = rows, "whole run"
        sm = [r[1] for r in inside]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max((r[2] for r in inside), default=None),
                "samples": len(sm), "scope": scope, "reasons": sorted({n for r in inside for n in r[3]})}


# ----------------------------------------------------------------------------------- CPU reference arm
def cpu_full_schedule(layers, embed, prompt_len, decode_steps, vocab=VOCAB):
    """The oracle through a whole schedule (prompt in sequence mode, then greedy decode), timed."""
    from oracle.fastquant_oracle import OracleRWKV
    from rwkvstic_b200.synth import synth_checkpoint, synth_tokens
    t0 = time.perf_counter()
    model = OracleRWKV(synth_checkpoint(layers, embed, vocab=vocab, seed=1234))
    t_load = time.perf_counter() - t0
    state = model.emptyState.clone()
    t0 = time.perf_counter()
    logits, state = model.forward(synth_tokens(prompt_len, seed=38, vocab=vocab), state)
    t_prompt = time.perf_counter() - t0
    t0 = time.perf_counter()
    for _ in range(decode_steps):
        logits, state = model.forward(torch.tensor([int(torch.argmax(logits))]), state)
    t_dec = time.perf_counter() - t0
    return {"shape": f"L={layers} D={embed} V={vocab}", "load_quantise_s": t_load, "prompt_tokens": prompt_len, "prompt_s": t_prompt,
            "decode_steps": decode_steps, "decode_tokens_per_s": decode_steps / t_dec, "extrapolated": False}


def cpu_reference(shape, steps, warmup, with_1b5=False):
    """tokens/s of the CPU oracle at this shape, from a bounded sample (one block + head)."""
    from oracle.fastquant_oracle import OracleRWKV
    from rwkvstic_b200.synth import synth_checkpoint
    L, D = SHAPES[shape]
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    ck = synth_checkpoint(1, D, seed=1234)
    model = OracleRWKV(ck)
    del ck
    state = model.emptyState.clone()
    x = torch.randn(1, D, dtype=torch.float64)
    tok = torch.tensor([17])
    for _ in range(max(1, min(warmup, 2))):
        model.forward(tok, state)
        model.head(x)
    n = max(2, min(steps, 8))
    t0 = time.perf_counter()
    for _ in range(n):
        model.forward(tok, state)
    t_model = (time.perf_counter() - t0) / n
    t0 = time.perf_counter()
    for _ in range(n):
        model.head(x)
    t_head = (time.perf_counter() - t0) / n
    t_block = max(t_model - t_head, 1e-9)
    t_token = L * t_block + t_head
    del model
    # whole schedules where they fit the time budget: the 169M shape in full; the 1.5B shape (reference arm
    # only) with its 64-token prompt and a bounded number of decode steps
    full = {"169m": cpu_full_schedule(*SHAPES["169m"], 32, 64)}
    if with_1b5:
        full["1b5"] = cpu_full_schedule(*SHAPES["1b5"], 64, 8)
        full["1b5"]["note"] = "64-token prompt in full, 8 of the 512 decode steps"
    return {"value": 1.0 / t_token, "unit": UNIT, "cores": cores, "kind": "port", "extrapolated": True,
            "sample": f"oracle port of the reference FASTQUANT CPU path (uint8 weights cast to fp32 per call, "
                      f"fp32 matmul, fp64 vectors), {n} decode steps of a 1-block D={D} model + head: "
                      f"{t_block * 1e3:.1f} ms/block, {t_head * 1e3:.1f} ms/head, extrapolated to {L} blocks",
            "full_schedules": full}


def run_reference(args, rank):
    if rank != 0:
        return
    L, D = SHAPES[args.shape]
    base = cpu_reference(args.shape, args.steps, args.warmup, with_1b5=True)
    line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 / base["value"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8 weights, f32 matmul, f64 vectors",
            "data": "synthetic", "config": {"workload": f"RWKV-4 {args.shape} shape L={L} D={D} V={VOCAB}, batch-1 decode",
                                            "note": "CPU path of the reference; GPUs unused"},
            "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------- our arm
def time_isolated_kernels(model, reps=5):
    """Per matrix group: GB/s of the GEMV launches of all layers replayed back to back from a CUDA
    graph (one activation-preparation CTA + one streaming grid per launch), timed with CUDA
    events.  Successive launches walk over the layers, so each reads bytes that are not in L2;
    the head (a single matrix) is preceded by an L2 flush instead."""
    from rwkvstic_b200 import ops
    dev = model.device
    out = {}
    D, F = model.n_embd, model.n_ffn
    xs = {D: torch.randn(D, device=dev), F: torch.randn(F, device=dev)}
    groups = {"att_kvr 3x[D,D]": [[ly.mat[k] for k in ("att.key", "att.value", "att.receptance")] for ly in model.w.layers],
              "att_out [D,D]": [[ly.mat["att.output"]] for ly in model.w.layers],
              "ffn_key+rec [4D,D]+[D,D]": [[ly.mat["ffn.key"], ly.mat["ffn.receptance"]] for ly in model.w.layers],
              "ffn_value [D,4D]": [[ly.mat["ffn.value"]] for ly in model.w.layers],
              "head [V,D]": [[model.w.head]]}
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for name, launches in groups.items():
        ys = [torch.empty(m.n_out, device=dev) for m in launches[0]]
        nbytes = sum(m.qt.numel() for m in launches[0])

        def run():
            for mats in launches:
                ops.gemv_u8(mats, [xs[m.k_in] for m in mats], ys)
        run()                                            # also builds the cached workspace
        torch.cuda.synchronize(dev)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            run()
        times = []
        for r in range(reps):
            if len(launches) == 1:
                flush.fill_(r)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            e1.synchronize()
            times.append(e0.elapsed_time(e1) / len(launches))
        t = statistics.median(times)
        out[name] = {"bytes": nbytes, "us": round(t * 1e3, 2), "gbs": round(nbytes / t / 1e6, 1)}
    return out


def measured_tensor_peak():
    """Dense bf16 TFLOP/s measured on this pool (burst figure), or the stated fallback."""
    try:
        with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["bf16_tflops"])
    except Exception:
        return 1590.0


def matrix_params(L, D, V=VOCAB):
    """Matrix elements every activation row is multiplied with (7 matrices per block + head)."""
    F = 4 * D
    return L * (4 * D * D + 2 * D * F + D * D) + V * D


def library_baseline_ms(model, rows, head_rows=None, reps=3):
    """The reference's own GPU formulation of the network's matrices for `rows` activation rows
    (modules/matmul.py:57, :87-89): scale the activations by `range`, cast them and the uint8 weights
    to bf16, one cuBLAS GEMM per matrix, plus the offset term; timed with stock torch over all
    blocks + head.  A comparison figure (how fast the library path is on this box), not a product path."""
    dev = model.device
    D, F = model.n_embd, model.n_ffn
    xs = {D: torch.randn(rows, D, device=dev), F: torch.randn(rows, F, device=dev)}

    def one_pass():
        for ly in model.w.layers:
            for m in ly.mat.values():
                x = xs[m.k_in]
                y = ((x * m.ry).to(torch.bfloat16) @ m.qt.to(torch.bfloat16).t()).float()     # qt is [out][in]
                y += (x @ m.my).unsqueeze(1)
        h = model.w.head
        x = xs[D][:head_rows if head_rows else rows]
        y = ((x * h.ry).to(torch.bfloat16) @ h.qt.to(torch.bfloat16).t()).float()
        y += (x @ h.my).unsqueeze(1)
    one_pass()
    times = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(dev)
        e0.record()
        one_pass()
        e1.record()
        torch.cuda.synchronize(dev)
        times.append(e0.elapsed_time(e1))
    return statistics.median(times)


def time_decode_shape(shape, dev, steps=128, warm=8):
    """Batch-1 decode at another shape (graph-replayed steps, tokens resident): tokens/s and roofline."""
    from rwkvstic_b200.model import B200RWKV
    L, D = SHAPES[shape]
    model = B200RWKV.synthetic(L, D, seed=1234, device=dev, copy_logits=False)
    toks = torch.randint(0, VOCAB, (steps + warm,), generator=torch.Generator().manual_seed(11), dtype=torch.int64).to(dev)
    state = model.emptyState.clone()
    for i in range(warm):
        model.forward(toks[i:i + 1], state)
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(warm, warm + steps):
        model.forward(toks[i:i + 1], state)
    e1.record()
    torch.cuda.synchronize(dev)
    model.check_status()
    ms = e0.elapsed_time(e1) / steps
    _, total = decode_bytes_per_token(L, D)
    peak, _ = measured_peaks()
    gbs = total / (ms * 1e-3) / 1e9
    return {"workload": f"RWKV-4 {shape} shape L={L} D={D} V={VOCAB}, batch-1 decode", "value": 1e3 / ms, "unit": UNIT,
            "ms_per_step": ms, "steps": steps,
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                         "frac_of_nominal_8TBs": gbs / 8000.0}}


def time_dense_decode(shape, dev, dtype=torch.bfloat16, steps=64, warm=6):
    """Batch-1 decode with UNQUANTISED weights (the reference's TORCH mode) at `shape`: tokens/s, the HBM
    roofline at sizeof(dtype) bytes per weight, and beside it the same matrices through stock torch
    (one cuBLAS ``torch.mv`` per matrix, no vector work) as the library baseline."""
    from rwkvstic_b200.dense_model import B200DenseRWKV
    L, D = SHAPES[shape]
    model = B200DenseRWKV.synthetic(L, D, seed=1234, dtype=dtype, device=dev)
    toks = torch.randint(0, VOCAB, (steps + warm,), generator=torch.Generator().manual_seed(12), dtype=torch.int64).to(dev)
    state = model.emptyState.clone()
    for i in range(warm):
        model.forward(toks[i:i + 1], state)
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(warm, warm + steps):
        model._tok.copy_(toks[i:i + 1])
        model._step(state, True)
    e1.record()
    torch.cuda.synchronize(dev)
    model.check_status()
    ms = e0.elapsed_time(e1) / steps
    wbytes = model.weight_bytes()
    peak, _ = measured_peaks()
    gbs = wbytes / (ms * 1e-3) / 1e9
    mats = [v for k, v in model.t.items() if v.dim() == 2 and k != "emb.weight"]
    xs = {n: torch.randn(n, device=dev).to(dtype) for n in {m.shape[1] for m in mats}}
    for m in mats[:8]:
        torch.mv(m, xs[m.shape[1]])
    torch.cuda.synchronize(dev)
    e0.record()
    for _ in range(3):
        for m in mats:
            torch.mv(m, xs[m.shape[1]])
    e1.record()
    torch.cuda.synchronize(dev)
    lib_ms = e0.elapsed_time(e1) / 3
    name = str(dtype).replace("torch.", "")
    prompt = None
    if dtype != torch.float32:
        # a 1024-token prompt through the tensor-core rows path, and the same matrices through cuBLAS
        ptoks = torch.randint(0, VOCAB, (1, 1024), generator=torch.Generator().manual_seed(13), dtype=torch.int64).to(dev)
        pstate = model.empty_batch_state(1)
        model.forward_rows(ptoks, pstate)
        torch.cuda.synchronize(dev)
        e0.record()
        for _ in range(3):
            model.forward_rows(ptoks, pstate)
        e1.record()
        torch.cuda.synchronize(dev)
        model.check_status()
        p_ms = e0.elapsed_time(e1) / 3
        blocks = [m for m in mats if m.shape[0] != VOCAB]
        rows = {n: torch.randn(1024, n, device=dev).to(dtype) for n in {m.shape[1] for m in blocks}}
        for m in blocks[:4]:
            torch.matmul(rows[m.shape[1]], m.t())
        torch.cuda.synchronize(dev)
        e0.record()
        for _ in range(3):
            for m in blocks:
                torch.matmul(rows[m.shape[1]], m.t())
        e1.record()
        torch.cuda.synchronize(dev)
        plib_ms = e0.elapsed_time(e1) / 3
        flops = 2.0 * sum(m.numel() for m in blocks) * 1024 + 2.0 * VOCAB * D
        tf_peak = measured_tensor_peak()
        prompt = {"tokens": 1024, "ms": p_ms, "tokens_per_s": 1024 / (p_ms * 1e-3), "kernel": "dense_tile_gemm_kernel (tcgen05 kind::f16)",
                  "tensor": {"algorithmic_tflops": flops / (p_ms * 1e-3) / 1e12, "peak_bf16_tflops": tf_peak,
                             "frac_of_measured_bf16": flops / (p_ms * 1e-3) / 1e12 / tf_peak if tf_peak else None},
                  "library_baseline": {"what": "the blocks' matrices through torch.matmul (cuBLAS) on 1024 rows, no layer norm / "
                                               "mix / WKV work", "ms": plib_ms, "ours_over_library": p_ms / plib_ms}}
    return {"workload": f"RWKV-4 {shape} shape L={L} D={D} V={VOCAB}, {name} weights unquantised (TORCH mode), batch-1 decode",
            "prompt_1024": prompt,
            "value": 1e3 / ms, "unit": UNIT, "ms_per_step": ms, "steps": steps, "dtype": name,
            "gpu_launches_per_step": model.launches_per_step, "kernel": "dense_rows_kernel + dense_vec_kernel",
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                         "algorithmic_bytes_per_step": wbytes},
            "library_baseline": {"what": "the same matrices through torch.mv (cuBLAS), one call per matrix, no layer norm / "
                                         "mix / WKV work; stock torch, same box", "ms_per_step": lib_ms,
                                 "ours_over_library": ms / lib_ms}}


def trace_spans(model, dev):
    """Mean over the 4L+1 GEMV launches of a graph-replayed traced step: from "launch dependency resolved"
    (median over CTAs) to "epilogue done" (last CTA) = the launch's working span, and from "digit planes
    in shared memory" to "all rows summed" (medians) = the part in which weights stream."""
    state = model.emptyState.clone()
    tr = model.trace_step(17, state, graph=True).double()          # [4L+1, 1024, 8] ns
    grid = int((tr[0, :1023, 0] > 0).sum())
    g = tr[:, :grid]
    dep, planes, rows, epi = g[:, :, 1].median(dim=1).values, g[:, :, 4].median(dim=1).values, g[:, :, 5].median(dim=1).values, g[:, :, 6].max(dim=1).values
    return {"launch_us": float((epi - dep).mean() / 1e3), "stream_us": float((rows - planes).mean() / 1e3),
            "step_us_in_trace": float((g[-1, :, 6].max() - tr[0, 1023, 0]) / 1e3), "grid": grid}


def time_config4_one_gpu(dev, streams=64, steps=16):
    """The 14B shape whole on one GPU: `streams`-stream decode and a 2048-token prompt (512-token pieces),
    the figures the layer split over several GPUs is to be read against."""
    from rwkvstic_b200.model import B200RWKV
    L, D = SHAPES["14b"]
    model = B200RWKV.synthetic(L, D, seed=1234, device=dev, copy_logits=False)
    tok = torch.randint(0, VOCAB, (streams, 1), generator=torch.Generator().manual_seed(5), dtype=torch.int64).to(dev)
    state = model.empty_batch_state(streams)
    for _ in range(3):
        tok = model.forward_rows(tok, state).argmax(dim=1, keepdim=True)
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        tok = model.forward_rows(tok, state).argmax(dim=1, keepdim=True)
    e1.record()
    torch.cuda.synchronize(dev)
    dec_ms = e0.elapsed_time(e1) / steps
    prompt = torch.randint(0, VOCAB, (1, 2048), generator=torch.Generator().manual_seed(6), dtype=torch.int64).to(dev)
    model.rows_per_call = 512
    pst = model.empty_batch_state(1)
    model.forward_rows(prompt, pst)
    torch.cuda.synchronize(dev)
    e0.record()
    model.forward_rows(prompt, model.empty_batch_state(1))
    e1.record()
    torch.cuda.synchronize(dev)
    model.check_rows_status()
    pre_ms = e0.elapsed_time(e1)
    # one stream, one token per step: the one-row streaming path
    st1 = model.emptyState.clone()
    t1 = torch.tensor([7], dtype=torch.int64, device=dev)
    for _ in range(4):
        model.forward(t1, st1)
    torch.cuda.synchronize(dev)
    e0.record()
    for _ in range(32):
        model.forward(t1, st1)
    e1.record()
    torch.cuda.synchronize(dev)
    model.check_status()
    b1_ms = e0.elapsed_time(e1) / 32
    return {"workload": f"RWKV-4 14b shape L={L} D={D}, all blocks on one GPU", "streams": streams, "decode_ms_per_step": dec_ms,
            "decode_tokens_per_s": streams / (dec_ms * 1e-3), "prefill_tokens": 2048, "prefill_ms": pre_ms,
            "prefill_tokens_per_s": 2048 / (pre_ms * 1e-3), "b1_decode_ms_per_step": b1_ms}


def time_layer_split(rank, world, dev, streams=64, steps=16):
    """The 14B shape with its blocks partitioned over the ranks: decode of `streams` streams and a
    2048-token prompt in 512-token pieces.  CUDA events, max over ranks."""
    import torch.distributed as dist
    from rwkvstic_b200 import layer_split as LS
    from rwkvstic_b200.synth import iter_synth_tensors
    L, D = SHAPES["14b"]
    model = LS.build_stage(iter_synth_tensors(L, D, VOCAB, 1234, device=str(dev)), rank, world, L, dev)
    pipe = LS.make_pipeline(model, rank, world)

    def timed(fn):
        torch.cuda.synchronize(dev); dist.barrier(); torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize(dev); dist.barrier()
        t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    state = LS.empty_stage_state(model, streams)
    tok = torch.randint(0, VOCAB, (streams, 1), generator=torch.Generator().manual_seed(5), dtype=torch.int64)
    pipe.decode_greedy(tok, state, 3, 1)
    dec_ms = timed(lambda: pipe.decode_greedy(tok, state, steps, 1)) / steps
    pstate = LS.empty_stage_state(model, 1)
    prompt = torch.randint(0, VOCAB, (1, 2048), generator=torch.Generator().manual_seed(6), dtype=torch.int64).to(dev)
    pipe.rows_per_item = 512
    pipe.forward_rows(prompt, pstate)
    pre_ms = timed(lambda: pipe.forward_rows(prompt, pstate))
    model.check_rows_status()
    # one stream, one token per step: every stage runs the one-row streaming step on its blocks
    s1 = LS.empty_stage_state(model, 1)
    one = torch.full((1, 1), 7, dtype=torch.int64)
    pipe.decode_greedy(one, s1, 3, 1)
    b1_ms = timed(lambda: pipe.decode_greedy(one, s1, 32, 1)) / 32
    model.check_status()
    del model, pipe, state, pstate, s1
    torch.cuda.empty_cache()
    return {"workload": f"RWKV-4 14b shape L={L} D={D}, blocks split contiguously over {world} GPUs, {streams} streams, "
                        "one stream group", "decode_ms_per_step": dec_ms, "decode_tokens_per_s": streams / (dec_ms * 1e-3),
            "prefill_tokens": 2048, "prefill_ms": pre_ms, "prefill_tokens_per_s": 2048 / (pre_ms * 1e-3),
            "b1_decode_ms_per_step": b1_ms,
            "handoff": "NCCL send/recv of the fp32 residual stream [rows, D] between consecutive ranks; sampled ids last -> first rank",
            "limit": "a decode step is a chain through all stages (each streams its blocks' weights once), so the split adds "
                     "capacity, not decode speed; the prompt's 512-token pieces pipeline across the stages"}


def time_split_decode(model, rank, world, dev, total_streams=256, steps=16):
    """A fixed total of `total_streams` independent streams SPLIT over the ranks
    (strong scaling), each rank decoding its shard on a replica; no collective on the data path."""
    import torch.distributed as dist
    from rwkvstic_b200.parallel import decode_sharded, stream_shard
    shard = stream_shard(total_streams, world, rank)
    gen = torch.Generator().manual_seed(21)
    toks = torch.randint(0, VOCAB, (total_streams, 1), generator=gen, dtype=torch.int64).to(dev)
    state = model.empty_batch_state(total_streams)[shard.start:shard.stop].contiguous()
    full_state_view = {"s": state}

    def step(tk):
        lg = model.forward_rows(tk, full_state_view["s"])
        return lg.argmax(dim=1, keepdim=True)
    tk = toks[shard.start:shard.stop].contiguous()
    for _ in range(3):
        tk = step(tk)
    torch.cuda.synchronize(dev); dist.barrier(); torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        tk = step(tk)
    e1.record()
    torch.cuda.synchronize(dev); dist.barrier()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t[0]) / steps
    return {"total_streams": total_streams, "streams_per_gpu": len(shard), "ms_per_step": ms,
            "value": total_streams / (ms * 1e-3), "unit": UNIT, "scaling": "strong",
            "api": "parallel.stream_shard + B200RWKV.forward_rows on each rank's shard (the kernels of parallel.decode_sharded)"}


def time_prefill(dev, tf_peak, B=8, T=1024):
    """Prompt ingestion at the 3B shape: B streams x T tokens in sequence mode through forward_rows."""
    from rwkvstic_b200.model import B200RWKV
    L, D = SHAPES["3b"]
    model = B200RWKV.synthetic(L, D, seed=1234, device=dev, copy_logits=False)
    toks = torch.randint(0, VOCAB, (B, T), generator=torch.Generator().manual_seed(7), dtype=torch.int64).to(dev)
    times = []
    for i in range(4):
        state = model.empty_batch_state(B)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(dev)
        e0.record()
        model.forward_rows(toks, state)
        e1.record()
        torch.cuda.synchronize(dev)
        if i:
            times.append(e0.elapsed_time(e1))
    ms = statistics.median(times)
    alg = 2.0 * (matrix_params(L, D) - VOCAB * D) * B * T / (ms * 1e-3) / 1e12   # the head runs on B rows only
    lib_ms = library_baseline_ms(model, B * T, head_rows=B, reps=2)
    return {"workload": f"RWKV-4 3b shape L={L} D={D}, {B} streams x {T} tokens, sequence mode", "ms": ms,
            "value": B * T / (ms * 1e-3), "unit": UNIT, "rows_per_call": model.rows_per_call,
            "tensor": {"algorithmic_tflops": alg, "peak_bf16_tflops": tf_peak, "frac_of_measured_bf16": alg / tf_peak},
            "library_baseline": {"what": "matrices only (all blocks + the head on the last rows): activations * range and uint8 weights "
                                         "cast to bf16 per call, cuBLAS GEMM, offset term; stock torch, same box",
                                 "ms": lib_ms, "ours_over_library": ms / lib_ms}}


def run_layer_split(args, rank, world, local_rank):
    """14B shape with its blocks partitioned contiguously over the ranks (launch with torchrun):
    64-stream decode and a 2048-token prompt; the residual stream hops GPUs over NCCL point-to-point."""
    import torch.distributed as dist
    from rwkvstic_b200 import layer_split as LS
    from rwkvstic_b200.synth import iter_synth_tensors

    L, D = SHAPES[args.shape]
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    model = LS.build_stage(iter_synth_tensors(L, D, VOCAB, 1234, device=str(dev)), rank, world, L, dev)
    pipe = LS.make_pipeline(model, rank, world)
    Bs, K, W, mb = args.streams, args.steps, max(args.warmup, 3), args.microbatches

    def timed(fn):
        torch.cuda.synchronize(dev); dist.barrier(); torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize(dev); dist.barrier()
        t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    state = LS.empty_stage_state(model, Bs)
    tok = torch.randint(0, VOCAB, (Bs, 1), generator=torch.Generator().manual_seed(5), dtype=torch.int64)
    pipe.decode_greedy(tok, state, W, mb)
    decode_ms = timed(lambda: pipe.decode_greedy(tok, state, K, mb))
    pstate = LS.empty_stage_state(model, 1)
    prompt = torch.randint(0, VOCAB, (1, 2048), generator=torch.Generator().manual_seed(6), dtype=torch.int64).to(dev)
    pipe.rows_per_item = 512
    pipe.forward_rows(prompt, pstate)
    prefill_ms = timed(lambda: pipe.forward_rows(prompt, pstate))
    model.check_rows_status()
    if rank == 0:
        print(json.dumps({
            "metric": "rwkv4_14b_layer_split_decode_tokens_per_s_b64", "value": Bs * K / (decode_ms * 1e-3), "unit": UNIT,
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": decode_ms / K, "higher_is_better": True,
            "scaling": "strong", "dtype": "u8", "data": "synthetic",
            "config": {"workload": f"RWKV-4 {args.shape} shape L={L} D={D}, blocks split contiguously over {world} GPUs, "
                                   f"{Bs} streams in {mb} micro-batches, greedy decode",
                       "handoff": "NCCL send/recv of the fp32 residual stream [rows, D] between consecutive ranks",
                       "timing": "CUDA events, max over ranks"},
            "prefill": {"tokens": 2048, "ms": prefill_ms, "value": 2048 / (prefill_ms * 1e-3), "unit": UNIT,
                        "tokens_per_piece": 512}}), flush=True)
    dist.destroy_process_group()


def run_ours(args, rank, world, local_rank):
    import torch.distributed as dist
    from rwkvstic_b200.model import B200RWKV

    L, D = SHAPES[args.shape]
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    model = B200RWKV.synthetic(L, D, seed=1234, device=dev, copy_logits=False)
    K, W = args.steps, max(args.warmup, 3)
    gen = torch.Generator().manual_seed(100 + rank)
    host_tokens = torch.randint(0, VOCAB, (K + W,), generator=gen, dtype=torch.int64).pin_memory()
    dev_tokens = host_tokens.to(dev)

    def barrier():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # ---- device-resident loop: tokens already in HBM, logits stay in HBM
    sampler = ClockSampler()
    if rank == 0:
        sampler.start()
    state = model.emptyState.clone()
    for i in range(W):
        model.forward(dev_tokens[i:i + 1], state)
    barrier()
    launches0 = model.launch_count
    w0 = time.time()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(W, W + K):
        model.forward(dev_tokens[i:i + 1], state)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    sampler.window(w0, time.time())
    launches = model.launch_count - launches0
    model.check_status()

    # ---- end to end through the public API with host buffers: every step copies its input token
    # from pinned host memory, runs the step, takes the arg-max on the device and reads the
    # sampled id (the step's result) back to the host, which feeds it to the next step
    state = model.emptyState.clone()
    tok = host_tokens[:1].clone().pin_memory()
    nxt = torch.zeros(1, dtype=torch.int64).pin_memory()

    def e2e_step():
        model.step_greedy(tok, state, nxt)               # H2D of the token, step + arg-max, D2H of the sampled id, sync
        tok[0] = int(nxt[0])                             # greedy feedback through the host

    for i in range(W):
        e2e_step()
    barrier()
    w0 = time.time()
    t0 = time.perf_counter()
    for i in range(K):
        e2e_step()
    torch.cuda.synchronize(dev)
    e2e_ms = (time.perf_counter() - t0) * 1e3
    sampler.window(w0, time.time())
    model.check_status()

    # ---- batched decode: B independent streams per GPU through the tensor-core rows path, greedy
    # feedback on the device (tokens and logits never leave HBM)
    Bs, Kb = args.streams, max(4, min(K, 32))
    bstate = model.empty_batch_state(Bs)
    btok = torch.randint(0, VOCAB, (Bs, 1), generator=gen, dtype=torch.int64).to(dev)
    for i in range(3):
        btok = model.forward_rows(btok, bstate).argmax(dim=1, keepdim=True)
    barrier()
    b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches_b0 = model.launch_count
    w0 = time.time()
    b0.record()
    for i in range(Kb):
        btok = model.forward_rows(btok, bstate).argmax(dim=1, keepdim=True)
    b1.record()
    barrier()
    batched_ms = b0.elapsed_time(b1)
    sampler.window(w0, time.time())
    clocks = sampler.stop(set(range(world))) if rank == 0 else None
    launches_b = model.launch_count - launches_b0
    del bstate
    model.check_rows_status()
    extra = {}
    if world > 1:
        extra["split_decode"] = time_split_decode(model, rank, world, dev, total_streams=args.streams)

    if world > 1:
        t = torch.tensor([ms, e2e_ms, batched_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms, batched_ms = float(t[0]), float(t[1]), float(t[2])
        cnt = torch.tensor([launches], device=dev, dtype=torch.int64)
        dist.all_reduce(cnt)
        launches = int(cnt[0])

    if rank == 0:
        w8, total_bytes = decode_bytes_per_token(L, D)
        peak, peak_src = measured_peaks()
        step_ms = ms / K
        n_gemv = 4 * L + 1   # streaming GEMV launches per step; the preparation CTAs run beside them
        traffic_ratio, traffic_src = measured_traffic_ratio()
        achieved = total_bytes / (step_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": world * K / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": step_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8",
            "data": "synthetic",
            "config": {"workload": f"RWKV-4 {args.shape} shape L={L} D={D} F={4 * D} V={VOCAB}, uint8 FASTQUANT weights, "
                                   f"batch-1 decode, one stream per GPU (data-parallel replicas)",
                       "l2": f"no flush needed: every step streams {w8 / 1e9:.2f} GB of weights, far larger than the 126 MB L2",
                       "timing": "CUDA events on the launching stream, max over ranks"},
            "e2e": {"value": world * K / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": 8,
                    "d2h_bytes_per_step": 8, "api": "B200RWKV.step_greedy (token in from pinned host memory, greedy id read back per step)"},
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         # DRAM read + write bytes per launch: algorithmic bytes x the ratio the committed ncu
                         # summary of one 83.9 MB launch of the current build states (traffic grows with the bytes streamed)
                         "traffic": (traffic_ratio * total_bytes / n_gemv) if traffic_ratio else None,
                         "traffic_source": traffic_src, "peak_source": peak_src,
                         "kernel": "stream_gemv_kernel", "launches_per_step": n_gemv,
                         "algorithmic_bytes_per_launch": total_bytes / n_gemv,
                         "avg_launch_us": step_ms * 1e3 / n_gemv,
                         "frac_of_nominal_8TBs": achieved / 8000.0},
        }
        tf_peak = measured_tensor_peak()
        macs = matrix_params(L, D)   # multiply-adds per activation row
        alg_tflops = 2.0 * macs * Bs * Kb / (batched_ms * 1e-3) / 1e12
        line["batched_decode"] = {
            "streams_per_gpu": Bs, "steps": Kb, "ms_per_step": batched_ms / Kb,
            "value": world * Bs * Kb / (batched_ms * 1e-3), "unit": UNIT, "gpu_launches_per_rank": launches_b,
            "kernel": "tile_gemm_kernel (tcgen05 kind::i8, three 8-bit activation digits per row)",
            "tensor": {"algorithmic_tflops": alg_tflops, "peak_bf16_tflops": tf_peak,
                       "frac_of_measured_bf16": alg_tflops / tf_peak if tf_peak else None}}
        line.update(extra)
        if world == 1:
            spans = trace_spans(model, dev)
            line["roofline"]["avg_launch_us"] = spans["launch_us"]
            line["roofline"]["avg_stream_us"] = spans["stream_us"]
            line["roofline"]["launch_span"] = ("graph-replayed traced step: per GEMV launch, dependency resolved (median CTA) -> "
                                               "epilogue done (last CTA); stream = digit planes in shared memory -> rows summed")
            lib_ms = library_baseline_ms(model, Bs)
            line["batched_decode"]["library_baseline"] = {
                "what": "matrices only (all blocks + head): activations * range and uint8 weights cast to bf16 per call, "
                        "cuBLAS GEMM, offset term; stock torch, same box", "ms_per_step": lib_ms,
                "ours_over_library": (batched_ms / Kb) / lib_ms}
            line["kernels"] = time_isolated_kernels(model)
    if world > 1:
        del model
        torch.cuda.empty_cache()
        ls = time_layer_split(rank, world, dev)
        if rank == 0:
            line["layer_split"] = ls
    elif rank == 0:
        del model
        torch.cuda.empty_cache()
        model = None
        line["decode_1b5"] = time_decode_shape("1b5", dev)
        torch.cuda.empty_cache()
        line["torch_mode_bf16"] = time_dense_decode(args.shape, dev)
        torch.cuda.empty_cache()
        if not args.no_prefill:
            line["prefill"] = time_prefill(dev, tf_peak)
            torch.cuda.empty_cache()
            line["config4_one_gpu"] = time_config4_one_gpu(dev)
        if not args.no_cpu_baseline:
            torch.cuda.empty_cache()
            line["cpu_baseline"] = cpu_reference(args.shape, 4, 1)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shape", default="7b", choices=list(SHAPES))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-prefill", action="store_true", help="skip the 3B-shape prompt-ingestion measurement (N=1 only)")
    ap.add_argument("--mode", default="replicas", choices=["replicas", "layer-split"],
                    help="replicas: the headline data-parallel decode; layer-split: 14B blocks partitioned over the ranks")
    ap.add_argument("--microbatches", type=int, default=1,
                    help="stream groups of the layer-split pipeline (decode re-streams the stage weights per group: 1 is fastest)")
    ap.add_argument("--streams", type=int, default=256, help="streams per GPU of the batched-decode measurement")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.mode == "layer-split":
        if world < 2:
            sys.exit("--mode layer-split needs torchrun with at least two ranks")
        if args.shape == "7b":
            args.shape = "14b"
        if args.streams == 256:
            args.streams = 64
        run_layer_split(args, rank, world, local_rank)
        return
    if world != args.gpus and world == 1 and args.gpus > 1:
        sys.exit("--gpus N > 1 must be launched with torchrun (one rank per GPU)")
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
