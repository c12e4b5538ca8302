"""Host-side mirror of the reference's FASTQUANT model object.

``B200RWKV`` has the interface ``rwkvstic.rwkvMaster.RWKVMaster`` consumes
(rwkvMaster.py:32-38, :71): ``forward(tokens, state) -> (logits, state)`` and an
``emptyState`` attribute, with the same meaning as ``OptRWKV(...)`` from
agnostic/backends/opt.py:15-119:

* ``tokens``  int64 ``[T]`` (list, CPU or CUDA tensor).  T > 1 is sequence mode; the
  logits are those of the last token (opt.py:71-73).
* ``state``   ``[L,5,D]``; rows 0/1 are the att/ffn token-shift carries, rows 2..4 the
  WKV accumulators, empty state ``(0,0,0,0,-1e30)`` exactly as opt.py:31-32.  It is
  updated IN PLACE and returned, like the reference does (opt.py:68-69).  Runtime dtype
  is fp32 (the reference uses fp64); the WKV rows use the max-trick convention of
  agnosticRwkv.py:68-103 - ``state_to_reference`` / ``state_from_reference`` convert.

All arithmetic happens in the CUDA library (``_lib``); this file only owns device
memory, CUDA-graph capture and the call sequence.  There is no CPU path.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Sequence, Tuple, Union

import torch

from . import _lib
from .quant import QuantMatrix, quantize_fastquant, quantize_two_axis
from .synth import VOCAB, iter_synth_tensors

MATRIX_KEYS = ("att.key", "att.value", "att.receptance", "att.output", "ffn.key", "ffn.receptance", "ffn.value")


@dataclass
class LayerWeights:
    vec: Dict[str, torch.Tensor] = field(default_factory=dict)   # f32 [D] each
    mat: Dict[str, QuantMatrix] = field(default_factory=dict)    # keyed by MATRIX_KEYS


@dataclass
class QuantizedWeights:
    """Everything the kernels read, resident on one device."""
    n_layer: int
    n_embd: int
    n_ffn: int
    n_vocab: int
    emb: Optional[torch.Tensor]              # None on a pipeline stage other than the first
    ln0: Tuple[torch.Tensor, torch.Tensor]
    ln_out: Tuple[torch.Tensor, torch.Tensor]
    head: Optional[QuantMatrix]              # None on a pipeline stage other than the last
    layers: List[LayerWeights]
    first_layer: int = 0                     # global index of layers[0] (layer split)

    def weight_bytes(self) -> int:
        """uint8 matrix bytes one decode step streams (13*L*D^2 + V*D for F = 4D)."""
        n = self.head.qt.numel() if self.head is not None else 0
        for ly in self.layers:
            n += sum(m.qt.numel() for m in ly.mat.values())
        return n


def _quantizer(scheme: str):
    if scheme == "fastquant":
        return quantize_fastquant
    if scheme == "two_axis":
        return quantize_two_axis
    raise ValueError(f"unknown quantisation scheme {scheme!r}")


def quantize_tensors(tensors: Iterable[Tuple[str, torch.Tensor]], device, scheme: str = "fastquant",
                     quant_device=None, layer_range: Optional[Tuple[int, int]] = None,
                     keep_emb: bool = True, keep_head: bool = True) -> QuantizedWeights:
    """Build ``QuantizedWeights`` from (name, tensor) pairs with the reference checkpoint key
    names (helpers/loadWeights.py:19-26, modules/block.py:13-47).  Consumes the iterable one
    tensor at a time, so large shapes never need the fp32 checkpoint in memory.

    ``layer_range=(l0, l1)`` keeps only blocks l0..l1-1 (one stage of a layer split); a stage that
    is not the first drops the embedding (``keep_emb=False``), one that is not the last drops the
    head (``keep_head=False``)."""
    q = _quantizer(scheme)
    dev = torch.device(device)
    qdev = torch.device(quant_device) if quant_device is not None else None
    layers: Dict[int, LayerWeights] = {}
    top: Dict[str, torch.Tensor] = {}
    head = None
    f32 = lambda t: t.detach().reshape(-1).to(torch.float32).to(dev).contiguous()
    n_vocab = 0
    for name, t in tensors:
        if name.startswith("blocks."):
            _, idx, rest = name.split(".", 2)
            if rest.startswith("ln0."):
                top[rest] = f32(t)
                continue
            if layer_range is not None and not (layer_range[0] <= int(idx) < layer_range[1]):
                continue
            ly = layers.setdefault(int(idx), LayerWeights())
            if rest.endswith(".weight") and rest[:-7] in MATRIX_KEYS:
                w = t.detach().float()
                ly.mat[rest[:-7]] = q(w.to(qdev) if qdev is not None else w).to(dev)
            elif rest == "att.time_decay":
                ly.vec[rest] = (-torch.exp(t.detach().double().reshape(-1))).to(torch.float32).to(dev).contiguous()
            elif rest == "att.time_decay_final":       # already w = -exp(raw) (helpers/loadWeights.py:63-64)
                ly.vec["att.time_decay"] = f32(t)
            elif rest.startswith("ln0."):
                top[rest] = f32(t)
            else:
                ly.vec[rest] = f32(t)
        elif name == "head.weight":
            n_vocab = t.shape[0]
            if keep_head:
                w = t.detach().float()
                head = q(w.to(qdev) if qdev is not None else w).to(dev)
        elif name == "emb.weight":
            n_vocab = t.shape[0]
            if keep_emb:
                top["emb"] = t.detach().to(torch.float32).to(dev).contiguous()
        else:
            top[name] = f32(t)
    first = min(layers)
    ordered = [layers[i] for i in range(first, first + len(layers))]
    D = ordered[0].mat["att.key"].k_in
    F = ordered[0].mat["ffn.key"].n_out
    return QuantizedWeights(n_layer=len(ordered), n_embd=D, n_ffn=F, n_vocab=n_vocab, emb=top.get("emb"),
                            ln0=(top["ln0.weight"], top["ln0.bias"]),
                            ln_out=(top["ln_out.weight"], top["ln_out.bias"]), head=head, layers=ordered,
                            first_layer=first)


def state_to_reference(state: torch.Tensor, time_decay: Sequence[torch.Tensor]) -> torch.Tensor:
    """Convert a max-trick state to the reference FASTQUANT meaning (modules/wkv.py:31-39):
    ``aa_ref = exp(w + pp) * aa``, same for bb; pp reported as the reference leaves it (-1e30)."""
    out = state.detach().double().clone()
    for i, w in enumerate(time_decay):
        e = torch.exp(w.double().to(out.device) + out[..., i, 4, :])
        out[..., i, 2, :] *= e
        out[..., i, 3, :] *= e
    out[..., 4, :] = float(torch.tensor(-1e30, dtype=torch.float32))
    return out


def state_from_reference(state: torch.Tensor, time_decay: Sequence[torch.Tensor]) -> torch.Tensor:
    """Inverse of ``state_to_reference``: ``aa = aa_ref, pp = -w`` (empty rows stay empty)."""
    out = state.detach().to(torch.float32).clone()
    for i, w in enumerate(time_decay):
        empty = (out[..., i, 2, :] == 0) & (out[..., i, 3, :] == 0)
        out[..., i, 4, :] = torch.where(empty, torch.full_like(out[..., i, 4, :], -1e30), -w.float().to(out.device))
    return out


class B200RWKV:
    """RWKV-4 with uint8 weights on one B200.  See the module docstring for the contract."""

    RnnOnly = False  # sequence mode is supported (rwkvMaster.py:97 looks this up)

    def __init__(self, weights: QuantizedWeights, use_graph: bool = True, copy_logits: bool = True,
                 decode_mode: str = "chained"):
        """``decode_mode``: how one-token steps run.  "chained" (default, the faster one on a B200):
        one streaming launch per matrix group, chained by programmatic dependent launch
        (b200rwkv_decode_step); "persistent": the whole step is one resident kernel whose weight
        stream runs on from matrix to matrix and whose CTAs exchange activations through tagged
        words in L2 (b200rwkv_decode_step_persistent).  Both compute the same step."""
        if decode_mode not in ("persistent", "chained"):
            raise ValueError("decode_mode must be 'persistent' or 'chained'")
        self.w = weights
        self.device = weights.ln0[0].device
        if self.device.type != "cuda":
            raise RuntimeError("B200RWKV needs a CUDA device: the kernels are sm_100a only and there is no CPU path")
        self._L = _lib.lib()
        self.n_layer, self.n_embd, self.n_ffn, self.n_vocab = weights.n_layer, weights.n_embd, weights.n_ffn, weights.n_vocab
        self.use_graph = use_graph
        self.copy_logits = copy_logits
        if weights.emb is None or weights.head is None:
            decode_mode = "chained"      # a pipeline stage: only the rows path applies to it
        self.decode_mode = decode_mode
        self.launches_per_step = 1 if decode_mode == "persistent" else 8 * self.n_layer + 3
        self.step_tuning = [0, 0, -1, 0]  # b200rwkv_decode_step_persistent's tuning words (0 / -1: library defaults)
        self.time_decay = [ly.vec["att.time_decay"] for ly in weights.layers]
        self.emptyState = torch.zeros(self.n_layer, 5, self.n_embd, dtype=torch.float32, device=self.device)
        self.emptyState[:, 4] = -1e30
        self._build_descriptor()
        self.stage_stream_rows = 2     # forward_rows_stage: up to this many rows go through the one-row step
        nbytes = int(self._L.b200rwkv_decode_workspace_bytes(C.byref(self._cmodel)))
        self._ws = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
        self._plan = None
        if decode_mode == "persistent":
            with torch.cuda.device(self.device):
                nplan = int(self._L.b200rwkv_step_plan_bytes(C.byref(self._cmodel)))
                self._plan = torch.zeros(nplan, dtype=torch.uint8, device=self.device)
                torch.cuda.synchronize(self.device)
                _lib.check(self._L.b200rwkv_step_plan_init(C.byref(self._cmodel), self._plan.data_ptr(), nplan))
        self._status_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self._tok = torch.zeros(1, dtype=torch.int64, device=self.device)
        self._logits = torch.zeros(self.n_vocab, dtype=torch.float32, device=self.device)
        self._rows_ws: Dict[Tuple[int, int], torch.Tensor] = {}
        self.rows_threshold = 3       # forward / forward_batch use the tensor-core rows path from this many rows (7B: 3 rows 3.8 ms against 3 x 1.7 ms)
        self.rows_per_call = 4096     # upper bound on rows (streams x tokens) of one rows-path call
        self._graphs: Dict[Tuple[int, bool], torch.cuda.CUDAGraph] = {}
        self._seen: Dict[int, int] = {}
        self.launch_count = 0  # kernels launched so far (for the benchmark's gpu_launches)

    # ------------------------------------------------------------------ construction helpers
    @classmethod
    def from_checkpoint(cls, ck: Union[str, Dict[str, torch.Tensor]], device="cuda:0", scheme: str = "fastquant",
                        **kw) -> "B200RWKV":
        """From a ``.pth`` path or an in-memory dict with the reference key names.  Quantisation
        runs on the CPU so the bytes are identical to the reference's (modules/matmul.py:26-40)."""
        if isinstance(ck, str):
            ck = torch.load(ck, map_location="cpu")
        return cls(quantize_tensors(ck.items(), device, scheme), **kw)

    @classmethod
    def synthetic(cls, layers: int, embed: int, vocab: int = VOCAB, seed: int = 1234, device="cuda:0",
                  scheme: str = "fastquant", **kw) -> "B200RWKV":
        """Seeded random-init model generated and quantised on the device, matrix by matrix."""
        gen = iter_synth_tensors(layers, embed, vocab, seed, device=str(device))
        return cls(quantize_tensors(gen, device, scheme), **kw)

    def _matrix(self, m: QuantMatrix) -> _lib.Matrix:
        for t in (m.qt, m.ry, m.my):
            assert t.is_contiguous() and t.device == self.device
        assert m.qt.dtype == torch.uint8 and m.ry.dtype == torch.float32 and m.my.dtype == torch.float32
        return _lib.Matrix(_lib.ptr(m.qt), _lib.ptr(m.ry), _lib.ptr(m.my), _lib.ptr(m.rx), _lib.ptr(m.mx),
                           float(m.half), m.n_out, m.k_in)

    def _build_descriptor(self) -> None:
        w = self.w
        self._clayers = (_lib.Layer * self.n_layer)()
        for i, ly in enumerate(w.layers):
            c = self._clayers[i]
            v = ly.vec
            c.ln1_w, c.ln1_b, c.ln2_w, c.ln2_b = (_lib.ptr(v[k]) for k in ("ln1.weight", "ln1.bias", "ln2.weight", "ln2.bias"))
            c.att_mix_k, c.att_mix_v, c.att_mix_r = (_lib.ptr(v[k]) for k in ("att.time_mix_k", "att.time_mix_v", "att.time_mix_r"))
            c.ffn_mix_k, c.ffn_mix_r = _lib.ptr(v["ffn.time_mix_k"]), _lib.ptr(v["ffn.time_mix_r"])
            c.time_decay, c.time_first = _lib.ptr(v["att.time_decay"]), _lib.ptr(v["att.time_first"])
            c.att_key, c.att_value, c.att_receptance, c.att_output = (self._matrix(ly.mat[k]) for k in MATRIX_KEYS[:4])
            c.ffn_key, c.ffn_receptance, c.ffn_value = (self._matrix(ly.mat[k]) for k in MATRIX_KEYS[4:])
        self._cmodel = _lib.Model(self.n_layer, self.n_embd, self.n_ffn, self.n_vocab, _lib.ptr(w.emb),
                                  _lib.ptr(w.ln0[0]), _lib.ptr(w.ln0[1]), _lib.ptr(w.ln_out[0]), _lib.ptr(w.ln_out[1]),
                                  self._matrix(w.head) if w.head is not None else _lib.Matrix(),
                                  C.cast(self._clayers, C.POINTER(_lib.Layer)))

    # ------------------------------------------------------------------ one decode step
    def _step_raw(self, tok_ptr: int, state_ptr: int, logits_ptr: Optional[int]) -> None:
        stream = torch.cuda.current_stream(self.device).cuda_stream
        if self._plan is not None:
            tuning = (C.c_int32 * 4)(*[int(v) for v in self.step_tuning])
            _lib.check(self._L.b200rwkv_decode_step_persistent(C.byref(self._cmodel), self._plan.data_ptr(), self._plan.numel(),
                                                               tok_ptr, state_ptr, logits_ptr, tuning, None, stream))
            return
        _lib.check(self._L.b200rwkv_decode_step(C.byref(self._cmodel), tok_ptr, state_ptr, logits_ptr,
                                                self._ws.data_ptr(), self._ws.numel(), stream))

    def _step(self, state: torch.Tensor, want_logits: bool) -> None:
        """Run one step on the token in ``self._tok``; logits (if any) land in ``self._logits``."""
        self.launch_count += self.launches_per_step - (0 if want_logits or self._plan is not None else 2)
        lp = self._logits.data_ptr() if want_logits else None
        if not self.use_graph:
            self._step_raw(self._tok.data_ptr(), state.data_ptr(), lp)
            return
        key = (state.data_ptr(), want_logits)
        g = self._graphs.get(key)
        if g is None:
            # Capture once a state buffer shows up for the second time (RWKVMaster.forward reuses
            # one buffer for every token; loadContext clones per chunk and just runs eagerly).
            n = self._seen.get(key, 0) + 1
            self._seen[key] = n
            if n < 2:
                self._step_raw(self._tok.data_ptr(), state.data_ptr(), lp)
                return
            if len(self._graphs) >= 16:
                self._graphs.clear()
                self._seen.clear()
            g = torch.cuda.CUDAGraph()
            torch.cuda.synchronize(self.device)
            with torch.cuda.graph(g):
                self._step_raw(self._tok.data_ptr(), state.data_ptr(), lp)
            self._graphs[key] = g
        g.replay()

    def trace_step(self, token: int, state: torch.Tensor, graph: bool = False) -> torch.Tensor:
        """Profiling: run one decode step and return the phase timeline, an int64 CPU tensor
        ``[4L+1 launches, 1024, 8]`` of %globaltimer nanoseconds: rows < grid are the GEMV CTAs, row 1023
        the preparation kernel (see b200rwkv_gemv_u8_traced).  ``graph=True`` captures the traced step
        in a CUDA graph and returns the timeline of its second replay (launch latencies as in production)."""
        n = 4 * self.n_layer + 1
        trace = torch.zeros(n, 1024, 8, dtype=torch.int64, device=self.device)
        self._tok.fill_(int(token))

        def step():
            stream = torch.cuda.current_stream(self.device).cuda_stream
            _lib.check(self._L.b200rwkv_decode_step_traced(C.byref(self._cmodel), self._tok.data_ptr(), state.data_ptr(),
                                                           self._logits.data_ptr(), self._ws.data_ptr(), self._ws.numel(),
                                                           trace.data_ptr(), stream))
        if not graph:
            step()
        else:
            step()
            g = torch.cuda.CUDAGraph()
            torch.cuda.synchronize(self.device)
            with torch.cuda.graph(g):
                step()
            g.replay()
            g.replay()
        torch.cuda.synchronize(self.device)
        return trace.cpu()

    def check_status(self) -> None:
        """Raise if any kernel reported an expired device-side wait (synchronises).  After that the
        state the failed step was given is undefined."""
        for buf in (self._ws, self._plan):
            if buf is None:
                continue
            self._status_host.copy_(buf[:4].view(torch.int32))
            bits = int(self._status_host[0])
            if bits:
                buf[:4].zero_()
                if buf is self._plan:       # the exchange buffers' use counts are stale after an abandoned step
                    _lib.check(self._L.b200rwkv_step_plan_init(C.byref(self._cmodel), self._plan.data_ptr(), self._plan.numel()))
                raise _lib.B200RWKVError(_lib.ETIMEOUT, f"device-side wait expired, status bits 0x{bits:x}")

    def _status_buffer(self) -> torch.Tensor:
        return self._plan if self._plan is not None else self._ws

    def _queue_step_status(self) -> None:
        """Non-blocking copy of the one-row path's status word to pinned host memory; looked at by the next
        call of forward / generate_* (or check_status) once the copy has completed, so an expired
        device-side wait is reported a call or two late instead of costing every call a device
        synchronisation.  The state a
        failed step was given is undefined."""
        if not hasattr(self, "_step_status_host"):
            self._step_status_host = torch.zeros(1, dtype=torch.int32).pin_memory()
            self._step_status_event = torch.cuda.Event()
        self._step_status_host.copy_(self._status_buffer()[:4].view(torch.int32), non_blocking=True)
        self._step_status_event.record(torch.cuda.current_stream(self.device))
        self._step_status_pending = True

    def _raise_step_status(self) -> None:
        if not getattr(self, "_step_status_pending", False) or not self._step_status_event.query():
            return                      # nothing queued, or the copy has not run yet: look again at the next call
        self._step_status_pending = False
        if int(self._step_status_host[0]):
            self.check_status()

    def trace_persistent_step(self, token: int, state: torch.Tensor, replays: int = 3) -> torch.Tensor:
        """Profiling: the %globaltimer timeline of one persistent decode step, an int64 CPU tensor
        ``[4L+1 launches, grid, 8]`` (slots as documented at b200rwkv_decode_step_persistent), taken from
        the last of ``replays`` replays of a CUDA graph of the traced step."""
        if self._plan is None:
            raise RuntimeError("trace_persistent_step needs decode_mode='persistent'")
        geo = (C.c_int64 * 8)()
        sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        _lib.check(self._L.b200rwkv_step_geometry(C.byref(self._cmodel), sms, geo))
        trace = torch.zeros(4 * self.n_layer + 1, int(geo[0]), 8, dtype=torch.int64, device=self.device)
        self._tok.fill_(int(token))
        tuning = (C.c_int32 * 4)(*[int(v) for v in self.step_tuning])

        def step():
            stream = torch.cuda.current_stream(self.device).cuda_stream
            _lib.check(self._L.b200rwkv_decode_step_persistent(C.byref(self._cmodel), self._plan.data_ptr(), self._plan.numel(),
                                                               self._tok.data_ptr(), state.data_ptr(), self._logits.data_ptr(),
                                                               tuning, trace.data_ptr(), stream))
        with torch.cuda.device(self.device):
            step()
            g = torch.cuda.CUDAGraph()
            torch.cuda.synchronize(self.device)
            with torch.cuda.graph(g):
                step()
            for _ in range(max(1, replays)):
                g.replay()
            torch.cuda.synchronize(self.device)
        return trace.cpu()

    # ------------------------------------------------------------------ public interface
    def _own_state(self, state: torch.Tensor) -> torch.Tensor:
        if (state.dtype == torch.float32 and state.device == self.device and state.is_contiguous()
                and tuple(state.shape) == (self.n_layer, 5, self.n_embd)):
            return state
        if tuple(state.shape) != (self.n_layer, 5, self.n_embd):
            raise ValueError(f"state must be [{self.n_layer},5,{self.n_embd}], got {tuple(state.shape)}")
        return state.to(device=self.device, dtype=torch.float32).contiguous()

    def _rows_launches(self, tokens_per_stream: int) -> int:
        """Kernels one rows-path call launches for its blocks: four preparation and four GEMM launches per
        block plus the WKV scan (one kernel up to 128 tokens per stream, two passes beyond)."""
        return (9 if tokens_per_stream <= 128 else 10) * self.n_layer

    def forward_rows(self, tokens: torch.Tensor, state: torch.Tensor) -> torch.Tensor:
        """Tensor-core path: ``tokens [B,T]`` int64, ``state [B,L,5,D]`` fp32 contiguous on the
        device (updated in place).  Every matrix is applied to all B*T rows at once
        (b200rwkv_forward_rows); prompts longer than ``rows_per_call // B`` tokens are fed in
        pieces.  Returns the logits ``[B,V]`` after each stream's last token."""
        if tokens.dim() != 2 or tokens.numel() == 0:
            raise ValueError("forward_rows needs tokens [B,T] with at least one token")
        B, T = tokens.shape
        if (state.dtype != torch.float32 or state.device != self.device or not state.is_contiguous()
                or tuple(state.shape) != (B, self.n_layer, 5, self.n_embd)):
            raise ValueError(f"forward_rows needs a contiguous fp32 state [{B},{self.n_layer},5,{self.n_embd}] on the model's device")
        if B > 65535:
            raise ValueError("forward_rows: at most 65535 streams per call")
        self._raise_rows_status()            # the previous call's status word, read back without blocking
        if T == 1 and self.use_graph:
            return self._rows_decode_replay(tokens, state)
        out = torch.empty(B, self.n_vocab, dtype=torch.float32, device=self.device)
        step = max(1, min(self.rows_per_call, 65535) // B)
        with torch.cuda.device(self.device):
            toks = tokens.to(device=self.device, dtype=torch.int64)
            for t0 in range(0, T, step):
                piece = toks[:, t0:t0 + step].contiguous()
                tp = piece.shape[1]
                ws = self._rows_workspace(B, tp)
                last = t0 + step >= T
                self._rows_call(piece, B, tp, state, out if last else None, ws)
            self._queue_rows_status(ws)
        return out

    def _rows_workspace(self, B: int, tp: int) -> torch.Tensor:
        ws = self._rows_ws.get((B, tp))
        if ws is None:
            n = int(self._L.b200rwkv_rows_workspace_bytes(C.byref(self._cmodel), B, tp))
            if len(self._rows_ws) >= 4:
                self._rows_ws.clear()
            ws = self._rows_ws[(B, tp)] = torch.zeros(n, dtype=torch.uint8, device=self.device)
        return ws

    def _rows_call(self, piece: torch.Tensor, B: int, tp: int, state: torch.Tensor, out: Optional[torch.Tensor],
                   ws: torch.Tensor) -> None:
        stream = torch.cuda.current_stream(self.device).cuda_stream
        _lib.check(self._L.b200rwkv_forward_rows(C.byref(self._cmodel), piece.data_ptr(), B, tp, state.data_ptr(),
                                                 state.stride(0), None if out is None else out.data_ptr(),
                                                 ws.data_ptr(), ws.numel(), stream))
        self.launch_count += self._rows_launches(tp) + 1 + (2 if out is not None else 0)

    def _queue_rows_status(self, ws: torch.Tensor) -> None:
        """Start a non-blocking copy of a rows workspace's status word to pinned host memory; the next
        rows call looks at it once the copy has completed (check_rows_status waits for it), so an expired
        device-side wait is reported a call or two late instead of costing every call a device
        synchronisation."""
        if not hasattr(self, "_rows_status_host"):
            self._rows_status_host = torch.zeros(1, dtype=torch.int32).pin_memory()
            self._rows_status_event = torch.cuda.Event()
        self._rows_status_host.copy_(ws[:4].view(torch.int32), non_blocking=True)
        self._rows_status_event.record(torch.cuda.current_stream(self.device))
        self._rows_status_ws = ws

    def _raise_rows_status(self) -> None:
        ws = getattr(self, "_rows_status_ws", None)
        if ws is None or not self._rows_status_event.query():
            return                      # nothing queued, or the copy has not run yet: look again at the next call
        self._rows_status_ws = None
        bits = int(self._rows_status_host[0])
        if bits:
            ws[:4].zero_()
            raise _lib.B200RWKVError(_lib.ETIMEOUT, f"device-side wait expired, status bits 0x{bits:x}")

    def _rows_decode_replay(self, tokens: torch.Tensor, state: torch.Tensor) -> torch.Tensor:
        """One token for each of B streams (batched decode) as a CUDA-graph replay: the ~9 launches per
        block are captured once per (B, state buffer) - from the second call with the same state buffer
        on - into static token and logits buffers.  Returns the logits ``[B,V]``; with
        ``copy_logits=False`` that is the static buffer, valid until the next call."""
        B = tokens.shape[0]
        key = (B, state.data_ptr())
        if not hasattr(self, "_rows_graphs"):
            self._rows_graphs: Dict[Tuple[int, int], dict] = {}
        ent = self._rows_graphs.get(key)
        with torch.cuda.device(self.device):
            if ent is None:
                if len(self._rows_graphs) >= 8:
                    self._rows_graphs.clear()
                ent = self._rows_graphs[key] = {"tok": torch.zeros(B, 1, dtype=torch.int64, device=self.device),
                                                "out": torch.empty(B, self.n_vocab, dtype=torch.float32, device=self.device),
                                                "ws": self._rows_workspace(B, 1), "graph": None, "seen": 0}
            ent["tok"].copy_(tokens.reshape(B, 1), non_blocking=True)
            ent["seen"] += 1
            if ent["graph"] is None and ent["seen"] >= 2:
                g = torch.cuda.CUDAGraph()
                torch.cuda.synchronize(self.device)
                count = self.launch_count
                with torch.cuda.graph(g):
                    self._rows_call(ent["tok"], B, 1, state, ent["out"], ent["ws"])
                self.launch_count = count       # the capture itself runs nothing
                ent["graph"] = g
            if ent["graph"] is not None:
                ent["graph"].replay()
                self.launch_count += self._rows_launches(1) + 3
            else:
                self._rows_call(ent["tok"], B, 1, state, ent["out"], ent["ws"])
            self._queue_rows_status(ent["ws"])
        return ent["out"].clone() if self.copy_logits else ent["out"]

    def forward_rows_stage(self, tokens: Optional[torch.Tensor], x: torch.Tensor, state: torch.Tensor,
                           want_logits: bool) -> Optional[torch.Tensor]:
        """One pipeline stage of ``forward_rows`` when this object holds only a contiguous range
        of blocks (layer split).  ``tokens [B,T]`` on the first stage, else None and ``x`` fp32
        ``[B*T, D]`` holds the residual stream received from the previous stage; ``x`` is updated
        in place for the next stage.  ``state [B, L_stage, 5, D]``.  Returns logits ``[B,V]`` when
        ``want_logits`` (last stage), else None.  Asynchronous on the current stream."""
        B = state.shape[0]
        if x.dim() != 2 or x.shape[1] != self.n_embd or x.shape[0] % B or not x.is_contiguous() or x.dtype != torch.float32:
            raise ValueError("forward_rows_stage needs x fp32 [B*T, D], contiguous")
        T = x.shape[0] // B
        if tuple(state.shape) != (B, self.n_layer, 5, self.n_embd) or not state.is_contiguous() or state.dtype != torch.float32:
            raise ValueError(f"forward_rows_stage needs a contiguous fp32 state [{B},{self.n_layer},5,{self.n_embd}]")
        if tokens is not None:
            if self.w.emb is None:
                raise ValueError("this stage holds no embedding: pass tokens=None and the previous stage's x")
            tokens = tokens.to(device=self.device, dtype=torch.int64).reshape(B, T).contiguous()
        if want_logits and self.w.head is None:
            raise ValueError("this stage holds no head")
        out = torch.empty(B, self.n_vocab, dtype=torch.float32, device=self.device) if want_logits else None
        if B * T <= self.stage_stream_rows:
            # one or two rows: the one-row streaming step per row (reads the stage's weights at HBM speed)
            # instead of tensor-core tiles that would be almost empty
            with torch.cuda.device(self.device):
                stream = torch.cuda.current_stream(self.device).cuda_stream
                for b in range(B):
                    for t in range(T):
                        r = b * T + t
                        lp = out[b].data_ptr() if (want_logits and t == T - 1) else None
                        _lib.check(self._L.b200rwkv_decode_step_stage(
                            C.byref(self._cmodel), None if tokens is None else tokens[b, t:t + 1].data_ptr(), x[r].data_ptr(),
                            state[b].data_ptr(), lp, self._ws.data_ptr(), self._ws.numel(), stream))
                        self.launch_count += self.launches_per_step - (0 if lp is not None else 2)
            return out
        with torch.cuda.device(self.device):
            ws = self._rows_ws.get((B, T))
            if ws is None:
                n = int(self._L.b200rwkv_rows_workspace_bytes(C.byref(self._cmodel), B, T))
                if n == 0:
                    raise ValueError("forward_rows_stage: at most 65535 rows per call")
                if len(self._rows_ws) >= 4:
                    self._rows_ws.clear()
                ws = self._rows_ws[(B, T)] = torch.zeros(n, dtype=torch.uint8, device=self.device)
            stream = torch.cuda.current_stream(self.device).cuda_stream
            _lib.check(self._L.b200rwkv_forward_rows_stage(
                C.byref(self._cmodel), None if tokens is None else tokens.data_ptr(), x.data_ptr(), B, T,
                state.data_ptr(), state.stride(0), None if out is None else out.data_ptr(), ws.data_ptr(), ws.numel(), stream))
            self.launch_count += self._rows_launches(T) + (1 if tokens is not None else 0) + (2 if want_logits else 0)
            self._last_rows_ws = ws
        return out

    def check_rows_status(self) -> None:
        """Raise if a kernel of the last ``forward_rows`` / ``forward_rows_stage`` call reported an expired
        wait (synchronises)."""
        if getattr(self, "_rows_status_ws", None) is not None:
            self._rows_status_event.synchronize()
        self._raise_rows_status()
        ws = getattr(self, "_last_rows_ws", None)
        if ws is None:
            return
        bits = int(ws[:4].view(torch.int32).item())
        if bits:
            ws[:4].zero_()
            raise _lib.B200RWKVError(_lib.ETIMEOUT, f"device-side wait expired, status bits 0x{bits:x}")

    # ------------------------------------------------------------------ greedy sampling on the device
    def argmax_token(self, logits: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Device int64[1]: index of the largest logit of the last ``forward`` (or of ``logits``),
        computed on the device so that only 8 bytes need to travel to the host per token."""
        lg = self._logits if logits is None else logits
        out = torch.empty(1, dtype=torch.int64, device=self.device)
        with torch.cuda.device(self.device):
            _lib.check(self._L.b200rwkv_argmax(lg.data_ptr(), 1, lg.numel(), lg.numel(), out.data_ptr(), None, None, 0,
                                               torch.cuda.current_stream(self.device).cuda_stream))
        self.launch_count += 1
        return out

    def step_greedy(self, token: torch.Tensor, state: torch.Tensor, out: torch.Tensor) -> None:
        """One decode step with the arg-max taken on the device, for a host-driven loop: the token
        (int64[1] on the host) goes to the device, the step and the arg-max kernel run, and the
        sampled id comes back into ``out`` (int64[1] on the host).  From the second call with the
        same ``state`` buffer on, all of it - both copies included, through pinned buffers this
        object owns - is one CUDA-graph replay.  Returns after the id has arrived; ``state`` is
        updated in place."""
        state = self._own_state(state)
        if not hasattr(self, "_next"):
            self._next = torch.zeros(1, dtype=torch.int64, device=self.device)
            self._tok_host = torch.zeros(1, dtype=torch.int64).pin_memory()
            self._next_host = torch.zeros(1, dtype=torch.int64).pin_memory()
            self._greedy_status = torch.zeros(1, dtype=torch.int32).pin_memory()
            self._greedy_graphs: Dict[int, torch.cuda.CUDAGraph] = {}
            self._greedy_seen: Dict[int, int] = {}
        self._tok_host[0] = int(token.reshape(-1)[0])
        with torch.cuda.device(self.device):
            def one():
                self._tok.copy_(self._tok_host, non_blocking=True)           # 8 bytes host -> device
                self._step_raw(self._tok.data_ptr(), state.data_ptr(), self._logits.data_ptr())
                _lib.check(self._L.b200rwkv_argmax(self._logits.data_ptr(), 1, self.n_vocab, self.n_vocab,
                                                   self._next.data_ptr(), None, None, 0,
                                                   torch.cuda.current_stream(self.device).cuda_stream))
                self._next_host.copy_(self._next, non_blocking=True)         # 8 bytes device -> host
                self._greedy_status.copy_(self._status_buffer()[:4].view(torch.int32), non_blocking=True)
            key = state.data_ptr()
            g = self._greedy_graphs.get(key) if self.use_graph else None
            if g is not None:
                g.replay()
            else:
                n = self._greedy_seen.get(key, 0) + 1
                self._greedy_seen[key] = n
                if self.use_graph and n >= 2:
                    if len(self._greedy_graphs) >= 16:
                        self._greedy_graphs.clear()
                        self._greedy_seen.clear()
                    g = torch.cuda.CUDAGraph()
                    torch.cuda.synchronize(self.device)
                    with torch.cuda.graph(g):
                        one()
                    self._greedy_graphs[key] = g
                    g.replay()
                else:
                    one()
            torch.cuda.current_stream(self.device).synchronize()
        if int(self._greedy_status[0]):
            self.check_status()              # raises: a device-side wait expired during this step
        out.reshape(-1)[0] = self._next_host[0]
        self.launch_count += self.launches_per_step + 1

    def generate_greedy(self, token, state: torch.Tensor, n: int) -> torch.Tensor:
        """``n`` greedy decode steps that never leave the device: feed ``token``, take the arg-max
        of the logits, feed it back, ...  Each step is one CUDA-graph replay (the decode step
        plus an arg-max kernel that writes the next token into the step's own input buffer and
        appends it to a history buffer).  Returns the ``n`` generated ids (device int64);
        ``state`` is updated in place.  Same tokens as calling ``forward`` + ``torch.argmax`` n times."""
        self._raise_step_status()
        state = self._own_state(state)
        hist = torch.zeros(max(n, 1), dtype=torch.int64, device=self.device)
        count = torch.zeros(1, dtype=torch.int32, device=self.device)
        with torch.cuda.device(self.device):
            self._tok.copy_(torch.as_tensor(token, dtype=torch.int64).reshape(1), non_blocking=True)
            stream = lambda: torch.cuda.current_stream(self.device).cuda_stream

            def one():
                self._step_raw(self._tok.data_ptr(), state.data_ptr(), self._logits.data_ptr())
                _lib.check(self._L.b200rwkv_argmax(self._logits.data_ptr(), 1, self.n_vocab, self.n_vocab,
                                                   self._tok.data_ptr(), hist.data_ptr(), count.data_ptr(), hist.numel(),
                                                   stream()))
            if self.use_graph and n >= 3:
                one()                                   # eager first step (also warms every lazy initialisation)
                g = torch.cuda.CUDAGraph()
                torch.cuda.synchronize(self.device)
                with torch.cuda.graph(g):
                    one()
                count.fill_(1)                          # the capture itself does not run the kernels
                for _ in range(n - 1):
                    g.replay()
            else:
                for _ in range(n):
                    one()
        self.launch_count += n * (self.launches_per_step + 1)
        with torch.cuda.device(self.device):
            self._queue_step_status()
        return hist[:n]

    def generate_typical(self, token, state: torch.Tensor, n: int, temp: float = 1.0, tau: float = 0.95,
                         seed: int = 0) -> torch.Tensor:
        """``n`` decode steps with typical sampling (the reference's sampler, samplers/typical.py:1-17)
        that never leave the device: like ``generate_greedy`` with the sampling kernel in the
        arg-max kernel's place.  The uniform numbers of all n draws come from one device
        generator seeded with ``seed`` before the loop, so a run is reproducible.  Returns the
        generated ids (device int64); ``state`` is updated in place."""
        self._raise_step_status()
        state = self._own_state(state)
        hist = torch.zeros(max(n, 1), dtype=torch.int64, device=self.device)
        count = torch.zeros(1, dtype=torch.int32, device=self.device)
        gen = torch.Generator(device=self.device)
        gen.manual_seed(seed)
        u = torch.rand(max(n, 1), device=self.device, dtype=torch.float32, generator=gen)
        with torch.cuda.device(self.device):
            self._tok.copy_(torch.as_tensor(token, dtype=torch.int64).reshape(1), non_blocking=True)
            stream = lambda: torch.cuda.current_stream(self.device).cuda_stream

            def one():
                self._step_raw(self._tok.data_ptr(), state.data_ptr(), self._logits.data_ptr())
                _lib.check(self._L.b200rwkv_sample_typical(self._logits.data_ptr(), 1, self.n_vocab, self.n_vocab,
                                                           float(temp), float(tau), u.data_ptr(), self._tok.data_ptr(),
                                                           None, hist.data_ptr(), count.data_ptr(), hist.numel(), stream()))
            if self.use_graph and n >= 3:
                one()
                g = torch.cuda.CUDAGraph()
                torch.cuda.synchronize(self.device)
                with torch.cuda.graph(g):
                    one()
                count.fill_(1)
                for _ in range(n - 1):
                    g.replay()
            else:
                for _ in range(n):
                    one()
        self.launch_count += n * (self.launches_per_step + 1)
        with torch.cuda.device(self.device):
            self._queue_step_status()
        return hist[:n]

    def forward(self, tokens, state: torch.Tensor):
        """``(logits f32[V] on the device, state)`` - see the module docstring."""
        if not torch.is_tensor(tokens):
            tokens = torch.tensor(tokens if isinstance(tokens, (list, tuple)) else [tokens], dtype=torch.int64)
        tokens = tokens.reshape(-1).to(torch.int64)
        if tokens.numel() == 0:
            raise ValueError("forward needs at least one token")
        self._raise_step_status()
        state = self._own_state(state)
        if tokens.numel() >= self.rows_threshold:
            self._logits.copy_(self.forward_rows(tokens.reshape(1, -1), state.unsqueeze(0))[0])
            return (self._logits.clone() if self.copy_logits else self._logits), state
        with torch.cuda.device(self.device):
            toks = tokens.to(self.device, non_blocking=True)
            T = toks.numel()
            for i in range(T):
                self._tok.copy_(toks[i:i + 1], non_blocking=True)
                self._step(state, want_logits=(i == T - 1))
            self._queue_step_status()
        return (self._logits.clone() if self.copy_logits else self._logits), state

    __call__ = forward

    def forward_batch(self, tokens: torch.Tensor, state: torch.Tensor, rows: Optional[bool] = None):
        """B independent streams: ``tokens [B]`` or ``[B,T]``, ``state [B,L,5,D]`` (in place).
        Returns ``(logits [B,V], state)``.  From ``rows_threshold`` rows (B*T) on, or when
        ``rows`` is True, every matrix is applied to all rows at once on the tensor cores
        (``forward_rows``); below it each stream runs the one-row streaming path, bit-identical
        to B separate ``forward`` calls."""
        tokens = tokens.reshape(tokens.shape[0], -1)
        B = tokens.shape[0]
        if state.dtype != torch.float32 or state.device != self.device or not state.is_contiguous():
            raise ValueError("forward_batch needs a contiguous fp32 state on the model's device")
        if rows is None:
            rows = tokens.numel() >= self.rows_threshold
        if rows:
            return self.forward_rows(tokens, state), state
        out = torch.empty(B, self.n_vocab, dtype=torch.float32, device=self.device)
        keep = self.copy_logits
        self.copy_logits = False
        try:
            for b in range(B):
                lg, _ = self.forward(tokens[b], state[b])
                out[b].copy_(lg)
        finally:
            self.copy_logits = keep
        return out, state

    def empty_batch_state(self, B: int) -> torch.Tensor:
        return self.emptyState.unsqueeze(0).repeat(B, 1, 1, 1).contiguous()

    def to_reference_state(self, state: torch.Tensor) -> torch.Tensor:
        return state_to_reference(state, self.time_decay)

    def from_reference_state(self, state: torch.Tensor) -> torch.Tensor:
        return state_from_reference(state.to(self.device), self.time_decay)
