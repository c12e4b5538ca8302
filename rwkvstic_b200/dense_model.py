"""RWKV-4 with unquantised weights on the sm_100a kernels: the reference's TORCH mode.

The reference builds this model with ``loadWeights(TORCH, path, dtype=..., runtimedtype=...)``
(helpers/loadWeights.py:11-85; op table ``RWKVCudaOps``, agnostic/backends/torch.py:125-166) and runs
it through ``AgnosticRWKV`` (agnostic/agnosticRwkv.py:123-187): matrices in ``dtype``, vectors and
state in ``runtimedtype``.  ``B200DenseRWKV`` keeps the matrices as the checkpoint has them
(``[out,in]``, rows contiguous) in bf16 / fp16 / fp32, everything else in fp32, and runs one token per
call of ``b200rwkv_dense_step`` (6 kernels per block, replayed from a CUDA graph).

    model = B200DenseRWKV.from_checkpoint("model.pth", dtype=torch.bfloat16)
    logits, state = model.forward(tokens, model.emptyState.clone())

``forward(tokens int64[T], state f32[L,5,D]) -> (logits f32[V] on the device, state)``; the state is
the reference's own (max-trick WKV rows 2..4, ``-1e30`` in row 4 when empty) and is updated in
place.  From ``rows_threshold`` tokens on, bf16 / fp16 models apply every matrix to all rows at once
on the tensor cores (``forward_rows``, ``b200rwkv_dense_forward_rows``: ``tcgen05.mma kind::f16``), as
the reference does with a sequence; fp32 models and shorter inputs are fed token by token.  There is
no CPU fallback: without the CUDA library the constructor raises.

``target_gb`` (the ``target`` of the reference README's TORCH_STREAM mode: "the amount of GB you want to
use for matrix storage, if the model is too large, matrixes will be stored in ram and moved to the GPU as
needed") keeps only the first blocks' matrices on the device; the others live in pinned host memory and
are copied, one block ahead of the kernels that use them, into two staging buffers on a copy stream
(``b200rwkv_dense_step_layers`` / ``b200rwkv_dense_forward_rows_layers`` run the blocks of a range).
Results are bit-identical to the resident model; a prompt crosses the bus once per piece of rows,
a decode step once per token.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, Iterable, Optional, Tuple, Union

import torch

from . import _lib
from .synth import VOCAB, iter_synth_tensors

DTYPES = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
_MATS = ("att.key", "att.value", "att.receptance", "att.output", "ffn.key", "ffn.receptance", "ffn.value")
_VECS = ("ln1.weight", "ln1.bias", "ln2.weight", "ln2.bias", "att.time_mix_k", "att.time_mix_v", "att.time_mix_r",
         "ffn.time_mix_k", "ffn.time_mix_r", "att.time_decay", "att.time_first")


class B200DenseRWKV:
    RnnOnly = False  # sequence mode is supported (rwkvMaster.py:97 looks this up)

    def __init__(self, tensors: Iterable[Tuple[str, torch.Tensor]], dtype: torch.dtype = torch.bfloat16, device="cuda:0",
                 use_graph: bool = True, decay_is_final: bool = False, target_gb: Optional[float] = None,
                 pin_memory: bool = True):
        """``tensors``: (name, tensor) pairs under the checkpoint's key names; matrices ``[out,in]``.
        ``decay_is_final``: ``att.time_decay`` already holds ``-exp(raw)`` (what loadWeights hands to the
        ops object, loadWeights.py:63-64) instead of the checkpoint's raw value."""
        if dtype not in DTYPES:
            raise ValueError("dtype must be torch.float32, torch.bfloat16 or torch.float16")
        self._L = _lib.lib()
        self.device = torch.device(device)
        self.dtype, self.use_graph = dtype, use_graph
        t: Dict[str, torch.Tensor] = {}
        self.n_res: Optional[int] = None          # blocks whose matrices stay on the device (None: all of them)
        if target_gb is not None:
            tensors = list(tensors)
            shapes = {n: tuple(v.shape) for n, v in tensors}
            n_layer = 1 + max(int(k.split(".")[1]) for k in shapes if k.startswith("blocks."))
            d, f = shapes["blocks.0.ffn.key.weight"][1], shapes["blocks.0.ffn.key.weight"][0]
            block_bytes = (5 * d * d + 2 * d * f) * torch.empty(0, dtype=dtype).element_size()
            self.n_res = min(n_layer, int(target_gb * 1e9) // block_bytes)
            if self.n_res == n_layer:
                self.n_res = None
        host: Dict[str, torch.Tensor] = {}
        for name, v in tensors:
            v = v.detach()
            if name.endswith("att.time_decay_final"):
                name, final = name[:-len("_final")], True
            else:
                final = decay_is_final
            if ".time_" in name:
                v = v.reshape(-1)
            if name.endswith("att.time_decay") and not final:
                v = -torch.exp(v.double())
            if v.dim() == 2 and name != "emb.weight":
                if self.n_res is not None and name.startswith("blocks.") and int(name.split(".")[1]) >= self.n_res:
                    host[name] = v.to(device="cpu", dtype=dtype).contiguous()     # streamed block: stays in host memory
                else:
                    t[name] = v.to(device=self.device, dtype=dtype).contiguous()   # initTensor, torch.py:146-152
            else:
                t[name] = v.to(device=self.device, dtype=torch.float32).contiguous()
        self.t = t
        self.n_layer = 1 + max(int(k.split(".")[1]) for k in t if k.startswith("blocks."))
        self.n_vocab, self.n_embd = t["emb.weight"].shape
        self.n_ffn = (t["blocks.0.ffn.key.weight"] if "blocks.0.ffn.key.weight" in t else host["blocks.0.ffn.key.weight"]).shape[0]
        # Streamed blocks: one pinned blob per block (its seven matrices at 256-byte aligned offsets) and two
        # staging buffers on the device; descriptor s addresses every streamed block inside staging buffer s.
        self._blob: Dict[int, torch.Tensor] = {}
        self._stage = []
        offsets: Dict[str, int] = {}
        if self.n_res is not None:
            off = 0
            for k in _MATS:
                offsets[k] = off
                off += (host[f"blocks.{self.n_res}.{k}.weight"].numel() * host[f"blocks.{self.n_res}.{k}.weight"].element_size() + 255) // 256 * 256
            for i in range(self.n_res, self.n_layer):
                blob = torch.empty(off, dtype=torch.uint8, pin_memory=pin_memory)
                for k in _MATS:
                    w = host.pop(f"blocks.{i}.{k}.weight")
                    view = blob[offsets[k]:offsets[k] + w.numel() * w.element_size()].view(dtype).view(w.shape)
                    view.copy_(w)
                    t[f"blocks.{i}.{k}.weight"] = view                 # host view: weight_bytes() still counts it
                self._blob[i] = blob
            self._stage = [torch.empty(off, dtype=torch.uint8, device=self.device) for _ in range(2)]
        self._clayers_slot, self._cmodel_slot = [], []
        for slot in range(2 if self.n_res is not None else 1):
            layers = (_lib.DenseLayer * self.n_layer)()
            for i in range(self.n_layer):
                c, p = layers[i], f"blocks.{i}."
                (c.ln1_w, c.ln1_b, c.ln2_w, c.ln2_b, c.att_mix_k, c.att_mix_v, c.att_mix_r, c.ffn_mix_k, c.ffn_mix_r,
                 c.time_decay, c.time_first) = (t[p + k].data_ptr() for k in _VECS)
                if i in self._blob:
                    base = self._stage[slot].data_ptr()
                    ptrs = [base + offsets[k] for k in _MATS]
                else:
                    ptrs = [t[p + k + ".weight"].data_ptr() for k in _MATS]
                (c.att_key, c.att_value, c.att_receptance, c.att_output, c.ffn_key, c.ffn_receptance, c.ffn_value) = ptrs
            self._clayers_slot.append(layers)
            self._cmodel_slot.append(_lib.DenseModel(self.n_layer, self.n_embd, self.n_ffn, self.n_vocab, DTYPES[dtype],
                                                     t["emb.weight"].data_ptr(), t["blocks.0.ln0.weight"].data_ptr(),
                                                     t["blocks.0.ln0.bias"].data_ptr(), t["ln_out.weight"].data_ptr(),
                                                     t["ln_out.bias"].data_ptr(), t["head.weight"].data_ptr(),
                                                     C.cast(layers, C.POINTER(_lib.DenseLayer))))
        self._clayers, self._cmodel = self._clayers_slot[0], self._cmodel_slot[0]
        if self.n_res is not None:
            self.use_graph = False                  # copies and events between the blocks: no graph replay
            self._copy_stream = torch.cuda.Stream(self.device)
            self._ready = [torch.cuda.Event(), torch.cuda.Event()]
            self._free = [torch.cuda.Event(), torch.cuda.Event()]
            self._seq = 0                           # streamed blocks handled so far: block j of the sequence uses buffer j % 2
            self._queued = 0                        # copies queued so far
            self.h2d_bytes = 0
        need = int(self._L.b200rwkv_dense_workspace_bytes(C.byref(self._cmodel)))
        self._ws = torch.zeros(need, dtype=torch.uint8, device=self.device)
        self._tok = torch.zeros(1, dtype=torch.int64, device=self.device)
        self._logits = torch.zeros(self.n_vocab, dtype=torch.float32, device=self.device)
        self.emptyState = torch.zeros(self.n_layer, 5, self.n_embd, dtype=torch.float32, device=self.device)
        self.emptyState[:, 4] = -1e30                                               # base.py:61-62
        self._graphs: Dict[Tuple[int, bool], torch.cuda.CUDAGraph] = {}
        self._seen: Dict[Tuple[int, bool], int] = {}
        self.launches_per_step = 6 * self.n_layer + 3
        self.rows_threshold = 4          # tokens per call from which the tensor-core rows path is used
        self.rows_per_call = 4096        # rows one rows call handles; longer prompts are fed in pieces
        self._rows_ws: Dict[Tuple[int, int], torch.Tensor] = {}
        self._status_host, self._status_event, self._status_pending = None, None, False
        self.launch_count = 0

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_checkpoint(cls, ck: Union[str, Dict[str, torch.Tensor]], dtype: torch.dtype = torch.bfloat16, device="cuda:0",
                        use_graph: bool = True, target_gb: Optional[float] = None, pin_memory: bool = True) -> "B200DenseRWKV":
        if isinstance(ck, str):
            ck = torch.load(ck, map_location="cpu")
        return cls(ck.items(), dtype=dtype, device=device, use_graph=use_graph, target_gb=target_gb, pin_memory=pin_memory)

    @classmethod
    def synthetic(cls, layers: int, embed: int, vocab: int = VOCAB, seed: int = 1234, dtype: torch.dtype = torch.bfloat16,
                  device="cuda:0", use_graph: bool = True) -> "B200DenseRWKV":
        """Seeded random weights of the RWKV-4 architecture, generated on the device one tensor at a time."""
        return cls(iter_synth_tensors(layers, embed, vocab=vocab, seed=seed, device=str(device)), dtype=dtype,
                   device=device, use_graph=use_graph)

    def weight_bytes(self) -> int:
        """Bytes of matrix weights one token reads (embedding row excluded)."""
        return sum(v.numel() * v.element_size() for k, v in self.t.items() if v.dim() == 2 and k != "emb.weight")

    # ------------------------------------------------------------------ one token
    def _step_raw(self, state_ptr: int, logits_ptr: Optional[int]) -> None:
        stream = torch.cuda.current_stream(self.device).cuda_stream
        _lib.check(self._L.b200rwkv_dense_step(C.byref(self._cmodel), self._tok.data_ptr(), state_ptr, logits_ptr,
                                               self._ws.data_ptr(), self._ws.numel(), stream))

    # ------------------------------------------------------------------ blocks streamed from host memory
    def _queue_copy(self) -> None:
        """Queue the copy of the next streamed block (in the circular order the kernels use them) into
        buffer `_queued % 2`, once the kernels that last read that buffer have finished."""
        n_str = self.n_layer - self.n_res
        layer = self.n_res + self._queued % n_str
        slot = self._queued % 2
        with torch.cuda.stream(self._copy_stream):
            self._copy_stream.wait_event(self._free[slot])
            self._stage[slot].copy_(self._blob[layer], non_blocking=True)
            self._ready[slot].record(self._copy_stream)
        self.h2d_bytes += self._blob[layer].numel()
        self._queued += 1

    def _run_streamed(self, call) -> None:
        """``call(cmodel, layer_begin, layer_end)`` for the resident blocks in one range, then for every
        streamed block as soon as its copy has landed; copies run two blocks ahead."""
        cur = torch.cuda.current_stream(self.device)
        call(self._cmodel_slot[0], 0, self.n_res)               # embedding + resident blocks (an empty range: embedding only)
        for layer in range(self.n_res, self.n_layer):
            while self._queued < self._seq + 2:
                self._queue_copy()
            slot = self._seq % 2
            cur.wait_event(self._ready[slot])
            call(self._cmodel_slot[slot], layer, layer + 1)
            self._free[slot].record(cur)
            self._seq += 1

    def _step(self, state: torch.Tensor, want_logits: bool) -> None:
        self.launch_count += self.launches_per_step - (0 if want_logits else 2)
        lp = self._logits.data_ptr() if want_logits else None
        if self.n_res is not None:
            stream = torch.cuda.current_stream(self.device).cuda_stream
            self._run_streamed(lambda cm, l0, l1: _lib.check(self._L.b200rwkv_dense_step_layers(
                C.byref(cm), l0, l1, self._tok.data_ptr(), state.data_ptr(), lp, self._ws.data_ptr(), self._ws.numel(), stream)))
            return
        if not self.use_graph:
            self._step_raw(state.data_ptr(), lp)
            return
        key = (state.data_ptr(), want_logits)
        g = self._graphs.get(key)
        if g is None:
            n = self._seen.get(key, 0) + 1          # capture when a state buffer shows up for the second time
            self._seen[key] = n
            if n < 2:
                self._step_raw(state.data_ptr(), lp)
                return
            if len(self._graphs) >= 16:
                self._graphs.clear()
                self._seen.clear()
            g = torch.cuda.CUDAGraph()
            torch.cuda.synchronize(self.device)
            with torch.cuda.graph(g):
                self._step_raw(state.data_ptr(), lp)
            self._graphs[key] = g
        g.replay()

    def check_status(self) -> None:
        """Raise if a kernel gave up a bounded device-side wait (synchronises).  The state the failed
        call was given is undefined after that."""
        for buf in [self._ws, *self._rows_ws.values()]:
            bits = int(buf[:4].view(torch.int32).cpu()[0])
            if bits:
                buf.zero_()                 # status word and, in a rows workspace, the tickets of an abandoned K split
                raise _lib.B200RWKVError(_lib.ETIMEOUT, f"device-side wait expired, status bits 0x{bits:x}")

    def _queue_status(self, buf: Optional[torch.Tensor] = None) -> None:
        """Non-blocking copy of a workspace's status word to pinned memory; looked at by a later call once it has landed."""
        buf = self._ws if buf is None else buf
        if self._status_host is None:
            self._status_host = torch.zeros(1, dtype=torch.int32).pin_memory()
            self._status_event = torch.cuda.Event()
        self._status_host.copy_(buf[:4].view(torch.int32), non_blocking=True)
        self._status_event.record(torch.cuda.current_stream(self.device))
        self._status_pending = True

    def _raise_status(self) -> None:
        if not self._status_pending or not self._status_event.query():
            return
        self._status_pending = False
        if int(self._status_host[0]):
            self.check_status()

    # ------------------------------------------------------------------ many rows at once
    def empty_batch_state(self, B: int) -> torch.Tensor:
        return self.emptyState.unsqueeze(0).repeat(B, 1, 1, 1).contiguous()

    def forward_rows(self, tokens: torch.Tensor, state: torch.Tensor) -> torch.Tensor:
        """``tokens [B,T]`` int64, ``state [B,L,5,D]`` fp32 contiguous on the device (updated in place):
        B independent sequences, every matrix applied to all B*T rows at once.  Returns the logits
        ``[B,V]`` after each sequence's last token.  bf16 / fp16 models only."""
        if self.dtype == torch.float32:
            raise ValueError("forward_rows needs bf16 or fp16 matrices; feed an fp32 model token by token")
        if tokens.dim() != 2 or tokens.numel() == 0:
            raise ValueError("forward_rows needs tokens [B,T] with at least one token")
        B, T = tokens.shape
        if (state.dtype != torch.float32 or state.device != self.device or not state.is_contiguous()
                or tuple(state.shape) != (B, self.n_layer, 5, self.n_embd)):
            raise ValueError(f"forward_rows needs a contiguous fp32 state [{B},{self.n_layer},5,{self.n_embd}] on the model's device")
        self._raise_status()
        out = torch.empty(B, self.n_vocab, dtype=torch.float32, device=self.device)
        piece = max(1, self.rows_per_call // B)
        with torch.cuda.device(self.device):
            toks = tokens.to(self.device, non_blocking=True)
            stream = torch.cuda.current_stream(self.device).cuda_stream
            for t0 in range(0, T, piece):
                tp = min(piece, T - t0)
                ws = self._rows_ws.get((B, tp))
                if ws is None:
                    if len(self._rows_ws) >= 4:
                        self._rows_ws.clear()
                    need = int(self._L.b200rwkv_dense_rows_workspace_bytes(C.byref(self._cmodel), B, tp))
                    if need == 0:
                        raise ValueError("forward_rows: at most 65535 rows per call")
                    ws = self._rows_ws[(B, tp)] = torch.zeros(need, dtype=torch.uint8, device=self.device)
                part = toks[:, t0:t0 + tp].contiguous()
                last = t0 + tp == T
                lp = out.data_ptr() if last else None
                if self.n_res is not None:
                    self._run_streamed(lambda cm, l0, l1: _lib.check(self._L.b200rwkv_dense_forward_rows_layers(
                        C.byref(cm), l0, l1, part.data_ptr(), B, tp, state.data_ptr(), state.stride(0), lp, ws.data_ptr(),
                        ws.numel(), stream)))
                else:
                    _lib.check(self._L.b200rwkv_dense_forward_rows(C.byref(self._cmodel), part.data_ptr(), B, tp, state.data_ptr(),
                                                                   state.stride(0), lp, ws.data_ptr(), ws.numel(), stream))
                self.launch_count += 12 * self.n_layer + 3
                self._rows_status_src = ws
            self._queue_status(self._rows_status_src)
        return out

    def forward(self, tokens, state: torch.Tensor):
        if not torch.is_tensor(tokens):
            tokens = torch.tensor(tokens if isinstance(tokens, (list, tuple)) else [tokens], dtype=torch.int64)
        tokens = tokens.reshape(-1).to(torch.int64)
        if tokens.numel() == 0:
            raise ValueError("forward needs at least one token")
        if tuple(state.shape) != (self.n_layer, 5, self.n_embd):
            raise ValueError(f"state must be [{self.n_layer},5,{self.n_embd}], got {tuple(state.shape)}")
        if state.dtype != torch.float32 or state.device != self.device or not state.is_contiguous():
            state = state.to(device=self.device, dtype=torch.float32).contiguous()
        if tokens.numel() >= self.rows_threshold and self.dtype != torch.float32 and self.n_embd % 64 == 0 and self.n_ffn % 64 == 0:
            return self.forward_rows(tokens.reshape(1, -1), state.unsqueeze(0))[0], state
        self._raise_status()
        with torch.cuda.device(self.device):
            toks = tokens.to(self.device, non_blocking=True)
            T = toks.numel()
            for i in range(T):
                self._tok.copy_(toks[i:i + 1], non_blocking=True)
                self._step(state, want_logits=(i == T - 1))
            self._queue_status()
        return self._logits.clone(), state

    __call__ = forward
