"""ctypes binding of ``libb200rwkv.so`` (C ABI declared in ``include/b200rwkv.h``).

The library is the product: there is no Python or CPU fallback.  If the shared object is
missing or fails to load, importing this module's ``lib()`` raises with the build command.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libb200rwkv.so")

OK, EINVAL, ECUDA, ETIMEOUT = 0, -1, -2, -3
STATUS_WAIT_FULL, STATUS_WAIT_EMPTY, STATUS_WAIT_PEER = 1, 2, 4

# Every symbol include/b200rwkv.h declares; tests check that the library exports all of them.
EXPORTS = (
    "b200rwkv_version", "b200rwkv_last_error", "b200rwkv_gemv_u8", "b200rwkv_wkv_scan", "b200rwkv_gemv_plan",
    "b200rwkv_gemv_u8_traced", "b200rwkv_gemv_workspace_bytes", "b200rwkv_gemv_u8_static",
    "b200rwkv_decode_workspace_bytes", "b200rwkv_decode_step", "b200rwkv_decode_step_traced", "b200rwkv_decode_step_stage",
    "b200rwkv_gemm_workspace_bytes", "b200rwkv_gemm_u8", "b200rwkv_rows_workspace_bytes", "b200rwkv_forward_rows", "b200rwkv_forward_rows_stage", "b200rwkv_argmax",
    "b200rwkv_sample_typical", "b200rwkv_gemv_dense",
    "b200rwkv_dense_workspace_bytes", "b200rwkv_dense_step", "b200rwkv_dense_rows_workspace_bytes", "b200rwkv_dense_forward_rows",
    "b200rwkv_dense_step_layers", "b200rwkv_dense_forward_rows_layers", "b200rwkv_wait_selftest", "b200rwkv_debug_expire_waits",
    "b200rwkv_step_plan_bytes", "b200rwkv_step_plan_init", "b200rwkv_decode_step_persistent", "b200rwkv_step_geometry",
)


class Matrix(C.Structure):
    _fields_ = [("qt", C.c_void_p), ("ry", C.c_void_p), ("my", C.c_void_p), ("rx", C.c_void_p),
                ("mx", C.c_void_p), ("half", C.c_float), ("n_out", C.c_int32), ("k_in", C.c_int32)]


class Layer(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in (
        "ln1_w", "ln1_b", "ln2_w", "ln2_b", "att_mix_k", "att_mix_v", "att_mix_r",
        "ffn_mix_k", "ffn_mix_r", "time_decay", "time_first")] + [
        (n, Matrix) for n in ("att_key", "att_value", "att_receptance", "att_output",
                              "ffn_key", "ffn_receptance", "ffn_value")]


class Model(C.Structure):
    _fields_ = [("n_layer", C.c_int32), ("n_embd", C.c_int32), ("n_ffn", C.c_int32), ("n_vocab", C.c_int32),
                ("emb", C.c_void_p), ("ln0_w", C.c_void_p), ("ln0_b", C.c_void_p),
                ("ln_out_w", C.c_void_p), ("ln_out_b", C.c_void_p), ("head", Matrix),
                ("layers", C.POINTER(Layer))]


class DenseLayer(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in (
        "ln1_w", "ln1_b", "ln2_w", "ln2_b", "att_mix_k", "att_mix_v", "att_mix_r", "ffn_mix_k", "ffn_mix_r",
        "time_decay", "time_first", "att_key", "att_value", "att_receptance", "att_output",
        "ffn_key", "ffn_receptance", "ffn_value")]


class DenseModel(C.Structure):
    _fields_ = [("n_layer", C.c_int32), ("n_embd", C.c_int32), ("n_ffn", C.c_int32), ("n_vocab", C.c_int32),
                ("dtype", C.c_int32), ("emb", C.c_void_p), ("ln0_w", C.c_void_p), ("ln0_b", C.c_void_p),
                ("ln_out_w", C.c_void_p), ("ln_out_b", C.c_void_p), ("head", C.c_void_p),
                ("layers", C.POINTER(DenseLayer))]


class B200RWKVError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"b200rwkv error {code}: {message}")
        self.code = code


_lib: Optional[C.CDLL] = None


def lib() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing; build it with `python -m rwkvstic_b200.build` "
                          "(needs nvcc; there is no CPU fallback)")
    L = C.CDLL(LIB_PATH)
    L.b200rwkv_version.restype = C.c_int
    L.b200rwkv_last_error.restype = C.c_char_p
    L.b200rwkv_gemv_u8.restype = C.c_int
    L.b200rwkv_gemv_u8.argtypes = [C.c_int, C.POINTER(Matrix), C.POINTER(C.c_void_p), C.POINTER(C.c_void_p),
                                   C.c_int, C.c_void_p, C.c_size_t, C.c_void_p]
    L.b200rwkv_gemv_workspace_bytes.restype = C.c_size_t
    L.b200rwkv_gemv_workspace_bytes.argtypes = [C.c_int, C.c_int]
    L.b200rwkv_gemv_u8_traced.restype = C.c_int
    L.b200rwkv_gemv_u8_traced.argtypes = [C.c_int, C.POINTER(Matrix), C.POINTER(C.c_void_p), C.POINTER(C.c_void_p),
                                          C.c_int, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p]
    L.b200rwkv_gemv_u8_static.restype = C.c_int
    L.b200rwkv_gemv_u8_static.argtypes = [C.c_int, C.POINTER(Matrix), C.POINTER(C.c_void_p), C.POINTER(C.c_void_p),
                                          C.c_int, C.c_void_p, C.c_void_p]
    L.b200rwkv_wkv_scan.restype = C.c_int
    L.b200rwkv_wkv_scan.argtypes = [C.c_int, C.c_int, C.c_int] + [C.c_void_p] * 8 + [C.c_int, C.c_void_p]
    L.b200rwkv_gemv_plan.restype = C.c_int
    L.b200rwkv_gemv_plan.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int64)]
    L.b200rwkv_decode_workspace_bytes.restype = C.c_size_t
    L.b200rwkv_decode_workspace_bytes.argtypes = [C.POINTER(Model)]
    L.b200rwkv_decode_step.restype = C.c_int
    L.b200rwkv_decode_step.argtypes = [C.POINTER(Model), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                       C.c_size_t, C.c_void_p]
    L.b200rwkv_decode_step_stage.restype = C.c_int
    L.b200rwkv_decode_step_stage.argtypes = [C.POINTER(Model), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                             C.c_size_t, C.c_void_p]
    L.b200rwkv_decode_step_traced.restype = C.c_int
    L.b200rwkv_decode_step_traced.argtypes = [C.POINTER(Model), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                              C.c_size_t, C.c_void_p, C.c_void_p]
    L.b200rwkv_step_plan_bytes.restype = C.c_size_t
    L.b200rwkv_step_plan_bytes.argtypes = [C.POINTER(Model)]
    L.b200rwkv_step_plan_init.restype = C.c_int
    L.b200rwkv_step_plan_init.argtypes = [C.POINTER(Model), C.c_void_p, C.c_size_t]
    L.b200rwkv_decode_step_persistent.restype = C.c_int
    L.b200rwkv_decode_step_persistent.argtypes = [C.POINTER(Model), C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p,
                                                  C.c_void_p, C.POINTER(C.c_int32), C.c_void_p, C.c_void_p]
    L.b200rwkv_step_geometry.restype = C.c_int
    L.b200rwkv_step_geometry.argtypes = [C.POINTER(Model), C.c_int, C.POINTER(C.c_int64)]
    L.b200rwkv_gemm_workspace_bytes.restype = C.c_size_t
    L.b200rwkv_gemm_workspace_bytes.argtypes = [C.c_int, C.c_int, C.c_int]
    L.b200rwkv_gemm_u8.restype = C.c_int
    L.b200rwkv_gemm_u8.argtypes = [C.c_int, C.POINTER(Matrix), C.POINTER(C.c_void_p), C.POINTER(C.c_void_p),
                                   C.c_int, C.c_void_p, C.c_size_t, C.c_void_p]
    L.b200rwkv_rows_workspace_bytes.restype = C.c_size_t
    L.b200rwkv_rows_workspace_bytes.argtypes = [C.POINTER(Model), C.c_int, C.c_int]
    L.b200rwkv_forward_rows.restype = C.c_int
    L.b200rwkv_forward_rows.argtypes = [C.POINTER(Model), C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int64,
                                        C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
    L.b200rwkv_forward_rows_stage.restype = C.c_int
    L.b200rwkv_forward_rows_stage.argtypes = [C.POINTER(Model), C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p,
                                              C.c_int64, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
    L.b200rwkv_argmax.restype = C.c_int
    L.b200rwkv_argmax.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,
                                  C.c_void_p]
    L.b200rwkv_sample_typical.restype = C.c_int
    L.b200rwkv_sample_typical.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int64, C.c_float, C.c_float, C.c_void_p,
                                          C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
    L.b200rwkv_gemv_dense.restype = C.c_int
    L.b200rwkv_gemv_dense.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int64, C.c_void_p, C.c_void_p,
                                      C.c_void_p]
    L.b200rwkv_dense_workspace_bytes.restype = C.c_size_t
    L.b200rwkv_dense_workspace_bytes.argtypes = [C.POINTER(DenseModel)]
    L.b200rwkv_dense_step.restype = C.c_int
    L.b200rwkv_dense_step.argtypes = [C.POINTER(DenseModel), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t,
                                      C.c_void_p]
    L.b200rwkv_dense_rows_workspace_bytes.restype = C.c_size_t
    L.b200rwkv_dense_rows_workspace_bytes.argtypes = [C.POINTER(DenseModel), C.c_int, C.c_int]
    L.b200rwkv_dense_forward_rows.restype = C.c_int
    L.b200rwkv_dense_forward_rows.argtypes = [C.POINTER(DenseModel), C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int64,
                                              C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
    L.b200rwkv_dense_step_layers.restype = C.c_int
    L.b200rwkv_dense_step_layers.argtypes = [C.POINTER(DenseModel), C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                             C.c_size_t, C.c_void_p]
    L.b200rwkv_dense_forward_rows_layers.restype = C.c_int
    L.b200rwkv_dense_forward_rows_layers.argtypes = [C.POINTER(DenseModel), C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_void_p,
                                                     C.c_int64, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
    L.b200rwkv_wait_selftest.restype = C.c_int
    L.b200rwkv_wait_selftest.argtypes = [C.c_uint64, C.c_void_p, C.c_void_p]
    L.b200rwkv_debug_expire_waits.restype = C.c_int
    L.b200rwkv_debug_expire_waits.argtypes = [C.c_int, C.c_uint64]
    _lib = L
    return L


def check(code: int) -> None:
    if code != OK:
        raise B200RWKVError(code, lib().b200rwkv_last_error().decode())


def ptr(t) -> Optional[int]:
    """Device (or host) address of a torch tensor, None for None."""
    return None if t is None else t.data_ptr()


PLAN_FIELDS = ("chunk_bytes", "chunks_per_row", "swizzle_bytes", "rows_per_stage",
               "ring_stages", "stage_bytes", "max_rows_per_cta", "grid", "shared_memory_bytes", "consumer_threads")


def gemv_plan(k_in: int, nmat: int, max_n_out: int, num_sms: int = 148) -> dict:
    out = (C.c_int64 * 10)()
    check(lib().b200rwkv_gemv_plan(k_in, nmat, max_n_out, num_sms, out))
    return dict(zip(PLAN_FIELDS, [int(v) for v in out]))
