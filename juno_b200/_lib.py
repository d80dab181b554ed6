"""ctypes binding of libjuno_b200.so — the same C ABI a Java host binds through Panama.

There is no CPU fallback: importing this module without the built library raises.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libjuno_b200.so")

OK, ERR_INVALID_ARG, ERR_OOM, ERR_CUDA, ERR_NCCL, ERR_TIMEOUT, ERR_CLOSED, ERR_UNSUPPORTED = 0, -1, -2, -3, -4, -5, -6, -7
TYPE_F32, TYPE_Q8_0, TYPE_Q4_K, TYPE_Q6_K = 0, 8, 12, 14

(T_TOKEN_EMBD, T_OUTPUT_NORM, T_OUTPUT, T_ATTN_NORM, T_FFN_NORM, T_ATTN_Q, T_ATTN_K, T_ATTN_V, T_ATTN_OUT,
 T_FFN_GATE, T_FFN_UP, T_FFN_DOWN) = range(12)


class ModelCfg(C.Structure):
    _fields_ = [("struct_size", C.c_int32), ("hidden", C.c_int32), ("n_layers", C.c_int32), ("n_heads", C.c_int32),
                ("n_kv_heads", C.c_int32), ("inter", C.c_int32), ("vocab", C.c_int32), ("rms_eps", C.c_float),
                ("rope_theta", C.c_float), ("max_batch", C.c_int32), ("max_seqs", C.c_int32), ("max_ctx", C.c_int32),
                ("kv_dtype", C.c_int32), ("tp_rank", C.c_int32), ("tp_world", C.c_int32), ("nccl_id", C.c_uint8 * 128)]


class Counters(C.Structure):
    _fields_ = [("kernel_launches", C.c_int64), ("gemv_calls", C.c_int64), ("forward_calls", C.c_int64),
                ("h2d_bytes", C.c_int64), ("d2h_bytes", C.c_int64)]


class ProfileEntry(C.Structure):
    _fields_ = [("launches", C.c_int64), ("ms", C.c_double), ("algo_bytes", C.c_double)]


PROF_NAMES = ["gemv_q4k", "gemv_q6k", "gemv_q8_0", "attention", "rope_append", "other", "gemm_tcgen05"]

P = C.c_void_p
PP = C.POINTER(C.c_void_p)
I32, I64 = C.c_int32, C.c_int64

# name -> (restype, argtypes); every symbol include/juno_b200.h declares
SIGNATURES = {
    "juno_last_error": (C.c_char_p, []),
    "juno_device_count": (C.c_int, [C.POINTER(I32)]),
    "juno_device_name": (C.c_int, [I32, C.c_char_p, I32]),
    "juno_device_total_mem": (C.c_int, [I32, C.POINTER(I64)]),
    "juno_ctx_create": (C.c_int, [I32, PP]),
    "juno_ctx_destroy": (C.c_int, [P]),
    "juno_ctx_device": (C.c_int, [P, C.POINTER(I32)]),
    "juno_ctx_synchronize": (C.c_int, [P]),
    "juno_ctx_counters": (C.c_int, [P, C.POINTER(Counters), I32]),
    "juno_ctx_stream": (C.c_int, [P, PP]),
    "juno_ctx_profile": (C.c_int, [P, I32]),
    "juno_ctx_profile_read": (C.c_int, [P, P, I32, I32]),
    "juno_qmat_upload": (C.c_int, [P, P, I32, I64, I64, PP]),
    "juno_qmat_free": (C.c_int, [P]),
    "juno_qmat_shape": (C.c_int, [P, C.POINTER(I64), C.POINTER(I64), C.POINTER(I32)]),
    "juno_gemv": (C.c_int, [P, P, P, I32, P]),
    "juno_gemv_device": (C.c_int, [P, P, P, I32, P, P]),
    "juno_dequantize": (C.c_int, [P, P, I64, I64, P]),
    "juno_sgemv_f32": (C.c_int, [P, P, P, I64, I64, P]),
    "juno_kvpool_create": (C.c_int, [P, I32, I32, I32, I32, I32, PP]),
    "juno_kvpool_free": (C.c_int, [P]),
    "juno_kvseq_create": (C.c_int, [P, I32, PP]),
    "juno_seq_free": (C.c_int, [P]),
    "juno_seq_length": (C.c_int, [P, C.POINTER(I32)]),
    "juno_seq_fork": (C.c_int, [P, I32, PP]),
    "juno_seq_append_kv": (C.c_int, [P, I32, I32, I32, P, P]),
    "juno_attn_decode": (C.c_int, [P, P, I32, I32, PP, I32, P, P]),
    "juno_attn_decode_static": (C.c_int, [P, P, I32, I32, PP, I32, P, P]),
    "juno_tp_slice": (C.c_int, [I32, I32, I32, I32, I32, I32, I32, I32, C.POINTER(I64)]),
    "juno_nccl_unique_id": (C.c_int, [P]),
    "juno_model_create": (C.c_int, [P, C.POINTER(ModelCfg), PP]),
    "juno_model_set_tensor": (C.c_int, [P, I32, I32, P, I32, I64, I64]),
    "juno_model_finalize": (C.c_int, [P]),
    "juno_model_free": (C.c_int, [P]),
    "juno_model_tp_mode": (C.c_int, [P, C.POINTER(I32)]),
    "juno_model_seq_create": (C.c_int, [P, PP]),
    "juno_forward": (C.c_int, [P, I32, PP, P, P, P, P]),
    "juno_decode_greedy": (C.c_int, [P, I32, PP, P, P, I32, P]),
    "juno_prefill": (C.c_int, [P, P, P, I32, I32, P, P]),
    "juno_model_last_hidden": (C.c_int, [P, I32, P]),
    "juno_gguf_open": (C.c_int, [C.c_char_p, PP]),
    "juno_gguf_close": (C.c_int, [P]),
    "juno_gguf_info": (C.c_int, [P, C.POINTER(I32), C.POINTER(I64), C.POINTER(I64), C.POINTER(I64)]),
    "juno_gguf_meta_int": (C.c_int, [P, C.c_char_p, I64, C.POINTER(I64)]),
    "juno_gguf_meta_float": (C.c_int, [P, C.c_char_p, C.c_double, C.POINTER(C.c_double)]),
    "juno_gguf_meta_string": (C.c_int, [P, C.c_char_p, C.c_char_p, I32, C.POINTER(I32)]),
    "juno_gguf_meta_array_len": (C.c_int, [P, C.c_char_p, C.POINTER(I64)]),
    "juno_gguf_tensor_name": (C.c_int, [P, I64, C.c_char_p, I32]),
    "juno_gguf_has_tensor": (C.c_int, [P, C.c_char_p, C.POINTER(I32)]),
    "juno_gguf_tensor": (C.c_int, [P, C.c_char_p, C.POINTER(I32), C.POINTER(I32), C.POINTER(I64), PP, C.POINTER(I64)]),
    "juno_gguf_raw_byte_count": (C.c_int, [I32, I64, C.POINTER(I64)]),
    "juno_gguf_model_cfg": (C.c_int, [P, C.POINTER(ModelCfg)]),
    "juno_model_load_gguf": (C.c_int, [P, P]),
}

_lib = None


def load() -> C.CDLL:
    """Loads the shared library and attaches the signatures. Raises if it was not built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m juno_b200.build` "
                               "(this backend has no CPU fallback)")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


class JunoError(RuntimeError):
    """Non-zero status from the library (the Java host raises IllegalStateException, CudaBindings.java:247-250)."""

    def __init__(self, op: str, rc: int, msg: str):
        super().__init__(f"{op} failed: rc={rc} ({msg})")
        self.rc = rc


def last_error() -> str:
    return (load().juno_last_error() or b"").decode("utf-8", "replace")


def check(rc: int, op: str) -> None:
    if rc != OK:
        msg = last_error()
        if rc == ERR_INVALID_ARG:
            raise ValueError(f"{op}: {msg}")  # IllegalArgumentException in the Java contract
        raise JunoError(op, rc, msg)
