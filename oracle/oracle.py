"""ctypes binding of the CPU oracle (oracle/juno_oracle.c).

Test infrastructure only: imported by tests/, by the smoke test and by the
CPU-baseline leg of bench.py.  The product package never imports this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liboracle.so")

F32, Q8_0, Q4_K, Q6_K = 0, 8, 12, 14

# tensor kinds (same numbering as the engine's C ABI)
(T_TOKEN_EMBD, T_OUTPUT_NORM, T_OUTPUT, T_ATTN_NORM, T_FFN_NORM, T_ATTN_Q, T_ATTN_K, T_ATTN_V,
 T_ATTN_OUT, T_FFN_GATE, T_FFN_UP, T_FFN_DOWN) = range(12)


def build(force: bool = False) -> str:
    """Compile liboracle.so with the recipe of oracle/Makefile."""
    src = os.path.join(_HERE, "juno_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(
            ["gcc", "-O2", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off", "-fno-fast-math",
             "-std=c11", "-o", _SO, src, "-lm"])
    return _SO


class _Cfg(C.Structure):
    _fields_ = [("hidden", C.c_int), ("layers", C.c_int), ("heads", C.c_int), ("kv_heads", C.c_int),
                ("head_dim", C.c_int), ("inter", C.c_int), ("vocab", C.c_int), ("eps", C.c_float),
                ("theta", C.c_float), ("kv_f16", C.c_int), ("max_seq", C.c_int)]


_lib = None


def lib():
    global _lib
    if _lib is None:
        L = C.CDLL(build())
        L.jo_f16_to_f32.restype = C.c_float
        L.jo_f16_to_f32.argtypes = [C.c_uint16]
        L.jo_f32_to_f16.restype = C.c_uint16
        L.jo_f32_to_f16.argtypes = [C.c_float]
        L.jo_row_bytes.restype = C.c_int64
        L.jo_row_bytes.argtypes = [C.c_int, C.c_int64]
        L.jo_dequantize.argtypes = [C.c_int, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]
        L.jo_matvec.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64,
                                C.c_void_p]
        L.jo_matvec_batch.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int64,
                                      C.c_void_p]
        L.jo_rmsnorm.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_float, C.c_void_p]
        L.jo_rope.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_float]
        L.jo_softmax.argtypes = [C.c_void_p, C.c_int]
        L.jo_silu.restype = C.c_float
        L.jo_silu.argtypes = [C.c_float]
        L.jo_gqa.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                             C.c_void_p, C.c_void_p]
        L.jo_greedy.restype = C.c_int
        L.jo_greedy.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        L.jo_q4k_scale.argtypes = [C.c_void_p, C.c_int]
        L.jo_q4k_min.argtypes = [C.c_void_p, C.c_int]
        L.jo_model_create.restype = C.c_void_p
        L.jo_model_create.argtypes = [C.POINTER(_Cfg)]
        L.jo_model_free.argtypes = [C.c_void_p]
        L.jo_model_set_tensor.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int,
                                          C.c_int64, C.c_int64]
        L.jo_seq_create.restype = C.c_void_p
        L.jo_seq_create.argtypes = [C.c_void_p]
        L.jo_seq_free.argtypes = [C.c_void_p]
        L.jo_seq_fill.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_uint]
        L.jo_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        L.jo_generate_greedy.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                         C.c_void_p, C.c_void_p]
        L.jo_allreduce_sum.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        L.jo_num_threads.restype = C.c_int
        L.jo_set_num_threads.argtypes = [C.c_int]
        _lib = L
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _u8(a) -> np.ndarray:
    a = np.ascontiguousarray(a)
    return a.view(np.uint8).reshape(-1)


def f16_to_f32(bits: int) -> float:
    return float(lib().jo_f16_to_f32(bits & 0xFFFF))


def f32_to_f16(v: float) -> int:
    return int(lib().jo_f32_to_f16(float(v)))


def row_bytes(ggml_type: int, cols: int) -> int:
    return int(lib().jo_row_bytes(ggml_type, cols))


def dequantize(ggml_type: int, raw, rows: int, cols: int) -> np.ndarray:
    raw = _u8(raw)
    assert raw.size == rows * row_bytes(ggml_type, cols)
    out = np.empty((rows, cols), dtype=np.float32)
    assert lib().jo_dequantize(ggml_type, _p(raw), rows, cols, _p(out)) == 0
    return out


def matvec(ggml_type: int, raw, x, rows: int, cols: int, row_start: int = 0, row_end: int | None = None):
    """y[batch, rows'] for x[batch, cols] (or 1-D x → 1-D y)."""
    raw = _u8(raw)
    x = _f32(x)
    row_end = rows if row_end is None else row_end
    one = x.ndim == 1
    xb = x.reshape(-1, cols)
    y = np.empty((xb.shape[0], row_end - row_start), dtype=np.float32)
    for b in range(xb.shape[0]):
        rc = lib().jo_matvec(ggml_type, _p(raw), _p(xb[b]), row_start, row_end, cols, _p(y[b]))
        assert rc == 0
    return y[0] if one else y


def rmsnorm(x, w, eps: float) -> np.ndarray:
    x, w = _f32(x), _f32(w)
    out = np.empty_like(x)
    lib().jo_rmsnorm(_p(x), _p(w), x.size, eps, _p(out))
    return out


def rope(x, pos: int, n_heads: int, head_dim: int, theta: float) -> np.ndarray:
    x = _f32(x).copy()
    lib().jo_rope(_p(x), pos, n_heads, head_dim, theta)
    return x


def softmax(s) -> np.ndarray:
    s = _f32(s).copy()
    lib().jo_softmax(_p(s), s.size)
    return s


def silu(v: float) -> float:
    return float(lib().jo_silu(v))


def gqa(q, K, V, seq_len: int, n_heads: int, n_kv_heads: int, head_dim: int) -> np.ndarray:
    q, K, V = _f32(q), _f32(K), _f32(V)
    out = np.empty(n_heads * head_dim, dtype=np.float32)
    scores = np.empty(seq_len, dtype=np.float32)
    lib().jo_gqa(_p(q), _p(K), _p(V), seq_len, n_heads, n_kv_heads, head_dim, _p(out), _p(scores))
    return out


def greedy(logits) -> int:
    logits = _f32(logits)
    probs = np.empty_like(logits)
    return int(lib().jo_greedy(_p(logits), logits.size, _p(probs)))


def allreduce_sum(parts) -> np.ndarray:
    parts = _f32(parts)
    out = np.empty(parts.shape[1], dtype=np.float32)
    lib().jo_allreduce_sum(_p(parts), parts.shape[0], parts.shape[1], _p(out))
    return out


def num_threads() -> int:
    return int(lib().jo_num_threads())


def set_num_threads(n: int) -> None:
    lib().jo_set_num_threads(int(n))


class Model:
    """Oracle model: tensors are borrowed numpy buffers (kept alive here)."""

    def __init__(self, hidden, layers, heads, kv_heads, inter, vocab, eps, theta, kv_f16=False,
                 max_seq=2048):
        self.cfg = _Cfg(hidden, layers, heads, kv_heads, hidden // heads, inter, vocab, eps, theta,
                        1 if kv_f16 else 0, max_seq)
        self.h = lib().jo_model_create(C.byref(self.cfg))
        self._keep = []

    def set_tensor(self, kind: int, layer: int, data, ggml_type: int, rows: int, cols: int):
        buf = _u8(data)
        assert buf.size == rows * row_bytes(ggml_type, cols), (kind, layer, buf.size, rows, cols)
        self._keep.append(buf)
        assert lib().jo_model_set_tensor(self.h, kind, layer, _p(buf), ggml_type, rows, cols) == 0

    def new_seq(self):
        return Seq(self)

    def forward(self, seq, token: int, pos: int, want_logits=True, want_hidden=False):
        logits = np.empty(self.cfg.vocab, dtype=np.float32) if want_logits else None
        hidden = np.empty(self.cfg.hidden, dtype=np.float32) if want_hidden else None
        rc = lib().jo_forward(self.h, seq.h, token, pos, _p(logits) if want_logits else None,
                              _p(hidden) if want_hidden else None)
        assert rc == 0, "position beyond max_seq"
        if want_hidden:
            return logits, hidden
        return logits

    def generate_greedy(self, seq, prompt, steps: int):
        prompt = np.ascontiguousarray(prompt, dtype=np.int32)
        ids = np.empty(steps, dtype=np.int32)
        margins = np.empty(steps, dtype=np.float32)
        rc = lib().jo_generate_greedy(self.h, seq.h, _p(prompt), prompt.size, steps, _p(ids), _p(margins))
        assert rc == 0
        return ids, margins

    def close(self):
        if self.h:
            lib().jo_model_free(self.h)
            self.h = None

    def __del__(self):
        self.close()


class Seq:
    def __init__(self, model: Model):
        self.model = model
        self.h = lib().jo_seq_create(model.h)

    def fill(self, n_pos: int, seed: int = 1):
        """Benchmark helper: pseudo-random K/V for positions [0, n_pos) of every layer (no forward passes)."""
        lib().jo_seq_fill(self.h, self.model.h, int(n_pos), int(seed))

    def close(self):
        if self.h:
            lib().jo_seq_free(self.h)
            self.h = None

    def __del__(self):
        self.close()
