"""MatVec operator (boundary A) over the C ABI.

Mirrors node/src/main/java/cab/ml/juno/node/{MatVec,GpuMatVec,CudaMatVec,GpuContext}.java: a context per
device, resident matrices uploaded once, `sgemv` returning a fresh array.  Where the reference uploads a
dequantised FP16 copy (GpuMatVec.uploadHalf, DeviceHalfMatrix.java:66-91), `upload_quantized` keeps the
GGUF blocks themselves resident.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import check


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


class GpuContext:
    """One device context (GpuContext.java:109-153). `shared(device)` returns the process-wide instance."""

    _shared: dict[int, "GpuContext"] = {}

    def __init__(self, device: int = 0):
        self._L = _lib.load()
        h = C.c_void_p()
        check(self._L.juno_ctx_create(device, C.byref(h)), "juno_ctx_create")
        self.handle = h
        self.device = device
        self._is_shared = False

    @classmethod
    def shared(cls, device: int = 0) -> "GpuContext":
        if device not in cls._shared:
            ctx = cls(device)
            ctx._is_shared = True
            cls._shared[device] = ctx
        return cls._shared[device]

    @staticmethod
    def device_count() -> int:
        n = C.c_int32()
        check(_lib.load().juno_device_count(C.byref(n)), "juno_device_count")
        return n.value

    @staticmethod
    def device_name(device: int = 0) -> str:
        buf = C.create_string_buffer(256)
        check(_lib.load().juno_device_name(device, buf, 256), "juno_device_name")
        return buf.value.decode()

    def synchronize(self) -> None:
        check(self._L.juno_ctx_synchronize(self.handle), "juno_ctx_synchronize")

    def counters(self, reset: bool = False) -> dict:
        c = _lib.Counters()
        check(self._L.juno_ctx_counters(self.handle, C.byref(c), 1 if reset else 0), "juno_ctx_counters")
        return {k: getattr(c, k) for k, _ in c._fields_}

    def stream(self) -> int:
        """cudaStream_t (as an integer) all work of this context runs on."""
        h = C.c_void_p()
        check(self._L.juno_ctx_stream(self.handle, C.byref(h)), "juno_ctx_stream")
        return h.value or 0

    def profile(self, enable: bool) -> None:
        check(self._L.juno_ctx_profile(self.handle, 1 if enable else 0), "juno_ctx_profile")

    def profile_read(self, reset: bool = True) -> dict:
        arr = (_lib.ProfileEntry * len(_lib.PROF_NAMES))()
        check(self._L.juno_ctx_profile_read(self.handle, arr, len(arr), 1 if reset else 0), "juno_ctx_profile_read")
        return {n: {"launches": e.launches, "ms": e.ms, "algo_bytes": e.algo_bytes} for n, e in zip(_lib.PROF_NAMES, arr)}

    def close(self) -> None:
        """No-op on the shared instance, like GpuContext.close (GpuContext.java:229-243)."""
        if self._is_shared or self.handle is None:
            return
        check(self._L.juno_ctx_destroy(self.handle), "juno_ctx_destroy")
        self.handle = None


class DeviceQuantMatrix:
    """Resident quantised matrix; the counterpart of DeviceHalfMatrix (close() is idempotent, :108-114)."""

    def __init__(self, ctx: GpuContext, handle, rows: int, cols: int, ggml_type: int):
        self.ctx, self.handle, self.rows, self.cols, self.ggml_type = ctx, handle, rows, cols, ggml_type
        self.closed = False

    def close(self) -> None:
        if not self.closed:
            check(self.ctx._L.juno_qmat_free(self.handle), "juno_qmat_free")
            self.closed = True


class B200MatVec:
    """GpuMatVec implementation backed by libjuno_b200 (label for juno.MatVec events: "cuda-b200-quant")."""

    BACKEND_LABEL = "cuda-b200-quant"

    def __init__(self, ctx: GpuContext | None = None):
        self.ctx = ctx or GpuContext.shared(0)
        self._L = self.ctx._L

    # GpuMatVec.uploadHalf / upload counterpart
    def upload_quantized(self, blocks, ggml_type: int, rows: int, cols: int) -> DeviceQuantMatrix:
        buf = np.ascontiguousarray(blocks).view(np.uint8).reshape(-1)
        blk_e, blk_b = {0: (1, 4), 8: (32, 34), 12: (256, 144), 14: (256, 210)}.get(ggml_type, (0, 0))
        if blk_e == 0:
            raise ValueError(f"unsupported GGML type {ggml_type}")
        if rows < 1 or cols < 1 or cols % blk_e or buf.size != rows * (cols // blk_e) * blk_b:
            raise ValueError(f"blocks.length must equal rows*cols/{blk_e}*{blk_b} (rows={rows}, cols={cols}, "
                             f"bytes={buf.size})")
        h = C.c_void_p()
        check(self._L.juno_qmat_upload(self.ctx.handle, _ptr(buf), ggml_type, rows, cols, C.byref(h)), "juno_qmat_upload")
        return DeviceQuantMatrix(self.ctx, h, rows, cols, ggml_type)

    def supports_half_resident(self) -> bool:  # GpuMatVec.supportsHalfResident
        return False

    def sgemv(self, A, x, rows: int | None = None, cols: int | None = None) -> np.ndarray:
        """y = A·x.  A is a DeviceQuantMatrix (x may be [cols] or [batch, cols]) or a host float32 array with
        rows, cols given (MatVec.sgemv(float[] A, float[] x, rows, cols), MatVec.java:66)."""
        if isinstance(A, DeviceQuantMatrix):
            if A.closed:
                raise RuntimeError("matrix is closed")  # IllegalStateException
            xv = np.ascontiguousarray(x, dtype=np.float32)
            one = xv.ndim == 1
            xb = xv.reshape(1, -1) if one else xv
            if xb.ndim != 2 or xb.shape[1] != A.cols:
                raise ValueError(f"x.length must equal cols ({A.cols}), got {xb.shape[-1]}")
            y = np.empty((xb.shape[0], A.rows), dtype=np.float32)
            check(self._L.juno_gemv(self.ctx.handle, A.handle, _ptr(xb), xb.shape[0], _ptr(y)), "juno_gemv")
            return y[0] if one else y
        a = np.ascontiguousarray(A, dtype=np.float32).reshape(-1)
        xv = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
        if rows is None or cols is None or rows < 1 or cols < 1 or a.size != rows * cols:
            raise ValueError(f"A.length must equal rows*cols (A.length={a.size}, rows={rows}, cols={cols})")
        if xv.size != cols:
            raise ValueError(f"x.length must equal cols ({cols}), got {xv.size}")
        y = np.empty(rows, dtype=np.float32)
        check(self._L.juno_sgemv_f32(self.ctx.handle, _ptr(a), _ptr(xv), rows, cols, _ptr(y)), "juno_sgemv_f32")
        return y

    def dequantize(self, A: DeviceQuantMatrix, row_start: int = 0, n_rows: int | None = None) -> np.ndarray:
        """Bit-exact FP32 values of rows [row_start, row_start+n_rows) (LlamaTransformerHandler.dequantize)."""
        n_rows = A.rows - row_start if n_rows is None else n_rows
        out = np.empty((n_rows, A.cols), dtype=np.float32)
        check(self._L.juno_dequantize(self.ctx.handle, A.handle, row_start, n_rows, _ptr(out)), "juno_dequantize")
        return out


class PagedKvCache:
    """Device-resident paged KV pool + per-request sequences, with the GQA decode attention operator."""

    def __init__(self, ctx: GpuContext, n_layers: int, n_kv_heads: int, head_dim: int, n_pages: int, kv_dtype: str = "f16"):
        self.ctx, self._L = ctx, ctx._L
        self.n_layers, self.n_kv_heads, self.head_dim = n_layers, n_kv_heads, head_dim
        h = C.c_void_p()
        check(self._L.juno_kvpool_create(ctx.handle, n_layers, n_kv_heads, head_dim, n_pages,
                                         {"f16": 0, "f32": 1}[kv_dtype], C.byref(h)), "juno_kvpool_create")
        self.handle = h

    def new_sequence(self, max_tokens: int):
        h = C.c_void_p()
        check(self._L.juno_kvseq_create(self.handle, max_tokens, C.byref(h)), "juno_kvseq_create")
        return h

    def free_sequence(self, seq) -> None:
        check(self._L.juno_seq_free(seq), "juno_seq_free")

    def length(self, seq) -> int:
        n = C.c_int32()
        check(self._L.juno_seq_length(seq, C.byref(n)), "juno_seq_length")
        return n.value

    def append(self, seq, layer: int, pos: int, k, v) -> None:
        k = np.ascontiguousarray(k, dtype=np.float32).reshape(-1, self.n_kv_heads * self.head_dim)
        v = np.ascontiguousarray(v, dtype=np.float32).reshape(-1, self.n_kv_heads * self.head_dim)
        check(self._L.juno_seq_append_kv(seq, layer, pos, k.shape[0], _ptr(k), _ptr(v)), "juno_seq_append_kv")

    def attention(self, layer: int, seqs, q, n_heads: int) -> np.ndarray:
        q = np.ascontiguousarray(q, dtype=np.float32).reshape(len(seqs), n_heads * self.head_dim)
        out = np.empty_like(q)
        arr = (C.c_void_p * len(seqs))(*[s.value if isinstance(s, C.c_void_p) else s for s in seqs])
        check(self._L.juno_attn_decode(self.ctx.handle, self.handle, layer, len(seqs), arr, n_heads, _ptr(q), _ptr(out)),
              "juno_attn_decode")
        return out

    def close(self) -> None:
        if self.handle is not None:
            check(self._L.juno_kvpool_free(self.handle), "juno_kvpool_free")
            self.handle = None
