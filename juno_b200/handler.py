"""Forward-pass operator (boundaries B and C) over the C ABI.

`B200TransformerHandler` mirrors node/.../ForwardPassHandler.java:33-70 as implemented by
LlamaTransformerHandler (:602-628): forward(ForwardRequest, ShardContext) -> ForwardResult keyed by
requestId, evict(requestId), releaseGpuResources().  `B200InferencePipeline` mirrors
node/.../InferencePipeline.java:34-76 (forward, forwardBatch, vocabSize) and is what a GenerationLoop calls.
"""
from __future__ import annotations

import ctypes as C
import time
from dataclasses import dataclass, field

import numpy as np

from . import _lib, synth
from ._lib import check
from .matvec import GpuContext, _ptr


@dataclass
class ForwardRequest:
    """ForwardRequest.java:26-48 — only the last token id is used (LlamaTransformerHandler.java:653-655)."""
    request_id: str
    token_ids: list
    start_position: int


@dataclass
class ForwardResult:
    """ForwardResult.java:25-43."""
    request_id: str
    logits: np.ndarray
    nanos: int


@dataclass
class TensorShardContext:
    """Geometry of node/.../TensorShardContext.java:41-117."""
    num_heads: int
    hidden_dim: int
    tensor_rank: int = 0
    tensor_world_size: int = 1

    def __post_init__(self):
        if self.num_heads < 1 or self.hidden_dim < 1:
            raise ValueError("numHeads and hiddenDim must be >= 1")
        if self.tensor_world_size < 1:
            raise ValueError("tensorWorldSize must be >= 1")
        if not 0 <= self.tensor_rank < self.tensor_world_size:
            raise ValueError(f"tensorRank ({self.tensor_rank}) must be < tensorWorldSize ({self.tensor_world_size})")
        if self.num_heads % 2:
            raise ValueError(f"numHeads ({self.num_heads}) must be divisible by 2 for tensor-parallel mode")

    def heads_per_node(self) -> int:
        return self.num_heads // self.tensor_world_size

    def head_start(self) -> int:
        return self.tensor_rank * self.heads_per_node()

    def head_end(self) -> int:
        return self.head_start() + self.heads_per_node()

    def head_dim(self) -> int:
        return self.hidden_dim // self.num_heads

    def slice_dim(self) -> int:
        return self.hidden_dim // self.tensor_world_size


class B200TransformerHandler:
    """LLaMA-family decode on one B200 (or one tensor-parallel rank)."""

    def __init__(self, arch: synth.Arch, ctx: GpuContext | None = None, max_batch: int = 1, max_seqs: int = 8,
                 max_ctx: int = 2048, kv_dtype: str = "f16", tp_rank: int = 0, tp_world: int = 1,
                 nccl_id: bytes | None = None):
        self.arch = arch
        self.ctx = ctx or GpuContext.shared(0)
        self._L = self.ctx._L
        cfg = _lib.ModelCfg()
        cfg.struct_size = C.sizeof(_lib.ModelCfg)
        cfg.hidden, cfg.n_layers, cfg.n_heads, cfg.n_kv_heads = arch.hidden, arch.n_layers, arch.n_heads, arch.n_kv_heads
        cfg.inter, cfg.vocab, cfg.rms_eps, cfg.rope_theta = arch.inter, arch.vocab, arch.rms_eps, arch.rope_theta
        cfg.max_batch, cfg.max_seqs, cfg.max_ctx = max_batch, max_seqs, max_ctx
        cfg.kv_dtype = {"f16": 0, "f32": 1}[kv_dtype]
        cfg.tp_rank, cfg.tp_world = tp_rank, tp_world
        if tp_world > 1:
            if nccl_id is None or len(nccl_id) != 128:
                raise ValueError("tensor parallelism needs the 128-byte ncclUniqueId shared by all ranks")
            C.memmove(cfg.nccl_id, nccl_id, 128)
        h = C.c_void_p()
        check(self._L.juno_model_create(self.ctx.handle, C.byref(cfg), C.byref(h)), "juno_model_create")
        self.handle = h
        self.max_batch = max_batch
        self._seqs: dict[str, C.c_void_p] = {}
        self._released = False

    @staticmethod
    def nccl_unique_id() -> bytes:
        buf = (C.c_uint8 * 128)()
        check(_lib.load().juno_nccl_unique_id(buf), "juno_nccl_unique_id")
        return bytes(buf)

    # ── loading ────────────────────────────────────────────────────────────────
    def set_tensor(self, kind: int, layer: int, blocks, ggml_type: int, rows: int, cols: int) -> None:
        buf = np.ascontiguousarray(blocks).view(np.uint8).reshape(-1)
        check(self._L.juno_model_set_tensor(self.handle, kind, layer, _ptr(buf), ggml_type, rows, cols),
              "juno_model_set_tensor")

    def load(self, tensors) -> "B200TransformerHandler":
        """tensors: iterable of (kind, layer, ggml_type, rows, cols, blocks), e.g. synth.random_model."""
        for kind, layer, t, rows, cols, blocks in tensors:
            self.set_tensor(kind, layer, blocks, t, rows, cols)
        check(self._L.juno_model_finalize(self.handle), "juno_model_finalize")
        return self

    def load_gguf(self, gguf) -> "B200TransformerHandler":
        """Every tensor the reference constructor reads (LlamaTransformerHandler.java:238-275), straight from the mapped
        file (gguf: gguf_file.GgufFile)."""
        check(self._L.juno_model_load_gguf(self.handle, gguf.handle), "juno_model_load_gguf")
        check(self._L.juno_model_finalize(self.handle), "juno_model_finalize")
        return self

    @classmethod
    def from_gguf(cls, path, ctx: GpuContext | None = None, **kw) -> "B200TransformerHandler":
        """The reference's load path in one call: GgufReader.open, LlamaConfig.from, the handler constructor."""
        from .gguf_file import GgufFile
        with GgufFile(path) as g:
            h = cls(g.arch(), ctx, **kw)
            try:
                return h.load_gguf(g)
            except Exception:
                h.release_gpu_resources()  # a file the library refuses must not leave a half-built model behind
                raise

    # ── ForwardPassHandler ─────────────────────────────────────────────────────
    def is_ready(self) -> bool:
        return not self._released

    def _seq(self, request_id: str):
        s = self._seqs.get(request_id)
        if s is None:
            s = C.c_void_p()
            check(self._L.juno_model_seq_create(self.handle, C.byref(s)), "juno_model_seq_create")
            self._seqs[request_id] = s
        return s

    def forward(self, request: ForwardRequest, context=None) -> ForwardResult:
        t0 = time.perf_counter_ns()
        logits = self.forward_batch([request.request_id], [request.token_ids], [request.start_position])[0]
        return ForwardResult(request.request_id, logits, time.perf_counter_ns() - t0)

    def forward_batch(self, request_ids, tokens, positions, want_logits: bool = True, want_argmax: bool = False):
        """n requests in one step (the seam of InferencePipeline.forwardBatch)."""
        n = len(request_ids)
        if not (n == len(tokens) == len(positions)) or n < 1:
            raise ValueError("requestIds, tokens and positions must have the same non-zero length")
        seqs = (C.c_void_p * n)(*[self._seq(r).value for r in request_ids])
        tok = np.array([t[-1] if hasattr(t, "__len__") else t for t in tokens], dtype=np.int32)
        pos = np.asarray(positions, dtype=np.int32)
        logits = np.empty((n, self.arch.vocab), dtype=np.float32) if want_logits else None
        ids = np.empty(n, dtype=np.int32) if want_argmax else None
        check(self._L.juno_forward(self.handle, n, seqs, _ptr(tok), _ptr(pos), _ptr(logits) if want_logits else None,
                                   _ptr(ids) if want_argmax else None), "juno_forward")
        if want_logits and want_argmax:
            return logits, ids
        return logits if want_logits else ids

    def prefill(self, request_id: str, token_ids, start_pos: int = 0, want_logits: bool = False):
        """Chunked prompt prefill (juno_prefill): positions start_pos.. of one request in passes of up to
        min(max_batch, 64) positions.  Returns the logits of the last position fed, or None."""
        toks = np.ascontiguousarray(np.asarray(token_ids, dtype=np.int32))
        logits = np.empty(self.arch.vocab, dtype=np.float32) if want_logits else None
        check(self._L.juno_prefill(self.handle, self._seq(request_id), _ptr(toks), len(toks), int(start_pos),
                                   _ptr(logits) if want_logits else None, None), "juno_prefill")
        return logits

    def decode_greedy(self, request_ids, first_tokens, positions, steps: int) -> np.ndarray:
        """`steps` greedy tokens per request with the loop kept on the device; returns [steps, n] ids."""
        n = len(request_ids)
        seqs = (C.c_void_p * n)(*[self._seq(r).value for r in request_ids])
        tok = np.asarray(first_tokens, dtype=np.int32)
        pos = np.asarray(positions, dtype=np.int32)
        out = np.empty((steps, n), dtype=np.int32)
        check(self._L.juno_decode_greedy(self.handle, n, seqs, _ptr(tok), _ptr(pos), steps, _ptr(out)), "juno_decode_greedy")
        return out

    def last_hidden(self, n: int = 1) -> np.ndarray:
        out = np.empty((n, self.arch.hidden), dtype=np.float32)
        check(self._L.juno_model_last_hidden(self.handle, n, _ptr(out)), "juno_model_last_hidden")
        return out

    def tp_mode(self) -> int:
        """0 = one GPU, 1 = NCCL all-reduce, 2 = partial products pushed into peer-mapped inboxes."""
        mode = C.c_int32()
        check(self._L.juno_model_tp_mode(self.handle, C.byref(mode)), "juno_model_tp_mode")
        return mode.value

    def fork(self, source_id: str, request_id: str, n_tokens: int) -> None:
        """A new request that starts with the first n_tokens cached positions of another live request (prefix-cache hit
        across requests): pages are shared, nothing is copied until one of the two writes into a shared page."""
        if request_id in self._seqs:
            raise ValueError(f"request {request_id} already holds a KV sequence")
        if source_id not in self._seqs:
            raise ValueError(f"request {source_id} holds no KV sequence")
        s = C.c_void_p()
        check(self._L.juno_seq_fork(self._seqs[source_id], int(n_tokens), C.byref(s)), "juno_seq_fork")
        self._seqs[request_id] = s

    def evict(self, request_id: str) -> None:
        """LlamaTransformerHandler.evict (:498-505): drops the request's KV pages; unknown ids are ignored."""
        s = self._seqs.pop(request_id, None)
        if s is not None:
            check(self._L.juno_seq_free(s), "juno_seq_free")

    def release_gpu_resources(self) -> None:
        """Idempotent, like LlamaTransformerHandler.releaseGpuResources (:424-448)."""
        if self._released:
            return
        self._seqs.clear()
        check(self._L.juno_model_free(self.handle), "juno_model_free")
        self._released = True


class B200InferencePipeline:
    """InferencePipeline (InferencePipeline.java:34-76) over one handler."""

    def __init__(self, handler: B200TransformerHandler):
        self.handler = handler

    def vocab_size(self) -> int:
        return self.handler.arch.vocab

    def forward(self, request_id: str, tokens, start_pos: int) -> np.ndarray:
        return self.handler.forward_batch([request_id], [tokens], [start_pos])[0]

    def forward_batch(self, request_ids, tokens, positions) -> np.ndarray:
        return self.handler.forward_batch(request_ids, tokens, positions)


def generate_greedy(pipeline: B200InferencePipeline, request_id: str, prompt, steps: int, chunked_prefill: bool = False) -> list:
    """Decode driver of coordinator/.../GenerationLoop.java:306-334: prefill positions 0..P-2 token by token
    (logits discarded), then greedy steps from position P-1.  chunked_prefill feeds the same positions through
    juno_prefill instead (batched kernels, FP16 operands)."""
    h = pipeline.handler
    P = len(prompt)
    if chunked_prefill and P > 1:
        h.prefill(request_id, prompt[:-1], 0)
    else:
        for p in range(P - 1):
            h.forward_batch([request_id], [[prompt[p]]], [p], want_logits=False, want_argmax=True)
    return h.decode_greedy([request_id], [prompt[-1]], [P - 1], steps)[:, 0].tolist()
