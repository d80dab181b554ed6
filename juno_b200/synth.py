"""Seeded synthetic GGUF blocks and random-init LLaMA-architecture models.

No checkpoint is available offline, so the benchmark configurations are stood in for by
random-init tensors of the same shapes and block formats.  Field distributions: Q4_K nibbles
uniform in [0,15], 6-bit sub-block scales and mins uniform in [0,63], fp16 d/dmin uniform in
[1e-3, 2e-2]; Q8_0 int8 uniform in [-127,127] with the same d; Q6_K ql/qh uniform bytes, int8
scales uniform in [-127,127], same d.  Generator: numpy PCG64 (default_rng(seed)), tensors drawn
in the order written in `random_model`.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

F32, Q8_0, Q4_K, Q6_K = 0, 8, 12, 14
BLOCK_ELEMS = {F32: 1, Q8_0: 32, Q4_K: 256, Q6_K: 256}
BLOCK_BYTES = {F32: 4, Q8_0: 34, Q4_K: 144, Q6_K: 210}


def row_bytes(ggml_type: int, cols: int) -> int:
    return cols // BLOCK_ELEMS[ggml_type] * BLOCK_BYTES[ggml_type]


def pack_q4k_scales(sc: np.ndarray, mn: np.ndarray) -> np.ndarray:
    """Inverse of the 6-bit unpack of LlamaTransformerHandler.q4kScaleRaw/q4kMinRaw (:1471-1482).
    sc, mn: [..., 8] uint8 in [0,63] -> [..., 12] uint8."""
    out = np.zeros(sc.shape[:-1] + (12,), dtype=np.uint8)
    for j in range(4):
        out[..., j] = (sc[..., j] & 63) | ((sc[..., j + 4] >> 4) << 6)
        out[..., j + 4] = (mn[..., j] & 63) | ((mn[..., j + 4] >> 4) << 6)
        out[..., j + 8] = (sc[..., j + 4] & 15) | ((mn[..., j + 4] & 15) << 4)
    return out


def _d_f16(rng, n) -> np.ndarray:
    return rng.uniform(1e-3, 2e-2, n).astype(np.float16).view(np.uint16)


def random_blocks(rng: np.random.Generator, ggml_type: int, rows: int, cols: int) -> np.ndarray:
    """Raw row-major GGUF blocks (uint8, rows*row_bytes) for a rows x cols matrix."""
    nblk = rows * cols // BLOCK_ELEMS[ggml_type]
    if ggml_type == Q4_K:
        out = np.empty((nblk, 144), dtype=np.uint8)
        d, dmin = _d_f16(rng, nblk), _d_f16(rng, nblk)
        out[:, 0], out[:, 1], out[:, 2], out[:, 3] = d & 255, d >> 8, dmin & 255, dmin >> 8
        sc = rng.integers(0, 64, (nblk, 8), dtype=np.uint8)
        mn = rng.integers(0, 64, (nblk, 8), dtype=np.uint8)
        out[:, 4:16] = pack_q4k_scales(sc, mn)
        out[:, 16:] = rng.integers(0, 256, (nblk, 128), dtype=np.uint8)
    elif ggml_type == Q6_K:
        out = np.empty((nblk, 210), dtype=np.uint8)
        out[:, :192] = rng.integers(0, 256, (nblk, 192), dtype=np.uint8)
        out[:, 192:208] = rng.integers(-127, 128, (nblk, 16), dtype=np.int8).view(np.uint8)
        d = _d_f16(rng, nblk)
        out[:, 208], out[:, 209] = d & 255, d >> 8
    elif ggml_type == Q8_0:
        out = np.empty((nblk, 34), dtype=np.uint8)
        d = _d_f16(rng, nblk)
        out[:, 0], out[:, 1] = d & 255, d >> 8
        out[:, 2:] = rng.integers(-127, 128, (nblk, 32), dtype=np.int8).view(np.uint8)
    elif ggml_type == F32:
        return (rng.standard_normal(rows * cols) * 0.02).astype(np.float32).view(np.uint8)
    else:
        raise ValueError(f"unsupported GGML type {ggml_type}")
    return out.reshape(-1)


@dataclass
class Arch:
    hidden: int
    n_layers: int
    n_heads: int
    n_kv_heads: int
    inter: int
    vocab: int
    rms_eps: float = 1e-5
    rope_theta: float = 10000.0

    @property
    def head_dim(self) -> int:
        return self.hidden // self.n_heads

    @property
    def kv_dim(self) -> int:
        return self.n_kv_heads * self.head_dim


TINYLLAMA = Arch(2048, 22, 32, 4, 5632, 32000, 1e-5, 10000.0)
LLAMA3_8B = Arch(4096, 32, 32, 8, 14336, 128256, 1e-5, 500000.0)
LLAMA3_70B = Arch(8192, 80, 64, 8, 28672, 128256, 1e-5, 500000.0)

# tensor kind ids shared with the C ABI
(T_TOKEN_EMBD, T_OUTPUT_NORM, T_OUTPUT, T_ATTN_NORM, T_FFN_NORM, T_ATTN_Q, T_ATTN_K, T_ATTN_V, T_ATTN_OUT,
 T_FFN_GATE, T_FFN_UP, T_FFN_DOWN) = range(12)
T_ATTN_Q_BIAS, T_ATTN_K_BIAS, T_ATTN_V_BIAS = 12, 13, 14  # optional (Qwen2-style files)

GGUF_NAMES = {T_TOKEN_EMBD: "token_embd.weight", T_OUTPUT_NORM: "output_norm.weight", T_OUTPUT: "output.weight",
              T_ATTN_NORM: "blk.{}.attn_norm.weight", T_FFN_NORM: "blk.{}.ffn_norm.weight",
              T_ATTN_Q: "blk.{}.attn_q.weight", T_ATTN_K: "blk.{}.attn_k.weight", T_ATTN_V: "blk.{}.attn_v.weight",
              T_ATTN_OUT: "blk.{}.attn_output.weight", T_FFN_GATE: "blk.{}.ffn_gate.weight",
              T_FFN_UP: "blk.{}.ffn_up.weight", T_FFN_DOWN: "blk.{}.ffn_down.weight",
              T_ATTN_Q_BIAS: "blk.{}.attn_q.bias", T_ATTN_K_BIAS: "blk.{}.attn_k.bias", T_ATTN_V_BIAS: "blk.{}.attn_v.bias"}


def q4_k_m_type(kind: int) -> int:
    """Type map of the benchmark configs: attn_v and ffn_down in Q6_K, every other matrix in Q4_K."""
    return Q6_K if kind in (T_ATTN_V, T_FFN_DOWN) else Q4_K


def tensor_shape(arch: Arch, kind: int):
    H, I, V, kv = arch.hidden, arch.inter, arch.vocab, arch.kv_dim
    return {T_TOKEN_EMBD: (V, H), T_OUTPUT: (V, H), T_ATTN_Q: (H, H), T_ATTN_K: (kv, H), T_ATTN_V: (kv, H),
            T_ATTN_OUT: (H, H), T_FFN_GATE: (I, H), T_FFN_UP: (I, H), T_FFN_DOWN: (H, I),
            T_OUTPUT_NORM: (1, H), T_ATTN_NORM: (1, H), T_FFN_NORM: (1, H),
            T_ATTN_Q_BIAS: (1, H), T_ATTN_K_BIAS: (1, kv), T_ATTN_V_BIAS: (1, kv)}[kind]


def random_model(arch: Arch, seed: int, type_map=q4_k_m_type, norm: str = "ones", qkv_bias: bool = False):
    """Yields (kind, layer, ggml_type, rows, cols, uint8 blocks) in a fixed order:
    token_embd, output_norm, output, then per layer attn_norm, ffn_norm, q, k, v, o, gate, up, down.
    norm="ones": RMSNorm weights of 1.0 (the benchmark configurations); norm="random": 1 + 0.3*N(0,1), drawn per
    vector from a generator of their own, so that the matrices of a seed are the same either way.
    qkv_bias: after each layer's matrices also attn_{q,k,v}.bias (F32, N(0,1) from the same side generator), as
    Qwen2-style files carry them."""
    rng = np.random.default_rng(seed)
    rng_norm = np.random.default_rng([seed, 0x6E6F726D])

    def norm_vec():
        if norm == "ones":
            return np.ones(arch.hidden, dtype=np.float32).view(np.uint8)
        return (1.0 + 0.3 * rng_norm.standard_normal(arch.hidden)).astype(np.float32).view(np.uint8)

    def mat(kind, layer):
        rows, cols = tensor_shape(arch, kind)
        t = type_map(kind)
        return kind, layer, t, rows, cols, random_blocks(rng, t, rows, cols)

    yield mat(T_TOKEN_EMBD, 0)
    yield T_OUTPUT_NORM, 0, F32, 1, arch.hidden, norm_vec()
    yield mat(T_OUTPUT, 0)
    for l in range(arch.n_layers):
        yield T_ATTN_NORM, l, F32, 1, arch.hidden, norm_vec()
        yield T_FFN_NORM, l, F32, 1, arch.hidden, norm_vec()
        for kind in (T_ATTN_Q, T_ATTN_K, T_ATTN_V, T_ATTN_OUT, T_FFN_GATE, T_FFN_UP, T_FFN_DOWN):
            yield mat(kind, l)
        if qkv_bias:
            for kind in (T_ATTN_Q_BIAS, T_ATTN_K_BIAS, T_ATTN_V_BIAS):
                n = tensor_shape(arch, kind)[1]
                yield kind, l, F32, 1, n, rng_norm.standard_normal(n).astype(np.float32).view(np.uint8)
