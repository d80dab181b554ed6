"""Tensor-parallel slicing rules, host-side mirror of what `juno_model_set_tensor` keeps for one rank.

Geometry of node/.../TensorShardContext.java:74-100 (headsPerNode = numHeads / world, sliceDim = hidden / world)
turned into real slices: column-parallel (rows of) attn_q/k/v, ffn_gate/up and the output projection; row-parallel
(whole 256-column super-blocks of) attn_output and ffn_down.  Raw GGUF rows are contiguous, so a row slice is a
byte range and a column slice is a per-row byte range.
"""
from __future__ import annotations

import numpy as np

from . import synth
from .synth import (T_ATTN_K, T_ATTN_OUT, T_ATTN_Q, T_ATTN_V, T_FFN_DOWN, T_FFN_GATE, T_FFN_UP, T_OUTPUT)


def check(arch: synth.Arch, world: int) -> None:
    if world < 1:
        raise ValueError("tensorWorldSize must be >= 1")
    if world == 1:
        return
    if arch.n_heads % 2:
        raise ValueError(f"numHeads ({arch.n_heads}) must be divisible by 2 for tensor-parallel mode")
    if arch.n_heads % world or arch.n_kv_heads % world:
        raise ValueError(f"heads ({arch.n_heads} query, {arch.n_kv_heads} kv) do not divide over {world} ranks")
    if (arch.hidden // world) % 256 or arch.inter % world or (arch.inter // world) % 256:
        raise ValueError("hidden/world and feed_forward_length/world must be multiples of 256 (whole super-blocks)")


def slice_spec(arch: synth.Arch, kind: int, rank: int, world: int):
    """(row0, nrows, col0, ncols) this rank keeps of a full tensor of the given kind."""
    rows, cols = synth.tensor_shape(arch, kind)
    hd = arch.head_dim
    if kind == T_ATTN_Q:
        n = arch.n_heads // world * hd
        return rank * n, n, 0, cols
    if kind in (T_ATTN_K, T_ATTN_V):
        n = arch.n_kv_heads // world * hd
        return rank * n, n, 0, cols
    if kind in (T_FFN_GATE, T_FFN_UP):
        n = arch.inter // world
        return rank * n, n, 0, cols
    if kind == T_ATTN_OUT:
        n = arch.hidden // world
        return 0, rows, rank * n, n
    if kind == T_FFN_DOWN:
        n = arch.inter // world
        return 0, rows, rank * n, n
    if kind == T_OUTPUT and arch.vocab % world == 0:
        n = arch.vocab // world
        return rank * n, n, 0, cols
    return 0, rows, 0, cols


def slice_blocks(blocks, ggml_type: int, rows: int, cols: int, row0: int, nrows: int, col0: int, ncols: int) -> np.ndarray:
    """Raw blocks of the sub-matrix [row0:row0+nrows, col0:col0+ncols] (column bounds on block boundaries)."""
    be, bb = synth.BLOCK_ELEMS[ggml_type], synth.BLOCK_BYTES[ggml_type]
    if col0 % be or ncols % be:
        raise ValueError("column slice must fall on block boundaries")
    a = np.ascontiguousarray(blocks).view(np.uint8).reshape(rows, cols // be * bb)
    return np.ascontiguousarray(a[row0:row0 + nrows, col0 // be * bb:(col0 + ncols) // be * bb]).reshape(-1)
