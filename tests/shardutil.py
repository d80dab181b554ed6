"""Test helper: cuts the slice of a full tensor that one tensor-parallel rank keeps, by the library's own rule
(juno_tp_slice, host-only) - so the multi-process CPU tests exercise the product's slicer, not a copy of it."""
from __future__ import annotations

import ctypes as C

import numpy as np

from juno_b200 import _lib, synth


def slice_spec(arch: synth.Arch, kind: int, rank: int, world: int):
    """(row0, nrows, col0, ncols) this rank keeps of a full tensor of the given kind; ValueError as the library reports."""
    out = (C.c_int64 * 6)()
    _lib.check(_lib.load().juno_tp_slice(arch.hidden, arch.n_heads, arch.n_kv_heads, arch.inter, arch.vocab, kind, rank, world, out),
               "juno_tp_slice")
    rows, cols = synth.tensor_shape(arch, kind)
    assert (out[0], out[1]) == (rows, cols)
    return out[2], out[3], out[4], out[5]


def slice_blocks(blocks, ggml_type: int, rows: int, cols: int, row0: int, nrows: int, col0: int, ncols: int) -> np.ndarray:
    """Raw blocks of the sub-matrix [row0:row0+nrows, col0:col0+ncols] (column bounds on block boundaries)."""
    be, bb = synth.BLOCK_ELEMS[ggml_type], synth.BLOCK_BYTES[ggml_type]
    if col0 % be or ncols % be:
        raise ValueError("column slice must fall on block boundaries")
    a = np.ascontiguousarray(blocks).view(np.uint8).reshape(rows, cols // be * bb)
    return np.ascontiguousarray(a[row0:row0 + nrows, col0 // be * bb:(col0 + ncols) // be * bb]).reshape(-1)
