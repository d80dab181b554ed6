"""CPU checks of the product library: it loads and exports every symbol the header declares (and nothing else with
the juno_ prefix); the tile layout round-trips bit-exactly through a host build of the device index maps."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from juno_b200 import _lib, synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    L = _lib.load()
    hdr = open(os.path.join(ROOT, "include", "juno_b200.h")).read()
    declared = set(re.findall(r"\b(juno_[a-z0-9_]+)\s*\(", hdr))
    assert len(declared) >= 30
    for name in declared:
        assert hasattr(L, name), name
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    # no undeclared juno_* export (debug hooks do not belong in the product library)
    import subprocess
    out = subprocess.run(["nm", "-D", "--defined-only", _lib.LIB_PATH], capture_output=True, text=True).stdout
    exported = {ln.split()[-1] for ln in out.splitlines() if ln.split() and ln.split()[-1].startswith("juno_")}
    assert exported == declared, exported ^ declared


def test_cfg_struct_matches_header():
    assert C.sizeof(_lib.ModelCfg) == 4 * 15 + 128
    assert C.sizeof(_lib.Counters) == 40


def test_device_probe_fails_soft():
    n = C.c_int32(-1)
    assert _lib.load().juno_device_count(C.byref(n)) == _lib.OK and n.value >= 0
    if n.value == 0:  # no GPU: the context refuses loudly, there is no CPU fallback
        h = C.c_void_p()
        assert _lib.load().juno_ctx_create(0, C.byref(h)) == _lib.ERR_CUDA
        assert "no CPU fallback" in _lib.last_error()


def test_null_and_closed_handles_return_codes():
    L = _lib.load()
    assert L.juno_qmat_free(None) == _lib.ERR_INVALID_ARG
    assert L.juno_ctx_destroy(None) == _lib.ERR_INVALID_ARG
    assert L.juno_model_free(None) == _lib.ERR_INVALID_ARG
    assert L.juno_seq_free(None) == _lib.ERR_INVALID_ARG


@pytest.mark.parametrize("t", [synth.Q4_K, synth.Q6_K, synth.Q8_0])
@pytest.mark.parametrize("rows,cols", [(16, 256), (37, 512), (5, 1024)])
def test_tile_layout_round_trip_bit_exact(oracle, layout_host, t, rows, cols):
    L = layout_host
    raw = synth.random_blocks(np.random.default_rng(t), t, rows, cols)
    n = L.layout_tiled_bytes(t, rows, cols)
    assert n == ((rows + 15) // 16) * (cols // 256) * {12: 2368, 14: 3360, 8: 4352}[t]
    tiles = np.zeros(n, dtype=np.uint8)
    assert L.layout_repack(t, raw.ctypes.data, rows, cols, tiles.ctypes.data) == 0
    out = np.empty((rows, cols), dtype=np.float32)
    assert L.layout_dequant_tiled(t, tiles.ctypes.data, rows, cols, out.ctypes.data) == 0
    ref = oracle.dequantize(t, raw, rows, cols)
    assert np.array_equal(out.view(np.uint32), ref.view(np.uint32))


def test_synthetic_block_distributions(oracle):
    rng = np.random.default_rng(0)
    raw = synth.random_blocks(rng, synth.Q4_K, 64, 1024).reshape(-1, 144)
    d = raw[:, 0:2].copy().view(np.float16).astype(np.float32)
    assert 1e-3 * 0.99 <= d.min() and d.max() <= 2e-2 * 1.01
    sc = np.array([[oracle.lib().jo_q4k_scale(np.ascontiguousarray(b[4:16]).ctypes.data, j) for j in range(8)] for b in raw[:50]])
    assert sc.min() >= 0 and sc.max() <= 63 and sc.max() > 40
    q8 = synth.random_blocks(rng, synth.Q8_0, 8, 256).reshape(-1, 34)[:, 2:].view(np.int8)
    assert q8.min() >= -127 and q8.max() <= 127


def test_tensor_shard_context_geometry():
    from juno_b200.handler import TensorShardContext
    c = TensorShardContext(num_heads=32, hidden_dim=4096, tensor_rank=3, tensor_world_size=8)
    assert (c.heads_per_node(), c.head_start(), c.head_end(), c.head_dim(), c.slice_dim()) == (4, 12, 16, 128, 512)
    with pytest.raises(ValueError):
        TensorShardContext(32, 4096, 8, 8)
    with pytest.raises(ValueError):
        TensorShardContext(31, 4096, 0, 1)


def test_gemv_work_split_covers_every_tile_once(layout_host):
    """The split of a fused dequant-GEMV launch over CTAs, chunks and warps (csrc/qsplit.cuh, the same functions the
    kernel calls, built for the host): every (row tile, block) exactly once, the request order of a warp equals its use
    order, the finisher reads exactly the partial-sum slots that were written, and the busiest warp carries at most one
    row tile's worth of rounding more than the mean."""
    import ctypes as C
    import random
    L = layout_host
    L.qsplit_check.restype = C.c_int
    L.qsplit_check.argtypes = [C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int)]
    # (row tiles, blocks of K, CTAs): the decode-step products of the 8B and 70B architectures on 148 SMs x 1 or 2 CTAs,
    # their tensor-parallel shards, and degenerate shapes
    cases = [(384, 16, 148), (256, 16, 256), (1792, 16, 296), (256, 56, 148), (8016, 16, 296), (640, 32, 148), (3584, 32, 296),
             (512, 112, 148), (896, 16, 296), (128, 8, 128), (1002, 16, 296), (64, 1, 64), (8016, 1, 296), (300, 16, 296),
             (1, 16, 1), (3, 2, 3), (17, 3, 4), (33, 5, 2), (5000, 7, 296)]
    rng = random.Random(1)
    cases += [(rt := rng.randint(1, 3000), rng.randint(1, 60), min(rng.choice([1, 2, 7, 148, 296]), rt)) for _ in range(200)]
    for rt, nb, grid in cases:
        busiest = C.c_int()
        assert L.qsplit_check(rt, nb, grid, C.byref(busiest)) == 0, (rt, nb, grid)
        per_cta = -(-rt // grid)  # row tiles of the busiest CTA
        chunks = -(-per_cta // 16)
        assert busiest.value <= -(-per_cta * nb // 16) + chunks, (rt, nb, grid, busiest.value)
