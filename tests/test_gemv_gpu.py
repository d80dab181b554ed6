"""Parity of the fused dequant-GEMV and the dequantise kernel with the CPU oracle (through the C ABI)."""
import numpy as np
import pytest

from conftest import rel_err
from juno_b200 import synth

pytestmark = pytest.mark.gpu
TYPES = [synth.Q4_K, synth.Q6_K, synth.Q8_0]
TOL = 1e-3  # GEMV bar: 1e-3 relative with FP32 accumulation


@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("rows,cols", [(16, 256), (37, 512), (300, 4096)])
def test_dequantize_bit_exact(mv, oracle, t, rows, cols):
    rng = np.random.default_rng(100 + t)
    raw = synth.random_blocks(rng, t, rows, cols)
    A = mv.upload_quantized(raw, t, rows, cols)
    got = mv.dequantize(A)
    ref = oracle.dequantize(t, raw, rows, cols)
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))
    part = mv.dequantize(A, 5, min(7, rows - 5))
    assert np.array_equal(part.view(np.uint32), ref[5:5 + part.shape[0]].view(np.uint32))
    A.close()


@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("rows,cols", [(16, 256), (1000, 1024), (4096, 4096), (64, 14336), (4100, 2048)])
@pytest.mark.parametrize("batch", [1, 2, 4])
def test_gemv_matches_oracle(mv, oracle, t, rows, cols, batch):
    rng = np.random.default_rng(1)
    raw = synth.random_blocks(rng, t, rows, cols)
    x = rng.standard_normal((batch, cols)).astype(np.float32)
    A = mv.upload_quantized(raw, t, rows, cols)
    y = mv.sgemv(A, x)
    ref = oracle.matvec(t, raw, x, rows, cols)
    assert y.shape == (batch, rows)
    assert rel_err(y, ref) < TOL, rel_err(y, ref)
    A.close()


@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("batch", [16, 64])
def test_gemv_large_batch(mv, oracle, t, batch):
    rows, cols = 512, 4096
    rng = np.random.default_rng(2)
    raw = synth.random_blocks(rng, t, rows, cols)
    x = rng.standard_normal((batch, cols)).astype(np.float32)
    A = mv.upload_quantized(raw, t, rows, cols)
    y = mv.sgemv(A, x)
    ref = oracle.matvec(t, raw, x, rows, cols)
    assert rel_err(y, ref) < TOL, rel_err(y, ref)
    A.close()


@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("rows,cols,batch", [(9616, 4096, 48), (9601, 2048, 64), (14336, 4096, 50)])
def test_gemm_tcgen05_route_matches_oracle(ctx, mv, oracle, t, rows, cols, batch):
    """Batches of 48..64 sequences on matrices with at least sm_count/2 blocks of 128 rows take the tcgen05/TMEM
    kernel: ragged row counts, a batch that is not a multiple of 16, all three block formats, and the launch is
    seen in the profile category of that kernel."""
    rng = np.random.default_rng(7)
    raw = synth.random_blocks(rng, t, rows, cols)
    x = rng.standard_normal((batch, cols)).astype(np.float32)
    A = mv.upload_quantized(raw, t, rows, cols)
    ctx.profile(True)
    ctx.profile_read()
    y = mv.sgemv(A, x)
    prof = ctx.profile_read()
    ctx.profile(False)
    assert prof["gemm_tcgen05"]["launches"] >= 1, prof
    ref = oracle.matvec(t, raw, x, rows, cols)
    assert rel_err(y, ref) < TOL, rel_err(y, ref)
    A.close()


@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("rows,cols", [(14336, 4096), (4096, 14336), (128256, 4096)])
def test_gemv_sweep_shapes_batched(mv, oracle, t, rows, cols):
    """The operator sweep's shapes at batch 16 and 64 (one upload per shape; on the largest shape the oracle
    checks a sample of the sequences)."""
    rng = np.random.default_rng(1)
    raw = synth.random_blocks(rng, t, rows, cols)
    A = mv.upload_quantized(raw, t, rows, cols)
    for batch in (16, 64):
        x = rng.standard_normal((batch, cols)).astype(np.float32)
        y = mv.sgemv(A, x)
        pick = list(range(batch)) if rows < 100000 else [0, batch // 2, batch - 1]
        ref = oracle.matvec(t, raw, x[pick], rows, cols)
        assert rel_err(y[pick], ref) < TOL, (batch, rel_err(y[pick], ref))
    A.close()


@pytest.mark.parametrize("t", TYPES)
def test_gemv_exact_path_batches_up_to_eight(mv, oracle, t):
    """1..8 sequences run on the integer tensor-core kernel, whose products are exact: the result differs from the
    oracle only by FP32 summation order (1e-5), outliers in the activation included."""
    rows, cols = 1000, 4096
    rng = np.random.default_rng(9)
    raw = synth.random_blocks(rng, t, rows, cols)
    A = mv.upload_quantized(raw, t, rows, cols)
    for batch in (1, 2, 3, 5, 8):
        x = rng.standard_normal((batch, cols)).astype(np.float32)
        x[:, ::7] *= 30.0
        x[:, 5] = 0.0
        y = mv.sgemv(A, x)
        ref = oracle.matvec(t, raw, x, rows, cols)
        assert rel_err(y, ref) < 1e-5, (batch, rel_err(y, ref))
    zero = mv.sgemv(A, np.zeros(cols, dtype=np.float32))
    assert not zero.any()
    A.close()


def test_gemv_sweep_shape_logits(mv, oracle):
    """The largest shape of the operator sweep: 128256 x 4096 Q4_K, batch 1."""
    rows, cols = 128256, 4096
    rng = np.random.default_rng(1)
    raw = synth.random_blocks(rng, synth.Q4_K, rows, cols)
    x = rng.standard_normal(cols).astype(np.float32)
    A = mv.upload_quantized(raw, synth.Q4_K, rows, cols)
    y = mv.sgemv(A, x)
    ref = oracle.matvec(synth.Q4_K, raw, x, rows, cols)
    assert rel_err(y, ref) < TOL
    A.close()


def test_gemv_repeatable_and_inputs_untouched(mv):
    rng = np.random.default_rng(3)
    raw = synth.random_blocks(rng, synth.Q4_K, 4096, 4096)
    x = rng.standard_normal(4096).astype(np.float32)
    raw0, x0 = raw.copy(), x.copy()
    A = mv.upload_quantized(raw, synth.Q4_K, 4096, 4096)
    y1, y2 = mv.sgemv(A, x), mv.sgemv(A, x)
    assert y1 is not y2 and np.array_equal(y1, y2)  # fixed reduction order: bitwise repeatable
    assert np.array_equal(raw, raw0) and np.array_equal(x, x0)
    A.close()


def test_gemv_linearity(mv):
    """Size-independent property at a full sweep shape: A(ax + bz) == a·Ax + b·Az within FP32 rounding."""
    rows, cols = 14336, 4096
    rng = np.random.default_rng(4)
    raw = synth.random_blocks(rng, synth.Q6_K, rows, cols)
    x, z = rng.standard_normal((2, cols)).astype(np.float32)
    A = mv.upload_quantized(raw, synth.Q6_K, rows, cols)
    lhs = mv.sgemv(A, (2 * x - 3 * z).astype(np.float32))
    rhs = 2 * mv.sgemv(A, x).astype(np.float64) - 3 * mv.sgemv(A, z).astype(np.float64)
    assert rel_err(lhs, rhs) < 1e-4
    A.close()


def test_reference_known_answers_on_device(mv, oracle):
    """The reference's own one-block cases (PhiQuantizedMatVecTest) through the device path."""
    import json, os
    g = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "quant_known_answers.json")))
    blk = np.array(g["q6k_golden"]["block"], dtype=np.uint8)
    A = mv.upload_quantized(blk, synth.Q6_K, 1, 256)
    out = mv.dequantize(A)[0]
    for i, v in g["q6k_golden"]["expected"]:
        assert abs(out[i] - v) < g["q6k_golden"]["eps"]
    y = mv.sgemv(A, np.ones(256, dtype=np.float32))
    assert abs(y[0] - out.sum(dtype=np.float64)) < 1e-3 * max(1.0, abs(out.sum()))
    A.close()
    rows3 = np.array(g["q4k_three_rows"]["blocks"], dtype=np.uint8)
    A = mv.upload_quantized(rows3, synth.Q4_K, 3, 256)
    y = mv.sgemv(A, np.ones(256, dtype=np.float32))
    ref = oracle.matvec(synth.Q4_K, rows3, np.ones(256, dtype=np.float32), 3, 256)
    assert np.allclose(y, ref, atol=1e-3)
    A.close()
    # Q8_0 single 32-column block goes through the raw-layout kernel
    q8 = np.array(g["q8_0_half_i"]["block"], dtype=np.uint8)
    A = mv.upload_quantized(q8, synth.Q8_0, 1, 32)
    assert np.allclose(mv.dequantize(A)[0], g["q8_0_half_i"]["expected"], atol=1e-3)
    A.close()


# ── MatVec contract (MatVecBackendContractTest.java:73-212) on the FP32 host-matrix entry ──────────────
def _scalar(A, x, rows, cols):
    y = np.zeros(rows, dtype=np.float32)
    A = A.reshape(rows, cols)
    for r in range(rows):
        acc = np.float32(0)
        for c in range(cols):
            acc = np.float32(acc + np.float32(A[r, c] * x[c]))
        y[r] = acc
    return y


@pytest.mark.parametrize("rows,cols", [(7, 5), (32, 32), (256, 256), (1, 512), (128, 1)])
def test_f32_contract_shapes(mv, rows, cols):
    rng = np.random.default_rng(20)
    A = (rng.standard_normal(rows * cols) * 0.02).astype(np.float32)
    x = (rng.standard_normal(cols) * 0.02).astype(np.float32)
    y = mv.sgemv(A, x, rows, cols)
    assert y.shape == (rows,)
    assert np.allclose(y, _scalar(A, x, rows, cols), atol=1e-4)


def test_f32_contract_known_values_and_errors(mv):
    y = mv.sgemv(np.array([1, 0, 0, 0, 1, 0], dtype=np.float32), np.array([3, 5, 7], dtype=np.float32), 2, 3)
    assert abs(y[0] - 3) < 1e-6 and abs(y[1] - 5) < 1e-6
    assert not mv.sgemv(np.zeros(64 * 64, dtype=np.float32), np.ones(64, dtype=np.float32), 64, 64).any()
    with pytest.raises(ValueError, match="rows\\*cols"):
        mv.sgemv(np.zeros(10, dtype=np.float32), np.zeros(4, dtype=np.float32), 3, 4)
    with pytest.raises(ValueError, match="cols"):
        mv.sgemv(np.zeros(12, dtype=np.float32), np.zeros(5, dtype=np.float32), 3, 4)


def test_closed_matrix_and_dimension_errors(mv):
    rng = np.random.default_rng(5)
    raw = synth.random_blocks(rng, synth.Q4_K, 16, 256)
    A = mv.upload_quantized(raw, synth.Q4_K, 16, 256)
    with pytest.raises(ValueError):
        mv.sgemv(A, np.zeros(255, dtype=np.float32))
    A.close()
    A.close()  # idempotent
    with pytest.raises(RuntimeError):
        mv.sgemv(A, np.zeros(256, dtype=np.float32))
    # the C ABI itself reports CLOSED for a freed handle instead of crashing
    from juno_b200 import _lib
    assert mv._L.juno_qmat_free(A.handle) == _lib.ERR_CLOSED
    with pytest.raises(ValueError):
        mv.upload_quantized(raw[:-1], synth.Q4_K, 16, 256)
