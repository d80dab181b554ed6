package cab.ml.juno.node;

import static java.lang.foreign.ValueLayout.ADDRESS;
import static java.lang.foreign.ValueLayout.JAVA_BYTE;
import static java.lang.foreign.ValueLayout.JAVA_FLOAT;

import java.lang.foreign.Arena;
import java.lang.foreign.MemorySegment;
import java.util.concurrent.atomic.AtomicBoolean;

/**
 * MatVec backend that keeps GGUF blocks (Q4_K, Q6_K, Q8_0) resident on the GPU as they are and multiplies through
 * juno_gemv, instead of dequantising to FP16 at load (CudaMatVec.uploadHalf) and calling cuBLAS per product.
 *
 * Needs `B200MatVec` in the permits list of the sealed GpuMatVec. The FP32/FP16 upload methods of GpuMatVec exist for
 * LoRA and for handlers that have no quantised path; they are not what this backend is for and are left to throw.
 *
 * NOT COMPILED: written without a JDK at hand; see integration/java/README.md.
 */
final class B200MatVec implements GpuMatVec, AutoCloseable {

	/** A quantised matrix resident on the device (the counterpart of DeviceHalfMatrix). */
	static final class DeviceQuantMatrix implements AutoCloseable {
		final MemorySegment handle;
		final int rows, cols, ggmlType;
		private final AtomicBoolean closed = new AtomicBoolean();

		DeviceQuantMatrix(MemorySegment handle, int rows, int cols, int ggmlType) {
			this.handle = handle;
			this.rows = rows;
			this.cols = cols;
			this.ggmlType = ggmlType;
		}

		boolean isClosed() {
			return closed.get();
		}

		@Override
		public void close() {
			if (closed.compareAndSet(false, true)) {
				try {
					B200Bindings.check((int) B200Bindings.qmatFree.invokeExact(handle), "juno_qmat_free");
				} catch (RuntimeException e) {
					throw e;
				} catch (Throwable t) {
					throw new IllegalStateException(t);
				}
			}
		}
	}

	private final MemorySegment ctx;
	private final AtomicBoolean closed = new AtomicBoolean();

	B200MatVec(int deviceIndex) {
		try (Arena a = Arena.ofConfined()) {
			MemorySegment out = a.allocate(ADDRESS);
			B200Bindings.check((int) B200Bindings.ctxCreate.invokeExact(deviceIndex, out), "juno_ctx_create");
			this.ctx = out.get(ADDRESS, 0);
		} catch (RuntimeException e) {
			throw e;
		} catch (Throwable t) {
			throw new IllegalStateException(t);
		}
	}

	MemorySegment context() {
		return ctx;
	}

	/** GgufReader.QuantizedTensor bytes, row-major GGUF blocks, kept as they are (no dequantisation). */
	DeviceQuantMatrix uploadQuantized(GgufReader.QuantizedTensor t, int rows, int cols) {
		byte[] raw = t.data();
		try (Arena a = Arena.ofConfined()) { // Panama rejects heap segments for native calls (CudaMatVec.java:158-160)
			MemorySegment host = a.allocate(raw.length, 64);
			MemorySegment.copy(raw, 0, host, JAVA_BYTE, 0, raw.length);
			MemorySegment out = a.allocate(ADDRESS);
			B200Bindings.check((int) B200Bindings.qmatUpload.invokeExact(ctx, host, t.type(), (long) rows, (long) cols, out),
					"juno_qmat_upload");
			return new DeviceQuantMatrix(out.get(ADDRESS, 0), rows, cols, t.type());
		} catch (RuntimeException e) {
			throw e;
		} catch (Throwable th) {
			throw new IllegalStateException(th);
		}
	}

	/** y = A x with A resident and quantised; inputs are not modified, the result is a fresh array. */
	float[] sgemv(DeviceQuantMatrix A, float[] x) {
		if (A.isClosed())
			throw new IllegalStateException("matrix is closed");
		if (x.length != A.cols)
			throw new IllegalArgumentException("x has " + x.length + " elements, the matrix has " + A.cols + " columns");
		try (Arena a = Arena.ofConfined()) {
			MemorySegment xs = a.allocate(JAVA_FLOAT, x.length);
			MemorySegment.copy(x, 0, xs, JAVA_FLOAT, 0, x.length);
			MemorySegment ys = a.allocate(JAVA_FLOAT, A.rows);
			B200Bindings.check((int) B200Bindings.gemv.invokeExact(ctx, A.handle, xs, 1, ys), "juno_gemv");
			return ys.toArray(JAVA_FLOAT);
		} catch (RuntimeException e) {
			throw e;
		} catch (Throwable th) {
			throw new IllegalStateException(th);
		}
	}

	/** MatVec.sgemv with a host FP32 matrix (the contract tests of MatVecBackendContractTest). */
	@Override
	public float[] sgemv(float[] A, float[] x, int rows, int cols) {
		if (A.length != (long) rows * cols || x.length != cols)
			throw new IllegalArgumentException("dimension mismatch: A=" + A.length + " x=" + x.length + " rows=" + rows + " cols=" + cols);
		try (Arena a = Arena.ofConfined()) {
			MemorySegment as = a.allocate(JAVA_FLOAT, A.length);
			MemorySegment.copy(A, 0, as, JAVA_FLOAT, 0, A.length);
			MemorySegment xs = a.allocate(JAVA_FLOAT, x.length);
			MemorySegment.copy(x, 0, xs, JAVA_FLOAT, 0, x.length);
			MemorySegment ys = a.allocate(JAVA_FLOAT, rows);
			B200Bindings.check((int) B200Bindings.sgemvF32.invokeExact(ctx, as, xs, (long) rows, (long) cols, ys), "juno_sgemv_f32");
			return ys.toArray(JAVA_FLOAT);
		} catch (RuntimeException e) {
			throw e;
		} catch (Throwable th) {
			throw new IllegalStateException(th);
		}
	}

	@Override
	public DeviceFloatMatrix upload(float[] host, int rows, int cols) {
		throw new UnsupportedOperationException("B200MatVec keeps quantised blocks resident: use uploadQuantized");
	}

	@Override
	public DeviceHalfMatrix uploadHalf(float[] host, int rows, int cols) {
		throw new UnsupportedOperationException("B200MatVec keeps quantised blocks resident: use uploadQuantized");
	}

	@Override
	public boolean supportsHalfResident() {
		return false;
	}

	@Override
	public void close() {
		if (closed.compareAndSet(false, true)) {
			try {
				B200Bindings.check((int) B200Bindings.ctxDestroy.invokeExact(ctx), "juno_ctx_destroy");
			} catch (RuntimeException e) {
				throw e;
			} catch (Throwable t) {
				throw new IllegalStateException(t);
			}
		}
	}
}
