package cab.ml.juno.node;

import static java.lang.foreign.ValueLayout.ADDRESS;
import static java.lang.foreign.ValueLayout.JAVA_DOUBLE;
import static java.lang.foreign.ValueLayout.JAVA_FLOAT;
import static java.lang.foreign.ValueLayout.JAVA_INT;
import static java.lang.foreign.ValueLayout.JAVA_LONG;

import java.lang.foreign.Arena;
import java.lang.foreign.FunctionDescriptor;
import java.lang.foreign.Linker;
import java.lang.foreign.MemoryLayout;
import java.lang.foreign.MemorySegment;
import java.lang.foreign.StructLayout;
import java.lang.foreign.SymbolLookup;
import java.lang.invoke.MethodHandle;

/**
 * Panama downcall handles for libjuno_b200.so — one handle per function of include/juno_b200.h that the Java host
 * uses. Plays the role CudaBindings plays for libcudart/libcublas: library lookup from a system property, one
 * status check, no state of its own.
 *
 * NOT COMPILED: written without a JDK at hand; see integration/java/README.md.
 */
final class B200Bindings {

	static final int OK = 0, ERR_INVALID_ARG = -1, ERR_OOM = -2, ERR_CUDA = -3, ERR_NCCL = -4, ERR_TIMEOUT = -5,
			ERR_CLOSED = -6, ERR_UNSUPPORTED = -7;

	/** GGML type ids the kernels accept (GgufReader.GGML_TYPE_*). */
	static final int TYPE_F32 = 0, TYPE_Q8_0 = 8, TYPE_Q4_K = 12, TYPE_Q6_K = 14;

	/** Tensor kinds of juno_model_set_tensor, in header order. */
	static final int T_TOKEN_EMBD = 0, T_OUTPUT_NORM = 1, T_OUTPUT = 2, T_ATTN_NORM = 3, T_FFN_NORM = 4, T_ATTN_Q = 5,
			T_ATTN_K = 6, T_ATTN_V = 7, T_ATTN_OUT = 8, T_FFN_GATE = 9, T_FFN_UP = 10, T_FFN_DOWN = 11, T_ATTN_Q_BIAS = 12,
			T_ATTN_K_BIAS = 13, T_ATTN_V_BIAS = 14;

	/** juno_model_cfg: fifteen 32-bit fields then uint8_t nccl_id[128] = 188 bytes. */
	static final StructLayout MODEL_CFG = MemoryLayout.structLayout(JAVA_INT.withName("struct_size"),
			JAVA_INT.withName("hidden"), JAVA_INT.withName("n_layers"), JAVA_INT.withName("n_heads"),
			JAVA_INT.withName("n_kv_heads"), JAVA_INT.withName("inter"), JAVA_INT.withName("vocab"),
			JAVA_FLOAT.withName("rms_eps"), JAVA_FLOAT.withName("rope_theta"), JAVA_INT.withName("max_batch"),
			JAVA_INT.withName("max_seqs"), JAVA_INT.withName("max_ctx"), JAVA_INT.withName("kv_dtype"),
			JAVA_INT.withName("tp_rank"), JAVA_INT.withName("tp_world"),
			MemoryLayout.sequenceLayout(128, java.lang.foreign.ValueLayout.JAVA_BYTE).withName("nccl_id"));

	private static final Linker LINKER = Linker.nativeLinker();
	private static final SymbolLookup LIB = SymbolLookup
			.libraryLookup(System.getProperty("juno.b200.library", "libjuno_b200.so"), Arena.global());

	private static MethodHandle h(String name, FunctionDescriptor d) {
		return LINKER.downcallHandle(
				LIB.find(name).orElseThrow(() -> new UnsatisfiedLinkError("libjuno_b200.so lacks " + name)), d);
	}

	private static FunctionDescriptor fn(MemoryLayout... args) {
		return FunctionDescriptor.of(JAVA_INT, args);
	}

	static final MethodHandle lastError = h("juno_last_error", FunctionDescriptor.of(ADDRESS));
	static final MethodHandle deviceCount = h("juno_device_count", fn(ADDRESS));
	static final MethodHandle ctxCreate = h("juno_ctx_create", fn(JAVA_INT, ADDRESS));
	static final MethodHandle ctxDestroy = h("juno_ctx_destroy", fn(ADDRESS));
	static final MethodHandle ctxSynchronize = h("juno_ctx_synchronize", fn(ADDRESS));
	static final MethodHandle qmatUpload = h("juno_qmat_upload", fn(ADDRESS, ADDRESS, JAVA_INT, JAVA_LONG, JAVA_LONG, ADDRESS));
	static final MethodHandle qmatFree = h("juno_qmat_free", fn(ADDRESS));
	static final MethodHandle gemv = h("juno_gemv", fn(ADDRESS, ADDRESS, ADDRESS, JAVA_INT, ADDRESS));
	static final MethodHandle sgemvF32 = h("juno_sgemv_f32", fn(ADDRESS, ADDRESS, ADDRESS, JAVA_LONG, JAVA_LONG, ADDRESS));
	static final MethodHandle dequantize = h("juno_dequantize", fn(ADDRESS, ADDRESS, JAVA_LONG, JAVA_LONG, ADDRESS));
	static final MethodHandle ncclUniqueId = h("juno_nccl_unique_id", fn(ADDRESS));
	static final MethodHandle ggufOpen = h("juno_gguf_open", fn(ADDRESS, ADDRESS));
	static final MethodHandle ggufClose = h("juno_gguf_close", fn(ADDRESS));
	static final MethodHandle ggufModelCfg = h("juno_gguf_model_cfg", fn(ADDRESS, ADDRESS));
	static final MethodHandle modelCreate = h("juno_model_create", fn(ADDRESS, ADDRESS, ADDRESS));
	static final MethodHandle modelSetTensor = h("juno_model_set_tensor", fn(ADDRESS, JAVA_INT, JAVA_INT, ADDRESS, JAVA_INT, JAVA_LONG, JAVA_LONG));
	static final MethodHandle modelLoadGguf = h("juno_model_load_gguf", fn(ADDRESS, ADDRESS));
	static final MethodHandle modelFinalize = h("juno_model_finalize", fn(ADDRESS));
	static final MethodHandle modelFree = h("juno_model_free", fn(ADDRESS));
	static final MethodHandle modelTpMode = h("juno_model_tp_mode", fn(ADDRESS, ADDRESS));
	static final MethodHandle modelSeqCreate = h("juno_model_seq_create", fn(ADDRESS, ADDRESS));
	static final MethodHandle seqFree = h("juno_seq_free", fn(ADDRESS));
	static final MethodHandle seqLength = h("juno_seq_length", fn(ADDRESS, ADDRESS));
	static final MethodHandle seqFork = h("juno_seq_fork", fn(ADDRESS, JAVA_INT, ADDRESS));
	static final MethodHandle forward = h("juno_forward", fn(ADDRESS, JAVA_INT, ADDRESS, ADDRESS, ADDRESS, ADDRESS, ADDRESS));
	static final MethodHandle prefill = h("juno_prefill", fn(ADDRESS, ADDRESS, ADDRESS, JAVA_INT, JAVA_INT, ADDRESS, ADDRESS));
	static final MethodHandle decodeGreedy = h("juno_decode_greedy", fn(ADDRESS, JAVA_INT, ADDRESS, ADDRESS, ADDRESS, JAVA_INT, ADDRESS));
	static final MethodHandle lastHidden = h("juno_model_last_hidden", fn(ADDRESS, JAVA_INT, ADDRESS));

	private B200Bindings() {
	}

	static String lastErrorMessage() {
		try {
			MemorySegment s = (MemorySegment) lastError.invokeExact();
			return s.equals(MemorySegment.NULL) ? "" : s.reinterpret(1024).getString(0);
		} catch (Throwable t) {
			return "(juno_last_error failed: " + t + ")";
		}
	}

	/**
	 * Status check with the exception types of the MatVec contract (MatVec.java:46-54): a bad argument is an
	 * IllegalArgumentException, a freed handle and every device failure an IllegalStateException. Out of memory
	 * keeps "cudaMalloc" in the message, which LlamaTransformerHandler.java:350-352 matches on.
	 */
	static void check(int rc, String op) {
		if (rc == OK)
			return;
		String msg = lastErrorMessage();
		if (rc == ERR_INVALID_ARG)
			throw new IllegalArgumentException(op + ": " + msg);
		throw new IllegalStateException(op + " failed: rc=" + rc + " (" + msg + ")");
	}
}
