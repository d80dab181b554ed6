package cab.ml.juno.node;

import static java.lang.foreign.ValueLayout.ADDRESS;
import static java.lang.foreign.ValueLayout.JAVA_FLOAT;
import static java.lang.foreign.ValueLayout.JAVA_INT;

import java.lang.foreign.Arena;
import java.lang.foreign.MemoryLayout.PathElement;
import java.lang.foreign.MemorySegment;
import java.nio.file.Path;
import java.util.Map;
import java.util.concurrent.ConcurrentHashMap;
import java.util.concurrent.atomic.AtomicBoolean;

/**
 * ForwardPassHandler for LLaMA-family GGUF models whose whole decode step runs inside libjuno_b200.so: embedding
 * lookup, every projection on the quantised blocks, RoPE, paged KV cache, attention, SiLU gate, output projection.
 * One juno_forward call per step replaces the ~155 matVec round trips of LlamaTransformerHandler.
 *
 * Loading: the library maps the GGUF file itself (juno_gguf_open, juno_gguf_model_cfg = LlamaConfig.from,
 * juno_model_load_gguf = the tensor reads of the LlamaTransformerHandler constructor), so no tensor passes through
 * the Java heap.
 *
 * Tensor parallelism: every node process builds its handler with its rank, the world size and the 128-byte
 * ncclUniqueId created by rank 0 (newNcclUniqueId()); all ranks then return the same logits and the coordinator's
 * allReduceSum goes away.
 *
 * NOT COMPILED: written without a JDK at hand; see integration/java/README.md.
 */
final class B200TransformerHandler implements ForwardPassHandler {

	private final B200MatVec backend;
	private final MemorySegment model;
	private final int vocab;
	private final Map<String, MemorySegment> sequences = new ConcurrentHashMap<>();
	private final AtomicBoolean released = new AtomicBoolean();
	private final Arena arena = Arena.ofShared();
	private final MemorySegment logits; // one row of vocab floats, reused under the lock
	private final Object lock = new Object();

	static byte[] newNcclUniqueId() {
		try (Arena a = Arena.ofConfined()) {
			MemorySegment id = a.allocate(128);
			B200Bindings.check((int) B200Bindings.ncclUniqueId.invokeExact(id), "juno_nccl_unique_id");
			return id.toArray(java.lang.foreign.ValueLayout.JAVA_BYTE);
		} catch (RuntimeException e) {
			throw e;
		} catch (Throwable t) {
			throw new IllegalStateException(t);
		}
	}

	B200TransformerHandler(Path gguf, B200MatVec backend, int maxBatch, int maxSeqs, int maxContext, boolean fp16Kv, int tpRank,
			int tpWorld, byte[] ncclId) {
		this.backend = backend;
		try (Arena a = Arena.ofConfined()) {
			MemorySegment out = a.allocate(ADDRESS);
			B200Bindings.check((int) B200Bindings.ggufOpen.invokeExact(a.allocateFrom(gguf.toString()), out), "juno_gguf_open");
			MemorySegment file = out.get(ADDRESS, 0);
			try {
				MemorySegment cfg = a.allocate(B200Bindings.MODEL_CFG);
				cfg.fill((byte) 0);
				set(cfg, "struct_size", (int) B200Bindings.MODEL_CFG.byteSize());
				B200Bindings.check((int) B200Bindings.ggufModelCfg.invokeExact(file, cfg), "juno_gguf_model_cfg");
				set(cfg, "max_batch", maxBatch);
				set(cfg, "max_seqs", maxSeqs);
				set(cfg, "max_ctx", maxContext);
				set(cfg, "kv_dtype", fp16Kv ? 0 : 1);
				set(cfg, "tp_rank", tpRank);
				set(cfg, "tp_world", tpWorld);
				if (tpWorld > 1) {
					if (ncclId == null || ncclId.length != 128)
						throw new IllegalArgumentException("tensor parallelism needs the 128-byte ncclUniqueId of rank 0");
					MemorySegment.copy(ncclId, 0, cfg, java.lang.foreign.ValueLayout.JAVA_BYTE,
							B200Bindings.MODEL_CFG.byteOffset(PathElement.groupElement("nccl_id")), 128);
				}
				this.vocab = cfg.get(JAVA_INT, B200Bindings.MODEL_CFG.byteOffset(PathElement.groupElement("vocab")));
				B200Bindings.check((int) B200Bindings.modelCreate.invokeExact(backend.context(), cfg, out), "juno_model_create");
				this.model = out.get(ADDRESS, 0);
				B200Bindings.check((int) B200Bindings.modelLoadGguf.invokeExact(model, file), "juno_model_load_gguf");
				B200Bindings.check((int) B200Bindings.modelFinalize.invokeExact(model), "juno_model_finalize");
			} finally {
				int ignored = (int) B200Bindings.ggufClose.invokeExact(file);
			}
		} catch (RuntimeException e) {
			throw e;
		} catch (Throwable t) {
			throw new IllegalStateException(t);
		}
		this.logits = arena.allocate(JAVA_FLOAT, vocab);
	}

	private static void set(MemorySegment cfg, String field, int v) {
		cfg.set(JAVA_INT, B200Bindings.MODEL_CFG.byteOffset(PathElement.groupElement(field)), v);
	}

	private MemorySegment sequence(String requestId) {
		return sequences.computeIfAbsent(requestId, id -> {
			try (Arena a = Arena.ofConfined()) {
				MemorySegment out = a.allocate(ADDRESS);
				B200Bindings.check((int) B200Bindings.modelSeqCreate.invokeExact(model, out), "juno_model_seq_create");
				return out.get(ADDRESS, 0);
			} catch (RuntimeException e) {
				throw e;
			} catch (Throwable t) {
				throw new IllegalStateException(t);
			}
		});
	}

	/**
	 * One position of one request, as LlamaTransformerHandler.forward: the last token id of the request at
	 * startPosition, logits out. A position beyond the cached ones is an IllegalArgumentException.
	 */
	@Override
	public ForwardResult forward(ForwardRequest request, ShardContext context) {
		if (released.get())
			throw new IllegalStateException("handler is released");
		if (!request.isFirstNode())
			throw new IllegalArgumentException("B200TransformerHandler runs the whole model: it takes token ids, not activations");
		long t0 = System.nanoTime();
		int[] ids = request.tokenIds();
		synchronized (lock) {
			try (Arena a = Arena.ofConfined()) {
				MemorySegment seqs = a.allocate(ADDRESS);
				seqs.set(ADDRESS, 0, sequence(request.requestId()));
				MemorySegment tok = a.allocateFrom(JAVA_INT, ids[ids.length - 1]);
				MemorySegment pos = a.allocateFrom(JAVA_INT, request.startPosition());
				B200Bindings.check((int) B200Bindings.forward.invokeExact(model, 1, seqs, tok, pos, logits, MemorySegment.NULL),
						"juno_forward");
				return ForwardResult.logits(request.requestId(), logits.toArray(JAVA_FLOAT), System.nanoTime() - t0);
			} catch (RuntimeException e) {
				throw e;
			} catch (Throwable t) {
				throw new IllegalStateException(t);
			}
		}
	}

	/**
	 * n requests in one step (the seam of InferencePipeline.forwardBatch): returns the greedy token of each request;
	 * pass a non-null logitsOut of n * vocab floats to get the logits too.
	 */
	int[] forwardBatch(String[] requestIds, int[] tokens, int[] positions, float[] logitsOut) {
		int n = requestIds.length;
		if (n == 0 || tokens.length != n || positions.length != n)
			throw new IllegalArgumentException("requestIds, tokens and positions must have the same non-zero length");
		synchronized (lock) {
			try (Arena a = Arena.ofConfined()) {
				MemorySegment seqs = a.allocate(ADDRESS, n);
				for (int i = 0; i < n; i++)
					seqs.setAtIndex(ADDRESS, i, sequence(requestIds[i]));
				MemorySegment tok = a.allocateFrom(JAVA_INT, tokens);
				MemorySegment pos = a.allocateFrom(JAVA_INT, positions);
				MemorySegment lg = logitsOut == null ? MemorySegment.NULL : a.allocate(JAVA_FLOAT, (long) n * vocab);
				MemorySegment arg = a.allocate(JAVA_INT, n);
				B200Bindings.check((int) B200Bindings.forward.invokeExact(model, n, seqs, tok, pos, lg, arg), "juno_forward");
				if (logitsOut != null)
					MemorySegment.copy(lg, JAVA_FLOAT, 0, logitsOut, 0, n * vocab);
				return arg.toArray(JAVA_INT);
			} catch (RuntimeException e) {
				throw e;
			} catch (Throwable t) {
				throw new IllegalStateException(t);
			}
		}
	}

	/** Prompt positions startPosition .. startPosition+n-1 in passes of up to 64 (GenerationLoop.java:306-317 does one forward per position). */
	void prefill(String requestId, int[] tokenIds, int startPosition) {
		synchronized (lock) {
			try (Arena a = Arena.ofConfined()) {
				MemorySegment tok = a.allocateFrom(JAVA_INT, tokenIds);
				B200Bindings.check((int) B200Bindings.prefill.invokeExact(model, sequence(requestId), tok, tokenIds.length, startPosition,
						MemorySegment.NULL, MemorySegment.NULL), "juno_prefill");
			} catch (RuntimeException e) {
				throw e;
			} catch (Throwable t) {
				throw new IllegalStateException(t);
			}
		}
	}

	/**
	 * A prefix-cache hit whose pages belong to another live request (PrefixCache.findLongestPrefix): the new request
	 * starts with the first matchedTokens cached positions of the source; pages are shared until one of the two writes.
	 */
	void adoptPrefix(String sourceRequestId, String requestId, int matchedTokens) {
		MemorySegment src = sequences.get(sourceRequestId);
		if (src == null)
			throw new IllegalArgumentException("request " + sourceRequestId + " holds no KV sequence");
		synchronized (lock) {
			try (Arena a = Arena.ofConfined()) {
				MemorySegment out = a.allocate(ADDRESS);
				B200Bindings.check((int) B200Bindings.seqFork.invokeExact(src, matchedTokens, out), "juno_seq_fork");
				if (sequences.putIfAbsent(requestId, out.get(ADDRESS, 0)) != null)
					throw new IllegalArgumentException("request " + requestId + " already holds a KV sequence");
			} catch (RuntimeException e) {
				throw e;
			} catch (Throwable t) {
				throw new IllegalStateException(t);
			}
		}
	}

	/** Frees the KV pages of a finished request (KVCacheManager eviction). */
	void evict(String requestId) {
		MemorySegment s = sequences.remove(requestId);
		if (s != null) {
			try {
				B200Bindings.check((int) B200Bindings.seqFree.invokeExact(s), "juno_seq_free");
			} catch (RuntimeException e) {
				throw e;
			} catch (Throwable t) {
				throw new IllegalStateException(t);
			}
		}
	}

	@Override
	public boolean isReady() {
		return !released.get();
	}

	/** Idempotent, as LlamaTransformerHandler.releaseGpuResources (:424-448). */
	@Override
	public void releaseGpuResources() {
		if (released.compareAndSet(false, true)) {
			synchronized (lock) {
				try {
					sequences.clear(); // the model owns its sequences: juno_model_free releases their pages
					B200Bindings.check((int) B200Bindings.modelFree.invokeExact(model), "juno_model_free");
				} catch (RuntimeException e) {
					throw e;
				} catch (Throwable t) {
					throw new IllegalStateException(t);
				} finally {
					arena.close();
				}
			}
		}
	}
}
