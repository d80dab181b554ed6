"""Forward-pass operator vs the oracle: logits within 1e-3 relative, greedy ids identical."""
import numpy as np
import pytest

from conftest import rel_err
from juno_b200 import synth
from juno_b200.handler import B200InferencePipeline, ForwardRequest, generate_greedy
from modelutil import SMALL128, TINY, build_pair

pytestmark = pytest.mark.gpu
TOL = 1e-3
# FP16 pages: engine and oracle round the same k, v values to binary16, but the values themselves differ in the last
# FP32 bits (summation order), so a few of them land on different sides of a rounding boundary: one binary16 ulp
# (5e-4) on single cache entries.  The random-init test models amplify that (their residual stream reaches 1e6 and the
# softmax is nearly one-hot), so whole-model comparisons with FP16 pages get a wider bound; FP32 pages keep 1e-3.
TOL_F16_KV = 5e-3


@pytest.mark.parametrize("arch", [TINY, SMALL128], ids=["hd64", "hd128"])
@pytest.mark.parametrize("kv_dtype", ["f32", "f16"])
def test_stepwise_logits_match_oracle(ctx, oracle, arch, kv_dtype):
    om, h = build_pair(oracle, arch, seed=11, kv_dtype=kv_dtype, max_ctx=64, ctx=ctx)
    rng = np.random.default_rng(0)
    toks = rng.integers(0, arch.vocab, 40).tolist()
    seq = om.new_seq()
    worst, tol = 0.0, (TOL if kv_dtype == "f32" else TOL_F16_KV)
    for p, t in enumerate(toks):
        ref, hid_ref = om.forward(seq, t, p, want_hidden=True)
        res = h.forward(ForwardRequest("r0", toks[: p + 1], p))
        worst = max(worst, rel_err(res.logits, ref))
        assert rel_err(h.last_hidden(1)[0], hid_ref) < tol
        assert int(np.argmax(res.logits)) == oracle.greedy(ref)
    assert worst < tol, worst
    h.release_gpu_resources()
    h.release_gpu_resources()  # idempotent


def test_token_id_clamped_like_reference(ctx, oracle):
    om, h = build_pair(oracle, TINY, seed=12, kv_dtype="f32", max_ctx=32, ctx=ctx)
    for tok in (-5, TINY.vocab + 7):
        ref = om.forward(om.new_seq(), tok, 0)
        got = h.forward(ForwardRequest(f"c{tok}", [tok], 0)).logits
        assert rel_err(got, ref) < TOL
    h.release_gpu_resources()


@pytest.mark.parametrize("kv_dtype", ["f32", "f16"])
def test_greedy_ids_identical(ctx, oracle, kv_dtype):
    om, h = build_pair(oracle, SMALL128, seed=13, kv_dtype=kv_dtype, max_ctx=128, ctx=ctx)
    rng = np.random.default_rng(1)
    prompt = rng.integers(0, SMALL128.vocab, 24).tolist()
    ref_ids, margins = om.generate_greedy(om.new_seq(), prompt, 48)
    got = generate_greedy(B200InferencePipeline(h), "g0", prompt, 48)
    assert got == ref_ids.tolist(), (got, ref_ids.tolist(), margins.min())
    h.release_gpu_resources()


def test_forward_batch_ragged_positions_and_evict(ctx, oracle):
    """Continuous batching: three requests at different positions in one step; one is evicted and restarted."""
    arch = TINY
    om, h = build_pair(oracle, arch, seed=14, kv_dtype="f16", max_ctx=64, max_batch=4, max_seqs=4, ctx=ctx)
    rng = np.random.default_rng(2)
    streams = {r: rng.integers(0, arch.vocab, n).tolist() for r, n in (("a", 20), ("b", 9), ("c", 14))}
    oseq = {r: om.new_seq() for r in streams}
    pos = {r: 0 for r in streams}
    # stagger: "a" runs alone for 6 steps, then all that still have tokens run together
    for _ in range(6):
        ref = om.forward(oseq["a"], streams["a"][pos["a"]], pos["a"])
        got = h.forward_batch(["a"], [[streams["a"][pos["a"]]]], [pos["a"]])[0]
        assert rel_err(got, ref) < TOL_F16_KV
        pos["a"] += 1
    while any(pos[r] < len(streams[r]) for r in streams):
        live = [r for r in streams if pos[r] < len(streams[r])]
        logits, ids = h.forward_batch(live, [[streams[r][pos[r]]] for r in live], [pos[r] for r in live],
                                      want_logits=True, want_argmax=True)
        for i, r in enumerate(live):
            ref = om.forward(oseq[r], streams[r][pos[r]], pos[r])
            assert rel_err(logits[i], ref) < TOL_F16_KV
            assert ids[i] == oracle.greedy(ref)
            pos[r] += 1
    h.evict("b")
    h.evict("b")  # unknown id: ignored
    fresh = om.new_seq()
    ref = om.forward(fresh, 5, 0)
    assert rel_err(h.forward_batch(["b"], [[5]], [0])[0], ref) < TOL_F16_KV
    with pytest.raises(ValueError):
        h.forward_batch(["a", "a"], [[1], [2]], [0, 0])
    with pytest.raises(ValueError):
        h.forward_batch(["a"], [[1]], [64])  # beyond max_ctx
    with pytest.raises(ValueError, match="gap"):
        h.forward_batch(["b"], [[1]], [7])  # "b" holds one position: 1..6 were never fed
    with pytest.raises(ValueError, match="gap"):
        h.prefill("b", [1, 2, 3], 4)
    h.release_gpu_resources()


def test_decode_greedy_batch_matches_stepwise(ctx, oracle):
    arch = TINY
    om, h = build_pair(oracle, arch, seed=15, kv_dtype="f32", max_ctx=96, max_batch=3, max_seqs=3, ctx=ctx)
    rng = np.random.default_rng(3)
    prompts = [rng.integers(0, arch.vocab, n).tolist() for n in (5, 17, 11)]
    refs = [om.generate_greedy(om.new_seq(), p, 20)[0].tolist() for p in prompts]
    names = ["x", "y", "z"]
    for r, p in zip(names, prompts):
        for i in range(len(p) - 1):
            h.forward_batch([r], [[p[i]]], [i], want_logits=False, want_argmax=True)
    out = h.decode_greedy(names, [p[-1] for p in prompts], [len(p) - 1 for p in prompts], 20)
    for i in range(3):
        assert out[:, i].tolist() == refs[i]
    h.release_gpu_resources()


def test_all_q4k_and_q8_models(ctx, oracle):
    """Other type maps on the same kernels: every matrix Q4_K (one fused QKV launch) and every matrix Q8_0."""
    for tm in (lambda k: synth.Q4_K, lambda k: synth.Q8_0):
        om, h = build_pair(oracle, TINY, seed=16, kv_dtype="f32", max_ctx=32, ctx=ctx, type_map=tm)
        seq = om.new_seq()
        for p, t in enumerate([3, 900, 17, 512]):
            ref = om.forward(seq, t, p)
            assert rel_err(h.forward_batch(["q"], [[t]], [p])[0], ref) < TOL
        h.release_gpu_resources()


def test_tinyllama_config0_greedy_64(ctx, oracle):
    """TinyLlama-1.1B architecture, random-init Q4_K_M from seed 0, 128 random prompt ids, 64 greedy steps:
    token ids identical to the CPU path (FP32 KV as the reference stores it, and the FP16-page engine against
    the oracle run with FP16 KV)."""
    arch = synth.TINYLLAMA
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, arch.vocab, 128).tolist()
    for kv in ("f32", "f16"):
        om, h = build_pair(oracle, arch, seed=0, kv_dtype=kv, max_ctx=256, ctx=ctx, norm="ones")  # the configuration fixes ones
        ref_ids, margins = om.generate_greedy(om.new_seq(), prompt, 64)
        got = generate_greedy(B200InferencePipeline(h), "t0", prompt, 64)
        h.release_gpu_resources()
        om.close()
        first_bad = next((i for i, (a, b) in enumerate(zip(got, ref_ids.tolist())) if a != b), None)
        assert first_bad is None, (kv, first_bad, float(margins.min()))


@pytest.mark.parametrize("n_seq", [9, 16, 37])
def test_forward_batched_path_matches_oracle(ctx, oracle, n_seq):
    """Batches above eight sequences take the one-pass dequant-GEMM path.  Its operands are rounded to FP16, about
    3e-4 relative per product; the random-init test model amplifies a perturbation by up to ~100x on some sequences
    (the exact batch-1 path shows 1e-6 per product and up to 2e-4 on the logits of the same sequences), and a sequence
    that has drifted keeps drifting through its own KV entries.  So the end-to-end bounds are statistical: median
    below 3e-3, 85 % of the (sequence, step) pairs below 3e-2, and a clear winner is always reproduced.  The
    per-product 1e-3 bound of this path is checked in test_gemv_gpu.py."""
    arch = SMALL128
    om, h = build_pair(oracle, arch, seed=21, kv_dtype="f16", max_ctx=48, max_batch=n_seq, max_seqs=n_seq, ctx=ctx)
    rng = np.random.default_rng(5)
    ids = [f"s{i}" for i in range(n_seq)]
    lens = {r: int(rng.integers(3, 10)) for r in ids}
    streams = {r: rng.integers(0, arch.vocab, lens[r]).tolist() for r in ids}
    oseq = {r: om.new_seq() for r in ids}
    # bring the sequences to different positions one by one (batch-1 path), then step them all together
    for r in ids:
        for p in range(lens[r] - 1):
            om.forward(oseq[r], streams[r][p], p)
            h.forward_batch([r], [[streams[r][p]]], [p])
    errs = []
    nxt = {}
    for step in range(3):
        pos = [lens[r] - 1 + step for r in ids]
        toks = [streams[r][-1] if step == 0 else nxt[r] for r in ids]
        logits, got = h.forward_batch(ids, [[t] for t in toks], pos, want_logits=True, want_argmax=True)
        for i, r in enumerate(ids):
            ref = om.forward(oseq[r], toks[i], pos[i])
            errs.append(rel_err(logits[i], ref))
            nxt[r] = oracle.greedy(ref)
            top2 = np.sort(ref)[-2:]
            if top2[1] - top2[0] > 0.1 * np.abs(ref).max():  # a clear winner must be reproduced
                assert got[i] == nxt[r]
    errs = np.sort(np.array(errs))
    assert float(np.median(errs)) < 3e-3 and errs[int(0.85 * len(errs))] < 3e-2, (float(np.median(errs)), errs[-4:])
    h.release_gpu_resources()


@pytest.mark.parametrize("max_batch,n_prompt", [(32, 100), (64, 64), (8, 21)])
def test_chunked_prefill_matches_token_by_token(ctx, oracle, max_batch, n_prompt):
    """juno_prefill (chunks of min(max_batch, 64) positions through the batched kernels, causal inside a chunk) leaves
    the sequence where the reference's token-by-token prefill leaves it: the logits of the last prompt position and
    of the following token-by-token decode steps match the oracle (FP16 operands on the prefill path: 5e-3 on a
    two-layer model), greedy choice included."""
    arch = TINY
    om, h = build_pair(oracle, arch, seed=31, kv_dtype="f16", max_ctx=160, max_batch=max_batch, max_seqs=2, ctx=ctx)
    rng = np.random.default_rng(7)
    prompt = rng.integers(0, arch.vocab, n_prompt).tolist()
    seq = om.new_seq()
    for p, t in enumerate(prompt):
        ref = om.forward(seq, t, p)
    got = h.prefill("p0", prompt, 0, want_logits=True)
    assert rel_err(got, ref) < 5e-3, rel_err(got, ref)
    assert int(np.argmax(got)) == oracle.greedy(ref)
    tok, pos = oracle.greedy(ref), n_prompt
    for _ in range(6):  # continue token by token on top of the prefilled cache
        ref = om.forward(seq, tok, pos)
        got = h.forward_batch(["p0"], [[tok]], [pos])[0]
        assert rel_err(got, ref) < 5e-3
        tok, pos = oracle.greedy(ref), pos + 1
    # a second request, prefilled in two calls (continuation from a non-zero start position)
    h.prefill("p1", prompt[:10], 0)
    got2 = h.prefill("p1", prompt[10:], 10, want_logits=True)
    seq2 = om.new_seq()
    for p, t in enumerate(prompt):
        ref2 = om.forward(seq2, t, p)
    assert rel_err(got2, ref2) < 5e-3
    h.release_gpu_resources()


# ── the benchmarked shapes ─────────────────────────────────────────────────────────────────────────────────────
LLAMA3_8B_2L = synth.Arch(4096, 2, 32, 8, 14336, 128256, 1e-5, 500000.0)
LLAMA3_70B_2L = synth.Arch(8192, 2, 64, 8, 28672, 128256, 1e-5, 500000.0)


@pytest.mark.parametrize("arch", [LLAMA3_8B_2L, LLAMA3_70B_2L], ids=["8b-shaped", "70b-shaped"])
def test_benchmark_shapes_two_layers(ctx, oracle, arch):
    """Llama-3-8B and -70B layer shapes (hidden 4096/8192, 32q/8kv and 64q/8kv heads, FFN 14336/28672, vocabulary
    128256), two layers, random norm weights: logits within 1e-3 of the oracle at every position, greedy ids equal."""
    om, h = build_pair(oracle, arch, seed=3, kv_dtype="f32", max_ctx=64, ctx=ctx)
    rng = np.random.default_rng(8)
    prompt = rng.integers(0, arch.vocab, 6).tolist()
    seq = om.new_seq()
    for p, t in enumerate(prompt):
        ref = om.forward(seq, t, p)
        got = h.forward_batch(["r"], [[t]], [p])[0]
        assert rel_err(got, ref) < TOL, (p, rel_err(got, ref))
    ref_ids, margins = om.generate_greedy(om.new_seq(), prompt, 8)
    got_ids = generate_greedy(B200InferencePipeline(h), "g", prompt, 8)
    assert got_ids == ref_ids.tolist(), (got_ids, ref_ids.tolist(), float(margins.min()))
    h.release_gpu_resources()
    om.close()


def test_llama3_8b_full_depth_few_steps(ctx, oracle):
    """The benchmarked model itself (32 layers, seed 3 as the 8B configuration, norm weights of 1.0): a 4-token
    prompt and 4 greedy steps against the oracle - ids equal, logits of the last prompt position within 1e-3."""
    arch = synth.LLAMA3_8B
    om, h = build_pair(oracle, arch, seed=3, kv_dtype="f32", max_ctx=32, ctx=ctx, norm="ones")
    rng = np.random.default_rng(9)
    prompt = rng.integers(0, arch.vocab, 4).tolist()
    seq = om.new_seq()
    for p, t in enumerate(prompt):
        ref = om.forward(seq, t, p)
        got = h.forward_batch(["r"], [[t]], [p])[0]
    assert rel_err(got, ref) < TOL, rel_err(got, ref)
    ref_ids, margins = om.generate_greedy(om.new_seq(), prompt, 4)
    got_ids = generate_greedy(B200InferencePipeline(h), "g", prompt, 4)
    assert got_ids == ref_ids.tolist(), (got_ids, ref_ids.tolist(), float(margins.min()))
    h.release_gpu_resources()
    om.close()


def test_batched_tcgen05_route_in_a_forward_pass(ctx, oracle):
    """48 sequences through a model whose paired gate/up matrix (2 x 4864 rows) and output projection (9728 rows)
    cross the row threshold of the tcgen05 kernel: its store and SiLU-pair epilogues inside a real step."""
    arch = synth.Arch(hidden=512, n_layers=2, n_heads=4, n_kv_heads=2, inter=4864, vocab=9728, rms_eps=1e-5, rope_theta=500000.0)
    n = 48
    om, h = build_pair(oracle, arch, seed=41, kv_dtype="f16", max_ctx=16, max_batch=n, max_seqs=n, ctx=ctx)
    rng = np.random.default_rng(6)
    toks = rng.integers(0, arch.vocab, n).tolist()
    ids = [f"s{i}" for i in range(n)]
    ctx.profile(True)
    ctx.profile_read()
    logits = h.forward_batch(ids, [[t] for t in toks], [0] * n)
    prof = ctx.profile_read()
    ctx.profile(False)
    assert prof["gemm_tcgen05"]["launches"] >= 3, prof  # gate/up of both layers and the output projection
    errs = np.sort([rel_err(logits[i], om.forward(om.new_seq(), toks[i], 0)) for i in range(n)])
    # FP16 operands on this path: about 1e-3 on most sequences, a few amplified by the random-init model
    assert float(np.median(errs)) < 2e-3 and errs[int(0.9 * n)] < 2e-2, (float(np.median(errs)), errs[-4:])
    h.release_gpu_resources()


@pytest.mark.parametrize("n_seq", [16, 64])
def test_greedy_identity_batch_16_and_64_exact_path(ctx, oracle, n_seq, monkeypatch):
    """Greedy ids of a whole batch for 64 steps.  On the exact integer path (here forced for every batch size: the
    sequences go through it eight at a time) the ids equal the oracle's, except where the oracle's own decision is a
    near-tie below the logits bar (measured: none of 16 TinyLlama sequences, 2 of 64 on the small model).  The default FP16 one-pass path of 9..64
    sequences is faster and is compared in test_forward_batched_path_matches_oracle; it does not promise identical
    ids (its measured agreement is reported in the design notes)."""
    monkeypatch.setenv("JUNO_GEMM_MIN_BATCH", "1000")
    arch = synth.TINYLLAMA if n_seq == 16 else SMALL128
    steps = 64
    om, h = build_pair(oracle, arch, seed=0, kv_dtype="f32", max_ctx=96, max_batch=n_seq, max_seqs=n_seq, ctx=ctx, norm="ones" if n_seq == 16 else "random")
    rng = np.random.default_rng(12)
    prompts = [rng.integers(0, arch.vocab, 4).tolist() for _ in range(n_seq)]
    names = [f"b{i}" for i in range(n_seq)]
    for r, p in zip(names, prompts):
        for i in range(len(p) - 1):
            h.forward_batch([r], [[p[i]]], [i], want_logits=False, want_argmax=True)
    out = h.decode_greedy(names, [p[-1] for p in prompts], [len(p) - 1 for p in prompts], steps)
    bad, n_near_ties = [], 0
    for i, p in enumerate(prompts):
        ref, margins = om.generate_greedy(om.new_seq(), p, steps)
        got = out[:, i].tolist()
        if got != ref.tolist():
            # the only excuse: at the first differing step the oracle's own top two logits are closer than the
            # parity bar of the logits (1e-3 of the largest one) - a near-tie that a different order of FP32
            # additions, amplified by the random-init model over the steps so far, may break the other way
            k = next(j for j in range(steps) if got[j] != int(ref[j]))
            seq = om.new_seq()
            toks = p + ref[:k].tolist()
            for pos, t in enumerate(toks):
                lg = om.forward(seq, t, pos)
            n_near_ties += 1
            if float(margins[k]) > TOL * float(np.abs(lg).max()):
                bad.append((i, k, float(margins[k]), float(np.abs(lg).max())))
    assert not bad, bad
    assert n_near_ties <= n_seq // 16, n_near_ties  # and such near-ties are rare
    h.release_gpu_resources()
    om.close()


@pytest.mark.parametrize("tied", [False, True], ids=["q6k-output", "tied-output"])
def test_model_loaded_from_a_gguf_file(ctx, oracle, tmp_path, tied):
    """The reference's load path end to end: a GGUF file on disk -> juno_gguf_open -> LlamaConfig.from ->
    juno_model_load_gguf.  The oracle reads the same file through the restated Java parser.  As in real Q4_K_M
    files, output.weight is Q6_K; without output.weight the projection is tied to token_embd."""
    from juno_b200 import gguf_file
    from juno_b200.handler import B200TransformerHandler
    from oracle import gguf_reader as oref

    def type_map(kind):
        return synth.Q6_K if kind == synth.T_OUTPUT else synth.q4_k_m_type(kind)

    arch = SMALL128
    path = tmp_path / "model.gguf"
    gguf_file.write_model(path, arch, synth.random_model(arch, 31, type_map, norm="random"), tied_output=tied)
    h = B200TransformerHandler.from_gguf(path, ctx, max_batch=2, max_seqs=2, max_ctx=64, kv_dtype="f32")
    assert (h.arch.hidden, h.arch.n_layers, h.arch.n_kv_heads, h.arch.vocab) == (arch.hidden, arch.n_layers, arch.n_kv_heads, arch.vocab)
    r = oref.GgufReader(path)
    c = oref.llama_config(r)
    om = oracle.Model(c["hidden"], c["n_layers"], c["n_heads"], c["n_kv_heads"], c["inter"], c["vocab"], c["rms_eps"], c["rope_theta"],
                      kv_f16=False, max_seq=64)
    for kind, layer, t, rows, cols, raw in oref.model_tensors(r, c["n_layers"]):
        om.set_tensor(kind, layer, raw, t, rows, cols)
    rng = np.random.default_rng(2)
    prompt = rng.integers(0, arch.vocab, 12).tolist()
    seq = om.new_seq()
    for p, t in enumerate(prompt):
        ref = om.forward(seq, t, p)
        got = h.forward(ForwardRequest("f", prompt[: p + 1], p)).logits
        assert rel_err(got, ref) < TOL
    ref_ids, _ = om.generate_greedy(om.new_seq(), prompt, 24)
    assert generate_greedy(B200InferencePipeline(h), "g", prompt, 24) == ref_ids.tolist()
    h.release_gpu_resources()


@pytest.mark.parametrize("via_gguf", [False, True], ids=["set_tensor", "gguf-file"])
def test_qkv_bias_models(ctx, oracle, tmp_path, via_gguf):
    """Qwen2-style attn_{q,k,v}.bias tensors (LlamaTransformerHandler.java:258-262): added to q, k, v before the rotation
    (:758-762).  Exact path token by token, the chunked prefill (batched kernels) and the greedy ids, against the oracle
    with the same biases; handed over tensor by tensor and read from a GGUF file."""
    from juno_b200 import gguf_file
    from juno_b200.handler import B200TransformerHandler
    from oracle import gguf_reader as oref
    arch = SMALL128
    if via_gguf:
        path = tmp_path / "bias.gguf"
        gguf_file.write_model(path, arch, synth.random_model(arch, 34, norm="random", qkv_bias=True))
        h = B200TransformerHandler.from_gguf(path, ctx, max_batch=8, max_seqs=2, max_ctx=64, kv_dtype="f32")
        r = oref.GgufReader(path)
        om = oracle.Model(arch.hidden, arch.n_layers, arch.n_heads, arch.n_kv_heads, arch.inter, arch.vocab, arch.rms_eps,
                          arch.rope_theta, kv_f16=False, max_seq=64)
        kinds = set()
        for kind, layer, t, rows, cols, raw in oref.model_tensors(r, arch.n_layers):
            om.set_tensor(kind, layer, raw, t, rows, cols)
            kinds.add(kind)
        assert {12, 13, 14} <= kinds
    else:
        om, h = build_pair(oracle, arch, seed=34, kv_dtype="f32", max_ctx=64, max_batch=8, max_seqs=2, ctx=ctx, qkv_bias=True)
    rng = np.random.default_rng(4)
    prompt = rng.integers(0, arch.vocab, 14).tolist()
    seq = om.new_seq()
    for p, t in enumerate(prompt):
        ref = om.forward(seq, t, p)
        got = h.forward(ForwardRequest("tok", prompt[: p + 1], p)).logits
        assert rel_err(got, ref) < TOL, (p, rel_err(got, ref))
    got = h.prefill("chunk", prompt, 0, want_logits=True)
    assert rel_err(got, ref) < 5e-3 and int(np.argmax(got)) == oracle.greedy(ref)
    ref_ids, _ = om.generate_greedy(om.new_seq(), prompt, 16)
    h.evict("tok")
    assert generate_greedy(B200InferencePipeline(h), "g", prompt, 16) == ref_ids.tolist()
    h.release_gpu_resources()


def test_incomplete_qkv_bias_is_refused(ctx):
    """A model with a bias for q but not for k and v cannot be finalized."""
    from juno_b200.handler import B200TransformerHandler
    arch = TINY
    h = B200TransformerHandler(arch, ctx, max_ctx=32)
    for kind, layer, t, rows, cols, blocks in synth.random_model(arch, 35):
        h.set_tensor(kind, layer, blocks, t, rows, cols)
    h.set_tensor(synth.T_ATTN_Q_BIAS, 0, np.zeros(arch.hidden, np.float32), synth.F32, 1, arch.hidden)
    with pytest.raises(ValueError, match="biases come together"):
        h.load([])
    h.release_gpu_resources()


def test_session_reuse_restarts_prefill_at_the_matched_prefix(ctx, oracle):
    """Multi-turn session as GenerationLoop runs it (GenerationLoop.java:283-294, 385-405): the KV state of a session
    stays under its key; the next turn's prompt begins with the previous prompt, so its prefill starts at the matched
    offset and overwrites the positions the previous turn generated into.  Logits of the second turn must equal a run
    from scratch on the whole second prompt, for the token-by-token prefill and for the chunked one."""
    arch = SMALL128
    rng = np.random.default_rng(9)
    p1 = rng.integers(0, arch.vocab, 20).tolist()
    p2 = p1 + rng.integers(0, arch.vocab, 12).tolist()
    om, h = build_pair(oracle, arch, seed=33, kv_dtype="f32", max_ctx=96, max_batch=8, max_seqs=3, ctx=ctx)
    pipe = B200InferencePipeline(h)
    # from scratch on the second prompt (oracle), positions 0..31
    seq = om.new_seq()
    for p, t in enumerate(p2):
        ref = om.forward(seq, t, p)
    for rid, chunked in (("session-a", False), ("session-b", True)):
        generate_greedy(pipe, rid, p1, 8)  # turn 1: prompt, then 8 generated positions 20..27 in the cache
        if chunked:
            h.prefill(rid, p2[len(p1):-1], len(p1))  # turn 2 restarts at the matched prefix (20) and rewrites 20..30
        else:
            for p in range(len(p1), len(p2) - 1):
                h.forward_batch([rid], [[p2[p]]], [p], want_logits=False, want_argmax=True)
        got = h.forward(ForwardRequest(rid, p2, len(p2) - 1)).logits
        tol = 5e-3 if chunked else TOL  # the chunked prefill runs FP16 operands (see the chunked-prefill test)
        assert rel_err(got, ref) < tol, (rid, rel_err(got, ref))
        assert int(np.argmax(got)) == oracle.greedy(ref)
    # eviction frees the session's pages for others (KVCacheManager eviction): a third session fits after one is evicted
    h.evict("session-a")
    got = h.forward(ForwardRequest("session-c", p2[:1], 0)).logits
    assert rel_err(got, om.forward(om.new_seq(), p2[0], 0)) < TOL
    h.release_gpu_resources()


@pytest.mark.parametrize("kv_dtype", ["f32", "f16"])
def test_shared_prefix_fork_and_copy_on_write(ctx, oracle, kv_dtype):
    """Prefix sharing between live requests (juno_seq_fork): request B adopts the first 24 cached positions of request A
    (one whole page and half of the next).  Both then go their own ways - B through the chunked prefill and token by
    token, A by decoding on and by REWRITING positions inside the shared pages - and each must match the oracle run
    from scratch on its own token sequence: a write into a shared page has to land in a private copy.  Freeing one
    holder leaves the other intact, and all pages come back in the end."""
    arch = SMALL128
    tol = TOL if kv_dtype == "f32" else TOL_F16_KV
    om, h = build_pair(oracle, arch, seed=36, kv_dtype=kv_dtype, max_ctx=64, max_batch=8, max_seqs=3, ctx=ctx)
    rng = np.random.default_rng(11)
    pa = rng.integers(0, arch.vocab, 40).tolist()
    tail_b = rng.integers(0, arch.vocab, 14).tolist()

    def oracle_logits(tokens):
        seq = om.new_seq()
        for p, t in enumerate(tokens):
            out = om.forward(seq, t, p)
        return out

    for p in range(len(pa) - 1):
        h.forward_batch(["A"], [[pa[p]]], [p], want_logits=False, want_argmax=True)
    h.fork("A", "B", 24)
    with pytest.raises(ValueError, match="cannot share"):
        h.fork("A", "C", 41)
    # B: positions 24..30 through the chunked prefill (first write into the half page -> private copy), then token by token
    tb = pa[:24] + tail_b
    h.prefill("B", tb[24:31], 24)
    for p in range(31, len(tb) - 1):
        h.forward_batch(["B"], [[tb[p]]], [p], want_logits=False, want_argmax=True)
    got_b = h.forward(ForwardRequest("B", tb, len(tb) - 1)).logits
    assert rel_err(got_b, oracle_logits(tb)) < max(tol, 5e-3)
    # A is untouched by B's writes
    got_a = h.forward(ForwardRequest("A", pa, len(pa) - 1)).logits
    assert rel_err(got_a, oracle_logits(pa)) < tol
    # A rewrites positions 10..39 (inside the page it still shares with B) with other tokens; B must not see them
    pa2 = pa[:10] + rng.integers(0, arch.vocab, 30).tolist()
    for p in range(10, len(pa2) - 1):
        h.forward_batch(["A"], [[pa2[p]]], [p], want_logits=False, want_argmax=True)
    got_a2 = h.forward(ForwardRequest("A", pa2, len(pa2) - 1)).logits
    assert rel_err(got_a2, oracle_logits(pa2)) < tol
    tb2 = tb + [5]
    got_b2 = h.forward(ForwardRequest("B", tb2, len(tb2) - 1)).logits
    assert rel_err(got_b2, oracle_logits(tb2)) < max(tol, 5e-3)
    # one holder leaves; the other still reads the shared first page
    h.evict("A")
    tb3 = tb2 + [6]
    assert rel_err(h.forward(ForwardRequest("B", tb3, len(tb3) - 1)).logits, oracle_logits(tb3)) < max(tol, 5e-3)
    h.evict("B")
    # every page is free again: three sequences can be filled to max_ctx
    for rid in ("x", "y", "z"):
        h.prefill(rid, rng.integers(0, arch.vocab, 64).tolist(), 0)
    h.release_gpu_resources()
