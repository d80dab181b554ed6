"""Pins the CPU oracle to the reference's own known-answer tests (transcribed into tests/golden/)."""
import json
import os

import numpy as np
import pytest

from juno_b200 import synth

G = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "quant_known_answers.json")))


def test_f16_exact_values(oracle):
    for bits, val in G["f16_exact"]:
        assert oracle.f16_to_f32(bits) == val


def test_f16_matches_ieee_for_all_finite_patterns(oracle):
    bits = np.arange(65536, dtype=np.uint16)
    ours = np.array([oracle.f16_to_f32(int(b)) for b in bits], dtype=np.float32)
    ref = bits.view(np.float16).astype(np.float32)
    finite = np.isfinite(ref)
    assert np.array_equal(ours[finite].view(np.uint32), ref[finite].view(np.uint32))
    assert np.isnan(ours[~finite & np.isnan(ref)]).all()


def test_q6k_golden_block(oracle):
    g = G["q6k_golden"]
    out = oracle.dequantize(synth.Q6_K, np.array(g["block"], dtype=np.uint8), 1, 256)[0]
    assert out.shape == (256,)
    for i, v in g["expected"]:
        assert abs(out[i] - v) < g["eps"]


def test_q6k_range(oracle):
    out = oracle.dequantize(synth.Q6_K, np.array(G["q6k_range"]["block"], dtype=np.uint8), 1, 256)
    assert np.abs(out).max() <= G["q6k_range"]["abs_max"]


def test_q4k_cases(oracle):
    out = oracle.dequantize(synth.Q4_K, np.array(G["q4k_all_zero"]["block"], dtype=np.uint8), 1, 256)
    assert (out == 0.0).all()
    out = oracle.dequantize(synth.Q4_K, np.array(G["q4k_nibble_split"]["block"], dtype=np.uint8), 1, 256)[0]
    assert out.size == G["q4k_nibble_split"]["size"] and out[0] == 0.0


def test_q8_0_case(oracle):
    g = G["q8_0_half_i"]
    out = oracle.dequantize(synth.Q8_0, np.array(g["block"], dtype=np.uint8), 1, 32)[0]
    assert np.abs(out - np.array(g["expected"])).max() < g["eps"]


@pytest.mark.parametrize("name,t", [("q4k_one_block_dot", synth.Q4_K), ("q6k_golden_dot", synth.Q6_K)])
def test_quantised_matvec_equals_dequant_matvec(oracle, name, t):
    g = G[name]
    blk = np.array(g["block"], dtype=np.uint8)
    x = np.ones(g["cols"], dtype=np.float32)
    deq = oracle.dequantize(t, blk, 1, g["cols"])
    expected = oracle.matvec(synth.F32, deq, x, 1, g["cols"])
    actual = oracle.matvec(t, blk, x, 1, g["cols"])
    assert abs(actual[0] - expected[0]) < g["eps"]


def test_row_range_matvec(oracle):
    g = G["q4k_three_rows"]
    blk = np.array(g["blocks"], dtype=np.uint8)
    x = np.ones(256, dtype=np.float32)
    deq = oracle.dequantize(synth.Q4_K, blk, 3, 256)
    r0 = oracle.matvec(synth.Q4_K, blk, x, 3, 256, 0, 1)
    r1 = oracle.matvec(synth.Q4_K, blk, x, 3, 256, 1, 2)
    r01 = oracle.matvec(synth.Q4_K, blk, x, 3, 256, 0, 2)
    assert abs(r0[0] - deq[0].sum()) < 1e-3 and abs(r1[0] - deq[1].sum()) < 1e-3
    assert r01.shape == (2,) and r01[0] == r0[0] and r01[1] == r1[0]


def test_raw_byte_counts(oracle):
    for c in G["raw_bytes"]:
        assert oracle.row_bytes(c["type"], c["nelems"]) == c["bytes"]


def test_second_opinion_gguf_package(oracle):
    """The python gguf package dequantises with the same operation order; values must agree bit for bit."""
    quants = pytest.importorskip("gguf.quants")
    import gguf
    rng = np.random.default_rng(7)
    for t, qt in ((synth.Q4_K, gguf.GGMLQuantizationType.Q4_K), (synth.Q6_K, gguf.GGMLQuantizationType.Q6_K),
                  (synth.Q8_0, gguf.GGMLQuantizationType.Q8_0)):
        raw = synth.random_blocks(rng, t, 4, 512)
        ours = oracle.dequantize(t, raw, 4, 512)
        theirs = quants.dequantize(raw.reshape(4, -1), qt)
        assert np.array_equal(ours, theirs.reshape(4, 512).astype(np.float32))


def test_primitives_against_numpy(oracle):
    rng = np.random.default_rng(8)
    x = rng.standard_normal(64).astype(np.float32)
    w = rng.standard_normal(64).astype(np.float32)
    ref = w * x / np.sqrt((x.astype(np.float64) ** 2).mean() + 1e-5)
    assert np.allclose(oracle.rmsnorm(x, w, 1e-5), ref, rtol=1e-5)
    s = oracle.softmax(x)
    assert abs(s.sum() - 1) < 1e-5 and s.argmax() == x.argmax()
    assert abs(oracle.silu(1.5) - 1.5 / (1 + np.exp(-1.5))) < 1e-6
    # adjacent-pair rotation, position 0 is the identity
    assert np.array_equal(oracle.rope(x, 0, 2, 32, 10000.0), x)
    r = oracle.rope(x, 3, 2, 32, 10000.0)
    assert np.allclose(np.hypot(r[0::2], r[1::2]), np.hypot(x[0::2], x[1::2]), rtol=1e-5)
    ang = 3.0  # pair 0 has frequency 1
    assert np.allclose(r[0], x[0] * np.cos(ang) - x[1] * np.sin(ang), rtol=1e-5)
    # greedy: first maximum wins
    assert oracle.greedy(np.array([0.1, 2.0, 2.0, -1.0], dtype=np.float32)) == 1
    parts = rng.standard_normal((3, 10)).astype(np.float32)
    assert np.allclose(oracle.allreduce_sum(parts), parts.sum(0), rtol=1e-6)


def test_gqa_against_numpy(oracle):
    rng = np.random.default_rng(9)
    nH, nKV, hd, T = 8, 2, 16, 37
    q = rng.standard_normal(nH * hd).astype(np.float32)
    K = rng.standard_normal((T, nKV * hd)).astype(np.float32)
    V = rng.standard_normal((T, nKV * hd)).astype(np.float32)
    out = oracle.gqa(q, K, V, T, nH, nKV, hd).reshape(nH, hd)
    for h in range(nH):
        kv = h // (nH // nKV)
        s = K[:, kv * hd:(kv + 1) * hd].astype(np.float64) @ q[h * hd:(h + 1) * hd] / np.sqrt(hd)
        p = np.exp(s - s.max())
        p /= p.sum()
        assert np.allclose(out[h], p @ V[:, kv * hd:(kv + 1) * hd], rtol=1e-4, atol=1e-5)


def test_oracle_forward_runs_and_kv_modes_differ_only_slightly(oracle):
    from modelutil import TINY, build_pair
    o32, _ = build_pair(oracle, TINY, 21, kv_dtype="f32", max_ctx=16, engine=False)
    o16, _ = build_pair(oracle, TINY, 21, kv_dtype="f16", max_ctx=16, engine=False)
    s32, s16 = o32.new_seq(), o16.new_seq()
    for p, t in enumerate([1, 2, 3, 4]):
        a, b = o32.forward(s32, t, p), o16.forward(s16, t, p)
    assert a.shape == (TINY.vocab,) and np.isfinite(a).all()
    assert np.abs(a - b).max() / np.abs(a).max() < 5e-2
    with pytest.raises(AssertionError):
        o32.forward(s32, 1, 16)  # beyond max_seq


def test_oracle_qkv_bias_is_added_before_the_rotation(oracle):
    """attn_{q,k,v}.bias (LlamaTransformerHandler.java:258-262, 758-762): zero biases leave every logit bit-identical; a
    bias on v alone shifts the attention output of position 0 (softmax over one position = 1) by exactly Wo * bias, which
    shows in the hidden state; a model without bias tensors is unchanged."""
    from juno_b200 import synth
    arch = synth.Arch(hidden=256, n_layers=1, n_heads=4, n_kv_heads=2, inter=512, vocab=512)
    tensors = list(synth.random_model(arch, 3, norm="random"))

    def model(bias):
        m = oracle.Model(arch.hidden, arch.n_layers, arch.n_heads, arch.n_kv_heads, arch.inter, arch.vocab, arch.rms_eps,
                         arch.rope_theta, kv_f16=False, max_seq=8)
        for kind, layer, t, rows, cols, blocks in tensors:
            m.set_tensor(kind, layer, blocks, t, 1 if kind in (1, 3, 4) else rows, cols)
        if bias is not None:
            bq, bk, bv = bias
            m.set_tensor(12, 0, bq.view(np.uint8), 0, 1, arch.hidden)
            m.set_tensor(13, 0, bk.view(np.uint8), 0, 1, arch.kv_dim)
            m.set_tensor(14, 0, bv.view(np.uint8), 0, 1, arch.kv_dim)
        return m

    z = lambda n: np.zeros(n, np.float32)
    base = model(None).forward(model(None).new_seq(), 7, 0)
    m0 = model((z(arch.hidden), z(arch.kv_dim), z(arch.kv_dim)))
    assert np.array_equal(m0.forward(m0.new_seq(), 7, 0).view(np.uint32), base.view(np.uint32))
    rng = np.random.default_rng(0)
    mb = model((z(arch.hidden), z(arch.kv_dim), rng.standard_normal(arch.kv_dim).astype(np.float32)))
    assert not np.array_equal(mb.forward(mb.new_seq(), 7, 0), base)
    # q and k biases do not matter at position 0 of a fresh sequence: one position, softmax weight exactly 1
    mqk = model((rng.standard_normal(arch.hidden).astype(np.float32), rng.standard_normal(arch.kv_dim).astype(np.float32), z(arch.kv_dim)))
    assert np.array_equal(mqk.forward(mqk.new_seq(), 7, 0).view(np.uint32), base.view(np.uint32))
