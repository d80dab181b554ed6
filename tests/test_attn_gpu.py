"""GQA flash-decode attention over the paged KV cache vs the oracle's gqa() (through the C ABI)."""
import numpy as np
import pytest

from conftest import rel_err
from juno_b200.matvec import PagedKvCache

pytestmark = pytest.mark.gpu
TOL = 1e-3


def _run(ctx, oracle, n_heads, n_kv, hd, lens, kv_dtype, seed=2):
    rng = np.random.default_rng(seed)
    kvdim = n_kv * hd
    pages = sum((l + 15) // 16 for l in lens) + 4
    cache = PagedKvCache(ctx, 2, n_kv, hd, pages, kv_dtype)
    seqs, Ks, Vs = [], [], []
    for l in lens:
        s = cache.new_sequence(l)
        K = rng.standard_normal((l, kvdim)).astype(np.float32)
        V = rng.standard_normal((l, kvdim)).astype(np.float32)
        # appended in two ragged pieces to exercise page boundaries
        cut = max(1, l // 3)
        cache.append(s, 1, 0, K[:cut], V[:cut])
        cache.append(s, 1, cut, K[cut:], V[cut:])
        assert cache.length(s) == l
        seqs.append(s)
        if kv_dtype == "f16":
            K, V = K.astype(np.float16).astype(np.float32), V.astype(np.float16).astype(np.float32)
        Ks.append(K)
        Vs.append(V)
    q = rng.standard_normal((len(lens), n_heads * hd)).astype(np.float32)
    out = cache.attention(1, seqs, q, n_heads)
    for i, l in enumerate(lens):
        ref = oracle.gqa(q[i], Ks[i], Vs[i], l, n_heads, n_kv, hd)
        assert rel_err(out[i], ref) < TOL, (i, l, rel_err(out[i], ref))
    for s in seqs:
        cache.free_sequence(s)
    cache.close()


@pytest.mark.parametrize("kv_dtype", ["f16", "f32"])
@pytest.mark.parametrize("lens", [[1], [15], [16], [17], [300, 512, 257]])
def test_attention_llama3_heads(ctx, oracle, kv_dtype, lens):
    _run(ctx, oracle, 32, 8, 128, lens, kv_dtype)


def test_attention_tinyllama_heads(ctx, oracle):
    _run(ctx, oracle, 32, 4, 64, [100, 33], "f16")


def test_attention_sweep_point(ctx, oracle):
    """One point of the attention sweep: context 2048, batch 8, lengths uniform in [ctx/2, ctx]."""
    rng = np.random.default_rng(2)
    lens = rng.integers(1024, 2049, 8).tolist()
    _run(ctx, oracle, 32, 8, 128, lens, "f16")


def test_attention_long_context_split(ctx, oracle):
    _run(ctx, oracle, 32, 8, 128, [8192], "f16")


@pytest.mark.parametrize("cluster", ["0", "8", "16"])
@pytest.mark.parametrize("lens", [[2049], [300, 2049, 17], [1025, 1040]])
def test_attention_merge_with_empty_split(ctx, oracle, lens, cluster, monkeypatch):
    """Lengths just above a multiple of the split size: the splits are rounded up to whole pages, so the last
    split of a sequence holds no position at all.  Both merges are covered: the separate merge kernel (the default)
    and, with JUNO_ATTN_CLUSTER set, the splits of a (sequence, kv head) as one thread-block cluster merged on chip,
    where the empty split must still take part."""
    monkeypatch.setenv("JUNO_ATTN_CLUSTER", cluster)
    _run(ctx, oracle, 32, 8, 128, lens, "f16")


def test_attention_sweep_long_and_wide(ctx, oracle):
    """Two more points of the attention sweep: context 32768 at batch 1, and batch 64 at context 2048 with lengths
    uniform in [ctx/2, ctx]."""
    _run(ctx, oracle, 32, 8, 128, [32768], "f16")
    rng = np.random.default_rng(3)
    _run(ctx, oracle, 32, 8, 128, rng.integers(1024, 2049, 64).tolist(), "f16")
