"""The allocation-free attention entry point (juno_attn_decode_static) against the regular one.

Some hosts give every byte of HBM to weights and KV pages and cannot let the library call cudaMalloc later; for them
the attention operator exists in a form whose scratch is a fixed array inside the library.  This file sorts last so a
run that stops at the first failure has already exercised everything else; it must also pass alone in a fresh process.
"""
import ctypes as C

import numpy as np
import pytest

from conftest import rel_err
from juno_b200.matvec import PagedKvCache, _ptr
from juno_b200._lib import check

pytestmark = pytest.mark.gpu
TOL = 1e-3  # the tolerance of the attention parity tests


@pytest.mark.parametrize("kv_dtype,lens", [("f16", [700, 129, 16, 2048]), ("f32", [700, 129, 16, 2048]), ("f16", [9000])],
                         ids=["f16-pages", "f32-pages", "long-context"])
def test_static_scratch_attention_matches_regular_entry_twice(ctx, kv_dtype, lens):
    """FP16 pages with few context splits merge on chip and leave the array idle; FP32 pages and a long context (more
    splits than one thread-block cluster holds) put their split partials into it."""
    import torch
    rng = np.random.default_rng(42)
    n_heads, n_kv, hd = 32, 8, 128
    cache = PagedKvCache(ctx, 1, n_kv, hd, sum((l + 15) // 16 for l in lens) + 2, kv_dtype)
    seqs = []
    for l in lens:
        s = cache.new_sequence(l)
        cache.append(s, 0, 0, rng.standard_normal((l, n_kv * hd)).astype(np.float32),
                     rng.standard_normal((l, n_kv * hd)).astype(np.float32))
        seqs.append(s)
    arr = (C.c_void_p * len(seqs))(*[s.value for s in seqs])
    L = ctx._L
    for call in range(2):  # two calls in a row share the same scratch array
        q = rng.standard_normal((len(lens), n_heads * hd)).astype(np.float32)
        want = cache.attention(0, seqs, q, n_heads)
        q_dev = torch.from_numpy(q).cuda()
        out_dev = torch.full_like(q_dev, float("nan"))
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        check(L.juno_attn_decode_static(ctx.handle, cache.handle, 0, len(seqs), arr, n_heads,
                                        C.c_void_p(q_dev.data_ptr()), C.c_void_p(out_dev.data_ptr())),
              "juno_attn_decode_static")
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after == free_before, (free_before, free_after)  # the call took no device memory (cudaMemGetInfo)
        got = out_dev.cpu().numpy()
        assert np.isfinite(got).all()
        assert rel_err(got, want) < TOL, (call, rel_err(got, want))
    # a call that cannot fit the fixed scratch is refused with a clear message, not served by allocating
    many = (C.c_void_p * 300)(*([seqs[0].value] * 300))
    rc = L.juno_attn_decode_static(ctx.handle, cache.handle, 0, 300, many, n_heads, C.c_void_p(q_dev.data_ptr()),
                                   C.c_void_p(out_dev.data_ptr()))
    assert rc == -1 and b"allocation-free" in L.juno_last_error()
    for s in seqs:
        cache.free_sequence(s)
    cache.close()
