"""Builds the same seeded random-init model in the CPU oracle and in the B200 engine."""
import numpy as np

from juno_b200 import synth


def build_pair(oracle, arch, seed, kv_dtype="f16", max_ctx=256, max_batch=1, max_seqs=4, engine=True, ctx=None,
               type_map=synth.q4_k_m_type, norm="random", qkv_bias=False):
    """RMSNorm weights are random and distinct per vector by default: a wrong vector, a wrong layer index or a dropped
    output_norm shows up in every forward test."""
    tensors = list(synth.random_model(arch, seed, type_map, norm=norm, qkv_bias=qkv_bias))
    om = oracle.Model(arch.hidden, arch.n_layers, arch.n_heads, arch.n_kv_heads, arch.inter, arch.vocab, arch.rms_eps,
                      arch.rope_theta, kv_f16=(kv_dtype == "f16"), max_seq=max_ctx)
    for kind, layer, t, rows, cols, blocks in tensors:
        om.set_tensor(kind, layer, blocks, t, rows if kind not in (1, 3, 4) and kind < 12 else 1, cols)
    h = None
    if engine:
        from juno_b200.handler import B200TransformerHandler
        h = B200TransformerHandler(arch, ctx, max_batch=max_batch, max_seqs=max_seqs, max_ctx=max_ctx, kv_dtype=kv_dtype)
        h.load(tensors)
    return om, h


TINY = synth.Arch(hidden=256, n_layers=2, n_heads=4, n_kv_heads=2, inter=512, vocab=1024, rms_eps=1e-5, rope_theta=10000.0)
SMALL128 = synth.Arch(hidden=512, n_layers=3, n_heads=4, n_kv_heads=2, inter=768, vocab=2048, rms_eps=1e-5,
                      rope_theta=500000.0)
