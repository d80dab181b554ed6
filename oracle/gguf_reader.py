"""TEST INFRASTRUCTURE ONLY — CPU restatement of the reference's GGUF parsing for the decode path.

Follows node/GgufReader.java (open :102-180, readMetadataValue :1189-1244, readArray :1246-1253, rawByteCount :347-360,
tensorRaw :329-340, meta accessors :190-216) and node/LlamaConfig.java (from :58-91, tokenizerTokenCount :98-101).
It is the checker for the library's own reader (juno_gguf_*) and feeds the CPU oracle model from a file; nothing the
product ships imports it.  The llamafile ZIP scan of the reference (:110-117) is not restated.

Parity: pinned by the reference's minimal-GGUF layout (GgufReaderTest.buildMinimalGguf :448-489, rebuilt byte for
byte in tests/test_gguf_file.py) and cross-read with the independent python `gguf` package where it is installed.
"""
from __future__ import annotations

import struct

import numpy as np

GGUF_MAGIC = 0x46554747  # GgufReader.java:50
ALIGNMENT = 32           # :51
# elements / bytes per block of each GGML type with a byte-size formula (rawByteCount :347-360)
_BYTES = {0: (1, 4), 1: (1, 2), 30: (1, 2), 8: (32, 34), 2: (32, 18), 10: (256, 84), 11: (256, 110), 12: (256, 144),
          13: (256, 176), 14: (256, 210)}


def raw_byte_count(ggml_type: int, n_elems: int) -> int:
    if ggml_type not in _BYTES:
        raise NotImplementedError(f"No byte-size formula for GGML type {ggml_type}")  # UnsupportedOperationException
    e, b = _BYTES[ggml_type]
    return n_elems // e * b


class _Cur:
    def __init__(self, buf):
        self.buf, self.pos = buf, 0

    def take(self, fmt):
        v = struct.unpack_from(fmt, self.buf, self.pos)[0]
        self.pos += struct.calcsize(fmt)
        return v

    def string(self):  # readString :1165-1171
        n = self.take("<Q")
        s = bytes(self.buf[self.pos:self.pos + n]).decode("utf-8", "replace")
        self.pos += n
        return s


def _value(c: _Cur, vtype: int):
    """readMetadataValue :1189-1244.  The reference reads 8- and 16-bit integers of either signedness as signed and
    32/64-bit ones into int/long (signed)."""
    if vtype in (0, 1):
        return c.take("<b")
    if vtype in (2, 3):
        return c.take("<h")
    if vtype in (4, 5):
        return c.take("<i")
    if vtype == 6:
        return float(np.float32(c.take("<f")))
    if vtype == 7:
        return c.take("<b") != 0
    if vtype == 8:
        return c.string()
    if vtype in (10, 11):
        return c.take("<q")
    if vtype == 12:
        return c.take("<d")
    if vtype == 9:  # readArray :1246-1253
        etype = c.take("<i")
        n = c.take("<Q")
        return [_value(c, etype) for _ in range(n)]
    raise IOError(f"Unknown metadata type: {vtype}")


class GgufReader:
    def __init__(self, path):
        self.buf = np.memmap(path, dtype=np.uint8, mode="r")
        c = _Cur(self.buf)
        magic, self.version = c.take("<I"), c.take("<i")
        n_tensors, n_kv = c.take("<Q"), c.take("<Q")
        if magic != GGUF_MAGIC:
            raise IOError(f"Not a GGUF file (magic=0x{magic:x} at offset 0)")
        if self.version < 2 or self.version > 3:
            raise IOError(f"Unsupported GGUF version: {self.version}")
        self.metadata = {}
        for _ in range(n_kv):
            key = c.string()
            vtype = c.take("<i")
            self.metadata[key] = _value(c, vtype)
        self.tensors = {}  # name -> (dims innermost first, type, offset in the data section, element count); file order
        for _ in range(n_tensors):
            name = c.string()
            nd = c.take("<i")
            dims = [c.take("<Q") for _ in range(nd)]
            t = c.take("<i")
            off = c.take("<Q")
            self.tensors[name] = (dims, t, off, int(np.prod(dims, dtype=np.int64)) if dims else 1)
        self.data_offset = (c.pos + ALIGNMENT - 1) // ALIGNMENT * ALIGNMENT  # :169-176

    # meta accessors :190-216: a value of another kind gives the default
    def meta_string(self, key):
        v = self.metadata.get(key)
        return v if isinstance(v, str) else None

    def meta_int(self, key, default):
        v = self.metadata.get(key)
        return int(v) if isinstance(v, (int, float)) and not isinstance(v, bool) else default

    def meta_float(self, key, default):
        v = self.metadata.get(key)
        return float(np.float32(v)) if isinstance(v, (int, float)) and not isinstance(v, bool) else default

    def has_tensor(self, name):
        return name in self.tensors

    def tensor_raw(self, name):
        """(GGML type, dims, uint8 bytes) — tensorRaw :329-340."""
        if name not in self.tensors:
            raise KeyError(f"Tensor not found: {name}  (available: {len(self.tensors)} tensors)")
        dims, t, off, n = self.tensors[name]
        nb = raw_byte_count(t, n)
        a = self.data_offset + off
        return t, dims, np.asarray(self.buf[a:a + nb])


def llama_config(r: GgufReader) -> dict:
    """LlamaConfig.from :58-91."""
    arch = r.meta_string("general.architecture") or "llama"
    p = arch + "."

    def geti(k, d):
        return r.meta_int(p + k, r.meta_int("llama." + k, d))

    def getf(k, d):
        return r.meta_float(p + k, r.meta_float("llama." + k, d))

    hidden = geti("embedding_length", 2048)
    heads = geti("attention.head_count", 32)
    toks = r.metadata.get("tokenizer.ggml.tokens")
    tok_count = len(toks) if isinstance(toks, list) else 0
    return dict(hidden=hidden, n_layers=geti("block_count", 22), n_heads=heads, n_kv_heads=geti("attention.head_count_kv", heads),
                vocab=max(geti("vocab_size", 32000), tok_count), inter=geti("feed_forward_length", hidden * 11 // 4),
                rms_eps=getf("attention.layer_norm_rms_epsilon", float(np.float32(1e-5))),
                rope_theta=getf("rope.freq_base", 10000.0), head_dim=hidden // heads, arch=arch)


_PER_LAYER = [("attn_norm", 3), ("ffn_norm", 4), ("attn_q", 5), ("attn_k", 6), ("attn_v", 7), ("attn_output", 8), ("ffn_gate", 9),
              ("ffn_up", 10), ("ffn_down", 11)]


def model_tensors(r: GgufReader, n_layers: int):
    """(kind, layer, type, rows, cols, bytes) for every tensor the reference constructor reads
    (LlamaTransformerHandler.java:238-275); output.weight falls back to token_embd.weight when absent (:463-470)."""
    def one(name, kind, layer):
        t, dims, raw = r.tensor_raw(name)
        return kind, layer, t, (dims[1] if len(dims) > 1 else 1), dims[0], raw

    yield one("token_embd.weight", 0, 0)
    yield one("output_norm.weight", 1, 0)
    yield one("output.weight" if r.has_tensor("output.weight") else "token_embd.weight", 2, 0)
    for l in range(n_layers):
        for suffix, kind in _PER_LAYER:
            yield one(f"blk.{l}.{suffix}.weight", kind, l)
        if r.has_tensor("blk.0.attn_q.bias"):  # the constructor decides by the first layer's attn_q.bias (:258-262)
            for suffix, kind in (("attn_q", 12), ("attn_k", 13), ("attn_v", 14)):
                yield one(f"blk.{l}.{suffix}.bias", kind, l)
