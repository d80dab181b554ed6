"""GGUF model files: a writer for the seeded synthetic models and the binding of the library's reader.

Writer: GGUF v3 (or v2), little endian, alignment 32, exactly the layout node/GgufReader.java parses (open :102-180):
header (magic "GGUF", version, tensor count, metadata count), metadata key/value pairs, the tensor table (name, ndims,
dims innermost first = [cols, rows], GGML type, offset relative to the data section) and the data section at the next
multiple of 32.  Metadata keys are the ones LlamaConfig.from reads (LlamaConfig.java:58-91); tensor names are the ones
the LlamaTransformerHandler constructor reads (LlamaTransformerHandler.java:238-275).

Reader: `GgufFile` wraps juno_gguf_* of libjuno_b200.so (host code, no GPU needed): the file is mapped once and tensors
are handed to the GPU loader as pointers into the mapping.
"""
from __future__ import annotations

import ctypes as C
import struct

import numpy as np

from . import _lib, synth
from ._lib import check

GGUF_MAGIC = 0x46554747
ALIGNMENT = 32
# metadata value type ids (GgufReader.java:66-78)
(MT_UINT8, MT_INT8, MT_UINT16, MT_INT16, MT_UINT32, MT_INT32, MT_FLOAT32, MT_BOOL, MT_STRING, MT_ARRAY, MT_UINT64, MT_INT64,
 MT_FLOAT64) = range(13)
_SCALAR_FMT = {MT_UINT8: "<B", MT_INT8: "<b", MT_UINT16: "<H", MT_INT16: "<h", MT_UINT32: "<I", MT_INT32: "<i",
               MT_FLOAT32: "<f", MT_BOOL: "<B", MT_UINT64: "<Q", MT_INT64: "<q", MT_FLOAT64: "<d"}
FILE_TYPE_Q4_K_M = 15


def _str(s: str) -> bytes:
    b = s.encode("utf-8")
    return struct.pack("<Q", len(b)) + b


def _value(vtype: int, v) -> bytes:
    if vtype == MT_STRING:
        return _str(v)
    if vtype == MT_ARRAY:
        etype, items = v
        return struct.pack("<iQ", etype, len(items)) + b"".join(_value(etype, x) for x in items)
    return struct.pack(_SCALAR_FMT[vtype], v)


def llama_metadata(arch: synth.Arch, arch_name: str = "llama", file_type: int = FILE_TYPE_Q4_K_M, name: str = "synthetic"):
    """The metadata LlamaConfig.from reads, as (key, value type, value) triples."""
    p = arch_name + "."
    return [("general.architecture", MT_STRING, arch_name), ("general.name", MT_STRING, name),
            ("general.file_type", MT_UINT32, file_type),
            (p + "embedding_length", MT_UINT32, arch.hidden), (p + "block_count", MT_UINT32, arch.n_layers),
            (p + "attention.head_count", MT_UINT32, arch.n_heads), (p + "attention.head_count_kv", MT_UINT32, arch.n_kv_heads),
            (p + "vocab_size", MT_UINT32, arch.vocab), (p + "feed_forward_length", MT_UINT32, arch.inter),
            (p + "attention.layer_norm_rms_epsilon", MT_FLOAT32, arch.rms_eps), (p + "rope.freq_base", MT_FLOAT32, arch.rope_theta)]


def write_gguf(path, metadata, tensors, version: int = 3) -> dict:
    """metadata: (key, value type, value) triples; tensors: (name, GGML type, dims innermost first, uint8 data).
    Returns {"data_offset": ..., "offsets": {name: absolute offset}}."""
    tensors = list(tensors)
    head = struct.pack("<IiQQ", GGUF_MAGIC, version, len(tensors), len(metadata))
    meta = b"".join(_str(k) + struct.pack("<i", t) + _value(t, v) for k, t, v in metadata)
    table, off, offsets = [], 0, []
    for name, ggml_type, dims, data in tensors:
        data = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        table.append(_str(name) + struct.pack("<i", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) +
                     struct.pack("<iQ", ggml_type, off))
        offsets.append(off)
        off = (off + data.size + ALIGNMENT - 1) // ALIGNMENT * ALIGNMENT
    pre = head + meta + b"".join(table)
    data_offset = (len(pre) + ALIGNMENT - 1) // ALIGNMENT * ALIGNMENT
    out = {"data_offset": data_offset, "offsets": {}}
    with open(path, "wb") as f:
        f.write(pre)
        f.write(b"\0" * (data_offset - len(pre)))
        pos = 0
        for (name, _, _, data), o in zip(tensors, offsets):
            f.write(b"\0" * (o - pos))
            raw = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
            f.write(raw.tobytes())
            pos = o + raw.size
            out["offsets"][name] = data_offset + o
    return out


def model_tensor_entries(model_tensors, tied_output: bool = False):
    """(kind, layer, type, rows, cols, blocks) of synth.random_model -> (name, type, dims, data) of write_gguf."""
    for kind, layer, t, rows, cols, blocks in model_tensors:
        if tied_output and kind == synth.T_OUTPUT:
            continue  # output.weight absent: the reference ties it to token_embd (LlamaTransformerHandler.java:463-470)
        name = synth.GGUF_NAMES[kind].format(layer)
        dims = [cols] if kind in (synth.T_OUTPUT_NORM, synth.T_ATTN_NORM, synth.T_FFN_NORM) or kind >= synth.T_ATTN_Q_BIAS else [cols, rows]
        yield name, t, dims, blocks


def write_model(path, arch: synth.Arch, model_tensors, arch_name: str = "llama", tied_output: bool = False,
                extra_metadata=(), version: int = 3) -> dict:
    """A whole seeded model (synth.random_model) as one GGUF file."""
    return write_gguf(path, llama_metadata(arch, arch_name) + list(extra_metadata), model_tensor_entries(model_tensors, tied_output),
                      version)


class GgufFile:
    """GgufReader of the reference, backed by the library's mapped-file reader (juno_gguf_*)."""

    def __init__(self, path):
        self._L = _lib.load()
        h = C.c_void_p()
        check(self._L.juno_gguf_open(str(path).encode(), C.byref(h)), "juno_gguf_open")
        self.handle = h
        v, nt, nm, do = C.c_int32(), C.c_int64(), C.c_int64(), C.c_int64()
        check(self._L.juno_gguf_info(h, C.byref(v), C.byref(nt), C.byref(nm), C.byref(do)), "juno_gguf_info")
        self.version, self.n_tensors, self.n_meta, self.data_offset = v.value, nt.value, nm.value, do.value

    def close(self) -> None:
        if self.handle:
            check(self._L.juno_gguf_close(self.handle), "juno_gguf_close")
            self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def meta_int(self, key: str, default: int = 0) -> int:
        out = C.c_int64()
        check(self._L.juno_gguf_meta_int(self.handle, key.encode(), default, C.byref(out)), "juno_gguf_meta_int")
        return out.value

    def meta_float(self, key: str, default: float = 0.0) -> float:
        out = C.c_double()
        check(self._L.juno_gguf_meta_float(self.handle, key.encode(), default, C.byref(out)), "juno_gguf_meta_float")
        return out.value

    def meta_string(self, key: str):
        n = C.c_int32()
        check(self._L.juno_gguf_meta_string(self.handle, key.encode(), None, 0, C.byref(n)), "juno_gguf_meta_string")
        if n.value < 0:
            return None
        buf = C.create_string_buffer(n.value + 1)
        check(self._L.juno_gguf_meta_string(self.handle, key.encode(), buf, n.value + 1, C.byref(n)), "juno_gguf_meta_string")
        return buf.raw[: n.value].decode("utf-8")

    def meta_array_len(self, key: str) -> int:
        n = C.c_int64()
        check(self._L.juno_gguf_meta_array_len(self.handle, key.encode(), C.byref(n)), "juno_gguf_meta_array_len")
        return n.value

    def tensor_names(self):
        buf = C.create_string_buffer(512)
        out = []
        for i in range(self.n_tensors):
            check(self._L.juno_gguf_tensor_name(self.handle, i, buf, 512), "juno_gguf_tensor_name")
            out.append(buf.value.decode("utf-8"))
        return out

    def has_tensor(self, name: str) -> bool:
        p = C.c_int32()
        check(self._L.juno_gguf_has_tensor(self.handle, name.encode(), C.byref(p)), "juno_gguf_has_tensor")
        return bool(p.value)

    def tensor_info(self, name: str):
        """(GGML type, dims innermost first) — tensorType / tensorDims."""
        t, nd = C.c_int32(), C.c_int32()
        dims = (C.c_int64 * 4)()
        check(self._L.juno_gguf_tensor(self.handle, name.encode(), C.byref(t), C.byref(nd), dims, None, None), "juno_gguf_tensor")
        return t.value, [dims[i] for i in range(nd.value)]

    def tensor_raw(self, name: str):
        """(GGML type, dims, uint8 view of the mapped bytes) — tensorRaw; the view is valid until close()."""
        t, nd, nb = C.c_int32(), C.c_int32(), C.c_int64()
        dims = (C.c_int64 * 4)()
        data = C.c_void_p()
        check(self._L.juno_gguf_tensor(self.handle, name.encode(), C.byref(t), C.byref(nd), dims, C.byref(data), C.byref(nb)),
              "juno_gguf_tensor")
        arr = np.ctypeslib.as_array(C.cast(data, C.POINTER(C.c_uint8)), shape=(nb.value,)) if nb.value else np.zeros(0, np.uint8)
        return t.value, [dims[i] for i in range(nd.value)], arr

    @staticmethod
    def raw_byte_count(ggml_type: int, n_elems: int) -> int:
        out = C.c_int64()
        check(_lib.load().juno_gguf_raw_byte_count(ggml_type, n_elems, C.byref(out)), "juno_gguf_raw_byte_count")
        return out.value

    def arch(self) -> synth.Arch:
        """LlamaConfig.from."""
        cfg = _lib.ModelCfg()
        check(self._L.juno_gguf_model_cfg(self.handle, C.byref(cfg)), "juno_gguf_model_cfg")
        return synth.Arch(cfg.hidden, cfg.n_layers, cfg.n_heads, cfg.n_kv_heads, cfg.inter, cfg.vocab, cfg.rms_eps, cfg.rope_theta)
