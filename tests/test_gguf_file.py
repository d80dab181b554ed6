"""GGUF files on the host (no GPU): the library's mapped-file reader against the CPU restatement of the reference's
parser, the writer for the seeded models, the model configuration, and damaged files."""
import struct

import numpy as np
import pytest

from juno_b200 import _lib, gguf_file, synth
from juno_b200.gguf_file import GgufFile
from oracle import gguf_reader as oref

ARCH = synth.Arch(hidden=256, n_layers=2, n_heads=4, n_kv_heads=2, inter=512, vocab=1024, rms_eps=1e-5, rope_theta=500000.0)


def minimal_gguf(path, name, ggml_type, nelems, data, version=3):
    """The single-tensor file of the reference's reader tests (GgufReaderTest.buildMinimalGguf :448-489): header with
    zero metadata entries, one 1-D tensor at data offset 0, padding to a multiple of 32, the tensor bytes."""
    nb = name.encode()
    pre = struct.pack("<IiQQ", 0x46554747, version, 1, 0) + struct.pack("<Q", len(nb)) + nb + struct.pack("<iQiQ", 1, nelems, ggml_type, 0)
    pad = (-len(pre)) % 32
    with open(path, "wb") as f:
        f.write(pre + b"\0" * pad + bytes(data))
    return len(pre) + pad


def test_minimal_q8_0_file_of_the_reference_tests(tmp_path, oracle):
    """Q8_0 block with d = 0.5 (FP16 0x3800) and values 0..31 -> 0.5 * i (GgufReaderTest :634-656)."""
    block = struct.pack("<H", 0x3800) + bytes(range(32))
    p = tmp_path / "q8test.gguf"
    data_off = minimal_gguf(p, "q8test", 8, 32, block)
    with GgufFile(p) as g:
        assert (g.version, g.n_tensors, g.n_meta, g.data_offset) == (3, 1, 0, data_off)
        assert g.tensor_names() == ["q8test"]
        t, dims, raw = g.tensor_raw("q8test")
        assert (t, dims) == (8, [32]) and raw.tobytes() == block
        vals = oracle.dequantize(8, raw, 1, 32)
    assert np.array_equal(vals.reshape(-1), 0.5 * np.arange(32, dtype=np.float32))
    r = oref.GgufReader(p)
    assert r.data_offset == data_off and r.tensor_raw("q8test")[2].tobytes() == block
    # with no metadata every field of the configuration is the TinyLlama default (LlamaConfig.java:58-91)
    with GgufFile(p) as g:
        a = g.arch()
    assert (a.hidden, a.n_layers, a.n_heads, a.n_kv_heads, a.inter, a.vocab) == (2048, 22, 32, 32, 5632, 32000)
    assert a.rms_eps == np.float32(1e-5) and a.rope_theta == 10000.0
    ref = oref.llama_config(r)
    assert (ref["hidden"], ref["n_layers"], ref["n_heads"], ref["n_kv_heads"], ref["inter"], ref["vocab"]) == (2048, 22, 32, 32, 5632, 32000)


@pytest.mark.parametrize("version", [2, 3])
@pytest.mark.parametrize("tied", [False, True], ids=["own-output", "tied-output"])
def test_model_file_round_trip(tmp_path, version, tied):
    tensors = list(synth.random_model(ARCH, 5, norm="random"))
    p = tmp_path / "m.gguf"
    where = gguf_file.write_model(p, ARCH, tensors, tied_output=tied, version=version)
    r = oref.GgufReader(p)
    with GgufFile(p) as g:
        assert g.version == version == r.version and g.data_offset == where["data_offset"] == r.data_offset
        assert g.data_offset % 32 == 0
        assert g.tensor_names() == list(r.tensors)
        assert g.has_tensor("output.weight") == (not tied)
        a = g.arch()
        assert (a.hidden, a.n_layers, a.n_heads, a.n_kv_heads, a.inter, a.vocab) == (ARCH.hidden, ARCH.n_layers, ARCH.n_heads,
                                                                                     ARCH.n_kv_heads, ARCH.inter, ARCH.vocab)
        assert np.float32(a.rms_eps) == np.float32(ARCH.rms_eps) and np.float32(a.rope_theta) == np.float32(ARCH.rope_theta)
        cfg = oref.llama_config(r)
        assert (cfg["hidden"], cfg["n_layers"], cfg["n_heads"], cfg["n_kv_heads"], cfg["inter"], cfg["vocab"]) == (
            ARCH.hidden, ARCH.n_layers, ARCH.n_heads, ARCH.n_kv_heads, ARCH.inter, ARCH.vocab)
        assert np.float32(cfg["rope_theta"]) == np.float32(ARCH.rope_theta) and cfg["head_dim"] == 64
        assert g.meta_string("general.architecture") == "llama" and g.meta_string("llama.block_count") is None
        assert g.meta_int("general.file_type", -1) == 15 and g.meta_int("no.such.key", 77) == 77
        for kind, layer, t, rows, cols, blocks in tensors:
            name = synth.GGUF_NAMES[kind].format(layer)
            if tied and kind == synth.T_OUTPUT:
                with pytest.raises(ValueError, match="Tensor not found"):
                    g.tensor_raw(name)
                continue
            gt, dims, raw = g.tensor_raw(name)
            rt, rdims, rraw = r.tensor_raw(name)
            assert gt == rt == t and dims == rdims == ([cols] if rows == 1 and kind in (1, 3, 4) else [cols, rows])
            assert raw.tobytes() == rraw.tobytes() == np.asarray(blocks).tobytes()
            assert raw.size == GgufFile.raw_byte_count(t, rows * cols) == oref.raw_byte_count(t, rows * cols)
            assert (where["offsets"][name] - g.data_offset) % 32 == 0
    # the restated constructor walk hands back the same tensors, with the tied projection read from token_embd
    got = {(k, l): (t, rows, cols, raw.tobytes()) for k, l, t, rows, cols, raw in oref.model_tensors(r, ARCH.n_layers)}
    for kind, layer, t, rows, cols, blocks in tensors:
        want = np.asarray(blocks).tobytes()
        if tied and kind == synth.T_OUTPUT:
            want = np.asarray(tensors[0][5]).tobytes()
        assert got[(kind, layer)] == (t, rows, cols, want)


def test_cross_read_with_the_gguf_package(tmp_path):
    """A second opinion on the writer: the independent python `gguf` reader sees the same fields and bytes."""
    gg = pytest.importorskip("gguf")
    tensors = list(synth.random_model(ARCH, 6))
    p = tmp_path / "m.gguf"
    gguf_file.write_model(p, ARCH, tensors)
    rd = gg.GGUFReader(str(p))
    by_name = {t.name: t for t in rd.tensors}
    for kind, layer, t, rows, cols, blocks in tensors:
        e = by_name[synth.GGUF_NAMES[kind].format(layer)]
        assert int(e.tensor_type) == t and int(e.n_elements) == rows * cols
        assert np.asarray(e.data).view(np.uint8).reshape(-1).tobytes() == np.asarray(blocks).tobytes()
    f = rd.fields["llama.embedding_length"]
    assert int(f.parts[f.data[0]][0]) == ARCH.hidden
    f = rd.fields["llama.rope.freq_base"]
    assert np.float32(f.parts[f.data[0]][0]) == np.float32(ARCH.rope_theta)


def test_a_file_written_by_the_gguf_package_reads_the_same(tmp_path):
    gg = pytest.importorskip("gguf")
    p = tmp_path / "w.gguf"
    w = gg.GGUFWriter(str(p), "llama")
    w.add_uint32("llama.embedding_length", 512)
    w.add_uint32("llama.block_count", 3)
    w.add_uint32("llama.attention.head_count", 8)
    w.add_float32("llama.rope.freq_base", 500000.0)
    w.add_array("tokenizer.ggml.tokens", [f"t{i}" for i in range(40000)])
    rng = np.random.default_rng(0)
    blocks = synth.random_blocks(rng, synth.Q4_K, 8, 512)
    w.add_tensor("blk.0.attn_q.weight", blocks.reshape(8, 512 // 256 * 144), raw_dtype=gg.GGMLQuantizationType.Q4_K)
    vec = rng.standard_normal(512).astype(np.float32)
    w.add_tensor("output_norm.weight", vec)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    r = oref.GgufReader(p)
    with GgufFile(p) as g:
        a = g.arch()
        # head_count_kv defaults to head_count, feed_forward_length to hidden*11/4, the vocabulary is the tokenizer's count
        assert (a.hidden, a.n_layers, a.n_heads, a.n_kv_heads, a.inter, a.vocab) == (512, 3, 8, 8, 1408, 40000)
        assert g.meta_array_len("tokenizer.ggml.tokens") == 40000 and g.meta_array_len("llama.block_count") == -1
        t, dims, raw = g.tensor_raw("blk.0.attn_q.weight")
        assert (t, dims) == (12, [512, 8]) and raw.tobytes() == blocks.tobytes() == r.tensor_raw("blk.0.attn_q.weight")[2].tobytes()
        t, dims, raw = g.tensor_raw("output_norm.weight")
        assert (t, dims) == (0, [512]) and raw.tobytes() == vec.tobytes()
    c = oref.llama_config(r)
    assert (c["hidden"], c["n_layers"], c["n_heads"], c["n_kv_heads"], c["inter"], c["vocab"]) == (512, 3, 8, 8, 1408, 40000)


def test_metadata_of_every_value_type(tmp_path):
    """Types 0-12 (GgufReader.java:66-78); as in the reference, narrow unsigned integers come back sign-extended."""
    G = gguf_file
    meta = [("u8", G.MT_UINT8, 200), ("i8", G.MT_INT8, -5), ("u16", G.MT_UINT16, 40000), ("i16", G.MT_INT16, -300),
            ("u32", G.MT_UINT32, 123456), ("i32", G.MT_INT32, -7), ("f32", G.MT_FLOAT32, 2.5), ("b", G.MT_BOOL, 1),
            ("s", G.MT_STRING, "héllo"), ("arr", G.MT_ARRAY, (G.MT_STRING, ["a", "bc", ""])),
            ("nest", G.MT_ARRAY, (G.MT_ARRAY, [(G.MT_INT32, [1, 2]), (G.MT_INT32, [3])])),
            ("u64", G.MT_UINT64, 1 << 40), ("i64", G.MT_INT64, -(1 << 40)), ("f64", G.MT_FLOAT64, 1e-5),
            ("general.architecture", G.MT_STRING, "qwen2"), ("qwen2.block_count", G.MT_UINT64, 7),
            ("llama.embedding_length", G.MT_FLOAT32, 640.0)]
    p = tmp_path / "meta.gguf"
    G.write_gguf(p, meta, [("t", 0, [4], np.arange(4, dtype=np.float32))])
    r = oref.GgufReader(p)
    with GgufFile(p) as g:
        for key, want in [("u8", 200 - 256), ("i8", -5), ("u16", 40000 - 65536), ("i16", -300), ("u32", 123456), ("i32", -7),
                          ("u64", 1 << 40), ("i64", -(1 << 40)), ("f32", 2)]:
            assert g.meta_int(key, 99) == want == r.meta_int(key, 99), key
        assert g.meta_int("b", 99) == 99 and g.meta_int("s", 99) == 99  # a Boolean or a String is not a Number
        assert g.meta_float("f32", 0) == 2.5 and g.meta_float("f64", 0) == pytest.approx(1e-5) and g.meta_float("i8", 0) == -5.0
        assert g.meta_string("s") == "héllo" and g.meta_string("u8") is None
        assert g.meta_array_len("arr") == 3 and g.meta_array_len("nest") == 2
        a = g.arch()  # "<arch>." first, then "llama.", then the default; numbers of any type convert
        assert (a.n_layers, a.hidden, a.n_heads) == (7, 640, 32)
        assert g.tensor_raw("t")[2].view(np.float32).tolist() == [0.0, 1.0, 2.0, 3.0]
    c = oref.llama_config(r)
    assert (c["n_layers"], c["hidden"], c["arch"]) == (7, 640, "qwen2")


def test_damaged_and_foreign_files(tmp_path):
    good = tmp_path / "good.gguf"
    gguf_file.write_model(good, ARCH, synth.random_model(ARCH, 7))
    raw = good.read_bytes()

    def expect(data, exc, match):
        p = tmp_path / "bad.gguf"
        p.write_bytes(data)
        with pytest.raises(exc, match=match):
            GgufFile(p)

    expect(b"PK\x03\x04" + raw[4:], ValueError, "Not a GGUF file")            # a ZIP / llamafile start
    expect(raw[:4] + struct.pack("<i", 1) + raw[8:], _lib.JunoError, "Unsupported GGUF version: 1")
    expect(raw[:4] + struct.pack("<i", 4) + raw[8:], _lib.JunoError, "Unsupported GGUF version: 4")
    expect(raw[:10], ValueError, "shorter than a GGUF header")
    expect(raw[:200], ValueError, "past the end|damaged")                       # cut inside the metadata
    expect(raw[: len(raw) // 2], ValueError, "runs past the end of the file")   # cut inside the data section
    expect(raw[:8] + struct.pack("<Q", 1 << 60) + raw[16:], ValueError, "exceed the file")
    with pytest.raises(ValueError, match="cannot open"):
        GgufFile(tmp_path / "missing.gguf")
    with pytest.raises(_lib.JunoError, match="No byte-size formula"):
        GgufFile.raw_byte_count(99, 256)
    with pytest.raises(NotImplementedError):
        oref.raw_byte_count(99, 256)
    # a tensor of a type without a size formula can be listed, but its bytes cannot be asked for (tensorRaw :329-340)
    p = tmp_path / "odd.gguf"
    gguf_file.write_gguf(p, [], [("odd", 99, [256], np.zeros(16, np.uint8))])
    with GgufFile(p) as g:
        assert g.tensor_info("odd") == (99, [256])
        with pytest.raises(_lib.JunoError, match="No byte-size formula"):
            g.tensor_raw("odd")
        h = g.handle
    with pytest.raises(_lib.JunoError):  # closed handle
        _lib.check(_lib.load().juno_gguf_close(h), "juno_gguf_close")


def test_raw_byte_counts_of_every_type():
    for t, (e, b) in {0: (1, 4), 1: (1, 2), 30: (1, 2), 8: (32, 34), 2: (32, 18), 10: (256, 84), 11: (256, 110), 12: (256, 144),
                      13: (256, 176), 14: (256, 210)}.items():
        assert GgufFile.raw_byte_count(t, 4096 * 256) == 4096 * 256 // e * b == oref.raw_byte_count(t, 4096 * 256)
