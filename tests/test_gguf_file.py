"""GGUF container reader / writer: round trips, agreement with gguf-py in both directions, and the reference's error
cases (crates/inference-tensor/src/quantized/gguf_file.rs: magic / version :45-78, tensor bounds :93-126, block-size
divisibility :100-105, alignment :705-715)."""
import io
import struct

import numpy as np
import pytest

from oracle import kquants as kq

from inference_rs_b200 import gguf_file as gf
from inference_rs_b200.gguf_file import Content, GgufError, Value, ValueType


def packed(type_id, n, k, seed):
    rng = np.random.default_rng(seed)
    return kq.quantize(type_id, (rng.standard_normal((n, k)) * 0.02).astype(np.float32))


def sample_file():
    meta = [("general.architecture", Value.string("llama")), ("llama.block_count", Value.u32(2)),
            ("llama.rope.freq_base", Value.f32(5e5)), ("flag", Value(ValueType.BOOL, True)),
            ("small", Value(ValueType.I8, -3)), ("big", Value(ValueType.U64, 2 ** 40 + 5)), ("pi", Value(ValueType.F64, 3.25)),
            ("tokens", Value.array([Value.string(f"tok{i}") for i in range(5)])),
            ("scores", Value.array([Value.f32(i / 4) for i in range(7)])),
            ("nested", Value.array([Value.array([Value.u32(1), Value.u32(2)]), Value.array([Value.u32(3)])]))]
    tensors = [("blk.0.attn_q.weight", kq.Q4_K, (8, 512), packed(kq.Q4_K, 8, 512, 1)),
               ("blk.0.attn_v.weight", kq.Q6_K, (3, 256), packed(kq.Q6_K, 3, 256, 2)),   # 630 bytes: needs padding
               ("blk.0.ffn_down.weight", kq.Q8_0, (5, 96), packed(kq.Q8_0, 5, 96, 3)),
               ("blk.0.attn_norm.weight", 0, (512,), np.arange(512, dtype=np.float32).view(np.uint8))]
    buf = io.BytesIO()
    gf.write(buf, meta, tensors)
    return buf, meta, tensors


def test_round_trip_keeps_metadata_and_bytes():
    buf, meta, tensors = sample_file()
    c = Content.read(buf)
    assert c.version == 2 and c.tensor_data_offset % 32 == 0
    assert list(c.metadata) == [k for k, _ in meta]
    for k, v in meta:
        assert c.metadata[k].type == v.type and c.metadata[k].plain() == v.plain()
    assert c.metadata["nested"].plain() == [[1, 2], [3]]
    for name, dtype, shape, data in tensors:
        info, raw = c.tensor_bytes(buf, name)
        assert info.ggml_dtype == dtype and info.shape == tuple(shape) and info.offset % 32 == 0
        assert raw.tobytes() == (data.tobytes() if isinstance(data, np.ndarray) else data)


def test_files_written_by_gguf_py_are_read():
    gguf = pytest.importorskip("gguf")
    import tempfile, os
    q4 = packed(kq.Q4_K, 4, 256, 5)
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "m.gguf")
        w = gguf.GGUFWriter(path, "llama")
        w.add_uint32("llama.block_count", 7)
        w.add_string("general.name", "tiny")
        w.add_array("tokenizer.ggml.tokens", ["a", "b", "c"])
        w.add_tensor("w_q4", q4.reshape(4, -1), raw_dtype=gguf.GGMLQuantizationType.Q4_K)
        w.add_tensor("norm", np.ones(256, dtype=np.float32))
        w.write_header_to_file()
        w.write_kv_data_to_file()
        w.write_tensors_to_file()
        w.close()
        with open(path, "rb") as f:
            c = Content.read(f)
            assert c.version == 3
            assert c.metadata["llama.block_count"].plain() == 7 and c.metadata["general.name"].plain() == "tiny"
            assert c.metadata["tokenizer.ggml.tokens"].plain() == ["a", "b", "c"]
            info, raw = c.tensor_bytes(f, "w_q4")
            assert info.ggml_dtype == kq.Q4_K and info.shape == (4, 256) and raw.tobytes() == q4.tobytes()
            info, raw = c.tensor_bytes(f, "norm")
            assert info.shape == (256,) and (raw.view(np.float32) == 1).all()


def test_files_written_here_are_read_by_gguf_py():
    gguf = pytest.importorskip("gguf")
    import tempfile, os
    buf, meta, tensors = sample_file()
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "m.gguf")
        with open(path, "wb") as f:
            f.write(buf.getvalue())
        r = gguf.GGUFReader(path)
        by_name = {t.name: t for t in r.tensors}
        for name, dtype, shape, data in tensors:
            t = by_name[name]
            assert int(t.tensor_type) == dtype
            assert bytes(np.asarray(t.data).reshape(-1).view(np.uint8)) == (data.tobytes() if isinstance(data, np.ndarray) else data)
            assert [int(x) for x in t.shape] == list(reversed(shape))  # gguf-py reports dimensions innermost first
        assert int(r.fields["llama.block_count"].parts[-1][0]) == 2


def test_version_1_lengths_are_32_bit():
    # one metadata string and no tensors, lengths as u32
    b = struct.pack("<IIII", gf.GGUF_MAGIC, 1, 0, 1) + struct.pack("<I", 4) + b"name" + struct.pack("<I", 8) + struct.pack("<I", 5) + b"tin\x00\x00"
    c = Content.read(io.BytesIO(b))
    assert c.version == 1 and c.metadata["name"].plain() == "tin"  # trailing NULs dropped


def test_alignment_comes_from_the_metadata():
    buf = io.BytesIO()
    gf.write(buf, [("general.alignment", Value.u32(64))], [])
    c = Content.read(buf)
    assert c.tensor_data_offset % 64 == 0


def test_malformed_files_are_refused():
    with pytest.raises(GgufError, match="unknown magic"):
        Content.read(io.BytesIO(struct.pack("<IIQQ", 0x12345678, 2, 0, 0)))
    with pytest.raises(GgufError, match="unsupported magic/version"):
        Content.read(io.BytesIO(struct.pack("<IIQQ", gf.GGUF_MAGIC, 9, 0, 0)))
    with pytest.raises(GgufError, match="end of file"):
        Content.read(io.BytesIO(struct.pack("<IIQ", gf.GGUF_MAGIC, 2, 0)))
    buf, _, _ = sample_file()
    whole = buf.getvalue()
    cut = io.BytesIO(whole[:-700])  # the last tensors no longer fit
    c = Content.read(cut)
    with pytest.raises(GgufError, match="remaining in file"):
        c.tensor_bytes(cut, "blk.0.attn_norm.weight")
    with pytest.raises(GgufError, match="cannot find tensor info"):
        c.tensor_bytes(cut, "nope")
    with pytest.raises(GgufError, match="not divisible by the block size"):
        gf.TensorInfo(kq.Q4_K, (3, 100), 0).size_in_bytes
    with pytest.raises(GgufError, match="needs 144 bytes"):
        gf.write(io.BytesIO(), [], [("w", kq.Q4_K, (1, 256), b"\x00" * 10)])
    bad = io.BytesIO()
    gf.write(bad, [("general.alignment", Value.string("x"))], [])
    with pytest.raises(GgufError, match="alignment"):
        Content.read(bad)
