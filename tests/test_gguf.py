"""GGUF header / tensor directory / expert slicing (`joshua_b200.gguf`) against files written by the writer that
mirrors the reference's raw test writer (tests/common/mod.rs:1257-1304), and the guards of its reader
(src/gguf_ext.rs:33-59,316-480)."""
import io
import struct

import numpy as np
import pytest

from joshua_b200 import ggml_decode, gguf, synth


def tiny_file(tmp_path, version=2):
    rng = np.random.default_rng(0)
    E, inter, h = 4, 256, 512
    tensors = [
        ("token_embd.weight", (8, h), synth.Q4_K, synth.random_weight(synth.Q4_K, 8, h, 1)),
        ("blk.0.attn_norm.weight", (h,), 0, rng.standard_normal(h).astype(np.float32).tobytes()),
        ("blk.0.ffn_gate_inp.weight", (E, h), 1, rng.standard_normal((E, h)).astype(np.float16).tobytes()),
        ("blk.0.ffn_gate_exps.weight", (E, inter, h), synth.IQ2_XXS, synth.random_weight(synth.IQ2_XXS, E * inter, h, 2)),
        ("blk.0.ffn_down_exps.weight", (E, h, inter), synth.MXFP4, synth.random_weight(synth.MXFP4, E * h, inter, 3)),
        ("blk.0.ffn_up_exps.weight", (E, inter, h), synth.IQ2_XXS, synth.random_weight(synth.IQ2_XXS, E * inter, h, 4)),
        ("blk.0.ffn_gate_tid2eid.weight", (6, 2), 26, np.arange(12, dtype=np.int32).tobytes()),
        ("output.weight", (8, h), synth.Q6_K, synth.random_weight(synth.Q6_K, 8, h, 5)),
    ]
    meta = {"general.architecture": "qwen3moe", "qwen3moe.block_count": 1, "qwen3moe.expert_count": E,
            "qwen3moe.attention.layer_norm_rms_epsilon": 1e-6, "qwen3moe.attention.norm_topk_prob": True,
            "tokenizer.ggml.tokens": ["a", "bc", ""], "general.alignment": 32}
    path = tmp_path / f"tiny_v{version}.gguf"
    gguf.write_gguf(path, meta, tensors, version=version)
    return path, meta, tensors


@pytest.mark.parametrize("version", [2, 3])
def test_header_round_trip(tmp_path, version):
    path, meta, tensors = tiny_file(tmp_path, version)
    with gguf.GgufFile(path) as f:
        h = f.header
        assert h.version == version and h.architecture() == "qwen3moe"
        assert h.metadata["qwen3moe.expert_count"] == 4 and h.metadata["qwen3moe.attention.norm_topk_prob"] is True
        assert abs(h.metadata["qwen3moe.attention.layer_norm_rms_epsilon"] - 1e-6) < 1e-12
        assert h.metadata["tokenizer.ggml.tokens"] == ["a", "bc", ""]
        assert h.tensor_data_offset % 32 == 0
        for name, dims, dtype, data in tensors:
            t = h.tensors[name]
            assert t.dims == tuple(dims) and t.dtype == dtype and t.offset % 32 == 0     # dims back in row-major
            assert bytes(f.tensor_bytes(name)) == bytes(data)
        assert h.unsupported_by_candle() == [16, 26, 39]
        # the three expert tensors of layer 0 are adjacent: one merged range up to the next tensor
        (begin, end), = h.layer_expert_ranges(1)
        assert begin == h.tensor_data_offset + h.tensors["blk.0.ffn_gate_exps.weight"].offset
        assert end == h.tensor_data_offset + h.tensors["blk.0.ffn_gate_tid2eid.weight"].offset
        assert h.layer_expert_ranges(2)[1] is None


def test_expert_slicing_is_pointer_arithmetic(tmp_path):
    path, _, tensors = tiny_file(tmp_path)
    raw = {name: np.frombuffer(bytes(data), np.uint8) for name, _, _, data in tensors}
    with gguf.GgufFile(path) as f:
        E, rows, cols, per = f.expert_layout("blk.0.ffn_gate_exps.weight")
        assert (E, rows, cols) == (4, 256, 512) and per == synth.tensor_bytes(synth.IQ2_XXS, 256, 512)
        for e in range(E):
            assert np.array_equal(f.expert_bytes("blk.0.ffn_gate_exps.weight", e, 1),
                                  raw["blk.0.ffn_gate_exps.weight"][e * per:(e + 1) * per])
        # a rank's share of an expert-parallel split: experts [2, 4) of the MXFP4 bank
        per_d = synth.tensor_bytes(synth.MXFP4, 512, 256)
        assert np.array_equal(f.expert_bytes("blk.0.ffn_down_exps.weight", 2, 2), raw["blk.0.ffn_down_exps.weight"][2 * per_d:])
        with pytest.raises(gguf.GgufError, match="outside the bank"):
            f.expert_bytes("blk.0.ffn_down_exps.weight", 3, 2)
        with pytest.raises(gguf.GgufError, match="expected \\[n_expert, out, in\\]"):
            f.expert_layout("token_embd.weight")
        with pytest.raises(gguf.GgufError, match="not found"):
            f.tensor_bytes("nope")


def test_small_tensors_decode_on_the_host(tmp_path):
    path, _, tensors = tiny_file(tmp_path)
    by = {name: (dims, dtype, data) for name, dims, dtype, data in tensors}
    with gguf.GgufFile(path) as f:
        norm = f.float_tensor("blk.0.attn_norm.weight")
        assert norm.dtype == np.float32 and norm.tobytes() == bytes(by["blk.0.attn_norm.weight"][2])
        router = f.float_tensor("blk.0.ffn_gate_inp.weight")
        want = np.frombuffer(by["blk.0.ffn_gate_inp.weight"][2], np.float16).astype(np.float32).reshape(4, 512)
        assert router.shape == (4, 512) and np.array_equal(router, want)
        out = f.float_tensor("output.weight")          # a quantized tensor through the numpy decoder
        assert np.array_equal(out.reshape(-1), ggml_decode.dequantize(synth.Q6_K, by["output.weight"][2]))
        assert np.array_equal(f.int_tensor("blk.0.ffn_gate_tid2eid.weight"), np.arange(12, dtype=np.int32).reshape(6, 2))
        with pytest.raises(gguf.GgufError, match="expected I32"):
            f.int_tensor("blk.0.attn_norm.weight")


def test_type_sizes():
    assert gguf.type_size_bytes(12, 4096 * 4096) == 9437184 and gguf.type_size_bytes(16, 256) == 66
    assert gguf.type_size_bytes(39, 32) == 17 and gguf.type_size_bytes(26, 5) == 20 and gguf.type_size_bytes(30, 3) == 6
    assert gguf.type_size_bytes(12, 100) is None and gguf.type_size_bytes(99, 256) is None


def header(version=3, tensors=0, kvs=0, magic=gguf.MAGIC):
    n = struct.pack("<II", tensors, kvs) if version == 1 else struct.pack("<QQ", tensors, kvs)
    return struct.pack("<II", magic, version) + n


def test_version_1_lengths_are_32_bit():
    key = b"general.architecture"
    body = header(1, 0, 1) + struct.pack("<I", len(key)) + key + struct.pack("<I", 8) + struct.pack("<I", 5) + b"llama"
    h = gguf.read_header(io.BytesIO(body))
    assert h.version == 1 and h.architecture() == "llama" and h.tensor_data_offset % 32 == 0


def test_hostile_headers_are_rejected_before_any_large_allocation():
    with pytest.raises(gguf.GgufError, match="bad magic"):
        gguf.read_header(io.BytesIO(header(magic=0x12345678)))
    with pytest.raises(gguf.GgufError, match="unsupported GGUF version 4"):
        gguf.read_header(io.BytesIO(header(version=4)))
    with pytest.raises(gguf.GgufError, match="implausible"):
        gguf.read_header(io.BytesIO(header(tensors=(1 << 24) + 1)))
    key = struct.pack("<Q", 1 << 40)                    # a key that claims a terabyte
    with pytest.raises(gguf.GgufError, match="exceeds max"):
        gguf.read_header(io.BytesIO(header(kvs=1) + key))
    key = struct.pack("<Q", 1000) + b"abc"              # longer than the file
    with pytest.raises(gguf.GgufError, match="bytes remaining"):
        gguf.read_header(io.BytesIO(header(kvs=1) + key))
    k = struct.pack("<Q", 1) + b"k"
    with pytest.raises(gguf.GgufError, match="array of"):
        gguf.read_header(io.BytesIO(header(kvs=1) + k + struct.pack("<IIQ", 9, 4, (1 << 24) + 1)))
    with pytest.raises(gguf.GgufError, match="unknown metadata value type 13"):
        gguf.read_header(io.BytesIO(header(kvs=1) + k + struct.pack("<I", 13)))
    nested = k + struct.pack("<I", 9) + struct.pack("<IQ", 9, 1) * 70 + struct.pack("<IQ", 4, 0)
    with pytest.raises(gguf.GgufError, match="nesting depth"):
        gguf.read_header(io.BytesIO(header(kvs=1) + nested))
    name = struct.pack("<Q", 1) + b"t"
    with pytest.raises(gguf.GgufError, match="claims 9 dimensions"):
        gguf.read_header(io.BytesIO(header(tensors=1) + name + struct.pack("<I", 9)))
    with pytest.raises(gguf.GgufError, match="invalid general.alignment"):
        ka = b"general.alignment"
        gguf.read_header(io.BytesIO(header(kvs=1) + struct.pack("<Q", len(ka)) + ka + struct.pack("<II", 4, 24)))
    with pytest.raises(gguf.GgufError, match="unexpected end"):
        gguf.read_header(io.BytesIO(header(tensors=1) + name))


def test_strings_are_read_leniently():
    key = b"k\0\0"                                       # NUL-terminated keys and invalid UTF-8 load, as in the reference
    val = b"caf\xff"
    body = header(kvs=1) + struct.pack("<Q", len(key)) + key + struct.pack("<I", 8) + struct.pack("<Q", len(val)) + val
    h = gguf.read_header(io.BytesIO(body))
    assert list(h.metadata) == ["k"] and h.metadata["k"].startswith("caf")


def test_a_truncated_file_is_reported(tmp_path):
    path, _, _ = tiny_file(tmp_path)
    data = path.read_bytes()
    cut = tmp_path / "cut.gguf"
    cut.write_bytes(data[: len(data) - 4096])
    with gguf.GgufFile(cut) as f:
        with pytest.raises(gguf.GgufError, match="outside the file"):
            f.tensor_bytes("output.weight")
