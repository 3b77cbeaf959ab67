"""GGUF header, tensor directory and expert slicing: what feeds real model files to the device kernels.

Host-side mirror of the reference's tolerant header reader (`read_header`, `GgufHeader`, `type_size_bytes`,
`layer_expert_ranges`; src/gguf_ext.rs:120-512) and of its per-expert slicing of `[n_expert, out, in]` tensors
(`split_experts`, src/quantized_qwen3_moe.rs:556-651, src/quantized_deepseek4.rs:2193-2379).  Only the header
is parsed; tensor bytes are borrowed from a read-only memory mapping of the file (the reference's
`borrowed_range*`, src/mmap_tensor.rs:551-655) and go to the device unmodified through `jq_weight_upload`.

What the reference keeps and this keeps too:
  * every tensor's dtype stays the raw GGUF id (16 = IQ2_XXS, 39 = MXFP4, 26 = I32 are not in candle's table);
  * dims are reversed to row-major (GGUF stores the fastest-varying first, src/gguf_ext.rs:441-443);
  * tensor data starts at the header end rounded up to `general.alignment` (default 32);
  * the guards against hostile headers: counts <= 2^24, strings <= 16 MiB and never longer than the file,
    arrays <= 2^24 elements, nesting <= 64 (src/gguf_ext.rs:33-59,316-390).
The dense / expert split of a file is the replicate / shard split of expert parallelism: dense tensors go to
every rank, of an expert bank a rank uploads only its contiguous run of experts.
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass
from pathlib import Path

import numpy as np

MAGIC = 0x46554747  # "GGUF", little endian
DEFAULT_ALIGNMENT = 32
MAX_COUNT = 1 << 24
MAX_STRING_LENGTH = 1 << 24
MAX_ARRAY_ELEMENTS = 1 << 24
MAX_VALUE_DEPTH = 64

# GGUF type id -> (elements per block, bytes per block)   (src/gguf_ext.rs:483-512)
TYPE_SIZES = {
    0: (1, 4), 1: (1, 2), 30: (1, 2),
    2: (32, 18), 3: (32, 20), 6: (32, 22), 7: (32, 24), 8: (32, 34), 9: (32, 36),
    10: (256, 84), 11: (256, 110), 12: (256, 144), 13: (256, 176), 14: (256, 210), 15: (256, 292),
    26: (1, 4), 16: (256, 66), 39: (32, 17),
}
TYPE_NAMES = {0: "f32", 1: "f16", 30: "bf16", 2: "q4_0", 3: "q4_1", 6: "q5_0", 7: "q5_1", 8: "q8_0", 9: "q8_1",
              10: "q2_k", 11: "q3_k", 12: "q4_k", 13: "q5_k", 14: "q6_k", 15: "q8_k", 26: "i32", 16: "iq2_xxs",
              39: "mxfp4"}
CANDLE_TYPES = {0, 1, 2, 3, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15, 30}   # src/gguf_ext.rs:64-66


class GgufError(ValueError):
    """Malformed or unsupported file (the reference's `JoshuaError::ModelLoad("GGUF header: ...")`)."""


def type_size_bytes(dtype: int, elems: int):
    """Bytes of a tensor of `elems` elements of type `dtype`; None for an unknown type or a partial block."""
    if dtype not in TYPE_SIZES:
        return None
    blck, nbytes = TYPE_SIZES[dtype]
    if elems % blck:
        return None
    return elems // blck * nbytes


@dataclass
class RawTensorInfo:
    dtype: int          # raw GGUF type id
    dims: tuple         # row-major (reversed from the file's order)
    offset: int         # bytes from tensor_data_offset

    @property
    def elem_count(self) -> int:
        n = 1
        for d in self.dims:
            n *= d
        return n


class GgufHeader:
    def __init__(self, version, metadata, tensors, tensor_data_offset):
        self.version, self.metadata, self.tensors, self.tensor_data_offset = version, metadata, tensors, tensor_data_offset

    def architecture(self):
        v = self.metadata.get("general.architecture")
        return v if isinstance(v, str) else None

    def layer_expert_ranges(self, n_layer: int):
        """Per layer the merged absolute byte range [begin, end) of its routed-expert tensors, or None
        (src/gguf_ext.rs:164-207): a tensor's size is the distance to the next tensor in file order."""
        starts = sorted(t.offset for t in self.tensors.values())
        nxt = {o: (starts[i + 1] if i + 1 < len(starts) else None) for i, o in enumerate(starts)}
        out = []
        for i in range(n_layer):
            begin, end = None, 0
            for nm in ("ffn_gate_exps", "ffn_down_exps", "ffn_up_exps"):
                t = self.tensors.get(f"blk.{i}.{nm}.weight")
                if t is None:
                    continue
                begin = t.offset if begin is None else min(begin, t.offset)
                e = nxt.get(t.offset)
                end = max(end, (1 << 64) - 1 if e is None else e)
            out.append(None if begin is None or end <= begin else
                       (self.tensor_data_offset + begin, self.tensor_data_offset + end))
        return out

    def unsupported_by_candle(self):
        return sorted({t.dtype for t in self.tensors.values() if t.dtype not in CANDLE_TYPES})


class _Reader:
    def __init__(self, f):
        self.f, self.version = f, 0
        f.seek(0, 2)
        self.end = f.tell()
        f.seek(0)

    def take(self, n: int) -> bytes:
        b = self.f.read(n)
        if len(b) != n:
            raise GgufError("GGUF header: unexpected end of file")
        return b

    def u32(self) -> int:
        return struct.unpack("<I", self.take(4))[0]

    def u64(self) -> int:
        return struct.unpack("<Q", self.take(8))[0]

    def length(self) -> int:
        return self.u32() if self.version == 1 else self.u64()   # v1 wrote 32-bit lengths

    def string(self) -> str:
        n = self.length()
        if n > MAX_STRING_LENGTH:
            raise GgufError(f"GGUF header: string of {n} bytes exceeds max {MAX_STRING_LENGTH}")
        if n > self.end - self.f.tell():
            raise GgufError(f"GGUF header: string of {n} bytes exceeds the {self.end - self.f.tell()} bytes remaining in the stream")
        return self.take(n).rstrip(b"\0").decode("utf-8", errors="replace")   # lenient, like the reference

    _SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 10: "<Q", 11: "<q", 12: "<d"}

    def value(self, ty: int, depth: int = 0):
        if depth > MAX_VALUE_DEPTH:
            raise GgufError(f"GGUF header: value nesting depth exceeds max {MAX_VALUE_DEPTH}")
        if ty in self._SCALAR:
            fmt = self._SCALAR[ty]
            return struct.unpack(fmt, self.take(struct.calcsize(fmt)))[0]
        if ty == 7:
            return self.take(1)[0] != 0
        if ty == 8:
            return self.string()
        if ty == 9:
            elem_ty = self.u32()
            n = self.length()
            if n > MAX_ARRAY_ELEMENTS:
                raise GgufError(f"GGUF header: array of {n} elements exceeds max {MAX_ARRAY_ELEMENTS}")
            return [self.value(elem_ty, depth + 1) for _ in range(n)]
        raise GgufError(f"GGUF header: unknown metadata value type {ty}")


def read_header(f) -> GgufHeader:
    """Parses a GGUF v1-v3 header from a seekable binary stream (src/gguf_ext.rs:400-480)."""
    rd = _Reader(f)
    if struct.unpack("<I", rd.take(4))[0] != MAGIC:
        raise GgufError("GGUF header: not a GGUF file (bad magic)")
    version = rd.u32()
    if not 1 <= version <= 3:
        raise GgufError(f"GGUF header: unsupported GGUF version {version}")
    rd.version = version
    tensor_count, kv_count = rd.length(), rd.length()
    if tensor_count > MAX_COUNT or kv_count > MAX_COUNT:
        raise GgufError("GGUF header: implausible tensor/metadata count")
    metadata = {}
    for _ in range(kv_count):
        key = rd.string()
        metadata[key] = rd.value(rd.u32())
    tensors = {}
    for _ in range(tensor_count):
        name = rd.string()
        n_dims = rd.u32()
        if n_dims > 8:
            raise GgufError(f"GGUF header: tensor `{name}` claims {n_dims} dimensions")
        dims = tuple(reversed([rd.length() for _ in range(n_dims)]))
        dtype = rd.u32()
        tensors[name] = RawTensorInfo(dtype, dims, rd.u64())
    alignment = metadata.get("general.alignment", DEFAULT_ALIGNMENT)
    if isinstance(alignment, bool) or not isinstance(alignment, int) or alignment < 0:
        alignment = DEFAULT_ALIGNMENT
    if alignment == 0 or alignment & (alignment - 1):
        raise GgufError(f"GGUF header: invalid general.alignment {alignment}")
    pos = f.tell()
    return GgufHeader(version, metadata, tensors, (pos + alignment - 1) // alignment * alignment)


class GgufFile:
    """A memory-mapped GGUF file: header + zero-copy views of tensor bytes."""

    def __init__(self, path):
        self.path = Path(path)
        self._f = open(self.path, "rb")
        self.header = read_header(self._f)
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self.bytes = np.frombuffer(self._map, dtype=np.uint8)

    def close(self):
        self.bytes = None
        try:
            self._map.close()
        except BufferError:      # views handed out are still alive; the mapping goes when they do
            pass
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def info(self, name: str) -> RawTensorInfo:
        try:
            return self.header.tensors[name]
        except KeyError:
            raise GgufError(f"tensor `{name}` not found in {self.path.name}") from None

    def tensor_bytes(self, name: str) -> np.ndarray:
        """The tensor's raw bytes as a view of the mapping, bounds-checked against the file like the reference's
        borrowed ranges (src/mmap_tensor.rs:551-600)."""
        t = self.info(name)
        size = type_size_bytes(t.dtype, t.elem_count)
        if size is None:
            raise GgufError(f"tensor `{name}`: {t.elem_count} elements of type {t.dtype} is not a whole number of blocks")
        begin = self.header.tensor_data_offset + t.offset
        if begin + size > self.bytes.size:
            raise GgufError(f"tensor `{name}` [{begin}, {begin + size}) lies outside the file ({self.bytes.size} bytes)")
        return self.bytes[begin:begin + size]

    def expert_layout(self, name: str):
        """(n_expert, rows, cols, bytes per expert) of a [n_expert, out, in] bank: experts are contiguous."""
        t = self.info(name)
        if len(t.dims) != 3:
            raise GgufError(f"tensor `{name}` has dims {t.dims}, expected [n_expert, out, in]")
        E, rows, cols = t.dims
        per = type_size_bytes(t.dtype, rows * cols)
        if per is None:
            raise GgufError(f"tensor `{name}`: one expert is not a whole number of blocks")
        return E, rows, cols, per

    def expert_bytes(self, name: str, first: int, count: int) -> np.ndarray:
        """Bytes of experts [first, first + count) of a bank: expert e = [base + e * per, + per)."""
        E, _, _, per = self.expert_layout(name)
        if first < 0 or count < 0 or first + count > E:
            raise GgufError(f"tensor `{name}`: experts [{first}, {first + count}) outside the bank's {E}")
        return self.tensor_bytes(name)[first * per:(first + count) * per]

    def float_tensor(self, name: str) -> np.ndarray:
        """A small tensor as float32 (norm weights, routers, biases): F32 / F16 / BF16 directly, block types
        through the CPU-side numpy decoders of `joshua_b200.ggml_decode` (routers are dequantised once at load,
        src/quantized_qwen3_moe.rs:654-657)."""
        t = self.info(name)
        raw = self.tensor_bytes(name)
        if t.dtype == 0:
            out = raw.view(np.float32).copy()
        elif t.dtype == 1:
            out = raw.view(np.float16).astype(np.float32)
        elif t.dtype == 30:
            out = (raw.view(np.uint16).astype(np.uint32) << 16).view(np.float32)
        else:
            from . import ggml_decode

            out = ggml_decode.dequantize(t.dtype, raw)
        return out.reshape(t.dims)

    def int_tensor(self, name: str) -> np.ndarray:
        t = self.info(name)
        if t.dtype != 26:
            raise GgufError(f"tensor `{name}` has type {t.dtype}, expected I32 (26)")
        return self.tensor_bytes(name).view(np.int32).reshape(t.dims).copy()

    # ── upload ──────────────────────────────────────────────────────────
    def upload(self, name: str, ctx=None):
        """A dense tensor -> `QTensor` on the device (replicated on every rank)."""
        from .qtensor import QTensor

        t = self.info(name)
        return QTensor.from_bytes(t.dtype, self.tensor_bytes(name), ctx)

    def upload_experts(self, name: str, rank: int = 0, world: int = 1, ctx=None):
        """This rank's contiguous run of experts of a bank (expert e lives on rank e // (E / world)) ->
        (`QTensor`, first expert, experts held)."""
        from .qtensor import QTensor

        E = self.expert_layout(name)[0]
        if E % world:
            raise GgufError(f"tensor `{name}`: {E} experts do not split evenly over {world} ranks")
        per = E // world
        return QTensor.from_bytes(self.info(name).dtype, self.expert_bytes(name, rank * per, per), ctx), rank * per, per


# ── writer (test fixtures and synthetic model files) ────────────────────────
_VALUE_TYPE = {bool: 7, str: 8, float: 6}


def _write_value(out: bytearray, v, ty=None):
    if ty is None:
        ty = value_type_id(v)
    if ty == 8:
        b = v.encode()
        out += struct.pack("<Q", len(b)) + b
    elif ty == 7:
        out += struct.pack("<B", 1 if v else 0)
    elif ty == 9:
        et = value_type_id(v[0]) if v else 4
        out += struct.pack("<IQ", et, len(v))
        for e in v:
            _write_value(out, e, et)
    else:
        out += struct.pack(_Reader._SCALAR[ty], v)


def value_type_id(v) -> int:
    if isinstance(v, bool):
        return 7
    if isinstance(v, str):
        return 8
    if isinstance(v, float):
        return 6
    if isinstance(v, (list, tuple)):
        return 9
    if isinstance(v, int):
        return 4 if 0 <= v < (1 << 32) else (5 if -(1 << 31) <= v < 0 else 10)
    raise TypeError(f"no GGUF value type for {type(v).__name__}")


def write_gguf(path, metadata: dict, tensors, version: int = 2, alignment: int = 32) -> None:
    """Writes a GGUF file: `tensors` = [(name, row-major dims, raw type id, bytes)].  Same layout as the
    reference's raw test writer (tests/common/mod.rs:1257-1304): dims stored reversed, tensor data aligned,
    offsets relative to the aligned start of the data section."""
    out = bytearray()
    out += struct.pack("<II", MAGIC, version)
    out += struct.pack("<QQ", len(tensors), len(metadata))
    for k, v in metadata.items():
        kb = k.encode()
        out += struct.pack("<Q", len(kb)) + kb + struct.pack("<I", value_type_id(v))
        _write_value(out, v)
    offset, offsets = 0, []
    for name, dims, dtype, data in tensors:
        nb = name.encode()
        out += struct.pack("<Q", len(nb)) + nb + struct.pack("<I", len(dims))
        for d in reversed(dims):
            out += struct.pack("<Q", d)
        out += struct.pack("<IQ", dtype, offset)
        offsets.append(offset)
        size = len(data)
        offset += (size + alignment - 1) // alignment * alignment
    out += bytes(-len(out) % alignment)
    start = len(out)
    for (name, dims, dtype, data), off in zip(tensors, offsets):
        assert len(out) - start == off
        out += bytes(data)
        out += bytes(-len(out) % alignment)
    Path(path).write_bytes(bytes(out))
