"""GGUF container: file <-> packed blocks, unchanged bytes.

Mirror of the reference's reader / writer for the part this path needs
(crates/inference-tensor/src/quantized/gguf_file.rs: `VersionedMagic` :57-84, `TensorInfo` :86-127, `Content` :136-143
and `Content::read` :775-822, `ValueType` / `Value` :169-216, `write` :886-905): little-endian only, versions 1-3 on
read (32-bit lengths in version 1), version 2 on write, dimensions stored innermost first, tensor data aligned to
`general.alignment` (32 by default), strings with trailing NULs dropped and invalid UTF-8 replaced. The packed bytes of
a tensor are neither reordered nor converted: a Q8_0 / Q4_K / Q6_K tensor becomes a `QTensor` holding exactly the
file's bytes (plus the device padding every upload appends), other types come back as raw bytes or, for F32 / F16 /
BF16, as a dense torch tensor.
"""
from __future__ import annotations

import dataclasses
import enum
import io
import os
import struct
from typing import Any, BinaryIO

import numpy as np

from .dtypes import GgmlDType

GGUF_MAGIC = 0x46554747  # "GGUF" read as a little-endian u32
DEFAULT_ALIGNMENT = 32
MAX_STRING_LENGTH = 1 << 30
MAX_ARRAY_ELEMENTS = 1 << 32

# ggml type id -> (values per block, bytes per block); the dense types have block size 1
TYPE_LAYOUT = {0: (1, 4), 1: (1, 2), 30: (1, 2), 8: (32, 34), 12: (256, 144), 14: (256, 210)}
DENSE_NUMPY = {0: np.float32, 1: np.float16}


class GgufError(ValueError):
    """Malformed or unsupported file (the reference's `Error::Msg` for this module)."""


class ValueType(enum.IntEnum):
    U8 = 0
    I8 = 1
    U16 = 2
    I16 = 3
    U32 = 4
    I32 = 5
    F32 = 6
    BOOL = 7
    STRING = 8
    ARRAY = 9
    U64 = 10
    I64 = 11
    F64 = 12


_SCALAR_FMT = {ValueType.U8: "<B", ValueType.I8: "<b", ValueType.U16: "<H", ValueType.I16: "<h", ValueType.U32: "<I",
               ValueType.I32: "<i", ValueType.F32: "<f", ValueType.U64: "<Q", ValueType.I64: "<q", ValueType.F64: "<d"}


_SCALAR_NUMPY = {ValueType.U8: "u1", ValueType.I8: "i1", ValueType.U16: "<u2", ValueType.I16: "<i2", ValueType.U32: "<u4",
                 ValueType.I32: "<i4", ValueType.F32: "<f4", ValueType.U64: "<u8", ValueType.I64: "<i8", ValueType.F64: "<f8"}


@dataclasses.dataclass(frozen=True)
class Value:
    """A metadata value with its on-disk type (an `Array` holds a list of `Value` of one type)."""
    type: ValueType
    value: Any

    @staticmethod
    def string(s: str) -> "Value":
        return Value(ValueType.STRING, s)

    @staticmethod
    def u32(v: int) -> "Value":
        return Value(ValueType.U32, int(v))

    @staticmethod
    def f32(v: float) -> "Value":
        return Value(ValueType.F32, float(v))

    @staticmethod
    def array(items: list["Value"]) -> "Value":
        if items and any(i.type != items[0].type for i in items):
            raise GgufError("gguf: arrays hold values of one type")
        return Value(ValueType.ARRAY, list(items))

    def plain(self):
        """The Python value without type tags (arrays as lists)."""
        return [v.plain() for v in self.value] if self.type == ValueType.ARRAY else self.value


@dataclasses.dataclass(frozen=True)
class TensorInfo:
    ggml_dtype: int          # ggml type id (8 = Q8_0, 12 = Q4_K, 14 = Q6_K, 0 = F32, 1 = F16, 30 = BF16)
    shape: tuple[int, ...]   # outermost first, as the model sees it
    offset: int              # from the start of the tensor data section

    @property
    def elem_count(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n

    @property
    def size_in_bytes(self) -> int:
        if self.ggml_dtype not in TYPE_LAYOUT:
            raise GgufError(f"gguf: ggml type {self.ggml_dtype} is not handled by this library")
        block, nbytes = TYPE_LAYOUT[self.ggml_dtype]
        if self.elem_count % block:
            raise GgufError(f"the number of elements {self.elem_count} is not divisible by the block size {block}")
        return self.elem_count // block * nbytes


class _Reader:
    def __init__(self, f: BinaryIO, version: int, file_size: int):
        self.f, self.version, self.file_size = f, version, file_size

    def take(self, n: int) -> bytes:
        b = self.f.read(n)
        if len(b) != n:
            raise GgufError("gguf: unexpected end of file")
        return b

    def scalar(self, fmt: str):
        return struct.unpack(fmt, self.take(struct.calcsize(fmt)))[0]

    def length(self) -> int:
        return self.scalar("<I") if self.version == 1 else self.scalar("<Q")

    def string(self) -> str:
        n = self.length()
        if n > MAX_STRING_LENGTH:
            raise GgufError(f"gguf: string length {n} exceeds max {MAX_STRING_LENGTH}")
        if n > self.file_size - self.f.tell():
            raise GgufError(f"gguf: string length {n} exceeds remaining file bytes {self.file_size - self.f.tell()}")
        return self.take(n).rstrip(b"\x00").decode("utf-8", errors="replace")

    def value(self, vt: ValueType) -> Value:
        if vt in _SCALAR_FMT:
            return Value(vt, self.scalar(_SCALAR_FMT[vt]))
        if vt == ValueType.BOOL:
            b = self.scalar("<B")
            if b > 1:
                raise GgufError(f"gguf: unexpected bool value {b}")
            return Value(vt, bool(b))
        if vt == ValueType.STRING:
            return Value(vt, self.string())
        if vt == ValueType.ARRAY:
            inner = self.value_type()
            n = self.length()
            if n > MAX_ARRAY_ELEMENTS:
                raise GgufError(f"gguf: array length {n} exceeds max {MAX_ARRAY_ELEMENTS}")
            if inner in _SCALAR_FMT:  # fixed-size elements: one bulk read
                dt = np.dtype(_SCALAR_NUMPY[inner])
                if n * dt.itemsize > self.file_size - self.f.tell():
                    raise GgufError("gguf: array exceeds remaining file bytes")
                data = np.frombuffer(self.take(n * dt.itemsize), dtype=dt)
                conv = float if inner in (ValueType.F32, ValueType.F64) else int
                return Value(vt, [Value(inner, conv(x)) for x in data])
            return Value(vt, [self.value(inner) for _ in range(n)])
        raise GgufError(f"gguf: unknown value type {vt}")

    def value_type(self) -> ValueType:
        raw = self.scalar("<I")
        try:
            return ValueType(raw)
        except ValueError:
            raise GgufError(f"gguf: unrecognized value-type {raw:#010x}") from None


@dataclasses.dataclass
class Content:
    """Header of a GGUF file: metadata, tensor directory and where the tensor data starts."""
    version: int
    metadata: dict[str, Value]
    tensor_infos: dict[str, TensorInfo]
    tensor_data_offset: int

    @classmethod
    def read(cls, f: BinaryIO) -> "Content":
        f.seek(0, os.SEEK_END)
        file_size = f.tell()
        f.seek(0)
        head = f.read(8)
        if len(head) != 8:
            raise GgufError("gguf: unexpected end of file")
        magic, version = struct.unpack("<II", head)
        if magic not in (GGUF_MAGIC, 0x47475546):
            raise GgufError(f"unknown magic 0x{magic:08x}")
        if magic != GGUF_MAGIC or version not in (1, 2, 3):
            raise GgufError(f"gguf: unsupported magic/version Gguf/{version}")
        r = _Reader(f, version, file_size)
        tensor_count, kv_count = r.length(), r.length()
        if tensor_count > MAX_ARRAY_ELEMENTS or kv_count > MAX_ARRAY_ELEMENTS:
            raise GgufError(f"gguf: tensor_count {tensor_count} / metadata count {kv_count} exceeds max {MAX_ARRAY_ELEMENTS}")
        metadata: dict[str, Value] = {}
        for _ in range(kv_count):
            key = r.string()
            metadata[key] = r.value(r.value_type())
        infos: dict[str, TensorInfo] = {}
        for _ in range(tensor_count):
            name = r.string()
            n_dims = r.scalar("<I")
            if n_dims > 8:
                raise GgufError(f"gguf: tensor {name} has {n_dims} dimensions")
            dims = [r.scalar("<I") if version == 1 else r.scalar("<Q") for _ in range(n_dims)]
            dtype = r.scalar("<I")
            offset = r.scalar("<Q")
            infos[name] = TensorInfo(dtype, tuple(reversed(dims)), offset)  # stored innermost first
        alignment = DEFAULT_ALIGNMENT
        if "general.alignment" in metadata:
            a = metadata["general.alignment"]
            if a.type not in (ValueType.U8, ValueType.U16, ValueType.U32, ValueType.I8, ValueType.I16, ValueType.I32) or a.value <= 0:
                raise GgufError(f"gguf: general.alignment has unexpected value {a}")
            alignment = int(a.value)
        pos = f.tell()
        return cls(version, metadata, infos, -(-pos // alignment) * alignment)

    def tensor_bytes(self, f: BinaryIO, name: str) -> tuple[TensorInfo, np.ndarray]:
        """The tensor's bytes exactly as the file holds them."""
        if name not in self.tensor_infos:
            raise GgufError(f"cannot find tensor info for {name}")
        info = self.tensor_infos[name]
        size = info.size_in_bytes
        start = self.tensor_data_offset + info.offset
        f.seek(0, os.SEEK_END)
        remaining = max(0, f.tell() - start)
        if size > remaining:
            raise GgufError(f"tensor needs {size} bytes at offset {start}, only {remaining} remaining in file")
        f.seek(start)
        return info, np.frombuffer(f.read(size), dtype=np.uint8)

    def tensor(self, f: BinaryIO, name: str, device="cuda"):
        """`Content::tensor` (gguf_file.rs:801-821): a `QTensor` on `device` for Q8_0 / Q4_K / Q6_K (2-D), a dense torch
        tensor for F32 / F16 / BF16."""
        import torch

        from .qmatmul import QTensor
        info, raw = self.tensor_bytes(f, name)
        if info.ggml_dtype in (int(GgmlDType.Q8_0), int(GgmlDType.Q4K), int(GgmlDType.Q6K)):
            if len(info.shape) != 2:
                raise GgufError(f"quantized tensor {name} has shape {info.shape}; the matmul path takes matrices")
            return QTensor.from_packed(raw, GgmlDType(info.ggml_dtype), (info.shape[0], info.shape[1]), device)
        if info.ggml_dtype in DENSE_NUMPY:
            return torch.from_numpy(raw.view(DENSE_NUMPY[info.ggml_dtype]).reshape(info.shape).copy()).to(device)
        if info.ggml_dtype == 30:
            return torch.from_numpy(raw.view(np.int16).reshape(info.shape).copy()).view(torch.bfloat16).to(device)
        raise GgufError(f"gguf: ggml type {info.ggml_dtype} is not handled by this library")


def _padding(n: int, alignment: int = DEFAULT_ALIGNMENT) -> int:
    return (alignment - n % alignment) % alignment


def _write_string(out: BinaryIO, s: str) -> None:
    b = s.encode("utf-8")
    out.write(struct.pack("<Q", len(b)))
    out.write(b)


def _write_value(out: BinaryIO, v: Value) -> None:
    if v.type in _SCALAR_FMT:
        out.write(struct.pack(_SCALAR_FMT[v.type], v.value))
    elif v.type == ValueType.BOOL:
        out.write(struct.pack("<B", 1 if v.value else 0))
    elif v.type == ValueType.STRING:
        _write_string(out, v.value)
    elif v.type == ValueType.ARRAY:
        items = v.value
        inner = items[0].type if items else ValueType.U8
        if any(i.type != inner for i in items):
            raise GgufError("gguf: arrays hold values of one type")
        out.write(struct.pack("<IQ", int(inner), len(items)))
        for i in items:
            _write_value(out, i)
    else:
        raise GgufError(f"gguf: unknown value type {v.type}")


def write(out: BinaryIO, metadata: list[tuple[str, Value]], tensors: list[tuple[str, int, tuple[int, ...], bytes | np.ndarray]]) -> None:
    """`write` (gguf_file.rs:886-905): version 2, metadata in the given order, then the tensor directory (dimensions
    innermost first, offsets from the start of the data section), zero padding to 32 bytes, then each tensor's bytes
    padded to 32. `tensors` = (name, ggml type id, shape outermost first, packed bytes)."""
    kv = io.BytesIO()
    for key, value in metadata:
        _write_string(kv, key)
        kv.write(struct.pack("<I", int(value.type)))
        _write_value(kv, value)
    blobs = []
    for name, dtype, shape, data in tensors:
        b = data.tobytes() if isinstance(data, np.ndarray) else bytes(data)
        need = TensorInfo(dtype, tuple(shape), 0).size_in_bytes
        if len(b) != need:
            raise GgufError(f"tensor {name} of shape {tuple(shape)} and type {dtype} needs {need} bytes, got {len(b)}")
        blobs.append(b)
    out.write(struct.pack("<IIQQ", GGUF_MAGIC, 2, len(tensors), len(metadata)))
    out.write(kv.getvalue())
    offset = 0
    for (name, dtype, shape, _), b in zip(tensors, blobs):
        _write_string(out, name)
        out.write(struct.pack("<I", len(shape)))
        for d in reversed(shape):
            out.write(struct.pack("<Q", d))
        out.write(struct.pack("<IQ", dtype, offset))
        offset += len(b) + _padding(len(b))
    out.write(b"\x00" * _padding(out.tell()))
    for b in blobs:
        out.write(b)
        out.write(b"\x00" * _padding(len(b)))


def write_qtensors(out: BinaryIO, metadata: list[tuple[str, Value]], tensors: list[tuple[str, Any]]) -> None:
    """The reference's signature: (name, QTensor) pairs; the packed bytes are copied back from the device unchanged."""
    items = []
    for name, q in tensors:
        items.append((name, int(q.dtype), tuple(q.shape), q.packed_bytes().cpu().numpy()))
    write(out, metadata, items)
