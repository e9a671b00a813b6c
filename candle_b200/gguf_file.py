"""GGUF files: ``Content.read`` and ``Content.tensor`` as in candle-core/src/quantized/gguf_file.rs:470-581.

Parsing and the upload live in libcandle_q_b200.so (csrc/host/gguf.cpp): the file is memory-mapped, and a tensor - or a
contiguous range of its rows, which is what a tensor-parallel rank wants - goes from the mapping to the device in one
copy.  Metadata arrives as JSON and is exposed as a plain dict (integers, floats, bools, strings, nested lists).
"""
from __future__ import annotations

import ctypes as C
import dataclasses
import json

import numpy as np
import torch

from . import capi
from .capi import CandleQError
from .quantized import GgmlDType, QTensor

DEFAULT_ALIGNMENT = 32


@dataclasses.dataclass
class TensorInfo:
    ggml_dtype: GgmlDType
    shape: tuple
    offset: int
    nbytes: int
    index: int


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise CandleQError(f"{what}: {capi.lib().cqh_gguf_last_error().decode()}")


class Content:
    """An open GGUF file.  ``magic`` is the container version (1, 2 or 3)."""

    def __init__(self, handle: int):
        L = capi.lib()
        self._h = C.c_void_p(handle)
        self.magic = int(L.cqh_gguf_version(self._h))
        self.tensor_data_offset = int(L.cqh_gguf_tensor_data_offset(self._h))
        self.metadata = json.loads(L.cqh_gguf_metadata_json(self._h).decode("utf-8", errors="replace"))
        self.tensor_infos: dict[str, TensorInfo] = {}
        name, dt, nd = C.c_char_p(), C.c_int(), C.c_int()
        dims, off, nb = (C.c_int64 * 4)(), C.c_uint64(), C.c_uint64()
        for i in range(int(L.cqh_gguf_tensor_count(self._h))):
            _check(L.cqh_gguf_tensor_info(self._h, i, C.byref(name), C.byref(dt), dims, C.byref(nd), C.byref(off), C.byref(nb)),
                   "gguf tensor info")
            self.tensor_infos[name.value.decode("utf-8", errors="replace")] = TensorInfo(
                GgmlDType.from_u32(dt.value), tuple(int(dims[j]) for j in range(nd.value)), int(off.value), int(nb.value), i)

    @classmethod
    def read(cls, path: str) -> "Content":
        h = C.c_void_p()
        _check(capi.lib().cqh_gguf_open(str(path).encode(), C.byref(h)), "gguf")
        return cls(h.value)

    def close(self) -> None:
        h, self._h = getattr(self, "_h", None), None
        if h:
            capi.lib().cqh_gguf_close(h)

    __del__ = close

    def _info(self, name: str) -> TensorInfo:
        if name not in self.tensor_infos:
            raise CandleQError(f"cannot find tensor info for {name}")
        return self.tensor_infos[name]

    def tensor(self, name: str, device="cuda:0", rows: tuple[int, int] | None = None) -> QTensor:
        """The tensor on `device`; `rows` = (start, count) loads only that range of the outermost dimension."""
        info = self._info(name)
        device = torch.device(device)
        start, count = rows if rows is not None else (0, -1)
        out = C.c_void_p()
        _check(capi.lib().cqh_gguf_load_tensor(self._h, info.index, device.index or 0, start, count, C.byref(out)), f"gguf tensor {name}")
        shape = info.shape if rows is None else (count, *info.shape[1:])
        return QTensor(out.value, info.ggml_dtype, shape, device)

    def tensor_bytes(self, name: str) -> np.ndarray:
        """The raw bytes of a tensor on the host (norm weights and other small float tensors are used this way)."""
        info = self._info(name)
        out = np.empty(info.nbytes, dtype=np.uint8)
        _check(capi.lib().cqh_gguf_read_tensor(self._h, info.index, out.ctypes.data, out.size), f"gguf tensor {name}")
        return out


# ---- writing (gguf_file.rs:190-260 `Value`, :376-411 `Value::write`, :583-638 `write`) ----------------------------------
_VALUE_TYPES = {"u8": (0, "<B"), "i8": (1, "<b"), "u16": (2, "<H"), "i16": (3, "<h"), "u32": (4, "<I"), "i32": (5, "<i"),
                "f32": (6, "<f"), "bool": (7, "<B"), "string": (8, None), "array": (9, None), "u64": (10, "<Q"), "i64": (11, "<q"),
                "f64": (12, "<d")}


class Value:
    """One metadata value with its GGUF type, as the reference's `Value` enum: `Value("u32", 7)`, `Value("string", "llama")`,
    `Value("array", [Value("f32", 1.0), ...])`.  An array's elements must share one type; an empty array is written as an
    array of u32, as the reference does."""

    def __init__(self, kind: str, v):
        if kind not in _VALUE_TYPES:
            raise CandleQError(f"unrecognized value-type {kind}")
        if kind == "array":
            v = list(v)
            if any(not isinstance(e, Value) for e in v):
                raise CandleQError("array elements must be Value objects")
        self.kind, self.v = kind, v

    def value_type(self) -> int:
        return _VALUE_TYPES[self.kind][0]

    def write(self, w) -> None:
        import struct
        code, fmt = _VALUE_TYPES[self.kind]
        if fmt is not None:
            w.write(struct.pack(fmt, (1 if self.v else 0) if self.kind == "bool" else self.v))
        elif self.kind == "string":
            _write_string(w, self.v)
        else:
            kinds = {e.kind for e in self.v}
            if len(kinds) > 1:
                raise CandleQError(f"multiple value-types in the same array {sorted(kinds)}")
            elem = _VALUE_TYPES[kinds.pop()][0] if kinds else _VALUE_TYPES["u32"][0]
            w.write(struct.pack("<IQ", elem, len(self.v)))
            for e in self.v:
                e.write(w)


def _write_string(w, s) -> None:
    import struct
    b = s.encode("utf-8") if isinstance(s, str) else bytes(s)
    w.write(struct.pack("<Q", len(b)))
    w.write(b)


@dataclasses.dataclass
class HostTensor:
    """GGUF blocks held in host memory: what `write` needs of a tensor (a `QTensor` is read back from its device)."""
    ggml_dtype: GgmlDType
    shape: tuple
    data: bytes


def write(w, metadata, tensors) -> None:
    """`gguf_file::write` (gguf_file.rs:590-638): a version-2 file on the seekable binary stream `w`.  metadata: (name,
    Value) pairs; tensors: (name, QTensor or HostTensor) pairs.  Dimensions are stored innermost first, tensor data is
    padded to 32 bytes, offsets are relative to the first tensor."""
    import struct
    metadata, tensors = list(metadata), list(tensors)
    w.write(struct.pack("<IIQQ", 0x46554747, 2, len(tensors), len(metadata)))
    for name, value in metadata:
        _write_string(w, name)
        w.write(struct.pack("<I", value.value_type()))
        value.write(w)
    offset, offsets, blobs = 0, [], []
    for name, t in tensors:
        if isinstance(t, HostTensor):
            dtype, shape, data = GgmlDType(t.ggml_dtype), tuple(t.shape), bytes(t.data)
        else:
            dtype, shape, data = t.dtype, tuple(t.shape), t.data()
        n = 1
        for d in shape:
            n *= int(d)
        if n % dtype.block_size() or n // dtype.block_size() * dtype.type_size() != len(data):
            raise CandleQError(f"tensor {name}: {len(data)} bytes do not match shape {list(shape)} of {dtype.name}")
        _write_string(w, name)
        w.write(struct.pack("<I", len(shape)))
        for d in reversed(shape):
            w.write(struct.pack("<Q", int(d)))
        w.write(struct.pack("<IQ", int(dtype), offset))
        offsets.append(offset)
        blobs.append(data)
        offset += len(data) + (31 - (31 + len(data)) % 32)
    pos = w.tell()
    w.write(b"\0" * (31 - (31 + pos) % 32))
    start = w.tell()
    for off, data in zip(offsets, blobs):
        if start + off != w.tell():
            raise CandleQError(f"internal error, unexpected current position {start} {off} {w.tell()}")
        w.write(data)
        w.write(b"\0" * (31 - (31 + len(data)) % 32))
