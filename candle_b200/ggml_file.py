"""The legacy GGML container (files older than GGUF): `Content.read` as in candle-core/src/quantized/ggml_file.rs:234-266.

Layout (little endian): magic [version] | seven u32 hyper-parameters | n_vocab x (u32 length, bytes, f32 score) | tensors
until the end of the file, each: n_dims, name length, ggml dtype, dims (innermost first), name, [padding to 32 bytes for
the "ggjt" files], blocks.  Host-side parsing only; a tensor goes to the device when it is taken out with `remove`.
"""
from __future__ import annotations

import dataclasses
import struct

from .capi import CandleQError
from .gguf_file import HostTensor
from .quantized import GgmlDType, QTensor

_MAGICS = {0x67676a74: "ggjt", 0x67676c61: "ggla", 0x67676d66: "ggmf", 0x67676d6c: "ggml", 0x6767736e: "ggsn"}
_VERSIONED = {("ggmf", 1): "GgmfV1", ("ggjt", 1): "GgjtV1", ("ggjt", 2): "GgjtV2", ("ggjt", 3): "GgjtV3"}
_SUPPORTED = {GgmlDType.F32, GgmlDType.F16, GgmlDType.BF16, GgmlDType.Q4_0, GgmlDType.Q4_1, GgmlDType.Q5_0, GgmlDType.Q5_1,
              GgmlDType.Q8_0, GgmlDType.Q2K, GgmlDType.Q3K, GgmlDType.Q4K, GgmlDType.Q5K, GgmlDType.Q6K}


@dataclasses.dataclass
class HParams:
    n_vocab: int
    n_embd: int
    n_mult: int
    n_head: int
    n_layer: int
    n_rot: int
    ftype: int


class _Reader:
    def __init__(self, data: bytes):
        self.data, self.pos = data, 0

    def take(self, n: int) -> bytes:
        if n < 0 or self.pos + n > len(self.data):
            raise CandleQError("ggml: failed to fill whole buffer")        # what read_exact reports at a short file
        out = self.data[self.pos:self.pos + n]
        self.pos += n
        return out

    def u32(self) -> int:
        return struct.unpack("<I", self.take(4))[0]

    def f32(self) -> float:
        return struct.unpack("<f", self.take(4))[0]


def _read_magic(r: _Reader) -> str:
    """`VersionedMagic::read` (ggml_file.rs:44-60)."""
    value = r.u32()
    if value not in _MAGICS:
        raise CandleQError(f"unknown magic {value:08x}")
    magic = _MAGICS[value]
    if magic == "ggml":
        return "GgmlUnversioned"
    version = r.u32()
    if (magic, version) not in _VERSIONED:
        raise CandleQError(f"ggml: unsupported magic/version {magic.capitalize()}/{version}")
    return _VERSIONED[(magic, version)]


def tensor_from_ggml(ggml_dtype: GgmlDType, raw: bytes, dims) -> HostTensor:
    """`qtensor_from_ggml` (ggml_file.rs:138-189) up to the upload: checks the shape against the block size."""
    elems = 1
    for d in dims:
        elems *= int(d)
    bs = ggml_dtype.block_size()
    if elems % bs != 0:
        raise CandleQError(f"the number of elements {elems} is not divisible by the block size {bs}")
    if ggml_dtype not in _SUPPORTED:
        raise CandleQError(f"quantized type {ggml_dtype.name} is not supported yet")
    return HostTensor(ggml_dtype, tuple(int(d) for d in dims), raw[:elems // bs * ggml_dtype.type_size()])


class Content:
    """A parsed GGML file: `magic` (GgmlUnversioned, GgmfV1, GgjtV1..3), `hparams`, `vocab` ((bytes, score) pairs) and the
    tensors by name, held in host memory."""

    def __init__(self, magic: str, hparams: HParams, vocab, tensors: dict, device=None):
        self.magic, self.hparams, self.vocab, self.tensors, self.device = magic, hparams, vocab, tensors, device

    @classmethod
    def read(cls, source, device=None) -> "Content":
        """`source`: a path, bytes, or a binary stream.  `device`: where `remove` puts tensors (e.g. "cuda:0")."""
        if isinstance(source, (bytes, bytearray, memoryview)):
            data = bytes(source)
        elif hasattr(source, "read"):
            data = source.read()
        else:
            with open(source, "rb") as f:
                data = f.read()
        r = _Reader(data)
        magic = _read_magic(r)
        hparams = HParams(*(r.u32() for _ in range(7)))
        vocab = []
        for _ in range(hparams.n_vocab):
            word = r.take(r.u32())
            vocab.append((word, r.f32()))
        align32 = magic.startswith("Ggjt")
        tensors: dict[str, HostTensor] = {}
        while r.pos != len(data):
            n_dims, name_len, dtype_u32 = r.u32(), r.u32(), r.u32()
            ggml_dtype = GgmlDType.from_u32(dtype_u32)
            dims = [r.u32() for _ in range(n_dims)][::-1]          # stored innermost first
            name = r.take(name_len).decode("utf-8", errors="replace")
            if align32:
                r.take((32 - r.pos % 32) % 32)
            elems = 1
            for d in dims:
                elems *= d
            raw = r.take(elems * ggml_dtype.type_size() // ggml_dtype.block_size())
            try:
                tensors[name] = tensor_from_ggml(ggml_dtype, raw, dims)
            except CandleQError as e:
                raise CandleQError(f"Error creating tensor {name}: {e}") from None
        return cls(magic, hparams, vocab, tensors, device)

    def remove(self, name: str, device=None):
        """Takes the tensor out of the file's table (ggml_file.rs:260-265): a `QTensor` on `device` (or on the device given to
        `read`), the `HostTensor` itself when neither names a device."""
        if name not in self.tensors:
            raise CandleQError(f"cannot find tensor with name '{name}'")
        t = self.tensors.pop(name)
        dev = device if device is not None else self.device
        if dev is None:
            return t
        return QTensor.from_data(t.data, t.ggml_dtype, t.shape, dev)
