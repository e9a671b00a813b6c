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
