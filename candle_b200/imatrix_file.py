"""Importance-matrix files (llama.cpp's `.imatrix` dumps): `load_imatrix` as in candle-core/src/quantized/imatrix_file.rs:10-85.

Layout (little endian): i32 entry count, then per entry: i32 name length, the UTF-8 name, i32 ncall, i32 nval, nval f32
values.  The values are the accumulated squared activations; they are divided by `ncall` when it is not zero.  The result
feeds `QTensor.quantize_imatrix` / `quantize_imatrix_onto`.
"""
from __future__ import annotations

import struct

import numpy as np

from .capi import CandleQError


def load_imatrix(fname) -> dict[str, np.ndarray]:
    """Tensor name -> f32 importance values (one per column of the weight matrix)."""
    try:
        with open(fname, "rb") as f:
            data = f.read()
    except OSError as e:
        raise CandleQError(f"Failed to open {fname}: {e}") from None
    pos = 0

    def i32(what: str) -> int:
        nonlocal pos
        if pos + 4 > len(data):
            raise CandleQError(f"Failed to read {what}: failed to fill whole buffer")
        v = struct.unpack_from("<i", data, pos)[0]
        pos += 4
        return v

    n_entries = i32("number of entries")
    if n_entries < 1:
        raise CandleQError(f"No data in file {fname}")
    out: dict[str, np.ndarray] = {}
    for i in range(1, n_entries + 1):
        length = i32(f"name length for entry {i}")
        if length < 0 or pos + length > len(data):
            raise CandleQError(f"Failed to read name for entry {i}: failed to fill whole buffer")
        raw = data[pos:pos + length]
        pos += length
        try:
            name = raw.decode("utf-8")
        except UnicodeDecodeError as e:
            raise CandleQError(f"Invalid UTF-8 name for entry {i}: {e}") from None
        ncall = i32(f"ncall for entry {i}")
        nval = i32(f"nval for entry {i}")
        if nval < 1:
            raise CandleQError(f"Invalid nval for entry {i}: {nval}")
        if pos + 4 * nval > len(data):
            raise CandleQError(f"Failed to read values for entry {i}: failed to fill whole buffer")
        values = np.frombuffer(data, dtype="<f4", count=nval, offset=pos).astype(np.float32)
        pos += 4 * nval
        out[name] = values if ncall == 0 else (values / np.float32(ncall)).astype(np.float32)
    return out
