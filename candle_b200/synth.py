"""Seeded synthetic GGUF blocks generated directly on the device.

Benchmarks need gigabytes of weights; quantizing that many f32 values on the host takes minutes, and
throughput does not depend on the values.  ``random_blocks`` therefore writes valid blocks straight
away: uniformly random quants and sub-scales, and f16 super-scales sized so that the de-quantized
weights have the spread of N(0, 0.02) weights run through the reference quantizers
(|w| mostly below 0.06).  Parity tests do not use this module: they quantize real f32 matrices.
"""
from __future__ import annotations

import torch

from .quantized import GgmlDType, QTensor

# f16 scale fields: (byte offset inside the block, typical magnitude)
_SCALES = {
    GgmlDType.Q4_0: [(0, 0.06 / 8)],
    GgmlDType.Q8_0: [(0, 0.06 / 127)],
    GgmlDType.Q4K: [(0, 0.12 / (63 * 15)), (2, 0.06 / 63)],
    GgmlDType.Q6K: [(208, 0.06 / (127 * 32))],
}


def random_blocks(dtype: GgmlDType, n: int, k: int, seed: int, device="cuda:0") -> torch.Tensor:
    """uint8 tensor [n, k / block * type_size] of valid `dtype` blocks."""
    dtype = GgmlDType(dtype)
    bs, ts = dtype.block_size(), dtype.type_size()
    assert k % bs == 0
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    nblk = n * (k // bs)
    blocks = torch.randint(0, 256, (nblk, ts), dtype=torch.uint8, device=device, generator=g)
    for off, mag in _SCALES[dtype]:
        d = (torch.rand(nblk, device=device, generator=g) * 0.5 + 0.75) * mag
        blocks[:, off:off + 2] = d.to(torch.float16).view(torch.uint8).view(nblk, 2)
    return blocks.view(n, (k // bs) * ts)


def random_qtensor(dtype: GgmlDType, n: int, k: int, seed: int, device="cuda:0") -> QTensor:
    return QTensor.from_device_blocks(random_blocks(dtype, n, k, seed, device), dtype, (n, k))
