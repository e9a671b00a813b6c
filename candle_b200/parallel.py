"""Column-parallel sharding of quantized projections inside one NVLink/NVSwitch box.

Every weight row of W[N, K] is an independent unit (a GGUF block never spans rows), so each rank keeps a
contiguous range of rows, computes y[:, rows] with the ordinary kernels and the slices are all-gathered.
The per-element summation order does not depend on the shard count, so results are bit-identical for any
world size - which K-sharding followed by an all-reduce (the scheme of candle's only multi-GPU example,
candle-examples/examples/llama_multiprocess/model.rs:13-137) cannot give.

Host logic here is device-free and is exercised on CPU with the gloo backend.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_rows(n: int, world: int, rank: int, unit: int = 1) -> tuple[int, int]:
    """Contiguous row range [start, start + count) of rank `rank`; `unit` rows stay together (e.g. one head)."""
    if n % (world * unit) != 0:
        raise ValueError(f"{n} rows cannot be split into {world} shards of whole units of {unit}")
    count = n // world
    return rank * count, count


def shard_block_rows(blocks, n: int, world: int, rank: int, unit: int = 1):
    """Slice the rows of a [n, row_bytes] block matrix (numpy or torch) for `rank`."""
    start, count = shard_rows(n, world, rank, unit)
    return blocks[start:start + count]


class Gatherer:
    """All-gather of column slices [rows, n_local] -> [rows, n_local * world], rank-major along the last dimension.

    Buffers are allocated once per shape so that the call can sit inside a CUDA graph."""

    def __init__(self, group=None, world: int | None = None):
        self.group = group
        self.world = world if world is not None else (dist.get_world_size(group) if dist.is_initialized() else 1)
        self._bufs: dict = {}

    def __call__(self, local: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return local
        rows, n_local = local.shape
        key = (rows, n_local, local.dtype, local.device)
        if key not in self._bufs:
            self._bufs[key] = (torch.empty((self.world * rows, n_local), dtype=local.dtype, device=local.device),
                               torch.empty((rows, self.world * n_local), dtype=local.dtype, device=local.device))
        stacked, full = self._bufs[key]
        dist.all_gather_into_tensor(stacked, local.contiguous(), group=self.group)
        if rows == 1:       # rank-major slices of a single row are already the gathered row
            return stacked.view(1, self.world * n_local)
        full.view(rows, self.world, n_local).copy_(stacked.view(self.world, rows, n_local).permute(1, 0, 2))
        return full


def argmax_sharded(local_logits: torch.Tensor, vocab_start: int, gather: Gatherer) -> torch.Tensor:
    """Greedy token over a vocabulary sharded by rows: gather (max, global index) pairs and break ties towards the
    lowest global index, which is what argmax over the whole row returns."""
    mx = local_logits.max(dim=-1).values
    ar = torch.arange(local_logits.shape[-1], device=local_logits.device)
    idx = torch.where(local_logits == mx.unsqueeze(-1), ar, ar.new_full((), 1 << 40)).min(dim=-1).values   # first maximum
    pair = torch.stack([mx, (idx + vocab_start).to(mx.dtype)], dim=-1)      # indices < 2^24 are exact in f32
    allp = gather(pair)                                                      # [rows, 2 * world]
    allp = allp.view(allp.shape[0], -1, 2)
    best = allp[..., 0].max(dim=-1, keepdim=True).values
    cand = torch.where(allp[..., 0] == best, allp[..., 1], torch.full_like(allp[..., 1], float("inf")))
    return cand.min(dim=-1).values.to(torch.int64)
