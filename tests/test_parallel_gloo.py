"""World-size-2 checks of the sharding / gathering host logic on CPU (gloo backend)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from candle_b200.parallel import Gatherer, argmax_sharded, shard_block_rows, shard_rows


def test_shard_rows_partition():
    for n, world, unit in ((4096, 8, 128), (1024, 2, 128), (128256, 8, 1), (14336, 4, 1)):
        seen = []
        for r in range(world):
            s, c = shard_rows(n, world, r, unit)
            assert c == n // world and s % unit == 0
            seen += list(range(s, s + c))
        assert seen == list(range(n))
    with pytest.raises(ValueError):
        shard_rows(100, 8, 0)
    blocks = np.arange(16 * 3).reshape(16, 3)
    assert np.array_equal(np.concatenate([shard_block_rows(blocks, 16, 4, r) for r in range(4)]), blocks)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = Gatherer()
        from candle_b200.parallel import make_gatherer
        assert type(make_gatherer(None, world, torch.device("cpu"))) is Gatherer      # the peer-memory kernel is for CUDA only
        full = torch.arange(3 * 8, dtype=torch.float32).view(3, 8) * 1.5
        s, c = shard_rows(8, world, rank)
        out = g(full[:, s:s + c].contiguous())
        ok = torch.equal(out, full)
        out2 = g((full[:, s:s + c] + 1).contiguous())          # buffers are reused across calls of the same shape
        ok = ok and torch.equal(out2, full + 1)
        # sharded greedy argmax with a tie across shards and inside a shard: lowest global index wins
        logits = torch.tensor([[0.0, 5.0, 1.0, 5.0, 5.0, 2.0, 0.0, 5.0], [9.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 9.0]])
        tok = argmax_sharded(logits[:, s:s + c].contiguous(), s, g)
        ok = ok and tok.tolist() == [1, 0]
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_gather_and_argmax_world2():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    res = sorted(q.get(timeout=10) for _ in range(2))
    assert res == [(0, True), (1, True)]
    assert all(p.exitcode == 0 for p in procs)


def _ep_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from candle_b200.parallel import make_gatherer
        experts, topk, rows, d = 8, 2, 5, 16
        e_local = experts // world
        e0 = rank * e_local
        gen = torch.Generator().manual_seed(5)
        ids = torch.stack([torch.randperm(experts, generator=gen)[:topk] for _ in range(rows)])           # [rows, topk]
        ids[0] = torch.tensor([0, 1])            # a token whose experts all sit on rank 0: the other rank owns none of its rows
        full = torch.randn(rows, topk, d, generator=gen) * (1.0 + ids.unsqueeze(-1))                      # what one GPU computes
        weights = torch.rand(rows, topk, generator=gen)
        # expert parallel: ids shifted by this rank's first expert; rows outside [0, e_local) are skipped and read as zero
        local = ids - e0
        mine = (local >= 0) & (local < e_local)
        y = torch.where(mine.unsqueeze(-1), full, torch.zeros_like(full))
        gather = make_gatherer(None, world, torch.device("cpu"))
        ok = getattr(gather, "exchange_rows", None) is None        # the CPU gatherer has no peer-memory exchange: all-reduce
        dist.all_reduce(y, op=dist.ReduceOp.SUM)
        ok = ok and torch.equal(y, full)                           # one value plus zeros per element: exact in any order
        ok = ok and int(mine.sum()) + 0 == int(((ids >= e0) & (ids < e0 + e_local)).sum())
        out = (y * weights.unsqueeze(-1)).sum(dim=1)
        ok = ok and torch.equal(out, (full * weights.unsqueeze(-1)).sum(dim=1))
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_expert_parallel_combine_world2():
    """Expert parallelism on the host side: every (token, slot) row is computed by the rank that holds its expert and is zero
    elsewhere, so the sum over ranks has the single-GPU bits; the weighted slot sum after it is the same tensor expression."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_ep_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    res = sorted(q.get(timeout=10) for _ in range(2))
    assert res == [(0, True), (1, True)]
    assert all(p.exitcode == 0 for p in procs)
