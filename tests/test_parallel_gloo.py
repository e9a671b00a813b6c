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
