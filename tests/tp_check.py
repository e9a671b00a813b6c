"""Token bit-consistency check: greedy tokens of a tensor-parallel run against a single-GPU run of the same model.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node=N --master-addr 127.0.0.1 tests/tp_check.py [--full]

Every rank builds its shard; rank 0 also builds the whole model on its own GPU and compares the token sequences.
Prints / writes "identical" or the first difference.
"""
import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from candle_b200.decoder import DecoderConfig, LlamaShapedDecoder  # noqa: E402
from candle_b200.moe_decoder import MoeDecoderConfig, MoeShapedDecoder  # noqa: E402


def check_gather(dev, rank, world) -> str:
    """Peer-memory gather against the library all-gather: ragged and aligned widths, 1-8 rows, strided slices, one shape
    twice in a row, eager and replayed from a CUDA graph.  All ranks return the same verdict."""
    from candle_b200.parallel import Gatherer, PeerGatherer
    ref, peer = Gatherer(None, world), PeerGatherer(None, world)
    gen = torch.Generator(device=dev).manual_seed(100 + rank)
    bad = []
    shapes = [(1, 4096), (2, 1024), (8, 16032), (3, 7), (5, 130), (1, 2), (4, 512), (4, 512), (4, 512), (8, 3584)]
    for it, (rows, n_local) in enumerate(shapes * 3):
        wide = torch.randn((rows, n_local + 12), device=dev, generator=gen)
        local = wide[:, 4:4 + n_local] if it % 2 else wide[:, :n_local].contiguous()
        want = ref(local).clone()
        got = peer(local)
        if not torch.equal(got, want):
            bad.append((it, rows, n_local))
    for rows, blocks in ((1, 16), (8, 112), (3, 5)):       # rows of 36-byte containers travel as 32-bit words
        u = torch.randint(0, 256, (rows, 36 * blocks), device=dev, dtype=torch.uint8, generator=gen)
        if not torch.equal(peer(u), ref(u)):
            bad.append(("u8", rows, blocks))
    # replayed from a graph: three gathers of different shapes, new data before every replay
    xs = [torch.zeros((r, n), device=dev) for (r, n) in ((2, 1024), (1, 4096), (8, 16032))]
    for x in xs:
        peer(x)
    side = torch.cuda.Stream(device=dev)
    outs = []
    with torch.cuda.stream(side):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            outs = [peer(x) for x in xs]
    for rep in range(4):
        for x in xs:
            x.copy_(torch.randn(x.shape, device=dev, generator=gen))
        torch.cuda.synchronize()
        g.replay()
        torch.cuda.synchronize()
        for x, o in zip(xs, outs):
            if not torch.equal(o, ref(x)):
                bad.append(("graph", rep, tuple(x.shape)))
    peer.check()
    # a graph that holds ONE gather, replayed many times: consecutive replays must not share a staging area (the kernel
    # alternates by its device-side epoch; a host-side choice would be frozen into the graph)
    x1 = torch.zeros((4, 512), device=dev)
    peer(x1)
    with torch.cuda.stream(side):
        g1 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g1, stream=side):
            o1 = peer(x1)
    for rep in range(40):
        x1.copy_(torch.randn(x1.shape, device=dev, generator=gen))
        torch.cuda.synchronize()
        if rep % 2 == rank % 2:        # ranks take turns being late
            torch.cuda._sleep(2_000_000)
        g1.replay()
        torch.cuda.synchronize()
        if not torch.equal(o1, ref(x1)):
            bad.append(("one-gather graph", rep))
    peer.check()
    # rows with one owner each (expert-parallel outputs): every rank must end up with each row as its owner holds it
    e_local = 5
    gen_all = torch.Generator(device=dev).manual_seed(77)       # the same on all ranks
    xrows = [(8, 2048), (8, 2048), (64, 96), (1, 3), (16, 2048)]
    for it, (rows, n) in enumerate(xrows * 3):
        experts = torch.randint(0, e_local * world, (rows,), device=dev, dtype=torch.int32, generator=gen_all)
        truth = torch.randn((rows, n), device=dev, generator=gen_all)
        owner = (experts - rank * e_local).contiguous()
        mine = (owner >= 0) & (owner < e_local)
        local = torch.where(mine[:, None], truth, torch.full_like(truth, float("nan")))     # the other rows hold nothing useful
        got = peer.exchange_rows(local, owner, e_local)
        if got is None or not torch.equal(got, truth):
            bad.append(("rows", it, rows, n))
    ex = torch.zeros((8, 2048), device=dev)
    ow = torch.zeros(8, dtype=torch.int32, device=dev)
    peer.exchange_rows(ex, ow, e_local)
    with torch.cuda.stream(side):
        g2 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g2, stream=side):
            o2 = peer.exchange_rows(ex, ow, e_local)
    for rep in range(30):
        experts = torch.randint(0, e_local * world, (8,), device=dev, dtype=torch.int32, generator=gen_all)
        if rep % 3 != 2:        # all rows on one rank, several exchanges in a row: the others own nothing and must still be waited for
            experts = torch.full_like(experts, ((rep // 3) % world) * e_local + 1)
        truth = torch.randn((8, 2048), device=dev, generator=gen_all)
        ow.copy_(experts - rank * e_local)
        ex.copy_(torch.where(((ow >= 0) & (ow < e_local))[:, None], truth, torch.zeros_like(truth)))
        torch.cuda.synchronize()
        if rep % 2 == rank % 2:
            torch.cuda._sleep(2_000_000)
        g2.replay()
        torch.cuda.synchronize()
        if not torch.equal(o2, truth):
            bad.append(("rows graph", rep))
    peer.check()
    # host buffers in, gathered host buffers out, with the copies on their own streams
    from candle_b200.parallel import ShardedHostForward
    from candle_b200.quantized import GgmlDType, QMatMul, QTensor
    from candle_b200.synth import random_blocks
    n_all, kk = 1024, 4096
    mm = QMatMul.from_qtensor(QTensor.from_device_blocks(random_blocks(GgmlDType.Q4K, n_all // world, kk, 5 + rank, dev), GgmlDType.Q4K,
                                                         (n_all // world, kk)))
    hf = ShardedHostForward(peer, dev)
    cpu_gen = torch.Generator().manual_seed(31)         # the same activations on every rank
    cases = []
    for b in (1, 8, 3, 1, 1, 8, 8, 2, 5, 1):
        hx = torch.randn((b, kk), generator=cpu_gen).pin_memory()
        hy = torch.full((b, n_all), float("nan")).pin_memory()
        hf(mm, hx, hy)
        cases.append((hx, hy))
    hf.flush()
    torch.cuda.synchronize()
    for i, (hx, hy) in enumerate(cases):
        if not torch.equal(hy, ref(mm.forward(hx.to(dev))).cpu()):
            bad.append(("host forward", i))
    peer.check()
    # cost of one gather: 100 alternating gathers of a decode-sized and a head-sized slice, replayed from a graph
    for name, g_ in (("peer", peer), ("nccl", ref)):
        a, b = torch.randn((1, 4096 // world), device=dev), torch.randn((1, 128256 // world), device=dev)
        g_(a); g_(b)
        with torch.cuda.stream(side):
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr, stream=side):
                for _ in range(50):
                    g_(a); g_(b)
            gr.replay()
            side.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(side)
            for _ in range(5):
                gr.replay()
            e1.record(side)
            side.synchronize()
        if rank == 0:
            print(f"{name} gather: {e0.elapsed_time(e1) * 1000.0 / 500:.2f} us per gather (world {world})", flush=True)
    peer.check()
    flag = torch.tensor([len(bad)], device=dev)
    dist.all_reduce(flag)
    return "identical" if int(flag.item()) == 0 else f"peer gather differs: {bad[:4]} (rank {rank})"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--full", action="store_true", help="Llama-3-8B shape instead of the tiny test shape")
    ap.add_argument("--steps", type=int, default=16)
    ap.add_argument("--prompt", type=int, default=32)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--moe", action="store_true", help="the mixture-of-experts harness (expert parallel) instead of the dense one")
    ap.add_argument("--out", default=None)
    ap.add_argument("--gather", action="store_true", help="check the peer-memory gather kernel against the NCCL all-gather")
    args = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    dist.init_process_group("nccl", device_id=dev)
    if args.gather:
        verdict = check_gather(dev, rank, world)
        if rank == 0:
            print(verdict)
            if args.out:
                open(args.out, "w").write(verdict + "\n")
        dist.barrier()
        dist.destroy_process_group()
        sys.exit(0 if verdict == "identical" else 1)
    if args.moe:
        cfg = MoeDecoderConfig.qwen3_30b_a3b() if args.full else MoeDecoderConfig.tiny()
        Model = MoeShapedDecoder
    else:
        cfg = DecoderConfig.llama3_8b() if args.full else DecoderConfig.tiny()
        Model = LlamaShapedDecoder
    prompt = torch.randint(0, cfg.vocab, (args.batch, args.prompt), device=dev, generator=torch.Generator(device=dev).manual_seed(2))
    tp = Model(cfg, dev, rank=rank, world=world, batch=args.batch, seed=1)
    toks_tp = tp.generate(prompt, args.steps)
    verdict = "identical"
    if rank == 0:
        del tp
        torch.cuda.empty_cache()
        single = Model(cfg, dev, rank=0, world=1, batch=args.batch, seed=1)
        toks_1 = single.generate(prompt, args.steps)
        if not torch.equal(toks_tp, toks_1):
            diff = (toks_tp != toks_1).nonzero()[0].tolist()
            verdict = f"differ at {diff}: tp {toks_tp[diff[0], diff[1]].item()} vs single {toks_1[diff[0], diff[1]].item()}"
        print(verdict)
        if args.out:
            open(args.out, "w").write(verdict + "\n")
    dist.barrier()
    dist.destroy_process_group()
    if verdict != "identical":
        sys.exit(1)


if __name__ == "__main__":
    main()
