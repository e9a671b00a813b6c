"""Token bit-consistency check: greedy tokens of a tensor-parallel run against a single-GPU run of the same model.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node=N --master-addr 127.0.0.1 candle_b200/tp_check.py [--full]

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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--full", action="store_true", help="Llama-3-8B shape instead of the tiny test shape")
    ap.add_argument("--steps", type=int, default=16)
    ap.add_argument("--prompt", type=int, default=32)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--moe", action="store_true", help="the mixture-of-experts harness (expert parallel) instead of the dense one")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    dist.init_process_group("nccl", device_id=dev)
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
