#!/usr/bin/env python
"""GPT-2 small data-parallel training step: tokens per second with the "hxccl" backend (fused
average AllReduce hook, overlapped with backward) or with NCCL.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench/ddp_gpt2.py --backend hxccl|nccl [--steps 20] [--warmup 5]

Random-initialised GPT-2 small (12 layers, d_model 768, 12 heads, MLP 3072, vocabulary 50257),
sequence length 1024, micro-batch 8 per GPU, token ids uniform over the vocabulary, bf16
autocast, AdamW, 25 MB gradient buckets. One step = forward, backward (with bucket
AllReduce), optimizer step. Timed with CUDA events between barriers, maximum over ranks;
rank 0 prints one JSON line. With one process the collectives drop out and the line is the
single-GPU baseline.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", default="hxccl", choices=["hxccl", "nccl"])
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--tiny", action="store_true", help="a two-layer toy model (smoke tests)")
    ap.add_argument("--exact", type=int, default=1)
    ap.add_argument("--max-ctas", type=int, default=48, help="grid bound of the hxccl kernels during training")
    ap.add_argument("--check", action="store_true", help="print the loss of every step")
    ap.add_argument("--compress", action="store_true",
                    help="average the buckets in bfloat16 (half the bytes): hxccl's one-kernel cast AllReduce, or "
                         "torch's bf16_compress_hook around NCCL")
    args = ap.parse_args()

    import torch
    import torch.distributed as dist
    from torch.nn.parallel import DistributedDataParallel as DDP

    from hxccl_b200.models import GPT2, GPT2Config

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29588")
    if args.backend == "hxccl":
        import hxccl_b200.parallel as hp

        hp.register()
    dist.init_process_group(args.backend, rank=rank, world_size=world,
                            device_id=torch.device("cuda", local) if args.backend == "nccl" else None)
    if args.backend == "hxccl" and world > 1:
        hp.tune(variant=0, exact=bool(args.exact), max_ctas=args.max_ctas)

    torch.manual_seed(0)  # the same initial weights on every rank
    cfg = GPT2Config.tiny() if args.tiny else GPT2Config.small()
    seq = min(args.seq, cfg.n_ctx)
    model = GPT2(cfg).cuda()
    ddp = DDP(model, device_ids=[local], bucket_cap_mb=25, gradient_as_bucket_view=True)
    if args.backend == "hxccl":
        from hxccl_b200.parallel import bf16_compress_average_hook, fused_average_hook

        ddp.register_comm_hook(None, bf16_compress_average_hook if args.compress else fused_average_hook)
    elif args.compress and world > 1:
        from torch.distributed.algorithms.ddp_comm_hooks.default_hooks import bf16_compress_hook

        ddp.register_comm_hook(None, bf16_compress_hook)
    opt = torch.optim.AdamW(ddp.parameters(), lr=3e-4, fused=True)
    g = torch.Generator(device="cuda").manual_seed(1000 + rank)

    def batch():
        x = torch.randint(0, cfg.vocab_size, (args.batch, seq + 1), device="cuda", generator=g)
        return x[:, :-1].contiguous(), x[:, 1:].contiguous()

    losses = []

    def step():
        x, y = batch()
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = ddp(x, y)
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        if args.check:
            losses.append(float(loss))

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / args.steps], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t[0])
    info = None
    if args.backend == "hxccl":
        info = hp.device_info()
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        print(json.dumps({"metric": "ddp_gpt2_tokens_per_s", "backend": args.backend, "n_gpus": world,
                          "value": round(world * args.batch * seq / (ms * 1e-3), 1), "ms_per_step": round(ms, 3),
                          "model": "gpt2-tiny" if args.tiny else "gpt2-small", "params": model.num_params(),
                          "micro_batch": args.batch, "seq_len": seq, "dtype": "bf16 autocast", "bucket_mb": 25,
                          "wire": "bf16" if args.compress else "fp32", "max_ctas": args.max_ctas,
                          "device_path": info, "losses": losses[:8]}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
