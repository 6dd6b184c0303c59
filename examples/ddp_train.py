#!/usr/bin/env python
"""Data-parallel training through the "hxccl" torch.distributed backend.

    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 8 examples/ddp_train.py            # one GPU per rank
    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 2 examples/ddp_train.py --cpu      # host buffers

A small MLP regresses a fixed random teacher; every rank draws its own batches, gradients are
averaged by the library (one AllReduce per bucket with the 1/N scaling inside the kernel,
overlapped with backward; `--compress` sends bfloat16). Rank 0 prints the loss every few steps and
finally checks that all ranks hold the same weights.
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--cpu", action="store_true", help="host tensors (no GPU needed)")
    ap.add_argument("--compress", action="store_true", help="bfloat16 gradient buckets")
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--width", type=int, default=256)
    args = ap.parse_args()

    import torch
    import torch.distributed as dist

    import hxccl_b200.parallel as hp

    hp.register()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    if args.cpu:
        device, ddp_device = torch.device("cpu"), None
    else:
        torch.cuda.set_device(local)
        device, ddp_device = torch.device("cuda", local), local
    dist.init_process_group("hxccl", rank=rank, world_size=world)

    torch.manual_seed(0)  # same initial weights and the same teacher everywhere
    teacher = torch.nn.Linear(args.width, 1).to(device)
    model = torch.nn.Sequential(torch.nn.Linear(args.width, args.width), torch.nn.Tanh(),
                                torch.nn.Linear(args.width, 1)).to(device)
    model = hp.wrap(model, device=ddp_device, bucket_cap_mb=1, compress=args.compress)
    opt = torch.optim.SGD(model.parameters(), lr=0.05)
    gen = torch.Generator(device="cpu").manual_seed(1000 + rank)  # different data per rank

    first = last = None
    for step in range(args.steps):
        x = torch.randn(64, args.width, generator=gen).to(device)
        with torch.no_grad():
            y = teacher(x)
        loss = torch.nn.functional.mse_loss(model(x), y)
        opt.zero_grad(set_to_none=True)
        loss.backward()  # bucket AllReduces run while backward continues
        opt.step()
        mean = loss.detach().clone()
        dist.all_reduce(mean, op=dist.ReduceOp.AVG)
        first = float(mean) if first is None else first
        last = float(mean)
        if rank == 0 and (step % 10 == 0 or step == args.steps - 1):
            print(f"step {step:3d}  loss {last:.5f}", flush=True)

    flat = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    lo, hi = flat.clone(), flat.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    same = bool(torch.equal(lo, hi))
    if rank == 0:
        print(f"loss {first:.5f} -> {last:.5f}; weights identical on all {world} ranks: {same}", flush=True)
    dist.destroy_process_group()
    return 0 if same and last < first else 1


if __name__ == "__main__":
    sys.exit(main())
