#!/usr/bin/env python
"""all_reduce through torch.distributed, one backend per row: "hxccl" (this library), "nccl",
"gloo". The call a PyTorch user makes, timed per size.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench/torch_allreduce.py --backends hxccl,nccl --sizes 4K,64K,1M,16M,256M

GPU tensors are timed with CUDA events on the current stream between barriers (calls return
before completion), CPU tensors (`--device cpu`) by the wall clock around a blocking call; both
as the maximum over ranks. Rank 0 prints one JSON line per (backend, size):
{"backend", "bytes", "us", "busbw_GBps"}. The counterpart of the reference's
python/bench_allreduce.py:1-43 (fp32 all_reduce, 4 KiB..256 MiB, warm-up 5, 20 timed).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def parse_size(s: str) -> int:
    mult = {"K": 1 << 10, "M": 1 << 20, "G": 1 << 30}
    return int(s[:-1]) * mult[s[-1]] if s[-1] in mult else int(s)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--backends", default="hxccl,nccl")
    ap.add_argument("--sizes", default="4K,64K,1M,4M,16M,64M,256M")
    ap.add_argument("--device", default="cuda", choices=["cuda", "cpu"])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    args = ap.parse_args()

    import torch
    import torch.distributed as dist

    import hxccl_b200.parallel as hp

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    cuda = args.device == "cuda"
    if cuda:
        torch.cuda.set_device(local)
        torch.zeros(1, device="cuda")  # the context exists before any communicator does
    hp.register()
    dist.init_process_group("gloo", rank=rank, world_size=world)  # plumbing: barriers, max over ranks
    dev = torch.device("cuda", local) if cuda else torch.device("cpu")
    sizes = [parse_size(s) for s in args.sizes.split(",")]
    buf = torch.rand(max(sizes) // 4, device=dev) * 2 - 1
    factor = 2.0 * (world - 1) / world if world > 1 else 1.0

    def max_over_ranks(v: float) -> float:
        t = torch.tensor([v], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    for name in args.backends.split(","):
        if name == "nccl" and not cuda:
            continue
        pg = dist.new_group(backend=name)
        for size in sizes:
            x = buf[: max(1, size // 4)]
            for _ in range(args.warmup):
                dist.all_reduce(x, group=pg)
            if cuda:
                torch.cuda.synchronize()
            dist.barrier()
            if cuda:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(args.iters):
                    dist.all_reduce(x, group=pg)
                e1.record()
                torch.cuda.synchronize()
                ms = e0.elapsed_time(e1) / args.iters
            else:
                t0 = time.perf_counter()
                for _ in range(args.iters):
                    dist.all_reduce(x, group=pg)
                ms = (time.perf_counter() - t0) * 1e3 / args.iters
            ms = max_over_ranks(ms)
            if rank == 0:
                nbytes = x.numel() * 4
                print(json.dumps({"backend": name, "device": args.device, "ranks": world, "bytes": nbytes,
                                  "us": round(ms * 1e3, 2),
                                  "busbw_GBps": round(nbytes / (ms * 1e-3) / 1e9 * factor, 3)}), flush=True)
            x.copy_(torch.rand_like(x))  # sums of sums would overflow over many sizes
        dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
