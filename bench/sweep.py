#!/usr/bin/env python
"""Tuning sweep: times AllReduce for several tuning settings and sizes in one launch.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench/sweep.py --sizes 16M,256M --configs 'MAX_CTAS=64;MAX_CTAS=128,THREADS=256'

Every configuration is a comma-separated list of HXCCL_<NAME>=<value> settings (read when the
communicator is created). Times are device-timed with CUDA events between barriers, maximum
over ranks; rank 0 prints one JSON line per (configuration, size). `--nccl` adds the
torch.distributed NCCL backend as a row of its own.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def parse_size(s: str) -> int:
    mult = {"K": 1 << 10, "M": 1 << 20, "G": 1 << 30}
    return int(s[:-1]) * mult[s[-1]] if s[-1] in mult else int(s)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", default="8,64K,1M,16M,256M")
    ap.add_argument("--configs", default="")
    ap.add_argument("--dtype", default="float32")
    ap.add_argument("--op", default="sum")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--nccl", action="store_true")
    ap.add_argument("--coll", default="allreduce", choices=["allreduce", "allgather", "reducescatter", "alltoall"])
    args = ap.parse_args()

    import torch
    import torch.distributed as dist

    import hxccl_b200 as hx

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29577")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    tdt = getattr(torch, args.dtype)
    es = torch.empty(0, dtype=tdt).element_size()
    sizes = [parse_size(s) for s in args.sizes.split(",")]
    op = {"sum": hx.SUM, "max": hx.MAX, "avg": hx.AVG}[args.op]
    stream = torch.cuda.current_stream()
    big = max(sizes)
    buf = (torch.rand(max(big // es, 16), device="cuda") * 2 - 1).to(tdt)
    out = torch.empty(max(big // es, 16) * (world if args.coll == "allgather" else 1), dtype=tdt, device="cuda")
    factor = {"allreduce": 2.0 * (world - 1) / world, "allgather": (world - 1) / world,
              "reducescatter": (world - 1) / world, "alltoall": (world - 1) / world}[args.coll]

    def timed(fn, iters):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(iters):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / iters], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    def report(name, size, ms, extra=None):
        if rank == 0:
            row = {"config": name, "coll": args.coll, "bytes": size, "us": round(ms * 1e3, 2),
                   "busbw_GBps": round(size / (ms * 1e-3) / 1e9 * factor, 1)}
            row.update(extra or {})
            print(json.dumps(row), flush=True)

    configs = [c for c in args.configs.split(";")] if args.configs else [""]
    for cfg in configs:
        saved = {}
        for kv in filter(None, cfg.split(",")):
            k, v = kv.split("=")
            saved["HXCCL_" + k] = os.environ.get("HXCCL_" + k)
            os.environ["HXCCL_" + k] = v
        uid = [hx.get_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(uid, src=0)
        comm = hx.Communicator.init_rank(uid[0], world, rank)
        for size in sizes:
            n_el = max(1, size // es)
            if args.coll == "allreduce":
                x = buf[:n_el]
                fn = lambda: comm.all_reduce(x, x, op=op)  # noqa: E731
            elif args.coll == "allgather":
                per = max(1, n_el // world)
                fn = lambda: comm.all_gather(buf[:per], out[: per * world])  # noqa: E731
            elif args.coll == "reducescatter":
                per = max(1, n_el // world)
                fn = lambda: comm.reduce_scatter(buf[: per * world], out[:per], op=op)  # noqa: E731
            else:
                per = max(1, n_el // world)
                fn = lambda: comm.all_to_all(buf[: per * world], out[: per * world], count=per)  # noqa: E731
            ms = timed(fn, args.iters if size >= (1 << 20) else 5 * args.iters)
            extra = {"variant": comm.device_info()["variant"], "err": comm.async_error()}
            if os.environ.get("HXCCL_TRACE"):
                tr = comm.read_trace()
                used = tr[tr[:, 7] > 0]
                if len(used):
                    calls = 5 + (args.iters if size >= (1 << 20) else 5 * args.iters)
                    names = ["in", "sigA", "waitA", "mid", "sigB", "waitB", "out", "all"]
                    extra["trace_us"] = {k: round(float(used[:, i].mean()) / calls / 1e3, 1) for i, k in enumerate(names)}
                    extra["ctas"] = int(len(used))
            report(cfg or "default", size, ms, extra)
        comm.destroy()
        for k, v in saved.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v
    if args.nccl:
        pg = dist.new_group(backend="nccl")
        for size in sizes:
            n_el = max(1, size // es)
            if args.coll == "allreduce":
                x = buf[:n_el]
                fn = lambda: dist.all_reduce(x, group=pg)  # noqa: E731
            elif args.coll == "allgather":
                per = max(1, n_el // world)
                fn = lambda: dist.all_gather_into_tensor(out[: per * world], buf[:per], group=pg)  # noqa: E731
            elif args.coll == "reducescatter":
                per = max(1, n_el // world)
                fn = lambda: dist.reduce_scatter_tensor(out[:per], buf[: per * world], group=pg)  # noqa: E731
            else:
                per = max(1, n_el // world)
                fn = lambda: dist.all_to_all_single(out[: per * world], buf[: per * world], group=pg)  # noqa: E731
            ms = timed(fn, args.iters if size >= (1 << 20) else 5 * args.iters)
            report("nccl", size, ms)
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
