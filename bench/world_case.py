#!/usr/bin/env python
"""One collective of the single-GPU world harness, run a few times: the small, single-process
case used for Nsight Compute captures of the collective kernels (a multi-rank job must never
run under ncu) and for timing them without any link in the way.

    python bench/world_case.py --n 2 --mb 256 --variant 2 --dtype float32 --iters 3
    python bench/world_case.py --n 8 --bytes 16384 --variant 7          # data-with-epoch lines
    python bench/world_case.py --n 4 --mb 64 --coll allgather           # also reducescatter, sendrecv, cast
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--n", type=int, default=2)
    ap.add_argument("--mb", type=int, default=256, help="message size per rank in MiB")
    ap.add_argument("--bytes", type=int, default=0, help="message size per rank in bytes (overrides --mb)")
    ap.add_argument("--order", type=int, default=0, help="0 ring order, 1 recursive doubling, -1 by size")
    ap.add_argument("--variant", type=int, default=2, help="1 one-shot, 2 two-shot")
    ap.add_argument("--dtype", default="float32")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--window-mb", type=int, default=256)
    ap.add_argument("--roles", action="store_true", help="force the three-role pipeline")
    ap.add_argument("--coll", default="allreduce", choices=["allreduce", "allgather", "reducescatter", "sendrecv", "cast"],
                    help="cast: fp32 buffers with bf16 on the wire; reducescatter runs the ring form")
    args = ap.parse_args()

    import torch

    import hxccl_b200 as hx
    from hxccl_b200.comm import dtype_of
    from hxccl_b200.ops.world import World

    tdt = getattr(torch, args.dtype)
    count = max(1, (args.bytes or (args.mb << 20)) // torch.empty(0, dtype=tdt).element_size())
    xs = [(torch.rand(count, device="cuda") * 2 - 1).to(tdt) for _ in range(args.n)]
    ys = [torch.empty_like(x) for x in xs]
    with World(args.n, window_mb=args.window_mb, wait_ms=20000) as w:
        w.tune(variant=args.variant, exact=True)
        if args.roles:
            w.knob("roles_min", 1)
        dt = dtype_of(xs[0])
        per = max(1, count // args.n)
        if args.coll == "allgather":
            gathered = [torch.empty(per * args.n, dtype=tdt, device="cuda") for _ in range(args.n)]
        if args.coll == "reducescatter":
            w.knob("rs_ring_min", 1)
        if args.coll == "cast":
            xs = [x.float() for x in xs]
            ys = [torch.empty_like(x) for x in xs]

        def call():
            if args.coll == "allreduce":
                w.all_reduce(xs, ys, count, dt, op=hx.SUM, order=args.order)
            elif args.coll == "allgather":
                w.all_gather([x[:per] for x in xs], gathered, per * xs[0].element_size())
            elif args.coll == "reducescatter":
                w.reduce_scatter([x[: per * args.n] for x in xs], [y[:per] for y in ys], per, dt, op=hx.SUM)
            elif args.coll == "sendrecv":  # ring shift: rank r sends its buffer to r+1
                nb = count * xs[0].element_size()
                w.send_recv([(r, (r + 1) % args.n, xs[r], nb, ys[(r + 1) % args.n], nb) for r in range(args.n)])
            else:
                w.all_reduce_cast(xs, ys, count, hx.BFLOAT16, op=hx.AVG)

        times = []
        for _ in range(args.iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            call()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        ok = all(w.status(r) == (0, 0) for r in range(args.n))
        info = w.info()
    if args.coll == "allreduce":
        err = float((ys[0].double() - sum(x.double() for x in xs)).abs().max())
    elif args.coll == "allgather":
        err = float((gathered[0].double() - torch.cat([x[:per] for x in xs]).double()).abs().max())
    elif args.coll == "reducescatter":
        err = float((ys[0][:per].double() - sum(x[:per].double() for x in xs)).abs().max())
    elif args.coll == "sendrecv":
        err = float((ys[1].double() - xs[0].double()).abs().max())
    else:  # an average of bf16-rounded values: compare loosely with the fp32 mean
        err = float((ys[0].double() - sum(x.double() for x in xs) / args.n).abs().max())
    print(json.dumps({"n": args.n, "coll": args.coll, "bytes_per_rank": args.bytes or (args.mb << 20), "order": args.order, "dtype": args.dtype, "variant": info["variant"],
                      "ms": [round(t, 3) for t in times], "status_ok": ok, "max_abs_err": err}))
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
