#!/usr/bin/env python
"""One collective of the single-GPU world harness, run a few times: the small, single-process
case used for Nsight Compute captures of the collective kernels (a multi-rank job must never
run under ncu) and for timing them without any link in the way.

    python bench/world_case.py --n 2 --mb 256 --variant 2 --dtype float32 --iters 3
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
        times = []
        for _ in range(args.iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            w.all_reduce(xs, ys, count, dt, op=hx.SUM, order=args.order)
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        ok = all(w.status(r) == (0, 0) for r in range(args.n))
        info = w.info()
    ref = sum(x.double() for x in xs)
    err = float((ys[0].double() - ref).abs().max())
    print(json.dumps({"n": args.n, "bytes_per_rank": args.bytes or (args.mb << 20), "order": args.order, "dtype": args.dtype, "variant": info["variant"],
                      "ms": [round(t, 3) for t in times], "status_ok": ok, "max_abs_err": err}))
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
