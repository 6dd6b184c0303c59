#!/usr/bin/env python
"""Peer-copy bandwidth between two GPUs of one node: the link-rate denominator of the roofline
fractions quoted for the collective kernels (next to NVLink 5's nominal 900 GB/s per direction).

    python bench/peer_copy.py [--mb 1024] [--iters 10]

One process, two devices: a device-to-device copy 0 -> 1 (the copy engine's path over NVLink),
then both directions at once on two streams. Timed with CUDA events on the copying stream after
three warm-up copies; prints one JSON line.
"""
from __future__ import annotations

import argparse
import json


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--mb", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()

    import torch

    if torch.cuda.device_count() < 2:
        print(json.dumps({"unavailable": "needs two GPUs"}))
        return 0
    n = args.mb << 20
    a0 = torch.empty(n, dtype=torch.uint8, device="cuda:0").fill_(1)
    b1 = torch.empty(n, dtype=torch.uint8, device="cuda:1")
    a1 = torch.empty(n, dtype=torch.uint8, device="cuda:1").fill_(2)
    b0 = torch.empty(n, dtype=torch.uint8, device="cuda:0")
    s0, s1 = torch.cuda.Stream(device=0), torch.cuda.Stream(device=1)

    def one_way(iters):
        with torch.cuda.stream(s0):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(s0)
            for _ in range(iters):
                b1.copy_(a0, non_blocking=True)
            e1.record(s0)
        e1.synchronize()
        return e0.elapsed_time(e1) / iters

    def both_ways(iters):
        torch.cuda.synchronize(0)
        torch.cuda.synchronize(1)
        ev = []
        for s, dst, src in ((s0, b1, a0), (s1, b0, a1)):
            with torch.cuda.stream(s):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(s)
                for _ in range(iters):
                    dst.copy_(src, non_blocking=True)
                e1.record(s)
                ev.append((e0, e1))
        for _, e1 in ev:
            e1.synchronize()
        return max(e0.elapsed_time(e1) for e0, e1 in ev) / iters

    one_way(3)
    ms1 = one_way(args.iters)
    both_ways(3)
    ms2 = both_ways(args.iters)
    ok = bool((b1[:: n // 64] == 1).all()) and bool((b0[:: n // 64] == 2).all())
    print(json.dumps({"bytes": n, "one_direction_GBps": round(n / (ms1 * 1e-3) / 1e9, 1),
                      "both_directions_each_GBps": round(n / (ms2 * 1e-3) / 1e9, 1), "copied_ok": ok,
                      "nominal_GBps_per_direction": 900}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
