#!/usr/bin/env python
"""Throughput of the standalone elementwise kernels (dst = dst op src, scale, divide) against
the measured copy bandwidth of the GPU (MEASURED_PEAKS.json when present, else 6650 GB/s).

    python bench/elementwise.py [--mb 1024] [--iters 10]
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--mb", type=int, default=1024, help="bytes of each operand in MiB")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--only", default="", help="one dtype name, e.g. float32")
    args = ap.parse_args()

    import torch

    from hxccl_b200 import _lib as L

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    peak, src = 6650.0, "fallback"
    try:
        peak, src = float(json.load(open(os.path.join(root, "MEASURED_PEAKS.json")))["hbm_gbs"]), "measured"
    except (OSError, KeyError, ValueError):
        pass
    lib = L.lib()
    nbytes = args.mb << 20
    a = torch.randint(0, 255, (nbytes,), dtype=torch.uint8, device="cuda")
    b = torch.randint(0, 255, (nbytes,), dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    rows = []
    for name, dt in (("float32", L.FLOAT32), ("bfloat16", L.BFLOAT16), ("float16", L.FLOAT16), ("int32", L.INT32),
                     ("float64", L.FLOAT64), ("float8_e4m3", L.FLOAT8E4M3), ("int8", L.INT8)):
        if args.only and args.only != name:
            continue
        count = nbytes // L.DTYPE_SIZE[dt]
        for _ in range(3):
            lib.hxcclDevReduce(a.data_ptr(), b.data_ptr(), count, dt, L.SUM, stream)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            assert lib.hxcclDevReduce(a.data_ptr(), b.data_ptr(), count, dt, L.SUM, stream) == 0
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.iters
        gbs = 3 * nbytes / (ms * 1e-3) / 1e9  # two reads and one write per element
        rows.append({"kernel": "reduce sum", "dtype": name, "ms": round(ms, 4), "GBps": round(gbs, 1),
                     f"frac_of_{src}_copy_bw": round(gbs / peak, 3)})
    print(json.dumps({"operand_MiB": args.mb, "peak_GBps": peak, "peak_source": src, "rows": rows}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
