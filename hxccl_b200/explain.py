"""Which AllReduce kernel the tuner picks, size by size, without a GPU.

    python -m hxccl_b200.explain --ranks 8 [--dtype float32] [--fast] [--no-nvls] [--from 8] [--to 1G]

Prints one line per size (doubling): the variant, whether a row of the tuning table decided or
the fixed thresholds did, and the launch shape the row sets (grid limit, CTA width, bytes per
CTA and step). The compiled-in table is used, then `HXCCL_TUNE_FILE` when set, exactly as a
communicator does at creation (src/device/planner.cc: choose_variant, find_row, with_row).
"""
from __future__ import annotations

import argparse
import ctypes as C
import sys

from . import _lib as L

VARIANTS = {0: "auto", 1: "oneshot", 2: "twoshot", 3: "nvls", 4: "twoshot_roles", 5: "nvls_roles", 6: "ring", 7: "lines"}
DTYPES = {"int8": L.INT8, "uint8": L.UINT8, "int32": L.INT32, "uint32": L.UINT32, "int64": L.INT64,
          "uint64": L.UINT64, "float16": L.FLOAT16, "float32": L.FLOAT32, "float64": L.FLOAT64,
          "bfloat16": L.BFLOAT16, "float8e4m3": L.FLOAT8E4M3, "float8e5m2": L.FLOAT8E5M2}


def parse_size(s: str) -> int:
    mult = {"K": 1 << 10, "M": 1 << 20, "G": 1 << 30}
    return int(s[:-1]) * mult[s[-1].upper()] if s[-1].upper() in mult else int(s)


def choose(nbytes: int, dtype: int, ranks: int, exact: bool = True, nvls: bool = True):
    """(variant name, decided by a table row, [grid limit, CTA width, bytes per CTA and step])."""
    lib = L.lib()
    lib.hxcclTestChooseVariant.argtypes = [C.c_size_t, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int),
                                           C.POINTER(C.c_int), C.POINTER(C.c_size_t)]
    v, tab = C.c_int(), C.c_int()
    shape = (C.c_size_t * 3)()
    rc = lib.hxcclTestChooseVariant(nbytes, dtype, ranks, int(exact), int(nvls), C.byref(v), C.byref(tab), shape)
    if rc:
        raise ValueError(f"hxcclTestChooseVariant: result {rc} (ranks 2..16, a readable HXCCL_TUNE_FILE)")
    return VARIANTS.get(v.value, str(v.value)), bool(tab.value), list(shape)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--ranks", type=int, default=8)
    ap.add_argument("--dtype", default="float32", choices=sorted(DTYPES))
    ap.add_argument("--fast", action="store_true", help="HXCCL_EXACT=0: in-switch float sums allowed")
    ap.add_argument("--no-nvls", action="store_true", help="a node without NVSwitch multicast")
    ap.add_argument("--from", dest="lo", default="8")
    ap.add_argument("--to", dest="hi", default="1G")
    args = ap.parse_args(argv)
    size, hi = parse_size(args.lo), parse_size(args.hi)
    print(f"{'bytes':>12}  {'variant':<14} {'decided by':<11} grid limit  CTA width  bytes per CTA and step")
    last = None
    while size <= hi:
        name, tabled, (ctas, threads, sub) = choose(size, DTYPES[args.dtype], args.ranks, not args.fast, not args.no_nvls)
        row = (name, tabled, ctas, threads, sub)
        mark = "" if row != last else "  (as above)"
        print(f"{size:>12}  {name:<14} {'table row' if tabled else 'thresholds':<11} {ctas:>10}  "
              f"{threads if threads else 'by size':>9}  {sub:>10}{mark}")
        last = row
        size *= 2
    return 0


if __name__ == "__main__":
    sys.exit(main())
