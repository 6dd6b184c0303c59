#!/usr/bin/env python
"""Host-buffer AllReduce (fp32 sum), this library against the unmodified reference library, both
over their socket bootstraps on this machine's CPUs: no GPU involved. The reference is the build
of baseline/build_ref.py (baseline/_ref/libhxccl_ref.so).

    python bench/host_vs_reference.py [--ranks 4] [--iters 20] [--coll allreduce]

Inputs are uniform in (-1, 1) from seed 1234 + rank in `--dtype` (float32 unless given). `--coll` is allreduce, allgather, reducescatter, broadcast or alltoall; `bytes` is the size of the
larger of the two buffers of a rank (the whole gathered vector for allgather, the whole input for
reducescatter and alltoall).

Every rank times `iters` calls per size after 5 warm-up calls between barriers (a one-element
AllReduce of the same library); a run's figure is the median over calls of the maximum over ranks,
as in the reference's bench/hxccl_perf.cc:36-49. The libraries alternate for `--rounds` runs each
and the best run of each is printed, one JSON line per size.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import multiprocessing as mp
import os
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
REF = ROOT / "baseline" / "_ref" / "libhxccl_ref.so"
STUB = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "lib64" / "stubs" / "libcuda.so"


# name -> (hxcclDataType_t, element bytes)
DTYPES = {"int32": (2, 4), "float16": (6, 2), "float32": (7, 4), "float64": (8, 8), "bfloat16": (9, 2),
          "float8e4m3": (10, 1)}


class Id(C.Structure):
    _fields_ = [("internal", C.c_char * 128)]


def load(which: str):
    if which == "reference":
        try:
            C.CDLL("libcuda.so.1", mode=C.RTLD_GLOBAL)
        except OSError:
            C.CDLL(str(STUB), mode=C.RTLD_GLOBAL)  # its CUDA build links the driver; the host path never calls it
        lib = C.CDLL(str(REF))
    else:
        from hxccl_b200 import _lib  # noqa: PLC0415

        lib = _lib.lib()
    vp = C.c_void_p
    lib.hxcclGetUniqueId.argtypes = [C.POINTER(Id)]
    lib.hxcclCommInitRank.argtypes = [C.POINTER(vp), C.c_int, Id, C.c_int]
    lib.hxcclAllReduce.argtypes = [vp, vp, C.c_size_t, C.c_int, C.c_int, vp, vp]
    lib.hxcclAllGather.argtypes = [vp, vp, C.c_size_t, C.c_int, vp, vp]
    lib.hxcclReduceScatter.argtypes = [vp, vp, C.c_size_t, C.c_int, C.c_int, vp, vp]
    lib.hxcclBroadcast.argtypes = [vp, vp, C.c_size_t, C.c_int, C.c_int, vp, vp]
    lib.hxcclAlltoAll.argtypes = [vp, vp, C.c_size_t, C.c_int, vp, vp]
    lib.hxcclCommDestroy.argtypes = [vp]
    return lib


def child(which, coll, op, dtype, rank, n, sizes, iters, id_q, out_q):
    import numpy as np

    os.environ["HXCCL_DEVICE"] = "0"
    lib = load(which)
    uid = Id()
    if rank == 0:
        assert lib.hxcclGetUniqueId(C.byref(uid)) == 0
        for _ in range(n - 1):
            id_q.put(bytes(uid))
    else:
        uid = Id.from_buffer_copy(id_q.get(timeout=60))
    comm = C.c_void_p()
    assert lib.hxcclCommInitRank(C.byref(comm), n, uid, rank) == 0
    one = np.zeros(1, dtype=np.float32)

    def barrier():
        assert lib.hxcclAllReduce(one.ctypes.data, one.ctypes.data, 1, 7, 0, comm, None) == 0

    rows = []
    for size in sizes:
        code, es = DTYPES[dtype]
        whole = max(n, size // es // n * n)  # elements, a multiple of the rank count
        u = np.random.default_rng(1234 + rank).uniform(-1.0, 1.0, whole)
        if dtype == "bfloat16":      # the upper half of the fp32 pattern
            x = (u.astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
        elif dtype == "float8e4m3":  # small finite codes of either sign
            x = (np.random.default_rng(1234 + rank).integers(0, 256, whole) & 0xBF).astype(np.uint8)
        elif dtype == "int32":
            x = (u * 1000).astype(np.int32)
        else:
            x = u.astype({"float32": np.float32, "float16": np.float16, "float64": np.float64}[dtype])
        y = np.empty_like(x)
        xp, yp, part = x.ctypes.data, y.ctypes.data, whole // n
        call = {
            "allreduce": lambda: lib.hxcclAllReduce(xp, yp, whole, code, op, comm, None),
            "allgather": lambda: lib.hxcclAllGather(xp, yp, part, code, comm, None),
            "reducescatter": lambda: lib.hxcclReduceScatter(xp, yp, part, code, op, comm, None),
            "broadcast": lambda: lib.hxcclBroadcast(xp, yp, whole, code, 0, comm, None),
            "alltoall": lambda: lib.hxcclAlltoAll(xp, yp, part, code, comm, None),
        }[coll]
        times = []
        for it in range(iters + 5):
            barrier()
            t0 = time.perf_counter()
            assert call() == 0
            if it >= 5:
                times.append(time.perf_counter() - t0)
        rows.append(times)
    lib.hxcclCommDestroy(comm)
    out_q.put((rank, rows))


def run(which, coll, op, dtype, n, sizes, iters):
    ctx = mp.get_context("spawn")
    id_q, out_q = ctx.Queue(), ctx.Queue()
    procs = [ctx.Process(target=child, args=(which, coll, op, dtype, r, n, sizes, iters, id_q, out_q)) for r in range(n)]
    for p in procs:
        p.start()
    got = dict(out_q.get(timeout=600) for _ in range(n))
    for p in procs:
        p.join(10)
    med = []
    for k in range(len(sizes)):
        worst = sorted(max(got[r][k][i] for r in range(n)) for i in range(iters))
        med.append(worst[len(worst) // 2])
    return med


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ranks", type=int, default=4)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--coll", default="allreduce",
                    choices=["allreduce", "allgather", "reducescatter", "broadcast", "alltoall"])
    ap.add_argument("--dtype", default="float32", choices=sorted(DTYPES))
    ap.add_argument("--op", default="sum", choices=["sum", "avg"], help="for allreduce and reducescatter")
    ap.add_argument("--rounds", type=int, default=3, help="alternating runs of each library")
    ap.add_argument("--sizes", default="256,16384,65536,1048576,4194304,16777216,67108864")
    args = ap.parse_args()
    sizes = [int(s) for s in args.sizes.split(",")]
    # the two libraries take turns, and the best median of each counts: other tenants of the
    # machine move single runs by tens of per cent
    ours, ref = None, None
    for _ in range(max(1, args.rounds)):
        op = {"sum": 0, "avg": 4}[args.op]
        a = run("hxccl", args.coll, op, args.dtype, args.ranks, sizes, args.iters)
        ours = a if ours is None else [min(x, y) for x, y in zip(ours, a)]
        if REF.exists():
            b = run("reference", args.coll, op, args.dtype, args.ranks, sizes, args.iters)
            ref = b if ref is None else [min(x, y) for x, y in zip(ref, b)]
    if ref is None:
        ref = [None] * len(sizes)
    n = args.ranks
    f = {"allreduce": 2.0 * (n - 1) / n, "broadcast": 1.0}.get(args.coll, (n - 1) / n)
    for size, a, b in zip(sizes, ours, ref):
        print(json.dumps({"coll": args.coll, "op": args.op, "dtype": args.dtype, "ranks": args.ranks, "bytes": size, "hxccl_us": round(a * 1e6, 1),
                          "hxccl_busbw_GBps": round(size / a / 1e9 * f, 3),
                          "reference_us": None if b is None else round(b * 1e6, 1),
                          "reference_busbw_GBps": None if b is None else round(size / b / 1e9 * f, 3),
                          "hxccl_time_over_reference": None if b is None else round(a / b, 2)}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
