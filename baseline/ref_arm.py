"""Reference arm of bench.py: the same AllReduce measurement through the unmodified reference
library (baseline/_ref/libhxccl_ref.so, built by baseline/build_ref.py from the reference's own
sources) and its own public C API: hxcclGetUniqueId, hxcclCommInitRank, hxcclAllReduce on device
buffers. Nothing of this repository's library is loaded in this process. The reference's calls
block until the data has arrived, so the CUDA events around the timed loop measure completed
work."""
from __future__ import annotations

import ctypes as C
import json
import os
from pathlib import Path

LIB = Path(__file__).resolve().parent / "_ref" / "libhxccl_ref.so"


class UniqueId(C.Structure):
    _fields_ = [("internal", C.c_char * 128)]


# published device AllReduce of the reference at 256 MiB fp32 as bus bandwidth (its README's device
# table: 43028 us with two ranks, 110449 us with four, all on one RTX 3060 Ti); nothing else matches
PUBLISHED_BUSBW_256MIB = {2: 268435456 / 43028e-6 / 1e9 * 1.0, 4: 268435456 / 110449e-6 / 1e9 * 1.5}


def vs_published(value: float, world: int, nbytes: int, dtype: str):
    ref = PUBLISHED_BUSBW_256MIB.get(world) if (nbytes == 268435456 and dtype == "float32") else None
    return round(value / ref, 2) if ref else None


def unavailable(rank: int, why: str) -> int:
    if rank == 0:
        print(json.dumps({"impl": "reference", "unavailable": why[:300]}))
    return 0


def run(args, rank: int, world: int, local: int, config_of=None) -> int:
    if not LIB.exists():
        return unavailable(rank, "baseline/_ref/libhxccl_ref.so is missing: the reference has no setup.py/pyproject "
                                 "(pip install refuses it) and baseline/build_ref.py was not run where its sources are")
    import torch
    import torch.distributed as dist

    torch.cuda.set_device(local)
    torch.zeros(1, device="cuda")
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        lib = C.CDLL(str(LIB))
    except OSError as e:
        return unavailable(rank, f"cannot load the reference library: {e}")
    vp = C.c_void_p
    lib.hxcclGetUniqueId.argtypes = [C.POINTER(UniqueId)]
    lib.hxcclCommInitRank.argtypes = [C.POINTER(vp), C.c_int, UniqueId, C.c_int]
    lib.hxcclAllReduce.argtypes = [vp, vp, C.c_size_t, C.c_int, C.c_int, vp, vp]
    lib.hxcclCommDestroy.argtypes = [vp]
    lib.hxcclGetLastError.argtypes = [vp]
    lib.hxcclGetLastError.restype = C.c_char_p

    uid = UniqueId()
    if rank == 0 and lib.hxcclGetUniqueId(C.byref(uid)) != 0:
        return unavailable(rank, "the reference's hxcclGetUniqueId failed")
    box = [bytes(uid)]
    if world > 1:
        dist.broadcast_object_list(box, src=0)
    uid = UniqueId.from_buffer_copy(box[0])
    comm = vp()
    rc = lib.hxcclCommInitRank(C.byref(comm), world, uid, rank)
    if rc != 0:
        return unavailable(rank, f"the reference's hxcclCommInitRank returned {rc}")

    tdt = getattr(torch, args.dtype)
    dt_code = {"float32": 7, "bfloat16": 9, "float16": 6}[args.dtype]
    es = torch.empty(0, dtype=tdt).element_size()
    count = args.bytes // es
    nbytes = count * es
    g = torch.Generator(device="cuda").manual_seed(1234 + rank)
    src = torch.rand(count, generator=g, device="cuda", dtype=torch.float32).mul_(2).sub_(1).to(tdt)
    dst = src.clone()
    stream = torch.cuda.current_stream()

    def allreduce(a, b):
        r = lib.hxcclAllReduce(a.data_ptr(), b.data_ptr(), a.numel(), dt_code, 0, comm, stream.cuda_stream)
        if r != 0:
            raise RuntimeError(f"reference hxcclAllReduce failed ({r}): {lib.hxcclGetLastError(comm).decode()}")

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    def max_over_ranks(v):
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        barrier()
        return max_over_ranks(e0.elapsed_time(e1) / steps)

    try:
        # same form as the library's own arm: in place, except with one rank (no work in place)
        step = (lambda: allreduce(src, dst)) if world == 1 else (lambda: allreduce(dst, dst))
        ms = timed(step, args.steps, max(args.warmup, 3))
        host_in = torch.empty(count, dtype=tdt).pin_memory()
        host_in.copy_(src.cpu())
        host_out = torch.empty(4096 // es, dtype=tdt).pin_memory()
        dev_in = torch.empty_like(src)

        def e2e_step():
            dev_in.copy_(host_in, non_blocking=True)
            allreduce(dev_in, dst)
            host_out.copy_(dst[: host_out.numel()], non_blocking=True)
            stream.synchronize()

        e2e_ms = timed(e2e_step, max(3, args.steps // 2), 3)
    except RuntimeError as e:
        return unavailable(rank, str(e))
    factor = 2.0 * (world - 1) / world if world > 1 else 1.0
    algbw = nbytes / (ms * 1e-3) / 1e9
    lib.hxcclCommDestroy(comm)
    if world > 1:
        dist.destroy_process_group()
    config = config_of(world, nbytes, count) if config_of else {"bytes_per_rank": nbytes}
    if rank == 0:
        print(json.dumps({
            "metric": "allreduce_busbw_GBps", "value": round(algbw * factor, 3), "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": vs_published(algbw * factor, world, nbytes, args.dtype), "dtype": args.dtype, "data": "synthetic U(-1,1), seed 1234+rank",
            "impl": "reference",
            "config": config,
            "impl_note": "unmodified reference sources (MPI stand-in header at compile time, socket bootstrap, "
                         "CUDA IPC staging path); its calls block, events bracket completed work",
            "algbw_GBps": round(algbw, 3),
            "e2e": {"value": round(nbytes / (e2e_ms * 1e-3) / 1e9 * factor, 3), "unit": "GB/s",
                    "ms_per_step": round(e2e_ms, 4), "h2d_bytes_per_step": nbytes,
                    "d2h_bytes_per_step": host_out.numel() * es},
            "gpu_launches": 0}))
    return 0
