#!/usr/bin/env python
"""Tuning sweep: times AllReduce for several tuning settings and sizes in one launch.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench/sweep.py --sizes 16M,256M --configs 'MAX_CTAS=64;MAX_CTAS=128,THREADS=256'

Every configuration is a comma-separated list of HXCCL_<NAME>=<value> settings (read when the
communicator is created). Times are device-timed with CUDA events between barriers, maximum
over ranks; rank 0 prints one JSON line per (configuration, size). `--nccl` adds the
torch.distributed NCCL backend as a row of its own.

`--emit-tune FILE` is the tuner's measurement: for AllReduce (exact and fast mode), AllGather,
ReduceScatter and Broadcast it times every candidate variant and launch shape at every size
from 8 B to `--tune-max` (doubling), keeps the fastest per size (a challenger must beat the
previous size's winner by 3 % to take over), merges runs of equal winners and appends the rows
for this rank count to FILE in the format of HXCCL_TUNE_FILE / src/device/tune_default.inc.
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


DEFAULT_KNOBS = {"max_ctas": 128, "threads": 0, "ring_sub": 512 * 1024, "sub_max": 256 * 1024, "roles_min": 96 << 20,
                 "roles_min_ranks": 8, "roles_sub": 64 * 1024, "rs_ring_min": 256 << 20, "mc_force": -1, "grain": 16 * 1024}


def tune_candidates(coll: str, world: int, nbytes: int):
    """(label, forced variant, exact, knobs, row fields) of everything worth timing at this size."""
    ll_most = ((8 << 20) // 2 // world // 256 * 256) // 2
    c = []
    if coll in ("allreduce", "allreduce_fast"):
        if nbytes <= ll_most:
            c.append(("lines", 7, True, {}, {"variant": "lines"}))
        if nbytes <= (2 << 20):
            c.append(("oneshot", 1, True, {}, {"variant": "oneshot"}))
            if nbytes >= (32 << 10):
                c.append(("oneshot g4K", 1, True, {"grain": 4096}, {"variant": "oneshot", "grain": 4096}))
        if nbytes >= (16 << 10):
            c.append(("twoshot", 2, True, {"roles_min": 1 << 40}, {"variant": "twoshot"}))
            if (128 << 10) <= nbytes <= (64 << 20):
                c.append(("twoshot g4K", 2, True, {"roles_min": 1 << 40, "grain": 4096}, {"variant": "twoshot", "grain": 4096}))
            if nbytes >= (1 << 20):
                c.append(("twoshot c64", 2, True, {"roles_min": 1 << 40, "max_ctas": 64}, {"variant": "twoshot", "ctas": 64}))
        if nbytes >= (32 << 20) and world > 2:
            c.append(("twoshot_roles", 2, True, {"roles_min": 1, "roles_min_ranks": 2}, {"variant": "twoshot_roles"}))
        if nbytes >= (256 << 10):
            for threads, ctas, sub in ((512, 128, 512 << 10), (512, 128, 128 << 10), (512, 128, 64 << 10),
                                       (256, 256, 128 << 10), (256, 256, 64 << 10), (256, 256, 32 << 10)):
                c.append((f"ring t{threads} c{ctas} s{sub >> 10}K", 6, True,
                          {"threads": threads, "max_ctas": ctas, "ring_sub": sub},
                          {"variant": "ring", "threads": threads, "ctas": ctas, "sub": sub}))
        if coll == "allreduce_fast" and nbytes >= (16 << 10) and nbytes % 16 == 0 and world > 2:
            c.append(("nvls", 3, False, {"roles_min": 1 << 40}, {"variant": "nvls"}))
            if nbytes >= (32 << 20):
                c.append(("nvls_roles", 3, False, {"roles_min": 1}, {"variant": "nvls_roles"}))
    elif coll in ("allgather", "broadcast"):
        c.append(("unicast", 0, True, {"mc_force": 0}, {"variant": "unicast"}))
        c.append(("multicast", 0, True, {"mc_force": 1}, {"variant": "multicast"}))
        if (64 << 10) <= nbytes <= (64 << 20):
            c.append(("unicast g4K", 0, True, {"mc_force": 0, "grain": 4096}, {"variant": "unicast", "grain": 4096}))
            c.append(("multicast g4K", 0, True, {"mc_force": 1, "grain": 4096}, {"variant": "multicast", "grain": 4096}))
        if nbytes >= (1 << 20):
            c.append(("unicast t256 c256", 0, True, {"mc_force": 0, "threads": 256, "max_ctas": 256},
                      {"variant": "unicast", "threads": 256, "ctas": 256}))
            c.append(("multicast c64", 0, True, {"mc_force": 1, "max_ctas": 64}, {"variant": "multicast", "ctas": 64}))
    elif coll == "reducescatter":
        c.append(("push", 0, True, {"rs_ring_min": 0}, {"variant": "push"}))
        if (64 << 10) <= nbytes <= (64 << 20):
            c.append(("push g4K", 0, True, {"rs_ring_min": 0, "grain": 4096}, {"variant": "push", "grain": 4096}))
        if nbytes >= (64 << 10):
            c.append(("ring_rs", 0, True, {"rs_ring_min": 1}, {"variant": "ring_rs"}))
            for threads, ctas, sub in ((512, 128, 128 << 10), (256, 256, 128 << 10), (256, 256, 32 << 10)):
                c.append((f"ring_rs t{threads} c{ctas} s{sub >> 10}K", 0, True,
                          {"rs_ring_min": 1, "threads": threads, "max_ctas": ctas, "ring_sub": sub},
                          {"variant": "ring_rs", "threads": threads, "ctas": ctas, "sub": sub}))
    return c


def emit_tune(args, rank, world, buf, out, tdt, es, timed) -> None:
    import torch.distributed as dist

    import hxccl_b200 as hx

    uid = [hx.get_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(uid, src=0)
    comm = hx.Communicator.init_rank(uid[0], world, rank)
    comm.knob("table", 0)  # the candidates are forced; no row may reshape them
    nvls = "nvls" in comm.device_info()["kind"]
    top = parse_size(args.tune_max)
    lines = [f"# {world} ranks, {args.dtype}, measured by bench/sweep.py --emit-tune (us per call, winner first)"]
    for coll in args.tune_colls.split(","):
        if coll == "allreduce_fast" and (not nvls or world <= 2):
            continue
        rows, incumbent = [], None
        size = 8
        while size <= top:
            n_el = max(1, size // es)
            per = max(1, n_el // world)
            # what a table row is keyed by: the message for AllReduce / Broadcast, the block per rank otherwise
            key_bytes = n_el * es if coll in ("allreduce", "allreduce_fast", "broadcast") else per * es
            results = []
            for label, variant, exact, knobs, fields in tune_candidates(coll, world, n_el * es):
                if fields["variant"] == "multicast" and not nvls:
                    continue
                for k, v in DEFAULT_KNOBS.items():
                    comm.knob(k, knobs.get(k, v))
                comm.tune(variant=variant, exact=exact)
                if coll.startswith("allreduce"):
                    x = buf[:n_el]
                    fn = lambda: comm.all_reduce(x, x, op=hx.SUM)  # noqa: E731
                elif coll == "allgather":
                    fn = lambda: comm.all_gather(buf[:per], out[: per * world])  # noqa: E731
                elif coll == "reducescatter":
                    fn = lambda: comm.reduce_scatter(buf[: per * world], out[:per], op=hx.SUM)  # noqa: E731
                else:
                    x = buf[:n_el]
                    fn = lambda: comm.bcast(x, root=0)  # noqa: E731
                if size < (1 << 20):  # shorter than a launch: kernel time behind a backlog, best of three
                    ms = min(timed.backlogged(fn, 25) for _ in range(3))
                else:
                    ms = timed(fn, 10 if size >= (16 << 20) else 25)
                if comm.async_error():
                    raise RuntimeError(f"{coll} {label} at {size} bytes failed: {comm.last_error()}")
                results.append((ms, label, fields))
            results.sort(key=lambda r: r[0])
            best = results[0]
            if incumbent is not None:  # hysteresis: stay unless clearly beaten
                same = [r for r in results if r[2] == incumbent]
                if same and same[0][0] <= best[0] * (1.01 if size >= (16 << 20) else 1.03 if size >= (1 << 20) else 1.06):
                    best = same[0]
            incumbent = best[2]
            if rank == 0:
                print(json.dumps({"tune": coll, "bytes": size, "key_bytes": key_bytes, "winner": best[1],
                                  "us": {lab: round(ms * 1e3, 2) for ms, lab, _ in results}}), flush=True)
            if not rows or rows[-1][1] != best[2]:
                rows.append((0 if not rows else key_bytes, best[2], best[1], round(best[0] * 1e3, 2)))
            size *= 2
        name, mode = ("allreduce", "fast") if coll == "allreduce_fast" else (coll, "exact" if coll == "allreduce" else "any")
        for start, fields, label, us in rows:
            extra = " ".join(f"{k}={v}" for k, v in fields.items() if k != "variant")
            lines.append(f"row {name} n={world} mode={mode} from={start} variant={fields['variant']}"
                         + (f" {extra}" if extra else "") + f"  # {label}: {us} us at the first size")
    comm.destroy()
    if rank == 0:
        with open(args.emit_tune, "a") as f:
            f.write("\n".join(lines) + "\n")


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", default="8,64K,1M,16M,256M")
    ap.add_argument("--configs", default="")
    ap.add_argument("--dtype", default="float32")
    ap.add_argument("--op", default="sum")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--nccl", action="store_true")
    ap.add_argument("--emit-tune", default="", help="measure the candidates and append table rows to this file")
    ap.add_argument("--tune-max", default="1G", help="largest message of the tuning measurement")
    ap.add_argument("--tune-colls", default="allreduce,allreduce_fast,allgather,reducescatter,broadcast")
    ap.add_argument("--coll", default="allreduce",
                    choices=["allreduce", "allgather", "reducescatter", "alltoall", "broadcast"])
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
    if args.emit_tune:
        sizes = [parse_size(args.tune_max)]
    op = {"sum": hx.SUM, "max": hx.MAX, "avg": hx.AVG}[args.op]
    stream = torch.cuda.current_stream()
    big = max(sizes)
    buf = (torch.rand(max(big // es, 16), device="cuda") * 2 - 1).to(tdt)
    out = torch.empty(max(big // es, 16) * (world if args.coll == "allgather" else 1), dtype=tdt, device="cuda")
    factor = {"allreduce": 2.0 * (world - 1) / world, "allgather": (world - 1) / world,
              "reducescatter": (world - 1) / world, "alltoall": (world - 1) / world, "broadcast": 1.0}[args.coll]
    # An in-place sum grows by a factor of `world` per call: the buffer is restored before each
    # timing and the calls per timing are bounded so that the values stay finite.
    pristine = buf.clone() if args.coll == "allreduce" else None
    most_calls = int(120 / max(1.0, __import__("math").log2(max(world, 2))))

    def timed(fn, iters):
        if pristine is not None:
            buf.copy_(pristine)
            iters = max(1, min(iters, most_calls - 5))
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

    def timed_backlogged(fn, iters):
        """Device time per call for calls far shorter than the interpreter's cost of issuing them:
        a spin kernel of a couple of milliseconds goes first, the calls queue up behind it and
        then run back to back, so the events bracket kernel time only, not launch gaps."""
        if pristine is not None:
            buf.copy_(pristine)
            iters = max(1, min(iters, most_calls - 5))
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda._sleep(6_000_000)  # about 3 ms at 1.97 GHz
        e0.record(stream)
        for _ in range(iters):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / iters], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    timed.backlogged = timed_backlogged

    def report(name, size, ms, extra=None):
        if rank == 0:
            row = {"config": name, "coll": args.coll, "bytes": size, "us": round(ms * 1e3, 2),
                   "busbw_GBps": round(size / (ms * 1e-3) / 1e9 * factor, 1)}
            row.update(extra or {})
            print(json.dumps(row), flush=True)

    if args.emit_tune:
        emit_tune(args, rank, world, buf, out, tdt, es, timed)
        dist.destroy_process_group()
        return 0

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
            elif args.coll == "broadcast":
                x = buf[:n_el]
                fn = lambda: comm.bcast(x, root=0)  # noqa: E731
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
            elif args.coll == "broadcast":
                x = buf[:n_el]
                fn = lambda: dist.broadcast(x, src=0, group=pg)  # noqa: E731
            else:
                per = max(1, n_el // world)
                fn = lambda: dist.all_to_all_single(out[: per * world], buf[: per * world], group=pg)  # noqa: E731
            ms = timed(fn, args.iters if size >= (1 << 20) else 5 * args.iters)
            report("nccl", size, ms)
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
