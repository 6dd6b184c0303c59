#!/usr/bin/env python
"""Headline benchmark: AllReduce bus bandwidth (and small-message latency) on N B200s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--bytes B] [--dtype float32]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One step is one in-place fp32 sum AllReduce of `--bytes` per rank (default 256 MiB, larger
than the 126 MB L2, so consecutive steps do not hit in cache). K steps are timed with CUDA
events on the launching stream between barriers, the maximum over ranks is taken, and rank 0
prints one JSON line. `value` is the bus bandwidth in GB/s by the nccl-tests convention,
algbw * 2(N-1)/N; with one GPU that factor is zero, so there `value` is the algorithm bandwidth
of the local AllReduce (a copy) and `config.note` says so. The `e2e` figure repeats the
measurement through the public Python API with the input copied from pinned host memory and a
slice of the result read back every step. Before anything is timed the full-size result is
checked: bit for bit against a replay of the reduction order on rank 0 (`verified`), and by
tolerance against an fp64 sum for the in-switch `fast_mode`. The `nccl` block repeats a short
size sweep with torch's NCCL backend in the same process, next to this library's `sweep`.
`--impl reference` runs the unmodified reference library (built by baseline/build_ref.py from
its sources) instead when that build is present, else reports why not.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--bytes", type=int, default=256 << 20)
    ap.add_argument("--dtype", default="float32")
    ap.add_argument("--impl", default="hxccl", choices=["hxccl", "reference", "nccl"])
    ap.add_argument("--exact", type=int, default=1, help="1: bit-exact reduction order; 0: NVLS fast mode")
    ap.add_argument("--no-sweep", action="store_true", help="skip the small size sweep in the extras")
    ap.add_argument("--no-nccl", action="store_true", help="skip the NCCL comparison in the extras")
    ap.add_argument("--bind-numa", type=int, default=1,
                    help="1: pin the rank to the CPUs next to its GPU before host buffers are allocated")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons of this rank's GPU while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            pass

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def reference_unavailable(reason: str) -> None:
    print(json.dumps({"impl": "reference", "unavailable": reason}))


# The reference's published device AllReduce (fp32 sum, 256 MiB) as bus bandwidth: 43028 us with
# two ranks and 110449 us with four, all ranks sharing one RTX 3060 Ti (its README, device table).
# Nothing is published for one or eight ranks, for other sizes of this benchmark, or for B200.
PUBLISHED_BUSBW_256MIB = {2: 268435456 / 43028e-6 / 1e9 * 1.0, 4: 268435456 / 110449e-6 / 1e9 * 1.5}


def bench_config(world: int, nbytes: int, count: int) -> dict:
    """The workload, in the same words for every arm."""
    return {"model": "AllReduce sum, in place" if world > 1 else "AllReduce sum, out of place (one rank)",
            "global_batch": nbytes * world, "seq_len": count,
            "parallelism": f"{world} ranks, one per GPU", "bytes_per_rank": nbytes,
            "note": ("one GPU: value is the algorithm bandwidth of the local out-of-place AllReduce (bus factor is 0)"
                     if world == 1 else "value = algbw * 2(N-1)/N (nccl-tests bus bandwidth)")}


def vs_published(value: float, world: int, nbytes: int, dtype: str):
    ref = PUBLISHED_BUSBW_256MIB.get(world) if (nbytes == 268435456 and dtype == "float32") else None
    return round(value / ref, 2) if ref else None



def main() -> int:
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        try:
            import ref_arm  # noqa: PLC0415
        except Exception as e:  # noqa: BLE001
            if rank == 0:
                reference_unavailable(f"reference arm could not be loaded: {e!r}"[:200])
            return 0
        return ref_arm.run(args, rank, world, local, bench_config)

    import torch  # noqa: PLC0415
    import torch.distributed as dist  # noqa: PLC0415

    torch.cuda.set_device(local)
    torch.zeros(1, device="cuda")
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("gloo", rank=rank, world_size=world)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    def max_over_ranks(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    tdt = getattr(torch, args.dtype)
    es = torch.empty(0, dtype=tdt).element_size()
    count = args.bytes // es
    nbytes = count * es

    if args.impl == "nccl":
        comm = None
        os.environ.setdefault("MASTER_PORT", "29533")
        nccl_pg = dist.new_group(backend="nccl") if world > 1 else None

        def allreduce(src, dst):
            # torch's all_reduce is in place; the timed loops below pass src is dst
            if src is not dst:
                dst.copy_(src)
            if nccl_pg is not None:
                dist.all_reduce(dst, group=nccl_pg)
        launches_of = lambda: 0  # noqa: E731
    else:
        import hxccl_b200 as hx  # noqa: PLC0415

        uid = [hx.get_unique_id() if rank == 0 else None]
        if world > 1:
            dist.broadcast_object_list(uid, src=0)
        comm = hx.Communicator.init_rank(uid[0], world, rank)
        comm.tune(variant=0, exact=bool(args.exact))
        info = comm.device_info()
        if info["kind"] == "none":
            raise RuntimeError("the hxccl device path did not start (libhxccl.so without a GPU?)")

        def allreduce(src, dst):
            comm.all_reduce(src, dst, op=hx.SUM)
        launches_of = lambda: comm.device_info()["launches"]  # noqa: E731

    g = torch.Generator(device="cuda").manual_seed(1234 + rank)
    src = torch.rand(count, generator=g, device="cuda", dtype=torch.float32).mul_(2).sub_(1).to(tdt)
    dst = torch.empty_like(src)
    stream = torch.cuda.current_stream()

    def timed(fn, steps: int, warmup: int) -> float:
        """ms per step, device-timed, max over ranks."""
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

    # ---- correctness of the full-size result, before any timing ------------------------------
    def replay_on_rank0():
        """The reference's ring order (block c starts at rank c, then c+1, c+2, ... each added as
        the left operand) replayed with plain tensor adds from the regenerated inputs of all
        ranks; fp32 / bf16 adds round once per hop exactly as the kernels do. Also an fp64 sum."""
        xs = []
        for r in range(world):
            gr = torch.Generator(device="cuda").manual_seed(1234 + r)
            xs.append(torch.rand(count, generator=gr, device="cuda", dtype=torch.float32).mul_(2).sub_(1).to(tdt))
        exact = torch.empty_like(xs[0])
        wide = torch.zeros(count, dtype=torch.float64, device="cuda")
        base, extra = divmod(count, world)
        for c in range(world):
            lo = c * base + min(c, extra)
            hi = lo + base + (1 if c < extra else 0)
            acc = xs[c][lo:hi].clone()
            for k in range(1, world):
                acc = xs[(c + k) % world][lo:hi] + acc
            exact[lo:hi] = acc
        for x in xs:
            wide += x.double()
        return exact, wide

    def check_result(expect_exact: bool):
        """Runs one out-of-place AllReduce of the full message and compares rank 0's result."""
        dst.zero_()
        allreduce(src, dst)
        torch.cuda.synchronize()
        out = None
        if rank == 0:
            exact, wide = replay_on_rank0()
            if expect_exact:
                same = bool(torch.equal(dst, exact))
                out = True if same else {"max_abs_diff": float((dst.double() - exact.double()).abs().max())}
            else:
                err = float((dst.double() - wide).abs().max())
                tol = world * (2.0 ** -22 if tdt == torch.float32 else 2.0 ** -7) * 4
                out = {"max_abs_err_vs_fp64": err, "tolerance": tol, "ok": err <= tol}
            del exact, wide
        barrier()
        return out

    verified = check_result(True) if (comm is not None and nbytes >= (64 << 10)) else None
    variant_checked = comm.device_info()["variant"] if comm is not None else None

    # ---- headline: kernel-only -------------------------------------------------------------
    sampler = ClockSampler(local) if rank == 0 else None
    for _ in range(max(args.warmup, 3)):
        allreduce(src, dst)
    barrier()
    l0 = launches_of()
    # in place on `dst`, the form torch.distributed offers, so that every arm does the same work.
    # With one rank an in-place AllReduce is no work at all (in this library and in the reference),
    # so the single-GPU run is out of place: the whole message is read and written once.
    dst.copy_(src)
    step = (lambda: allreduce(src, dst)) if world == 1 else (lambda: allreduce(dst, dst))
    ms = timed(step, args.steps, 0)
    launches = launches_of() - l0
    headline_path = comm.device_info() if comm is not None else {"kind": "nccl"}
    factor = 2.0 * (world - 1) / world if world > 1 else 1.0
    algbw = nbytes / (ms * 1e-3) / 1e9
    value = algbw * factor

    # ---- end to end: pinned host -> device, AllReduce, slice of the result back -------------
    numa = None
    if comm is not None and args.bind_numa:
        from hxccl_b200.utils.env import bind_to_gpu_numa  # noqa: PLC0415

        numa = bind_to_gpu_numa(local)  # before the pinned buffers exist: they follow the CPUs
    host_in = torch.empty(count, dtype=tdt).pin_memory()
    host_in.copy_(src.cpu())
    host_out = torch.empty(4096 // es, dtype=tdt).pin_memory()
    dev_in = torch.empty_like(src)

    def e2e_step():
        dev_in.copy_(host_in, non_blocking=True)
        allreduce(dev_in, dst)
        host_out.copy_(dst[: host_out.numel()], non_blocking=True)
        stream.synchronize()  # the caller reads the result every step

    e2e_ms = timed(e2e_step, max(3, args.steps // 2), 3)
    e2e_value = nbytes / (e2e_ms * 1e-3) / 1e9 * factor

    # ---- extras: the same step with bit-exactness switched off (NVLS in-switch reduction) -------
    fast = None
    if comm is not None and world > 2 and args.exact and "nvls" in info["kind"]:
        comm.tune(variant=0, exact=False)
        fast_check = check_result(False)
        dst.copy_(src)
        fast_ms = timed(lambda: allreduce(dst, dst), args.steps, 3)
        fast = {"value": round(nbytes / (fast_ms * 1e-3) / 1e9 * factor, 2), "unit": "GB/s",
                "ms_per_step": round(fast_ms, 4), "variant": comm.device_info()["variant"], "checked": fast_check,
                "note": "HXCCL_EXACT=0: float sums combined by the switch, order unspecified"}
        comm.tune(variant=0, exact=True)

    # ---- extras: latency and a short sweep ------------------------------------------------------
    # In place like the headline. A sum in place grows by a factor of N per call, so the values
    # are reset before each size and the calls per size are bounded to keep them finite.
    sweep_sizes = (8, 1024, 64 << 10, 1 << 20, 16 << 20, 64 << 20)
    sweep_warmup = 5
    most_calls = int(120 / max(1.0, __import__("math").log2(max(world, 2))))

    def sweep_with(fn) -> list:
        rows = []
        for sz in sweep_sizes:
            n_el = max(1, sz // es)
            a, b = src[:n_el], dst[:n_el]
            b.copy_(a)
            steps = min(50 if sz <= (1 << 20) else 20, most_calls - sweep_warmup)
            t = timed((lambda: fn(a, b)) if world == 1 else (lambda: fn(b, b)), steps, sweep_warmup)
            rows.append({"bytes": n_el * es, "us": round(t * 1e3, 2),
                         "busbw_GBps": round(n_el * es / (t * 1e-3) / 1e9 * factor, 2)})
        return rows

    sweep = sweep_with(allreduce) if not args.no_sweep else []

    # ---- extras: the same step through the neighbour-ring kernel (bit-exact like the headline).
    # Last of all measurements and guarded: whatever happens here cannot cost the figures above.
    ring = None
    if comm is not None and world > 1 and args.exact:
        try:
            comm.tune(variant=6, exact=True)
            ring_check = check_result(True)
            dst.copy_(src)
            ring_ms = timed(lambda: allreduce(dst, dst), args.steps, 3)
            ring = {"value": round(nbytes / (ring_ms * 1e-3) / 1e9 * factor, 2), "unit": "GB/s",
                    "ms_per_step": round(ring_ms, 4), "variant": comm.device_info()["variant"], "verified": ring_check,
                    "note": "HXCCL_VARIANT=ring: reduce-scatter and all-gather around the ring, same bits"}
            comm.tune(variant=0, exact=True)
        except Exception as e:  # noqa: BLE001
            ring = {"error": str(e)[:200]}

    clocks = sampler.stop() if sampler else None
    if comm is not None:
        err = comm.async_error()
        comm.destroy()
    else:
        err = 0

    # ---- extras: torch's NCCL backend on the same sizes, same process, same timing -------------
    nccl = None
    if args.impl == "hxccl" and world > 1 and not args.no_sweep and not args.no_nccl:
        saved_stdout = None
        try:
            os.environ.setdefault("MASTER_PORT", "29533")
            # NCCL prints its banner (and, with NCCL_DEBUG set, its log) on stdout: this program's
            # stdout is one JSON line, so while NCCL runs fd 1 is stderr's file
            sys.stdout.flush()
            saved_stdout = os.dup(1)
            os.dup2(2, 1)
            pg = dist.new_group(backend="nccl")

            def nccl_allreduce(a, b):
                dist.all_reduce(b, group=pg)

            rows = sweep_with(nccl_allreduce)
            dst.copy_(src)
            big_ms = timed(lambda: nccl_allreduce(dst, dst), args.steps, 3)
            rows.append({"bytes": nbytes, "us": round(big_ms * 1e3, 2),
                         "busbw_GBps": round(nbytes / (big_ms * 1e-3) / 1e9 * factor, 2)})
            nccl = {"version": ".".join(map(str, torch.cuda.nccl.version())), "sweep": rows,
                    "note": "torch.distributed all_reduce, NCCL backend, in place, fp32 sum"}
        except Exception as e:  # noqa: BLE001
            nccl = {"error": str(e)[:200]}
        finally:
            if saved_stdout is not None:
                torch.cuda.synchronize()
                os.dup2(saved_stdout, 1)
                os.close(saved_stdout)
    if world > 1:
        dist.destroy_process_group()
    if rank == 0:
        line = {
            "metric": "allreduce_busbw_GBps", "value": round(value, 2), "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 4),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": vs_published(value, world, nbytes, args.dtype),
            "dtype": args.dtype,
            "data": "synthetic U(-1,1), seed 1234+rank", "impl": args.impl,
            "config": bench_config(world, nbytes, count),
            "l2_policy": "message larger than L2 (126 MB): no flush needed",
            "exact_order": bool(args.exact), "device_path": headline_path,
            "verified": verified, "verified_variant": variant_checked,
            "algbw_GBps": round(algbw, 2),
            "e2e": {"value": round(e2e_value, 2), "unit": "GB/s", "ms_per_step": round(e2e_ms, 4),
                    "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": host_out.numel() * es, "numa": numa},
            "gpu_launches": int(launches), "clocks": clocks, "fast_mode": fast, "ring_mode": ring, "sweep": sweep, "nccl": nccl, "async_error": err,
        }
        print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
