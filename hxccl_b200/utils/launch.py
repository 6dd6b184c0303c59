"""Runs a function as N ranks in N fresh processes on this machine (no MPI, no torchrun).

Rank 0 creates the unique id and hands it to the others through a pipe; each rank builds its
communicator and calls `fn(comm, rank, nranks, *args)`. The parent collects the return values
(anything picklable) and re-raises the first failure. With `gpus=True` rank r uses CUDA device
r % device_count and creates its context before the communicator, so the device path starts.
This is the stand-in for `mpirun -np N` that the reference's tests use (CMakeLists.txt:47-142).

GPU ranks get two defaults unless the caller's `env` says otherwise: a short device-side wait
limit (HXCCL_WAIT_LIMIT_MS) and NVSwitch multicast off (HXCCL_NVLS=0; pass `nvls=True` for the
runs that are about multicast). When one rank fails, the survivors are given longer than that
wait limit to leave through their bounded waits and destroy their communicator (which unbinds
the window from the multicast object) before any process is killed: a rank must not be ended
while its kernels spin or while its memory is bound to a multicast object.
"""
from __future__ import annotations

import multiprocessing as mp
import os
import traceback
from typing import Any, Callable, Dict, List, Optional


def _child(rank: int, n: int, fn: Callable, args: tuple, uid_recv, uid_send: List, out, env: Dict[str, str],
           gpus: bool, make_comm: bool, one_gpu: bool = False) -> None:
    try:
        import faulthandler  # noqa: PLC0415

        faulthandler.enable()
        os.environ.update(env)
        os.environ["HXCCL_RANK"] = str(rank)
        log_dir = os.environ.get("HXCCL_RANK_LOG_DIR")
        if log_dir:  # per-rank stderr (native code included) for post-mortems
            os.makedirs(log_dir, exist_ok=True)
            fd = os.open(os.path.join(log_dir, f"rank{rank}.log"), os.O_WRONLY | os.O_CREAT | os.O_APPEND)
            os.dup2(fd, 2)
        from hxccl_b200 import comm as hc  # noqa: PLC0415

        if gpus:
            import torch  # noqa: PLC0415

            torch.cuda.set_device(0 if one_gpu else rank % torch.cuda.device_count())
            torch.cuda.init()
            torch.zeros(1, device="cuda")
        if rank == 0:
            uid = hc.get_unique_id()
            for c in uid_send:
                c.send(uid)
        else:
            uid = uid_recv.recv()
        if make_comm:
            comm = hc.Communicator.init_rank(uid, n, rank)
            try:
                res = fn(comm, rank, n, *args)
            finally:
                if comm.handle:
                    comm.destroy()
        else:
            res = fn(uid, rank, n, *args)
        out.send(("ok", res))
    except BaseException as e:  # noqa: BLE001
        out.send(("err", f"rank {rank}: {e!r}\n{traceback.format_exc()}"))


GPU_WAIT_LIMIT_MS = 5000  # default device-side wait limit of ranks started with gpus=True


def run_ranks(n: int, fn: Callable, *args: Any, env: Optional[Dict[str, str]] = None, gpus: bool = False,
              timeout: float = 120.0, make_comm: bool = True,
              rank_env: Optional[Dict[int, Dict[str, str]]] = None, nvls: bool = False,
              one_gpu: bool = False) -> List[Any]:
    """Returns [fn's result on rank 0, ..., on rank n-1]. `fn` must be importable (module level).
    `rank_env[r]` adds environment variables for rank r only. `nvls` leaves NVSwitch multicast
    on for GPU ranks (default off, see the module text). `one_gpu` puts every GPU rank on device
    0 (the ranks then cannot share windows and fall back to the staged path together)."""
    ctx = mp.get_context("spawn")
    env = dict(env or {})
    if gpus:
        env.setdefault("HXCCL_WAIT_LIMIT_MS", os.environ.get("HXCCL_WAIT_LIMIT_MS", str(GPU_WAIT_LIMIT_MS)))
        if not nvls:
            env.setdefault("HXCCL_NVLS", "0")
    # how long a survivor may need to notice a dead peer and leave on its own
    try:
        grace = (float(env.get("HXCCL_WAIT_LIMIT_MS", 0)) / 1000.0 if gpus else 0.0) + 5.0
    except ValueError:
        grace = 10.0
    uid_pipes = [ctx.Pipe(duplex=False) for _ in range(n - 1)]
    outs = [ctx.Pipe(duplex=False) for _ in range(n)]
    procs = []
    for r in range(n):
        e = dict(env or {})
        e.update((rank_env or {}).get(r, {}))
        p = ctx.Process(target=_child, args=(r, n, fn, args, uid_pipes[r - 1][0] if r else None,
                                             [w for _, w in uid_pipes] if r == 0 else [], outs[r][1], e,
                                             gpus, make_comm, one_gpu))
        p.start()
        procs.append(p)
    results: List[Any] = [None] * n
    errors = []
    import time  # noqa: PLC0415

    deadline = time.monotonic() + timeout
    pending = set(range(n))
    shortened = False
    while pending:
        for r in sorted(pending):
            if outs[r][0].poll(0.05):
                try:
                    kind, val = outs[r][0].recv()
                except Exception as e:  # noqa: BLE001  (a result that cannot be rebuilt here)
                    kind, val = "err", f"rank {r}: its result could not be received: {e!r}"
                if kind == "ok":
                    results[r] = val
                else:
                    errors.append(val)
                pending.discard(r)
            elif not procs[r].is_alive() and not outs[r][0].poll(0):
                errors.append(f"rank {r}: process ended with exit code {procs[r].exitcode} and no result")
                pending.discard(r)
        if errors and not shortened:  # one rank failed: the others get the grace period to report
            deadline = min(deadline, time.monotonic() + grace)
            shortened = True
        if time.monotonic() > deadline:
            break
    for r in sorted(pending):
        errors.append(f"rank {r}: no result" + ("" if errors else f" within {timeout} s"))
    # Ranks that reported are on their way out (communicator destroyed in _child); the others
    # get the grace period once more, in total, before the last resort.
    give_up = time.monotonic() + (grace if errors else 5.0)
    for p in procs:
        p.join(max(0.1, give_up - time.monotonic()))
    for p in procs:
        if p.is_alive():
            p.kill()  # this exact child, by handle
            p.join()
    if errors:
        raise RuntimeError("\n".join(errors))
    return results
