"""Host path under a random mix of collectives: every rank draws the same sequence of calls
(kind, size from 1 byte to 8 MiB, element type, in or out of place, root) and checks each
result against values computed from the ranks' deterministic inputs. Exercises the transport's
size-dependent paths (read-ahead, frames held for their receive, ring rounds) in whatever order
the draw brings them."""
import numpy as np
import pytest

import hxccl_b200 as hx
from hxccl_b200 import _lib as L
from hxccl_b200.utils import run_ranks


def body(comm, rank, n, iters, seed):  # noqa: C901
    rng = np.random.default_rng(seed)  # same sequence everywhere
    bad = []
    twin = comm.split(0, rank)
    for it in range(iters):
        kind = rng.choice(["allreduce", "allgather", "reducescatter", "broadcast", "alltoall", "shift", "twin"])
        size = int(2 ** rng.uniform(0, 23))
        dt = rng.choice(["f32", "i32", "u8"])
        npdt = {"f32": np.float32, "i32": np.int32, "u8": np.uint8}[dt]
        es = np.dtype(npdt).itemsize
        cnt = max(1, size // es)
        def data(r, c, salt=0):
            return ((np.arange(c, dtype=np.int64) * 7 + r * 13 + it + salt) % 11).astype(npdt)
        c = twin if kind == "twin" else comm
        if kind in ("allreduce", "twin"):
            x = data(rank, cnt); y = np.zeros_like(x)
            if rng.random() < 0.5: c.all_reduce(x, y, op=L.SUM)
            else: y = x.copy(); c.all_reduce(y, op=L.SUM)
            want = sum(data(r, cnt).astype(np.int64) for r in range(n)).astype(npdt)
            ok = np.array_equal(y, want)
        elif kind == "allgather":
            x = data(rank, cnt); y = np.zeros(cnt * n, dtype=npdt)
            c.all_gather(x, y)
            ok = np.array_equal(y, np.concatenate([data(r, cnt) for r in range(n)]))
        elif kind == "reducescatter":
            x = data(rank, cnt * n); y = np.zeros(cnt, dtype=npdt)
            c.reduce_scatter(x, y, op=L.SUM)
            want = sum(data(r, cnt * n).astype(np.int64) for r in range(n)).astype(npdt)[rank * cnt:(rank + 1) * cnt]
            ok = np.array_equal(y, want)
        elif kind == "broadcast":
            root = int(rng.integers(0, n))
            x = data(root, cnt) if rank == root else np.zeros(cnt, dtype=npdt)
            c.bcast(x, root)
            ok = np.array_equal(x, data(root, cnt))
        elif kind == "alltoall":
            x = data(rank, cnt * n); y = np.zeros(cnt * n, dtype=npdt)
            c.all_to_all(x, y, count=cnt)
            ok = all(np.array_equal(y[r * cnt:(r + 1) * cnt], data(r, cnt * n)[rank * cnt:(rank + 1) * cnt]) for r in range(n))
        else:  # ring shift in a group, sometimes two messages
            k = int(rng.integers(1, 3))
            outs = [data(rank, cnt, salt=j) for j in range(k)]; ins = [np.zeros(cnt, dtype=npdt) for _ in range(k)]
            hx.group_start()
            for o in outs: comm.send(o, (rank + 1) % n)
            for i_ in ins: comm.recv(i_, (rank - 1) % n)
            hx.group_end()
            ok = all(np.array_equal(ins[j], data((rank - 1) % n, cnt, salt=j)) for j in range(k))
        if not ok: bad.append((it, kind, size, dt))
    twin.destroy()
    return bad


@pytest.mark.parametrize("n,seed,env", [(3, 11, {}), (4, 12, {"HXCCL_RING_SLICE_KB": "64", "HXCCL_HOLD_US": "0"}),
                                        (2, 13, {"HXCCL_SPIN_US": "0"})])
def test_random_mix_of_host_collectives(n, seed, env):
    res = run_ranks(n, body, 120, seed, env=env, timeout=300)
    assert all(not bad for bad in res), res
