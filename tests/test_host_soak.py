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

KINDS = ["allreduce", "allgather", "reducescatter", "broadcast", "alltoall", "shift", "twin"]
TYPES = {"f32": np.float32, "i32": np.int32, "u8": np.uint8}


def _data(npdt, it, rank, count, salt=0):
    """Small whole numbers, a function of (call, rank, position): sums are exact in every type."""
    return ((np.arange(count, dtype=np.int64) * 7 + rank * 13 + it + salt) % 11).astype(npdt)


def _summed(npdt, it, n, count):
    return sum(_data(npdt, it, r, count).astype(np.int64) for r in range(n)).astype(npdt)


def _one_call(comm, twin, rank, n, it, rng):
    kind = rng.choice(KINDS)
    size = int(2 ** rng.uniform(0, 23))
    npdt = TYPES[rng.choice(list(TYPES))]
    count = max(1, size // np.dtype(npdt).itemsize)
    c = twin if kind == "twin" else comm  # the twin shares the parent's connections
    if kind in ("allreduce", "twin"):
        x = _data(npdt, it, rank, count)
        if rng.random() < 0.5:
            y = np.zeros_like(x)
            c.all_reduce(x, y, op=L.SUM)
        else:
            y = x.copy()
            c.all_reduce(y, op=L.SUM)
        return kind, size, np.array_equal(y, _summed(npdt, it, n, count))
    if kind == "allgather":
        y = np.zeros(count * n, dtype=npdt)
        c.all_gather(_data(npdt, it, rank, count), y)
        return kind, size, np.array_equal(y, np.concatenate([_data(npdt, it, r, count) for r in range(n)]))
    if kind == "reducescatter":
        y = np.zeros(count, dtype=npdt)
        c.reduce_scatter(_data(npdt, it, rank, count * n), y, op=L.SUM)
        want = _summed(npdt, it, n, count * n)[rank * count:(rank + 1) * count]
        return kind, size, np.array_equal(y, want)
    if kind == "broadcast":
        root = int(rng.integers(0, n))
        x = _data(npdt, it, root, count) if rank == root else np.zeros(count, dtype=npdt)
        c.bcast(x, root)
        return kind, size, np.array_equal(x, _data(npdt, it, root, count))
    if kind == "alltoall":
        y = np.zeros(count * n, dtype=npdt)
        c.all_to_all(_data(npdt, it, rank, count * n), y, count=count)
        ok = all(np.array_equal(y[r * count:(r + 1) * count],
                                _data(npdt, it, r, count * n)[rank * count:(rank + 1) * count]) for r in range(n))
        return kind, size, ok
    # a ring shift inside a group, one or two messages per neighbour
    k = int(rng.integers(1, 3))
    outs = [_data(npdt, it, rank, count, salt=j) for j in range(k)]
    ins = [np.zeros(count, dtype=npdt) for _ in range(k)]
    hx.group_start()
    for o in outs:
        comm.send(o, (rank + 1) % n)
    for i in ins:
        comm.recv(i, (rank - 1) % n)
    hx.group_end()
    return kind, size, all(np.array_equal(ins[j], _data(npdt, it, (rank - 1) % n, count, salt=j)) for j in range(k))


def _body(comm, rank, n, iters, seed):
    rng = np.random.default_rng(seed)  # the same draws on every rank
    twin = comm.split(0, rank)
    bad = []
    for it in range(iters):
        kind, size, ok = _one_call(comm, twin, rank, n, it, rng)
        if not ok:
            bad.append((it, kind, size))
    twin.destroy()
    return bad


@pytest.mark.parametrize("n,seed,env", [(3, 11, {}), (4, 12, {"HXCCL_RING_SLICE_KB": "64", "HXCCL_HOLD_US": "0"}),
                                        (2, 13, {"HXCCL_SPIN_US": "0"})])
def test_random_mix_of_host_collectives(n, seed, env):
    res = run_ranks(n, _body, 120, seed, env=env, timeout=300)
    assert all(not bad for bad in res), res
