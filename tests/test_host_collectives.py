"""Host path: every collective other than AllReduce, across processes, checked against values
computed from the ranks' deterministic inputs (reference: tests/test_collectives.cc:11-76,
tests/test_rooted.cc:12-121, tests/test_alltoall.cc:11-131)."""
import numpy as np
import pytest

from hxccl_b200 import _lib as L
from hxccl_b200.ops import oracle
from hxccl_b200.utils import run_ranks


def data(rank, count, dtype=np.float32, seed=0):
    return np.random.default_rng(1000 * seed + rank).integers(-50, 50, count).astype(dtype)


def _gather_scatter(comm, rank, n):
    out = {}
    for count in (0, 5, 400_000):  # 1.6 MB of fp32 crosses into the chain path
        x = data(rank, count)
        ag = np.zeros(count * n, dtype=np.float32)
        comm.all_gather(x, ag)
        inplace = np.zeros(count * n, dtype=np.float32)
        inplace[rank * count:(rank + 1) * count] = x
        comm.all_gather(inplace[rank * count:(rank + 1) * count], inplace, count=count)
        full = np.concatenate([data(r, count * n, seed=1) for r in range(1)]) if count else np.zeros(0, np.float32)
        rs_in = data(rank, count * n, seed=1)
        rs = np.zeros(count, dtype=np.float32)
        comm.reduce_scatter(rs_in, rs, op=L.SUM)
        rs_in2 = rs_in.copy()
        comm.reduce_scatter(rs_in2, rs_in2[rank * count:(rank + 1) * count], op=L.SUM, count=count)  # in place
        root = (n - 1) // 2
        b = x.copy() if rank == root else np.zeros(count, dtype=np.float32)
        comm.bcast(b, root)
        b2 = np.zeros(count, dtype=np.float32)
        comm.broadcast(x if rank == root else None, b2, root, count=count, dtype=L.FLOAT32)
        comm.reset_stats()
        red = np.zeros(count, dtype=np.float32) if rank == root else None
        comm.reduce(x, red, root, op=L.SUM, count=count, dtype=L.FLOAT32)
        red_stats = comm.stats()
        g = np.zeros(count * n, dtype=np.float32) if rank == root else None
        comm.gather(x, g, root, count=count, dtype=L.FLOAT32)
        sc_src = data(root, count * n, seed=2) if rank == root else None
        sc = np.zeros(count, dtype=np.float32)
        comm.scatter(sc_src, sc, root, count=count, dtype=L.FLOAT32)
        ia = np.full(count, rank * 3 - 4, dtype=np.int32)
        iavg = np.zeros(count, dtype=np.int32) if rank == root else None
        comm.reduce(ia, iavg, root, op=L.AVG, count=count, dtype=L.INT32)
        out[count] = dict(ag=ag, inplace=inplace, rs=rs, rs2=rs_in2[rank * count:(rank + 1) * count].copy(), b=b, b2=b2,
                          red=red, g=g, sc=sc, iavg=iavg, red_stats=red_stats)
    return out


@pytest.mark.parametrize("n", [1, 2, 3, 5, 8])
def test_gather_scatter_family(n):
    res = run_ranks(n, _gather_scatter)
    root = (n - 1) // 2
    for count in (0, 5, 400_000):
        xs = [data(r, count) for r in range(n)]
        want_ag = np.concatenate(xs) if count else np.zeros(0, np.float32)
        rs_want = oracle.reducescatter([data(r, count * n, seed=1).view(np.uint32) for r in range(n)], L.FLOAT32, L.SUM) \
            if count else [np.zeros(0, np.uint32)] * n
        red_want = oracle.reduce([x.view(np.uint32) for x in xs], L.FLOAT32, L.SUM, root)
        for r in range(n):
            o = res[r][count]
            assert np.array_equal(o["ag"], want_ag) and np.array_equal(o["inplace"], want_ag)
            assert np.array_equal(o["rs"].view(np.uint32), rs_want[r]) and np.array_equal(o["rs2"].view(np.uint32), rs_want[r])
            assert np.array_equal(o["b"], xs[root]) and np.array_equal(o["b2"], xs[root])
            assert np.array_equal(o["sc"], data(root, count * n, seed=2)[r * count:(r + 1) * count])
        o = res[root][count]
        assert np.array_equal(o["red"].view(np.uint32), red_want)
        assert np.array_equal(o["g"], want_ag)
        if count:
            tot = sum(r * 3 - 4 for r in range(n))
            assert o["iavg"].tolist() == [int(tot / n)] * count  # truncation toward zero, at the root only
        # traffic of Reduce: nothing at the root; one message (tree) or the chain's pieces elsewhere
        nbytes = count * 4
        for r in range(n):
            b, m = res[r][count]["red_stats"]
            if r == root or n == 1 or count == 0:
                assert (b, m) == (0, 0)
            elif nbytes < 512 * 1024:
                assert (b, m) == (nbytes, 1)
            else:
                assert b == nbytes and m == -(-nbytes // (512 * 1024))


def _alltoall(comm, rank, n):
    out = {}
    count = 3
    s = np.arange(n * count, dtype=np.int32) + 1000 * rank
    r1 = np.zeros(n * count, dtype=np.int32)
    comm.all_to_all(s, r1)
    r2 = np.zeros(n * count, dtype=np.int32)
    comm.all_to_all(s, r2, rccl_spelling=True)
    inplace = s.copy()
    comm.all_to_all(inplace, inplace, count=count)
    # uneven blocks with gaps: rank r sends (r + j) % 4 elements to rank j
    sc = [(rank + j) % 4 for j in range(n)]
    rc = [(i + rank) % 4 for i in range(n)]
    sd = [5 * j for j in range(n)]
    rd = [6 * i for i in range(n)]
    sv = np.arange(5 * n, dtype=np.int64) + 100 * rank
    rv = np.full(6 * n, -1, dtype=np.int64)
    comm.reset_stats()
    comm.all_to_allv(sv, sc, sd, rv, rc, rd)
    out["stats"] = comm.stats()
    # zero everywhere: nothing moves
    comm.reset_stats()
    comm.all_to_all(np.zeros(0, np.int32), np.zeros(0, np.int32), count=0, dtype=L.INT32)
    out["zero_stats"] = comm.stats()
    # one rank passes a bad argument: everyone must reject together and send nothing
    comm.reset_stats()
    bad = comm.all_to_allv(None if rank == 0 else sv, sc, sd, rv, rc, rd, dtype=L.INT64, check=False)
    out.update(r1=r1, r2=r2, inplace=inplace, rv=rv, bad=bad, bad_stats=comm.stats())
    return out


@pytest.mark.parametrize("n", [2, 3, 4, 8])
def test_alltoall_family(n):
    res = run_ranks(n, _alltoall)
    for r in range(n):
        want = np.concatenate([np.arange(r * 3, r * 3 + 3, dtype=np.int32) + 1000 * i for i in range(n)])
        assert np.array_equal(res[r]["r1"], want) and np.array_equal(res[r]["r2"], want)
        assert np.array_equal(res[r]["inplace"], want)
        rv = np.full(6 * n, -1, dtype=np.int64)
        for i in range(n):
            c = (i + r) % 4
            rv[6 * i:6 * i + c] = np.arange(5 * r, 5 * r + c) + 100 * i
        assert np.array_equal(res[r]["rv"], rv)
        assert res[r]["stats"] == (8 * sum((r + j) % 4 for j in range(n) if j != r), n - 1)
        assert res[r]["zero_stats"] == (0, 0)
        assert res[r]["bad"] == L.INVALID_ARGUMENT and res[r]["bad_stats"] == (0, 0)
