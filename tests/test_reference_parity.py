"""Bit-for-bit parity with the reference library itself, on host buffers and without a GPU: the
unmodified reference (built by baseline/build_ref.py into baseline/_ref/libhxccl_ref.so) and
this library run the same collectives on the same random bytes as real multi-process jobs over
their socket bootstraps; every result byte and every traffic counter (bytes and messages each
rank sent) must agree. This pins the element rules
(src/elem.h, src/fp.h, src/reduce.cc of the reference) AND the reduction orders of its
algorithms (src/algo_ring.cc, src/algo_rd.cc, src/algo_rooted.cc) at once.

Skipped where the reference build or the CUDA stub driver library is absent (the reference's
CUDA build links libcuda; without a GPU the toolkit's stub stands in and its host path never
calls it)."""
import ctypes as C
import multiprocessing as mp
import os
from pathlib import Path

import numpy as np
import pytest

from hxccl_b200 import _lib as L
from hxccl_b200.ops import oracle
from hxccl_b200.utils import run_ranks

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref" / "libhxccl_ref.so"
STUB = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "lib64" / "stubs" / "libcuda.so"

pytestmark = pytest.mark.skipif(not REF.exists(), reason="reference build absent (python baseline/build_ref.py)")


class RefId(C.Structure):
    _fields_ = [("internal", C.c_char * 128)]


def _load_reference():
    try:
        C.CDLL("libcuda.so.1", mode=C.RTLD_GLOBAL)
    except OSError:
        C.CDLL(str(STUB), mode=C.RTLD_GLOBAL)  # no driver on this machine: the toolkit's stub
    lib = C.CDLL(str(REF))
    vp = C.c_void_p
    lib.hxcclCommInitRank.argtypes = [C.POINTER(vp), C.c_int, RefId, C.c_int]
    lib.hxcclAllReduce.argtypes = [vp, vp, C.c_size_t, C.c_int, C.c_int, vp, vp]
    lib.hxcclReduceScatter.argtypes = [vp, vp, C.c_size_t, C.c_int, C.c_int, vp, vp]
    lib.hxcclReduce.argtypes = [vp, vp, C.c_size_t, C.c_int, C.c_int, C.c_int, vp, vp]
    lib.hxcclAllGather.argtypes = [vp, vp, C.c_size_t, C.c_int, vp, vp]
    lib.hxcclBroadcast.argtypes = [vp, vp, C.c_size_t, C.c_int, C.c_int, vp, vp]
    lib.hxcclAlltoAll.argtypes = [vp, vp, C.c_size_t, C.c_int, vp, vp]
    szp = C.POINTER(C.c_size_t)
    lib.hxcclAllToAllv.argtypes = [vp, szp, szp, vp, szp, szp, C.c_int, vp, vp]
    lib.hxcclGather.argtypes = [vp, vp, C.c_size_t, C.c_int, C.c_int, vp, vp]
    lib.hxcclScatter.argtypes = [vp, vp, C.c_size_t, C.c_int, C.c_int, vp, vp]
    lib.hxcclSend.argtypes = [vp, C.c_size_t, C.c_int, C.c_int, vp, vp]
    lib.hxcclRecv.argtypes = [vp, C.c_size_t, C.c_int, C.c_int, vp, vp]
    lib.hxcclRedOpCreatePreMulSum.argtypes = [C.POINTER(C.c_int), vp, C.c_int, C.c_int, vp]
    lib.hxcclCommDestroy.argtypes = [vp]
    lib.hxcclCommResetStats.argtypes = [vp]
    lib.hxcclCommGetStats.argtypes = [vp, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]
    return lib


def _ref_stats(lib, comm):
    b, m = C.c_uint64(), C.c_uint64()
    assert lib.hxcclCommGetStats(comm, C.byref(b), C.byref(m)) == 0
    return (b.value, m.value)


def inputs_for(n, count, dt, seed):
    es = L.DTYPE_SIZE[dt]
    return [np.random.default_rng(seed * 1000 + r).integers(0, 256, count * es, dtype=np.uint8) for r in range(n)]


def v_layout(n, rank, mean, seed):
    """Uneven AlltoAllv counts: rank i sends counts[i][j] elements to rank j, blocks packed with a gap of
    one element between them on both sides."""
    counts = np.random.default_rng(seed).integers(0, 2 * mean + 1, (n, n))
    scounts, rcounts = [int(c) for c in counts[rank]], [int(c) for c in counts[:, rank]]
    sdispls = [int(sum(scounts[:j]) + j) for j in range(n)]
    rdispls = [int(sum(rcounts[:j]) + j) for j in range(n)]
    return scounts, sdispls, rcounts, rdispls, sum(scounts) + n, sum(rcounts) + n


def _ref_child(rank, n, cases, id_q, out_q):
    try:
        os.environ["HXCCL_DEVICE"] = "0"
        lib = _load_reference()
        uid = RefId()
        if rank == 0:
            assert lib.hxcclGetUniqueId(C.byref(uid)) == 0
            for _ in range(n - 1):
                id_q.put(bytes(uid))
        else:
            uid = RefId.from_buffer_copy(id_q.get(timeout=60))
        comm = C.c_void_p()
        assert lib.hxcclCommInitRank(C.byref(comm), n, uid, rank) == 0
        res = []
        for (coll, dt, op, count, seed) in cases:
            es = L.DTYPE_SIZE[dt]
            lib.hxcclCommResetStats(comm)
            if coll == "allreduce":
                x = inputs_for(n, count, dt, seed)[rank].copy()
                rc = lib.hxcclAllReduce(x.ctypes.data, x.ctypes.data, count, dt, op, comm, None)
                res.append((rc, x))
            elif coll == "reducescatter":
                x = inputs_for(n, count * n, dt, seed)[rank].copy()
                y = np.zeros(count * es, dtype=np.uint8)
                rc = lib.hxcclReduceScatter(x.ctypes.data, y.ctypes.data, count, dt, op, comm, None)
                res.append((rc, y))
            elif coll == "alltoallv":
                sc, sd, rcn, rd, stot, rtot = v_layout(n, rank, count, seed)
                x = inputs_for(n, stot, dt, seed)[rank].copy()
                y = np.zeros(rtot * es, dtype=np.uint8)
                arr = lambda v: (C.c_size_t * n)(*v)  # noqa: E731
                rc = lib.hxcclAllToAllv(x.ctypes.data, arr(sc), arr(sd), y.ctypes.data, arr(rcn), arr(rd), dt, comm, None)
                res.append((rc, y))
            elif coll == "gather":
                x = inputs_for(n, count, dt, seed)[rank].copy()
                y = np.zeros(count * es * n, dtype=np.uint8)
                rc = lib.hxcclGather(x.ctypes.data, y.ctypes.data if rank == 0 else None, count, dt, 0, comm, None)
                res.append((rc, y if rank == 0 else None))
            elif coll == "scatter":
                x = inputs_for(n, count * n, dt, seed)[0].copy()
                y = np.zeros(count * es, dtype=np.uint8)
                rc = lib.hxcclScatter(x.ctypes.data if rank == 0 else None, y.ctypes.data, count, dt, 0, comm, None)
                res.append((rc, y))
            elif coll == "shift":  # ring shift: Send and Recv in one group
                x = inputs_for(n, count, dt, seed)[rank].copy()
                y = np.zeros(count * es, dtype=np.uint8)
                lib.hxcclGroupStart()
                lib.hxcclSend(x.ctypes.data, count, dt, (rank + 1) % n, comm, None)
                lib.hxcclRecv(y.ctypes.data, count, dt, (rank + n - 1) % n, comm, None)
                rc = lib.hxcclGroupEnd()
                res.append((rc, y))
            elif coll == "premul":  # `op` carries the scalar's bits
                k = np.array([op], dtype=np.uint64).view(np.uint8)[:es].copy()
                handle = C.c_int()
                assert lib.hxcclRedOpCreatePreMulSum(C.byref(handle), k.ctypes.data, dt, L.SCALAR_HOST_IMMEDIATE, comm) == 0
                x = inputs_for(n, count, dt, seed)[rank].copy()
                rc = lib.hxcclAllReduce(x.ctypes.data, x.ctypes.data, count, dt, handle.value, comm, None)
                res.append((rc, x))
            elif coll == "allgather":
                x = inputs_for(n, count, dt, seed)[rank].copy()
                y = np.zeros(count * es * n, dtype=np.uint8)
                rc = lib.hxcclAllGather(x.ctypes.data, y.ctypes.data, count, dt, comm, None)
                res.append((rc, y))
            elif coll == "broadcast":
                x = inputs_for(n, count, dt, seed)[rank].copy()
                y = np.zeros(count * es, dtype=np.uint8)
                rc = lib.hxcclBroadcast(x.ctypes.data, y.ctypes.data, count, dt, 1 % n, comm, None)
                res.append((rc, y))
            elif coll == "alltoall":
                x = inputs_for(n, count * n, dt, seed)[rank].copy()
                y = np.zeros(count * es * n, dtype=np.uint8)
                rc = lib.hxcclAlltoAll(x.ctypes.data, y.ctypes.data, count, dt, comm, None)
                res.append((rc, y))
            else:
                x = inputs_for(n, count, dt, seed)[rank].copy()
                y = np.zeros(count * es, dtype=np.uint8)
                rc = lib.hxcclReduce(x.ctypes.data, y.ctypes.data, count, dt, op, n - 1, comm, None)
                res.append((rc, y if rank == n - 1 else None))
            res[-1] = res[-1] + (_ref_stats(lib, comm),)
        lib.hxcclCommDestroy(comm)
        out_q.put((rank, "ok", res))
    except BaseException as e:  # noqa: BLE001
        out_q.put((rank, "err", repr(e)))


def run_reference(n, cases):
    ctx = mp.get_context("spawn")
    id_q, out_q = ctx.Queue(), ctx.Queue()
    procs = [ctx.Process(target=_ref_child, args=(r, n, cases, id_q, out_q)) for r in range(n)]
    for p in procs:
        p.start()
    got = {}
    try:
        for _ in range(n):
            rank, state, payload = out_q.get(timeout=180)
            assert state == "ok", payload
            got[rank] = payload
    finally:
        for p in procs:
            p.join(10)
            if p.is_alive():
                p.kill()
    return [got[r] for r in range(n)]


def _ours_body(comm, rank, n, cases):
    res = []
    for (coll, dt, op, count, seed) in cases:
        es = L.DTYPE_SIZE[dt]
        comm.reset_stats()
        if coll == "allreduce":
            x = inputs_for(n, count, dt, seed)[rank].copy()
            rc = comm.all_reduce(x, x, op=op, count=count, dtype=dt, check=False)
            res.append((rc, x))
        elif coll == "reducescatter":
            x = inputs_for(n, count * n, dt, seed)[rank].copy()
            y = np.zeros(count * es, dtype=np.uint8)
            rc = comm.reduce_scatter(x, y, op=op, count=count, dtype=dt, check=False)
            res.append((rc, y))
        elif coll == "alltoallv":
            sc, sd, rcn, rd, stot, rtot = v_layout(n, rank, count, seed)
            x = inputs_for(n, stot, dt, seed)[rank].copy()
            y = np.zeros(rtot * es, dtype=np.uint8)
            rc = comm.all_to_allv(x, sc, sd, y, rcn, rd, dtype=dt, check=False)
            res.append((rc, y))
        elif coll == "gather":
            x = inputs_for(n, count, dt, seed)[rank].copy()
            y = np.zeros(count * es * n, dtype=np.uint8)
            rc = comm.gather(x, y if rank == 0 else None, root=0, count=count, dtype=dt, check=False)
            res.append((rc, y if rank == 0 else None))
        elif coll == "scatter":
            x = inputs_for(n, count * n, dt, seed)[0].copy()
            y = np.zeros(count * es, dtype=np.uint8)
            rc = comm.scatter(x if rank == 0 else None, y, root=0, count=count, dtype=dt, check=False)
            res.append((rc, y))
        elif coll == "shift":
            import hxccl_b200 as hx  # noqa: PLC0415

            x = inputs_for(n, count, dt, seed)[rank].copy()
            y = np.zeros(count * es, dtype=np.uint8)
            hx.group_start()
            comm.send(x, (rank + 1) % n, count=count, dtype=dt)
            comm.recv(y, (rank + n - 1) % n, count=count, dtype=dt)
            rc = hx.group_end()
            res.append((rc, y))
        elif coll == "premul":
            k = np.array([op], dtype=np.uint64).view(np.uint8)[:es].copy()
            handle = comm.create_premul_sum(k, dtype=dt)
            x = inputs_for(n, count, dt, seed)[rank].copy()
            rc = comm.all_reduce(x, x, op=handle, count=count, dtype=dt, check=False)
            res.append((rc, x))
        elif coll == "allgather":
            x = inputs_for(n, count, dt, seed)[rank].copy()
            y = np.zeros(count * es * n, dtype=np.uint8)
            rc = comm.all_gather(x, y, count=count, dtype=dt, check=False)
            res.append((rc, y))
        elif coll == "broadcast":
            x = inputs_for(n, count, dt, seed)[rank].copy()
            y = np.zeros(count * es, dtype=np.uint8)
            rc = comm.broadcast(x, y, root=1 % n, count=count, dtype=dt, check=False)
            res.append((rc, y))
        elif coll == "alltoall":
            x = inputs_for(n, count * n, dt, seed)[rank].copy()
            y = np.zeros(count * es * n, dtype=np.uint8)
            rc = comm.all_to_all(x, y, count=count, dtype=dt, check=False)
            res.append((rc, y))
        else:
            x = inputs_for(n, count, dt, seed)[rank].copy()
            y = np.zeros(count * es, dtype=np.uint8)
            rc = comm.reduce(x, y, root=n - 1, op=op, count=count, dtype=dt, check=False)
            res.append((rc, y if rank == n - 1 else None))
        res[-1] = res[-1] + (tuple(comm.stats()),)
    return res


def make_cases():
    cases = []
    for dt in range(12):
        es = L.DTYPE_SIZE[dt]
        for op in (L.SUM, L.PROD, L.MAX, L.MIN, L.AVG):
            # 7 and 1000 elements take recursive doubling (< 64 KiB), the last count the ring
            for count in (7, 1000, (64 << 10) // es + 13):
                cases.append(("allreduce", dt, op, count, len(cases)))
        cases.append(("reducescatter", dt, L.SUM, 501, len(cases)))
        cases.append(("reducescatter", dt, L.AVG, 33, len(cases)))
        cases.append(("reduce", dt, L.SUM, 777, len(cases)))                    # tree toward the root
        cases.append(("reduce", dt, L.PROD, (512 << 10) // es + 5, len(cases)))  # chain in 512 KiB pieces
    for dt, count in ((L.UINT8, 300), (L.FLOAT64, 41)):
        cases.append(("allgather", dt, 0, count, len(cases)))
        cases.append(("alltoall", dt, 0, count, len(cases)))
        cases.append(("broadcast", dt, 0, count, len(cases)))                        # binomial tree
        cases.append(("alltoallv", dt, 0, count, len(cases)))                        # uneven counts, gaps
        cases.append(("gather", dt, 0, count, len(cases)))
        cases.append(("scatter", dt, 0, count, len(cases)))
        cases.append(("shift", dt, 0, count, len(cases)))
    cases.append(("broadcast", L.INT32, 0, (1600 << 10) // 4 + 3, len(cases)))      # chain in 512 KiB pieces
    # PreMulSum: scalar bits 0.125 (fp16), 0.5 (bf16), 3 (int32), 1.5 (e5m2), -0.25 (fp32), small and ring-sized
    for dt, bits in ((L.FLOAT16, 0x3000), (L.BFLOAT16, 0x3F00), (L.INT32, 3), (L.FLOAT8E5M2, 0x3E), (L.FLOAT32, 0xBE800000)):
        cases.append(("premul", dt, bits, 1001, len(cases)))
        cases.append(("premul", dt, bits, (64 << 10) // L.DTYPE_SIZE[dt] + 7, len(cases)))
    # ring blocks above 1 MiB travel in several rounds here; results and message counts stay the reference's
    cases.append(("allreduce", L.FLOAT32, L.SUM, (9 << 20) // 4 + 5, len(cases)))
    cases.append(("allreduce", L.BFLOAT16, L.AVG, (9 << 20) // 2 + 3, len(cases)))
    cases.append(("reducescatter", L.FLOAT32, L.SUM, 300_001, len(cases)))
    cases.append(("allgather", L.UINT8, 0, (3 << 19) + 3, len(cases)))
    return cases


@pytest.mark.parametrize("n", [2, 3, 4, 5, 8])
def test_host_collectives_equal_the_reference_bit_for_bit(n):
    if not STUB.exists():
        try:
            C.CDLL("libcuda.so.1")
        except OSError:
            pytest.skip("neither a CUDA driver nor the toolkit's stub library is here")
    cases = make_cases()
    ref = run_reference(n, cases)
    ours = run_ranks(n, _ours_body, cases, timeout=180)
    for k, (coll, dt, op, count, seed) in enumerate(cases):
        for r in range(n):
            rc_ref, out_ref, stats_ref = ref[r][k]
            rc_ours, out_ours, stats_ours = ours[r][k]
            assert rc_ref == 0 and rc_ours == 0, (n, coll, dt, op, count, r, rc_ref, rc_ours)
            assert stats_ref == stats_ours, (n, coll, dt, op, count, r, stats_ref, stats_ours)  # same schedule
            if out_ref is None:
                continue
            assert np.array_equal(out_ref, out_ours), (n, coll, dt, op, count, r)
        if coll == "allreduce":  # and the in-process oracle the GPU tests rely on says the same
            want = oracle.allreduce([x.view(oracle.raw_dtype(dt)) for x in inputs_for(n, count, dt, seed)], dt, op)
            assert np.array_equal(ref[0][k][1], want[0].view(np.uint8)), (n, dt, op, count)


def _invalid_calls(lib, comm, n):
    """A battery of calls that must be refused, the same way by both libraries. `lib` is a ctypes
    handle of either library (the public names and argument lists are identical)."""
    x = np.ones(16, dtype=np.float32)
    y = np.zeros(16, dtype=np.float32)
    p, q, none = x.ctypes.data, y.ctypes.data, None
    out = [
        ("allreduce null comm", lib.hxcclAllReduce(p, q, 16, L.FLOAT32, L.SUM, None, None)),
        ("allreduce bad dtype", lib.hxcclAllReduce(p, q, 16, 99, L.SUM, comm, None)),
        ("allreduce bad op", lib.hxcclAllReduce(p, q, 16, L.FLOAT32, 99, comm, None)),
        ("allreduce null send", lib.hxcclAllReduce(none, q, 16, L.FLOAT32, L.SUM, comm, None)),
        ("allreduce null recv", lib.hxcclAllReduce(p, none, 16, L.FLOAT32, L.SUM, comm, None)),
        ("allreduce size overflow", lib.hxcclAllReduce(p, q, 1 << 62, L.FLOAT64, L.SUM, comm, None)),
        ("allreduce zero count null buffers", lib.hxcclAllReduce(none, none, 0, L.FLOAT32, L.SUM, comm, None)),
        ("broadcast root too large", lib.hxcclBroadcast(p, q, 16, L.FLOAT32, n, comm, None)),
        ("broadcast negative root", lib.hxcclBroadcast(p, q, 16, L.FLOAT32, -1, comm, None)),
        ("reduce bad root", lib.hxcclReduce(p, q, 16, L.FLOAT32, L.SUM, n + 3, comm, None)),
        ("gather bad root", lib.hxcclGather(p, q, 4, L.FLOAT32, -2, comm, None)),
        ("send bad peer", lib.hxcclSend(p, 16, L.FLOAT32, n, comm, None)),
        ("recv bad peer", lib.hxcclRecv(q, 16, L.FLOAT32, -1, comm, None)),
        ("group end without start", lib.hxcclGroupEnd()),
        ("avg on a valid call", lib.hxcclAllReduce(p, q, 16, L.FLOAT32, L.AVG, comm, None)),
    ]
    # AllToAllv with a bad argument on ONE rank only: the ranks agree, everybody refuses, nothing moves
    rk = C.c_int(-1)
    lib.hxcclCommUserRank.argtypes = [C.c_void_p, C.POINTER(C.c_int)]
    lib.hxcclCommUserRank(comm, C.byref(rk))
    ones, disp = (C.c_size_t * n)(*([2] * n)), (C.c_size_t * n)(*[2 * j for j in range(n)])
    src, dst = np.ones(2 * n, dtype=np.float32), np.zeros(2 * n, dtype=np.float32)
    lib.hxcclCommResetStats.argtypes = [C.c_void_p]
    lib.hxcclCommGetStats.argtypes = [C.c_void_p, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]
    lib.hxcclCommResetStats(comm)
    rc = lib.hxcclAllToAllv(src.ctypes.data, None if rk.value == 1 else ones, disp, dst.ctypes.data, ones, disp,
                            L.FLOAT32, comm, None)
    sent, msgs = C.c_uint64(), C.c_uint64()
    lib.hxcclCommGetStats(comm, C.byref(sent), C.byref(msgs))
    out.append(("alltoallv one bad rank", rc, sent.value, msgs.value, dst.tolist()))
    rc = lib.hxcclAllToAllv(src.ctypes.data, ones, disp, dst.ctypes.data, ones, disp, L.FLOAT32, comm, None)
    out.append(("alltoallv good", rc, dst.tolist()))
    lib.hxcclGetErrorString.restype = C.c_char_p
    lib.hxcclGetErrorString.argtypes = [C.c_int]
    strings = [lib.hxcclGetErrorString(code).decode() for code in range(-1, 11)]
    version = C.c_int()
    lib.hxcclGetVersion(C.byref(version))
    return out, strings, version.value, y.tolist()


def _ref_invalid_child(rank, n, id_q, out_q):
    try:
        lib = _load_reference()
        uid = RefId()
        if rank == 0:
            lib.hxcclGetUniqueId(C.byref(uid))
            for _ in range(n - 1):
                id_q.put(bytes(uid))
        else:
            uid = RefId.from_buffer_copy(id_q.get(timeout=60))
        comm = C.c_void_p()
        assert lib.hxcclCommInitRank(C.byref(comm), n, uid, rank) == 0
        res = _invalid_calls(lib, comm, n)
        lib.hxcclCommDestroy(comm)
        out_q.put((rank, "ok", res))
    except BaseException as e:  # noqa: BLE001
        out_q.put((rank, "err", repr(e)))


def _ours_invalid_body(comm, rank, n):
    return _invalid_calls(L.lib(), C.c_void_p(comm.handle), n)


def test_refusals_and_error_strings_equal_the_reference():
    n = 2
    ctx = mp.get_context("spawn")
    id_q, out_q = ctx.Queue(), ctx.Queue()
    procs = [ctx.Process(target=_ref_invalid_child, args=(r, n, id_q, out_q)) for r in range(n)]
    for p in procs:
        p.start()
    ref = {}
    try:
        for _ in range(n):
            rank, state, payload = out_q.get(timeout=120)
            assert state == "ok", payload
            ref[rank] = payload
    finally:
        for p in procs:
            p.join(10)
            if p.is_alive():
                p.kill()
    ours = run_ranks(n, _ours_invalid_body, timeout=120)
    for r in range(n):
        assert ours[r][0] == ref[r][0], [(a, b) for a, b in zip(ours[r][0], ref[r][0]) if a != b]
        # hxcclGetErrorString, codes -1..10: the same words, except that hxcclSystemError (2) reads
        # "system (network) error" here and "system (MPI) error" there: this library has no MPI transport
        assert [s for i, s in enumerate(ours[r][1]) if i != 3] == [s for i, s in enumerate(ref[r][1]) if i != 3]
        assert ours[r][1][3] == "system (network) error" and ref[r][1][3] == "system (MPI) error"
        assert ours[r][2] == ref[r][2] == 200   # hxcclGetVersion
        assert ours[r][3] == ref[r][3] == [1.0] * 16  # the one valid call (Avg of ones)


def _lifecycle_calls(lib, comm, rank, n):
    """Communicator and operator lifecycle through the C API, written once for both libraries:
    returns every observable (codes, sizes, ranks, handle values, results)."""
    vp = C.c_void_p
    lib.hxcclCommSplit.argtypes = [vp, C.c_int, C.c_int, C.POINTER(vp), C.POINTER(L.Config)]
    lib.hxcclCommShrink.argtypes = [vp, C.POINTER(C.c_int), C.c_int, C.POINTER(vp), C.POINTER(L.Config), C.c_int]
    lib.hxcclCommCount.argtypes = [vp, C.POINTER(C.c_int)]
    lib.hxcclCommUserRank.argtypes = [vp, C.POINTER(C.c_int)]
    lib.hxcclCommGetAsyncError.argtypes = [vp, C.POINTER(C.c_int)]
    lib.hxcclCommFinalize.argtypes = [vp]
    lib.hxcclCommAbort.argtypes = [vp]
    lib.hxcclRedOpDestroy.argtypes = [C.c_int, vp]
    out = []

    def shape(c):
        cnt, rk = C.c_int(-1), C.c_int(-1)
        return (lib.hxcclCommCount(c, C.byref(cnt)), cnt.value, lib.hxcclCommUserRank(c, C.byref(rk)), rk.value)

    out.append(("world", shape(comm)))
    # split by parity with the order reversed inside each half
    half = vp()
    out.append(("split", lib.hxcclCommSplit(comm, rank % 2, -rank, C.byref(half), None), shape(half)))
    x = np.full(5, float(rank), dtype=np.float64)
    out.append(("split sum", lib.hxcclAllReduce(x.ctypes.data, x.ctypes.data, 5, L.FLOAT64, L.SUM, half, None), x.tolist()))
    # no colour on rank 0: no communicator there
    none = vp(123)
    out.append(("nocolor", lib.hxcclCommSplit(comm, L.SPLIT_NOCOLOR if rank == 0 else 7, 0, C.byref(none), None),
                none.value is None if rank == 0 else shape(none)))
    # configuration checks
    cfg = L.Config.initializer()
    cfg.blocking = 0
    bad = vp()
    out.append(("config blocking 0", lib.hxcclCommSplit(comm, 0, 0, C.byref(bad), C.byref(cfg))))
    cfg = L.Config.initializer()
    cfg.magic = 1
    out.append(("config magic", lib.hxcclCommSplit(comm, 0, 0, C.byref(bad), C.byref(cfg))))
    # shrink: argument errors, then the survivors without the last rank
    two = (C.c_int * 2)(n - 1, n - 1)
    out.append(("shrink duplicate", lib.hxcclCommShrink(comm, two, 2, C.byref(bad), None, 0)))
    me = (C.c_int * 1)(rank)
    out.append(("shrink self", lib.hxcclCommShrink(comm, me, 1, C.byref(bad), None, 0)))
    last = (C.c_int * 1)(n - 1)
    out.append(("shrink flags", lib.hxcclCommShrink(comm, last, 1, C.byref(bad), None, 1)))
    if rank != n - 1:
        small = vp()
        out.append(("shrink", lib.hxcclCommShrink(comm, last, 1, C.byref(small), None, 0), shape(small)))
        y = np.ones(3, dtype=np.int32)
        out.append(("shrink sum", lib.hxcclAllReduce(y.ctypes.data, y.ctypes.data, 3, L.INT32, L.SUM, small, None), y.tolist()))
        lib.hxcclCommDestroy(small)
    # operators: handle values, wrong type, destroyed, reuse of the slot, foreign communicator
    k = np.array([0.25], dtype=np.float32)
    op1, op2 = C.c_int(), C.c_int()
    out.append(("premul create", lib.hxcclRedOpCreatePreMulSum(C.byref(op1), k.ctypes.data, L.FLOAT32, L.SCALAR_HOST_IMMEDIATE, comm),
                op1.value))
    out.append(("premul second", lib.hxcclRedOpCreatePreMulSum(C.byref(op2), k.ctypes.data, L.FLOAT32, L.SCALAR_HOST_IMMEDIATE, comm),
                op2.value))
    f = np.full(4, 8.0, dtype=np.float32)
    out.append(("premul use", lib.hxcclAllReduce(f.ctypes.data, f.ctypes.data, 4, L.FLOAT32, op1.value, comm, None), f.tolist()))
    d = np.ones(4, dtype=np.float64)
    out.append(("premul wrong type", lib.hxcclAllReduce(d.ctypes.data, d.ctypes.data, 4, L.FLOAT64, op1.value, comm, None)))
    out.append(("premul foreign comm", lib.hxcclAllReduce(f.ctypes.data, f.ctypes.data, 4, L.FLOAT32, op1.value, half, None)))
    out.append(("premul destroy", lib.hxcclRedOpDestroy(op1.value, comm)))
    out.append(("premul destroyed use", lib.hxcclAllReduce(f.ctypes.data, f.ctypes.data, 4, L.FLOAT32, op1.value, comm, None)))
    out.append(("premul destroy twice", lib.hxcclRedOpDestroy(op1.value, comm)))
    op3 = C.c_int()
    out.append(("premul slot reuse", lib.hxcclRedOpCreatePreMulSum(C.byref(op3), k.ctypes.data, L.FLOAT32, L.SCALAR_HOST_IMMEDIATE, comm),
                op3.value == op1.value))
    out.append(("destroy builtin", lib.hxcclRedOpDestroy(L.SUM, comm)))
    # finalize: later calls are usage errors; abort of a child is local
    err = C.c_int(-1)
    out.append(("async error", lib.hxcclCommGetAsyncError(comm, C.byref(err)), err.value))
    out.append(("finalize", lib.hxcclCommFinalize(half)))
    out.append(("after finalize", lib.hxcclAllReduce(x.ctypes.data, x.ctypes.data, 5, L.FLOAT64, L.SUM, half, None)))
    out.append(("destroy finalized", lib.hxcclCommDestroy(half)))
    if rank != 0:
        out.append(("abort", lib.hxcclCommAbort(none)))
    return out


def _ref_lifecycle_child(rank, n, id_q, out_q):
    try:
        lib = _load_reference()
        uid = RefId()
        if rank == 0:
            lib.hxcclGetUniqueId(C.byref(uid))
            for _ in range(n - 1):
                id_q.put(bytes(uid))
        else:
            uid = RefId.from_buffer_copy(id_q.get(timeout=60))
        comm = C.c_void_p()
        assert lib.hxcclCommInitRank(C.byref(comm), n, uid, rank) == 0
        res = _lifecycle_calls(lib, comm, rank, n)
        lib.hxcclCommDestroy(comm)
        out_q.put((rank, "ok", res))
    except BaseException as e:  # noqa: BLE001
        import traceback

        out_q.put((rank, "err", repr(e) + traceback.format_exc()))


def _ours_lifecycle_body(comm, rank, n):
    return _lifecycle_calls(L.lib(), C.c_void_p(comm.handle), rank, n)


@pytest.mark.parametrize("n", [2, 5])
def test_lifecycle_observables_equal_the_reference(n):
    ctx = mp.get_context("spawn")
    id_q, out_q = ctx.Queue(), ctx.Queue()
    procs = [ctx.Process(target=_ref_lifecycle_child, args=(r, n, id_q, out_q)) for r in range(n)]
    for p in procs:
        p.start()
    ref = {}
    try:
        for _ in range(n):
            rank, state, payload = out_q.get(timeout=120)
            assert state == "ok", payload
            ref[rank] = payload
    finally:
        for p in procs:
            p.join(10)
            if p.is_alive():
                p.kill()
    ours = run_ranks(n, _ours_lifecycle_body, timeout=120)
    for r in range(n):
        assert ours[r] == ref[r], (r, [(a, b) for a, b in zip(ours[r], ref[r]) if a != b])


def _group_calls(lib, comm, rank, n):
    """Send/Recv and groups through the C API, once for both libraries (two ranks)."""
    lib.hxcclGetLastError.restype = C.c_char_p
    lib.hxcclGetLastError.argtypes = [C.c_void_p]
    out, other = [], 1 - rank
    # crossed exchange in one group (two blocking calls would deadlock)
    a = np.arange(100000, dtype=np.float32) + rank
    b = np.zeros_like(a)
    codes = [lib.hxcclGroupStart(), lib.hxcclSend(a.ctypes.data, a.size, L.FLOAT32, other, comm, None),
             lib.hxcclRecv(b.ctypes.data, b.size, L.FLOAT32, other, comm, None), lib.hxcclGroupEnd()]
    out.append(("crossed", codes, float(b[0]), float(b[-1])))
    # two messages to the same peer keep their order; nested groups; a collective in the same group
    s1, s2 = np.full(3, 10 + rank, dtype=np.int32), np.full(3, 20 + rank, dtype=np.int32)
    r1, r2 = np.zeros(3, dtype=np.int32), np.zeros(3, dtype=np.int32)
    red = np.ones(4, dtype=np.int64)
    codes = [lib.hxcclGroupStart(), lib.hxcclGroupStart(),
             lib.hxcclSend(s1.ctypes.data, 3, L.INT32, other, comm, None),
             lib.hxcclSend(s2.ctypes.data, 3, L.INT32, other, comm, None),
             lib.hxcclGroupEnd(),
             lib.hxcclAllReduce(red.ctypes.data, red.ctypes.data, 4, L.INT64, L.SUM, comm, None),
             lib.hxcclRecv(r1.ctypes.data, 3, L.INT32, other, comm, None),
             lib.hxcclRecv(r2.ctypes.data, 3, L.INT32, other, comm, None),
             lib.hxcclGroupEnd()]
    out.append(("ordered", codes, r1.tolist(), r2.tolist(), red.tolist()))
    # a refused call inside a group is skipped, the rest of the group runs
    t = np.full(2, 5.0 + rank, dtype=np.float64)
    u = np.zeros(2, dtype=np.float64)
    codes = [lib.hxcclGroupStart(), lib.hxcclSend(t.ctypes.data, 2, L.FLOAT64, 9, comm, None),
             lib.hxcclSend(t.ctypes.data, 2, L.FLOAT64, other, comm, None),
             lib.hxcclRecv(u.ctypes.data, 2, L.FLOAT64, other, comm, None), lib.hxcclGroupEnd()]
    out.append(("refused inside", codes, u.tolist()))
    # truncation: eight elements into room for five; only the receiver fails, the head arrives
    big, room = np.arange(8, dtype=np.int32), np.full(5, -1, dtype=np.int32)
    if rank == 1:
        rc = lib.hxcclSend(big.ctypes.data, 8, L.INT32, 0, comm, None)
        out.append(("truncated send", rc))
    else:
        rc = lib.hxcclRecv(room.ctypes.data, 5, L.INT32, 1, comm, None)
        out.append(("truncated recv", rc, room.tolist(), b"truncated" in lib.hxcclGetLastError(comm)))
    # the communicator still works afterwards
    z = np.full(3, rank + 1.0, dtype=np.float32)
    out.append(("after", lib.hxcclAllReduce(z.ctypes.data, z.ctypes.data, 3, L.FLOAT32, L.MAX, comm, None), z.tolist()))
    err = C.c_int(-1)
    lib.hxcclCommGetAsyncError.argtypes = [C.c_void_p, C.POINTER(C.c_int)]
    out.append(("async", lib.hxcclCommGetAsyncError(comm, C.byref(err)), err.value))
    return out


def _ref_group_child(rank, n, id_q, out_q):
    try:
        lib = _load_reference()
        uid = RefId()
        if rank == 0:
            lib.hxcclGetUniqueId(C.byref(uid))
            id_q.put(bytes(uid))
        else:
            uid = RefId.from_buffer_copy(id_q.get(timeout=60))
        comm = C.c_void_p()
        assert lib.hxcclCommInitRank(C.byref(comm), n, uid, rank) == 0
        res = _group_calls(lib, comm, rank, n)
        lib.hxcclCommDestroy(comm)
        out_q.put((rank, "ok", res))
    except BaseException as e:  # noqa: BLE001
        import traceback

        out_q.put((rank, "err", repr(e) + traceback.format_exc()))


def _ours_group_body(comm, rank, n):
    return _group_calls(L.lib(), C.c_void_p(comm.handle), rank, n)


def test_send_recv_and_groups_equal_the_reference():
    n = 2
    ctx = mp.get_context("spawn")
    id_q, out_q = ctx.Queue(), ctx.Queue()
    procs = [ctx.Process(target=_ref_group_child, args=(r, n, id_q, out_q)) for r in range(n)]
    for p in procs:
        p.start()
    ref = {}
    try:
        for _ in range(n):
            rank, state, payload = out_q.get(timeout=120)
            assert state == "ok", payload
            ref[rank] = payload
    finally:
        for p in procs:
            p.join(10)
            if p.is_alive():
                p.kill()
    ours = run_ranks(n, _ours_group_body, timeout=120)
    for r in range(n):
        assert ours[r] == ref[r], (r, [(a, b) for a, b in zip(ours[r], ref[r]) if a != b])


def _bootstrap_calls(lib, uid_struct, rank, n):
    """hxcclCommInitRank with bad arguments and with every rank claiming to be rank 0."""
    vp = C.c_void_p
    comm = vp()
    out = [("nranks 0", lib.hxcclCommInitRank(C.byref(comm), 0, uid_struct, 0)),
           ("rank too large", lib.hxcclCommInitRank(C.byref(comm), n, uid_struct, n)),
           ("negative rank", lib.hxcclCommInitRank(C.byref(comm), n, uid_struct, -1)),
           ("null comm", lib.hxcclCommInitRank(None, n, uid_struct, rank))]
    out.append(("duplicate ranks", lib.hxcclCommInitRank(C.byref(comm), n, uid_struct, 0)))
    return out


def _ref_bootstrap_child(rank, n, id_q, out_q):
    try:
        lib = _load_reference()
        uid = RefId()
        if rank == 0:
            lib.hxcclGetUniqueId(C.byref(uid))
            for _ in range(n - 1):
                id_q.put(bytes(uid))
        else:
            uid = RefId.from_buffer_copy(id_q.get(timeout=60))
        out_q.put((rank, "ok", _bootstrap_calls(lib, uid, rank, n)))
    except BaseException as e:  # noqa: BLE001
        out_q.put((rank, "err", repr(e)))


def _ours_bootstrap_body(uid, rank, n):
    from hxccl_b200._lib import UniqueId  # noqa: PLC0415

    return _bootstrap_calls(L.lib(), UniqueId.from_buffer_copy(uid), rank, n)


def test_bootstrap_refusals_equal_the_reference():
    n = 3
    ctx = mp.get_context("spawn")
    id_q, out_q = ctx.Queue(), ctx.Queue()
    procs = [ctx.Process(target=_ref_bootstrap_child, args=(r, n, id_q, out_q)) for r in range(n)]
    for p in procs:
        p.start()
    ref = {}
    try:
        for _ in range(n):
            rank, state, payload = out_q.get(timeout=120)
            assert state == "ok", payload
            ref[rank] = payload
    finally:
        for p in procs:
            p.join(10)
            if p.is_alive():
                p.kill()
    ours = run_ranks(n, _ours_bootstrap_body, make_comm=False, timeout=120)
    for r in range(n):
        assert ours[r] == ref[r], (r, ours[r], ref[r])
    assert ref[0][-1] == ("duplicate ranks", L.INVALID_USAGE)
