"""API semantics on the host path: Send/Recv and groups, Avg / PreMulSum, communicator
lifecycle (Split, Shrink, Abort, Finalize, config), error behaviour and the bootstrap.
Follows the reference's tests/test_p2p.cc, test_ops.cc, test_comm.cc, test_errors.cc,
test_init.cc and test_net_cancel.cc; failures are injected on the host only."""
import ctypes as C
import os

import numpy as np
import pytest

import hxccl_b200 as hx
from hxccl_b200 import _lib as L
from hxccl_b200.comm import Communicator, HxcclError
from hxccl_b200.utils import run_ranks


def test_version_and_enums():
    assert hx.get_version() == 200
    assert (L.SUCCESS, L.SYSTEM_ERROR, L.INVALID_ARGUMENT, L.INVALID_USAGE, L.REMOTE_ERROR, L.TIMEOUT) == (0, 2, 4, 5, 6, 8)
    assert (L.INT8, L.FLOAT16, L.FLOAT32, L.BFLOAT16, L.FLOAT8E5M2) == (0, 6, 7, 9, 11)
    assert L.lib().hxcclGetErrorString(4) == b"invalid argument"
    assert L.lib().hxcclGroupEnd() == L.INVALID_USAGE  # no group open


# ---- Send / Recv / groups -----------------------------------------------------------------------
def _p2p(comm, rank, n):
    out = {}
    right, left = (rank + 1) % n, (rank - 1) % n
    # crossed 4 MB exchange inside a group (would deadlock as two blocking calls)
    big = np.full(1 << 20, rank, dtype=np.int32)
    got = np.zeros(1 << 20, dtype=np.int32)
    hx.group_start()
    comm.send(big, right)
    comm.recv(got, left)
    assert hx.group_end() == 0
    out["cross"] = int(got[0]) == left and int(got[-1]) == left
    # ring shift traffic: one message of 400 bytes
    comm.reset_stats()
    a, b = np.full(100, rank, dtype=np.float32), np.zeros(100, dtype=np.float32)
    hx.group_start()
    comm.send(a, right)
    comm.recv(b, left)
    hx.group_end()
    out["shift"] = (b[0] == left, comm.stats())
    # two sends to the same peer arrive in order; nested groups run nothing at the inner end
    x1, x2 = np.array([1 + rank], dtype=np.int64), np.array([100 + rank], dtype=np.int64)
    y1, y2 = np.zeros(1, np.int64), np.zeros(1, np.int64)
    ar = np.array([rank], dtype=np.int32)
    hx.group_start()
    hx.group_start()
    comm.send(x1, right)
    comm.send(x2, right)
    assert hx.group_end() == 0 and y1[0] == 0
    comm.recv(y1, left)
    comm.recv(y2, left)
    comm.all_reduce(ar, op=L.SUM)  # collectives of a group run first
    # a rejected call is not queued; the rest of the group still runs
    bad = comm.send(x1, n + 3, check=False)
    assert hx.group_end() == 0
    out["order"] = (int(y1[0]), int(y2[0]), int(ar[0]), bad)
    # truncation: 8 elements into room for 5; the receiver fails, the sender does not
    if n >= 2:
        if rank == 0:
            out["trunc"] = comm.send(np.arange(8, dtype=np.int32), 1, check=False)
        elif rank == 1:
            t = np.zeros(5, dtype=np.int32)
            out["trunc"] = (comm.recv(t, 0, check=False), t.tolist(), comm.last_error())
        # and the communicator keeps working afterwards
        z = np.array([1], dtype=np.int32)
        comm.all_reduce(z)
        out["after"] = int(z[0])
    # blocking pair outside a group
    if rank == 0:
        comm.send(np.array([7.5]), 1 % n) if n > 1 else None
    elif rank == 1:
        v = np.zeros(1)
        comm.recv(v, 0)
        out["blocking"] = float(v[0])
    # a send to oneself pairs with one's own receive
    me_in, me_out = np.array([rank + 0.5]), np.zeros(1)
    hx.group_start()
    comm.send(me_in, rank)
    comm.recv(me_out, rank)
    hx.group_end()
    out["self"] = float(me_out[0])
    return out


@pytest.mark.parametrize("n", [2, 3, 4])
def test_send_recv_and_groups(n):
    res = run_ranks(n, _p2p)
    for r in range(n):
        left = (r - 1) % n
        assert res[r]["cross"] and res[r]["shift"] == (True, (400, 1))
        assert res[r]["order"] == (1 + left, 100 + left, sum(range(n)), L.INVALID_ARGUMENT)
        assert res[r]["after"] == n and res[r]["self"] == r + 0.5
    assert res[0]["trunc"] == 0
    rc, head, msg = res[1]["trunc"]
    assert rc == L.SYSTEM_ERROR and head == [0, 1, 2, 3, 4] and "truncated" in msg
    assert res[1]["blocking"] == 7.5


# sizes around the transport's thresholds: bodies under 4 KiB come through the 8 KiB read-ahead
# buffer (several frames per system call), larger ones go straight into the receive buffer, and
# from 64 KiB on an early frame waits in the socket for its receive
_BURST = [0, 1, 8, 4000, 4064, 4096, 4097, 8160, 8192, 8193, 16384, 65504, 65536, 65537, 300_001, 3, 1 << 20, 17, 5]


def _burst(comm, rank, n):
    peer = 1 - rank
    ins = [np.random.default_rng(50 * k + rank).integers(0, 255, sz).astype(np.uint8)
           for k, sz in enumerate(_BURST)]
    expect = [np.random.default_rng(50 * k + peer).integers(0, 255, sz).astype(np.uint8)
              for k, sz in enumerate(_BURST)]
    outs = [np.zeros(sz, dtype=np.uint8) for sz in _BURST]
    ok = []
    # all sends first: the messages queue up at the receiver before it asks for any of them
    hx.group_start()
    for x in ins:
        comm.send(x, peer)
    for y in outs:
        comm.recv(y, peer)
    assert hx.group_end() == 0
    ok.append(all(np.array_equal(a, b) for a, b in zip(outs, expect)))
    # and as blocking pairs, one message at a time, in both directions
    for k, sz in enumerate(_BURST):
        y = np.zeros(sz, dtype=np.uint8)
        if rank == 0:
            comm.send(ins[k], 1)
            comm.recv(y, 1)
        else:
            comm.recv(y, 0)
            comm.send(ins[k], 0)
        ok.append(np.array_equal(y, expect[k]))
    return all(ok)


@pytest.mark.parametrize("spin_us", ["0", "2000"])
def test_mixed_message_sizes_arrive_intact(spin_us):
    assert run_ranks(2, _burst, env={"HXCCL_SPIN_US": spin_us}) == [True, True]


def _early_large(comm, rank, n):
    """Large messages that arrive before anyone asks for them: taken straight into the receive
    posted next, parked when something behind them is wanted first, parked when nobody comes."""
    import time

    twin = comm.split(0, rank)  # same members, its own channel on the same connections
    big = lambda seed: np.random.default_rng(seed).integers(0, 255, 1 << 20).astype(np.uint8)  # noqa: E731
    out = {}
    if rank == 1:
        comm.send(big(1), 0)                    # (a) early, asked for next
        comm.send(big(2), 0)                    # (b) early, but the twin's message is wanted first
        twin.send(np.array([42], np.int32), 0)
        comm.send(big(3), 0)                    # (c) early, nobody asks while rank 0 waits for rank 2
    elif rank == 0:
        time.sleep(0.05)
        a = np.zeros(1 << 20, np.uint8)
        comm.recv(a, 1)
        small = np.zeros(1, np.int32)
        twin.recv(small, 1)
        b = np.zeros(1 << 20, np.uint8)
        comm.recv(b, 1)
        late = np.zeros(1, np.int32)
        comm.recv(late, 2)
        c = np.zeros(1 << 20, np.uint8)
        comm.recv(c, 1)
        out = {"a": np.array_equal(a, big(1)), "b": np.array_equal(b, big(2)),
               "c": np.array_equal(c, big(3)), "small": int(small[0]), "late": int(late[0])}
    else:
        time.sleep(0.15)
        comm.send(np.array([7], np.int32), 0)
    z = np.array([1], dtype=np.int32)
    comm.all_reduce(z)
    out["after"] = int(z[0])
    twin.destroy()
    return out


@pytest.mark.parametrize("hold_us", ["200", "0", "1000000"])
def test_large_messages_ahead_of_their_receives(hold_us):
    res = run_ranks(3, _early_large, env={"HXCCL_HOLD_US": hold_us})
    assert res[0] == {"a": True, "b": True, "c": True, "small": 42, "late": 7, "after": 3}
    assert res[1]["after"] == 3 and res[2]["after"] == 3


def _two_comm_group(comm, rank, n):
    """Crossed Send/Recv over two communicators in one group must not deadlock."""
    other = comm.split(0, rank)
    a, b = np.full(1 << 18, rank, np.int32), np.zeros(1 << 18, np.int32)
    c, d = np.full(1 << 18, 10 + rank, np.int32), np.zeros(1 << 18, np.int32)
    peer = 1 - rank
    hx.group_start()
    if rank == 0:
        comm.send(a, peer)
        other.recv(d, peer)
    else:
        other.send(c, peer)
        comm.recv(b, peer)
    assert hx.group_end() == 0
    other.destroy()
    return int(b[0]), int(d[0])


def test_group_over_two_communicators():
    res = run_ranks(2, _two_comm_group)
    assert res[0][1] == 11 and res[1][0] == 0


# ---- Avg and PreMulSum ------------------------------------------------------------------------------
def _ops(comm, rank, n):
    out = {}
    i = np.array([-7 + rank, 5], dtype=np.int32)
    comm.all_reduce(i, op=L.AVG)
    out["iavg"] = i.tolist()
    h = np.full(4, 60000.0, dtype=np.float16)
    comm.all_reduce(h, op=L.AVG)
    out["h60000"] = h.tolist()
    f = np.array([1.0 + rank, 2.0], dtype=np.float32)
    k = np.array([0.125], dtype=np.float32)
    op = comm.create_premul_sum(k)
    k[0] = 99.0  # host-immediate: the value was copied at creation
    comm.all_reduce(f, op=op)
    out["premul"] = f.tolist()
    # scalar by pointer: read when the collective is called
    kp = np.array([2.0], dtype=np.float64)
    op2 = comm.create_premul_sum(kp, residence=L.SCALAR_DEVICE)
    kp[0] = 3.0
    d = np.array([1.0], dtype=np.float64)
    comm.all_reduce(d, op=op2)
    out["by_ptr"] = float(d[0])
    # wrong datatype, destroyed op, handle reuse, op of another communicator
    out["wrong_dt"] = comm.all_reduce(np.zeros(1, np.float64), op=op, check=False)
    comm.destroy_op(op)
    out["destroyed"] = comm.all_reduce(f, op=op, check=False)
    out["reused"] = comm.create_premul_sum(np.array([1.0], dtype=np.float32)) == op
    sub = comm.split(0, rank)
    out["foreign"] = sub.all_reduce(f.copy(), op=op2, check=False)
    sub.destroy()
    # integer PreMulSum through ReduceScatter
    ki = np.array([3], dtype=np.int32)
    opi = comm.create_premul_sum(ki)
    src = np.arange(2 * n, dtype=np.int32) + rank
    dst = np.zeros(2, dtype=np.int32)
    comm.reduce_scatter(src, dst, op=opi)
    out["int_premul"] = dst.tolist()
    out["async"] = comm.async_error()
    return out


@pytest.mark.parametrize("n", [2, 3, 4])
def test_avg_and_premulsum(n):
    res = run_ranks(n, _ops)
    tot = sum(-7 + r for r in range(n))
    for r in range(n):
        o = res[r]
        assert o["iavg"] == [int(tot / n), 5]
        assert o["h60000"] == [60000.0] * 4
        assert o["premul"] == [0.125 * sum(1.0 + q for q in range(n)), 0.25 * n]
        assert o["by_ptr"] == 3.0 * n
        assert o["wrong_dt"] == o["destroyed"] == o["foreign"] == L.INVALID_ARGUMENT
        assert o["reused"] and o["async"] == 0  # argument errors never become asynchronous errors
        assert o["int_premul"] == [3 * sum(2 * r + k + q for q in range(n)) for k in range(2)]


# ---- communicator lifecycle -------------------------------------------------------------------------
def _comm(comm, rank, n):
    out = {}
    # split by parity with reversed keys
    sub = comm.split(rank % 2, -rank)
    x = np.array([rank], dtype=np.int32)
    sub.all_reduce(x)
    out["split"] = (sub.rank, sub.size, int(x[0]))
    sub.destroy()
    none = comm.split(L.SPLIT_NOCOLOR if rank == 0 else 0, 0)
    out["nocolor"] = none is None if rank == 0 else none.size
    if none is not None:
        none.destroy()
    h = C.c_void_p()
    out["bad_color"] = L.lib().hxcclCommSplit(comm.handle, -5, 0, C.byref(h), None)
    # shrink without the last rank; the excluded rank does not call
    if rank != n - 1:
        s = comm.shrink([n - 1])
        y = np.array([1], dtype=np.int32)
        s.all_reduce(y)
        out["shrink"] = (s.size, int(y[0]))
        s.destroy()
    ex = (C.c_int * 2)(0, 0)
    out["shrink_dup"] = L.lib().hxcclCommShrink(comm.handle, ex, 2, C.byref(h), None, 0)
    ex1 = (C.c_int * 1)(rank)
    out["shrink_self"] = L.lib().hxcclCommShrink(comm.handle, ex1, 1, C.byref(h), None, 0)
    out["shrink_flags"] = L.lib().hxcclCommShrink(comm.handle, ex1, 0, C.byref(h), None, 1)
    # config validation
    cfg = L.Config.initializer()
    cfg.blocking = 0
    out["cfg_blocking"] = L.lib().hxcclCommSplit(comm.handle, 0, 0, C.byref(h), C.byref(cfg))
    cfg = L.Config.initializer()
    cfg.magic = 1
    out["cfg_magic"] = L.lib().hxcclCommSplit(comm.handle, 0, 0, C.byref(h), C.byref(cfg))
    # local abort of a child never contacts anyone
    child = comm.split(0, rank)
    child.abort()
    # injected transport failure: SystemError now, and the asynchronous error stays set
    z = np.ones(100000, dtype=np.float32)
    fresh = comm.split(0, rank)
    if rank == 0:
        L.lib().hxcclTestFailSends(fresh.handle, 0)
        out["fail"] = (fresh.all_reduce(z, check=False), fresh.async_error(), fresh.last_error())
    fresh.abort()
    # finalize: every later call is a usage error, destroy still works
    fin = comm.split(0, rank)
    fin.finalize()
    out["finalized"] = (fin.all_reduce(z, check=False), fin.send(z, 0, check=False),
                        fin.all_to_allv(z, [0] * n, [0] * n, z, [0] * n, [0] * n, check=False))
    fin.destroy()
    return out


@pytest.mark.parametrize("n", [2, 4, 5])
def test_communicator_lifecycle(n):
    res = run_ranks(n, _comm)
    for r in range(n):
        o = res[r]
        members = sorted([q for q in range(n) if q % 2 == r % 2], key=lambda q: -q)
        assert o["split"] == (members.index(r), len(members), sum(members))
        assert o["nocolor"] is True if r == 0 else o["nocolor"] == n - 1
        assert o["bad_color"] == L.INVALID_ARGUMENT
        if r != n - 1:
            assert o["shrink"] == (n - 1, n - 1)
        assert o["shrink_dup"] == L.INVALID_ARGUMENT and o["shrink_self"] == L.INVALID_USAGE
        assert o["shrink_flags"] == L.INVALID_ARGUMENT
        assert o["cfg_blocking"] == L.INVALID_ARGUMENT and o["cfg_magic"] == L.INVALID_ARGUMENT
        assert o["finalized"] == (L.INVALID_USAGE,) * 3
    rc, async_err, msg = res[0]["fail"]
    assert rc == L.SYSTEM_ERROR and async_err == L.SYSTEM_ERROR and "injected" in msg


# ---- argument errors send nothing ----------------------------------------------------------------------
def _errors(comm, rank, n):
    out = {}
    x = np.zeros(4, dtype=np.float32)
    lib = L.lib()
    comm.reset_stats()
    codes = [
        lib.hxcclAllReduce(None, x.ctypes.data, 4, L.FLOAT32, L.SUM, comm.handle, None),   # null send
        lib.hxcclAllReduce(x.ctypes.data, x.ctypes.data, 4, 99, L.SUM, comm.handle, None),  # unknown dtype
        lib.hxcclAllReduce(x.ctypes.data, x.ctypes.data, 4, L.FLOAT32, 77, comm.handle, None),  # unknown op
        lib.hxcclAllReduce(x.ctypes.data, x.ctypes.data, 2 ** 63, L.FLOAT32, L.SUM, comm.handle, None),  # overflow
        lib.hxcclBroadcast(x.ctypes.data, x.ctypes.data, 4, L.FLOAT32, n, comm.handle, None),  # bad root
        lib.hxcclReduce(x.ctypes.data, x.ctypes.data, 4, L.FLOAT32, L.SUM, -1, comm.handle, None),
        lib.hxcclSend(x.ctypes.data, 4, L.FLOAT32, n, comm.handle, None),                      # bad peer
        lib.hxcclAllReduce(x.ctypes.data, x.ctypes.data, 4, L.FLOAT32, L.SUM, None, None),     # null comm
        # a message beyond the host transport's limit is refused by every rank alike
        lib.hxcclAllGather(x.ctypes.data, x.ctypes.data, 2 ** 31, L.INT8, comm.handle, None),
    ]
    out["codes"] = codes
    out["stats"] = comm.stats()
    out["async"] = comm.async_error()
    # zero counts with null buffers succeed and send nothing
    out["zero"] = [lib.hxcclAllReduce(None, None, 0, L.FLOAT32, L.SUM, comm.handle, None),
                   lib.hxcclGather(None, None, 0, L.FLOAT32, 0, comm.handle, None),
                   lib.hxcclSend(None, 0, L.FLOAT32, (rank + 1) % n, comm.handle, None) if False else 0]
    out["zero_stats"] = comm.stats()
    # non-root ranks may pass no receive buffer to Reduce / Gather and no send buffer to Scatter
    y = np.full(3, rank + 1, dtype=np.int32)
    r = np.zeros(3, dtype=np.int32)
    out["null_ok"] = [
        lib.hxcclReduce(y.ctypes.data, r.ctypes.data if rank == 0 else None, 3, L.INT32, L.SUM, 0, comm.handle, None),
        lib.hxcclScatter(np.arange(3 * n, dtype=np.int32).ctypes.data if rank == 0 else None, r.ctypes.data, 3,
                         L.INT32, 0, comm.handle, None)]
    return out


def test_argument_errors_send_nothing():
    n = 3
    res = run_ranks(n, _errors)
    for r in range(n):
        assert res[r]["codes"] == [L.INVALID_ARGUMENT] * 9
        assert res[r]["stats"] == (0, 0) and res[r]["async"] == 0
        assert res[r]["zero"] == [0, 0, 0] and res[r]["zero_stats"] == (0, 0)
        assert res[r]["null_ok"] == [0, 0]


# ---- bootstrap ---------------------------------------------------------------------------------------------
def _dup_ranks(uid, rank, n):
    h = C.c_void_p()
    use = 0 if rank == 1 else rank  # rank 1 claims to be rank 0 as well
    return L.lib().hxcclCommInitRank(C.byref(h), n, L.UniqueId.from_buffer_copy(uid), use)


def test_bootstrap_rejects_duplicate_ranks_everywhere():
    assert run_ranks(3, _dup_ranks, make_comm=False) == [L.INVALID_USAGE] * 3


def test_bootstrap_argument_checks():
    h = C.c_void_p()
    uid = L.UniqueId()
    assert L.lib().hxcclCommInitRank(C.byref(h), 2, uid, 2) == L.INVALID_ARGUMENT   # rank >= nranks
    assert L.lib().hxcclCommInitRank(C.byref(h), 1, uid, 0) == L.INVALID_ARGUMENT   # id not from GetUniqueId
    c = Communicator.init_rank(hx.get_unique_id(), 1, 0)                             # a world of one
    x = np.arange(5, dtype=np.float32)
    c.all_reduce(x, op=L.AVG)
    assert x.tolist() == [0, 1, 2, 3, 4] and c.stats() == (0, 0)
    c.destroy()


def _peer_loss(comm, rank, n):
    """A closed connection fails the transfers that involve that peer, with SystemError."""
    x = np.ones(1 << 16, dtype=np.float32)
    comm.all_reduce(x)
    if rank == 1:
        L.lib().hxcclTestSeverPeer(comm.handle, 0)
    rc = comm.all_reduce(x, check=False)
    return rc, comm.async_error()


def test_lost_peer_is_a_system_error_not_a_hang():
    res = run_ranks(2, _peer_loss, env={"HXCCL_NET_TIMEOUT_MS": "5000"})
    assert all(rc == L.SYSTEM_ERROR and a == L.SYSTEM_ERROR for rc, a in res)


def _cancel(comm, rank, n):
    """A send cancelled in mid-flight must not read the caller's buffer afterwards."""
    big = np.full(32 << 20, 7, dtype=np.uint8)
    if rank == 0:
        L.lib().hxcclTestFailSends(comm.handle, 1)  # the second send of the exchange fails
        hx.group_start()
        comm.send(big, 1)
        comm.send(big, 1)
        rc = hx.group_end()
        big[:] = 0  # if the library still read this buffer the peer would see zeros
        small = np.array([5], dtype=np.int32)
        comm.send(small, 1)
        return rc
    got = np.zeros(32 << 20, dtype=np.uint8)
    comm.recv(got, 0)
    tail = np.zeros(1, dtype=np.int32)
    comm.recv(tail, 0)
    return int(got.min()), int(got.max()), int(tail[0])


def test_cancelled_send_keeps_its_own_copy():
    res = run_ranks(2, _cancel)
    assert res[0] == L.SYSTEM_ERROR
    assert res[1] == (7, 7, 5)


def test_mpi_carrier_against_a_loopback_mpi(tmp_path):
    """No MPI is installed here, so the MPI carrier (the counterpart of the reference's MpiNet
    and MpiTransport) runs against tests/fake_mpi/fake_mpi.cc, a one-process MPI whose messages
    to self work: its matching, parking, truncation and cancel rules, and hxcclCommInitMPI with
    host collectives on top. The sources are compiled here with -DHXCCL_HAVE_MPI."""
    import subprocess
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    src = root / "src"
    exe = tmp_path / "carrier_check"
    host_sources = [str(p) for d in ("core", "ctrl", "host", "math") for p in sorted((src / d).glob("*.cc"))]
    stubs = tmp_path / "no_device.cc"
    stubs.write_text(
        '#include "core/devpath.h"\n'
        "namespace hx {\n"
        "MemKind classify(const void* p) { return p ? MemKind::Host : MemKind::Null; }\n"
        "MemKind classify_on(const void* p, int* o) { *o = -1; return classify(p); }\n"
        "int device_ordinal_of(const void*) { return -1; }\n"
        "bool cuda_context_exists() { return false; }\n"
        "std::unique_ptr<DevicePath> start_device_path(hxcclComm*, hxcclResult_t* rc, std::string* why) {\n"
        '  *rc = hxcclInvalidUsage; *why = "no device path in this build"; return nullptr; }\n'
        "}\n")
    cmd = ["g++", "-std=c++17", "-O1", "-DHXCCL_HAVE_MPI", "-DHXCCL_NO_NVTX", f"-I{root / 'baseline' / 'mpi_stub'}",
           f"-I{root / 'include'}", f"-I{src}", str(root / "tests" / "fake_mpi" / "fake_mpi.cc"),
           str(root / "tests" / "fake_mpi" / "carrier_check.cc"), str(stubs), *host_sources, "-pthread", "-o", str(exe)]
    built = subprocess.run(cmd, capture_output=True, text=True)
    assert built.returncode == 0, built.stderr[-3000:]
    ran = subprocess.run([str(exe)], capture_output=True, text=True, timeout=60)
    assert ran.returncode == 0 and ran.stdout.strip().endswith("ok"), ran.stdout + ran.stderr


def test_ranks_as_threads_of_one_process(tmp_path):
    """tests/tsan/ranks_as_threads.cc against the ordinary library: four ranks as threads of one
    process, a parent and its Split child used from two threads at once. The same program runs
    under ThreadSanitizer with `python -m hxccl_b200.build --tsan` (next test)."""
    import subprocess
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    L.lib()
    exe = tmp_path / "ranks_as_threads"
    lib_dir = root / "hxccl_b200" / "lib"
    subprocess.run(["g++", "-std=c++17", "-O1", f"-I{root / 'include'}", str(root / "tests" / "tsan" / "ranks_as_threads.cc"),
                    "-o", str(exe), f"-L{lib_dir}", "-lhxccl", f"-Wl,-rpath,{lib_dir}", "-pthread"], check=True)
    res = subprocess.run([str(exe), "4"], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0 and "4 ranks as threads: 0 failures" in res.stdout, (res.stdout, res.stderr[-2000:])


def test_ranks_as_threads_under_thread_sanitizer():
    import subprocess
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    exe = root / "build" / "ranks_as_threads"
    if not exe.exists() or not (root / "build" / "libhxccl_tsan.so").exists():
        pytest.skip("python -m hxccl_b200.build --tsan has not been run")
    env = dict(os.environ, TSAN_OPTIONS=f"suppressions={root / 'tests' / 'tsan' / 'suppressions.txt'} exitcode=66")
    env.pop("LD_PRELOAD", None)  # another sanitizer's runtime (the ASan run of this suite) cannot share the process
    res = subprocess.run([str(exe), "4"], capture_output=True, text=True, timeout=300, env=env)
    assert res.returncode == 0 and "ThreadSanitizer" not in res.stderr, res.stderr[-3000:]
