"""Scenarios around the device path that the reference covers with its repro programs and
its context test: a host-only program creates no CUDA context (tests/gpu_host_no_context.cc:28-55),
one rank failing its device set-up moves every rank to the staged path
(tests/repro_init_failure.cc, tests/gpu_no_ptracer.cc:14-47), a PreMulSum scalar in device
memory is read in stream order (tests/repro_device_scalar.cc), and a truncated receive in one
communicator of a group leaves the other communicator's transfer of the same group intact
(tests/repro_group_truncation.cc).
All failures are made on the host; nothing here faults a GPU."""
import ctypes

import numpy as np
import pytest

import hxccl_b200 as hx
from hxccl_b200 import _lib as L
from hxccl_b200.utils import run_ranks

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")
NGPU = torch.cuda.device_count() if torch.cuda.is_available() else 0
needs2 = pytest.mark.skipif(NGPU < 2, reason="needs two GPUs")


def _primary_context_active():
    cu = ctypes.CDLL("libcuda.so.1")
    assert cu.cuInit(0) == 0
    flags, active = ctypes.c_uint(0), ctypes.c_int(-1)
    assert cu.cuDevicePrimaryCtxGetState(0, ctypes.byref(flags), ctypes.byref(active)) == 0
    return active.value


def _host_only_body(comm, rank, n):
    x = np.full(1000, rank + 1.0, dtype=np.float32)
    comm.all_reduce(x)
    hx.group_start()
    comm.send(x, (rank + 1) % n)
    got = np.zeros(1000, dtype=np.float32)  # must outlive the group
    comm.recv(got, (rank - 1) % n)
    assert hx.group_end() == 0 and got[0] == x[0]
    return float(x[0]), comm.device_info()["kind"], _primary_context_active()


def test_host_only_program_creates_no_context():
    n = 2
    for r, (val, kind, active) in enumerate(run_ranks(n, _host_only_body, gpus=False, timeout=60)):
        assert val == 3.0 and kind == "none" and active == 0, (r, val, kind, active)


def _lazy_body(comm, rank, n):
    """HXCCL_DEVICE=0: nothing starts at creation although a context exists; the first device
    buffer starts the device path on every rank."""
    before = comm.device_info()["kind"]
    x = torch.full((16,), float(rank + 1), device="cuda")
    comm.all_reduce(x)
    torch.cuda.synchronize()
    return before, comm.device_info()["kind"], float(x[0])


def test_device_path_starts_late_when_told_not_to_start_at_creation():
    for before, after, val in run_ranks(2, _lazy_body, gpus=True, timeout=60, env={"HXCCL_DEVICE": "0"}):
        assert before == "none" and after != "none" and val == 3.0, (before, after, val)


def _sum_body(comm, rank, n):
    x = torch.full((5000,), float(rank + 1), device="cuda")
    comm.all_reduce(x)
    torch.cuda.synchronize()
    return comm.device_info()["kind"], float(x[0]), float(x[-1]), comm.async_error()


@needs2
def test_one_rank_failing_setup_moves_everyone_to_staged():
    res = run_ranks(2, _sum_body, gpus=True, timeout=90, rank_env={0: {"HXCCL_TEST_FAIL_DEVICE_INIT": "1"}})
    for kind, first, last, err in res:
        assert kind == "staged" and first == 3.0 and last == 3.0 and err == 0, (kind, first, last, err)


def _device_scalar_body(comm, rank, n):
    """The scalar sits in device memory and is written by work queued on the same stream just
    before the collective: the kernel must read it in stream order, not the host at call time."""
    out = {"kind": comm.device_info()["kind"]}
    k = torch.zeros(1, device="cuda", dtype=torch.float32)
    op = comm.create_premul_sum(k, residence=L.SCALAR_DEVICE)
    x = torch.full((70000,), float(rank + 1), device="cuda")
    big = torch.ones(1 << 24, device="cuda")
    for _ in range(8):  # keep the stream busy so the fill below is still queued at call time
        big.mul_(1.0001)
    k.fill_(0.5)
    comm.all_reduce(x, op=op)
    k.fill_(4.0)  # after the collective in stream order: must not be seen by it
    torch.cuda.synchronize()
    out["half"] = (float(x[0]), float(x[-1]))
    y = torch.full((9,), float(rank + 1), device="cuda")
    comm.all_reduce(y, op=op)
    torch.cuda.synchronize()
    out["four"] = float(y[0])
    out["err"] = comm.async_error()
    return out


@needs2
def test_premul_scalar_in_device_memory_is_read_in_stream_order():
    n = 2
    for o in run_ranks(n, _device_scalar_body, gpus=True, timeout=90):
        assert o["kind"].startswith("window"), o
        assert o["half"] == (1.5, 1.5) and o["four"] == 12.0 and o["err"] == 0, o


def _two_comms_body(comm, rank, n):
    """One group, two communicators: the transfer on A is too long for its Recv, the one on B
    fits. A reports the truncation on the receiver each round; B delivers each round."""
    other = comm.split(0, rank)
    out = []
    for rnd in range(3):
        a = torch.full((2000,), 10 + rnd, device="cuda", dtype=torch.int32)
        b = torch.full((1000,), 20 + rnd, device="cuda", dtype=torch.int32)
        ra = torch.zeros(1000, device="cuda", dtype=torch.int32)
        rb = torch.zeros(1000, device="cuda", dtype=torch.int32)
        hx.group_start()
        if rank == 1:
            comm.send(a, 0)
            other.send(b, 0)
        else:
            comm.recv(ra, 1)
            other.recv(rb, 1)
        hx.group_end()
        torch.cuda.synchronize()
        out.append((comm.async_error(), comm.last_error(), other.async_error(), int(ra[0]), int(ra[-1]),
                    int(rb[0]), int(rb[-1])))
    x = torch.full((3000,), float(rank + 1), device="cuda")
    rc = other.all_reduce(x, check=False)
    torch.cuda.synchronize()
    out.append((rc, float(x[0]), other.async_error()))
    other.destroy()
    return out


@needs2
def test_truncation_in_one_communicator_leaves_the_other_working():
    receiver, sender = run_ranks(2, _two_comms_body, gpus=True, timeout=90)
    for rnd in range(3):
        assert sender[rnd][0] == 0 and sender[rnd][2] == 0, sender[rnd]
        err_a, msg, err_b, a0, a1, b0, b1 = receiver[rnd]
        assert err_a == L.SYSTEM_ERROR and "truncated" in msg and err_b == 0, receiver[rnd]
        assert (a0, a1) == (10 + rnd, 10 + rnd)  # what fitted did arrive
        assert (b0, b1) == (20 + rnd, 20 + rnd)
    assert receiver[3] == (0, 3.0, 0) and sender[3] == (0, 3.0, 0)


def _single_rank_body(comm, rank, n):
    """One rank: out of place is one copy launch, in place is no launch at all, and neither changes
    a bit (no arithmetic runs, so NaN payloads stay as they are)."""
    out = []
    for count in (1, 7, 4099, (3 << 20) + 5):
        t = torch.randint(0, 255, (count,), dtype=torch.uint8, device="cuda")
        o = torch.zeros_like(t)
        before = comm.device_info()["launches"]
        comm.all_reduce(t, o, op=L.SUM, count=count, dtype=L.UINT8)
        mid = comm.device_info()["launches"]
        keep = t.clone()
        comm.all_reduce(t, t, op=L.MAX, count=count, dtype=L.UINT8)
        torch.cuda.synchronize()
        out.append((bool(torch.equal(o, t)), bool(torch.equal(t, keep)), mid - before, comm.device_info()["launches"] - mid))
    i = torch.arange(-5, 5, dtype=torch.int32, device="cuda")
    o = torch.zeros_like(i)
    comm.all_reduce(i, o, op=L.AVG)
    f = torch.tensor([1.5, float("nan"), -0.0], device="cuda")
    g = torch.zeros_like(f)
    comm.all_reduce(f, g, op=L.AVG)  # scaled by 1.0 through the general kernel
    torch.cuda.synchronize()
    return out, bool(torch.equal(i, o)), g.cpu().numpy().view(np.uint32).tolist(), comm.async_error()


def test_single_rank_allreduce_is_a_copy_or_nothing():
    (out, int_ok, fbits, err), = run_ranks(1, _single_rank_body, gpus=True, timeout=60)
    assert all(o == (True, True, 1, 0) for o in out), out
    assert int_ok and err == 0
    assert fbits[0] == 0x3FC00000 and (fbits[1] & 0x7FC00000) == 0x7FC00000 and fbits[2] == 0x80000000
