"""The production device path on real GPUs, one process per GPU: windows shared through file
descriptors, NVSwitch multicast when the node offers it, kernels on the caller's stream.
Results are compared bit for bit with the host schedules (floats in exact mode) or, for the
NVLS float variant, by tolerance against an fp64 sum."""
import numpy as np
import pytest

from conftest import gpu_count
from hxccl_b200 import _lib as L
from hxccl_b200.ops import oracle
from hxccl_b200.utils import run_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
NGPU = gpu_count()
needs2 = pytest.mark.skipif(NGPU < 2, reason="needs two GPUs")
WORLDS = [n for n in (2, 4, 8) if n <= NGPU]


def inputs_for(n, count, dt, seed, tame=False):
    es = L.DTYPE_SIZE[dt]
    out = []
    for r in range(n):
        x = np.random.default_rng(seed * 1000 + r).integers(0, 256, count * es, dtype=np.uint8).view(oracle.raw_dtype(dt))
        if tame and dt >= L.FLOAT16:  # clear the top exponent bit: moderate magnitudes
            x &= x.dtype.type(~(1 << (8 * es - 2)) & ((1 << (8 * es)) - 1))
        out.append(x)
    return out


def _allreduce_body(comm, rank, n, cases):
    import torch

    info = comm.device_info()
    outs = []
    for (dt, op, count, variant, seed) in cases:
        comm.tune(variant=variant, exact=True)
        x = torch.from_numpy(inputs_for(n, count, dt, seed, tame=count > 100000)[rank].view(np.uint8).copy()).cuda()
        y = torch.zeros_like(x)
        comm.reset_stats()
        comm.all_reduce(x, y, op=op, count=count, dtype=dt)
        torch.cuda.synchronize()
        outs.append((y.cpu().numpy(), comm.stats(), comm.device_info()["variant"]))
    return info, outs, comm.async_error()


@needs2
@pytest.mark.parametrize("n", WORLDS)
def test_allreduce_exact(n):
    cases = []
    for dt in range(12):
        for op in (L.SUM, L.MAX, L.AVG):
            for count, variant in ((1, 0), (4099, 1), (4099, 2), ((2 << 20) // L.DTYPE_SIZE[dt] + 3, 0),
                                   ((300 << 10) // L.DTYPE_SIZE[dt] + 5, 6)):  # 6 = neighbour ring
                cases.append((dt, op, count, variant, len(cases)))
    res = run_ranks(n, _allreduce_body, cases, gpus=True, timeout=120)
    assert res[0][0]["kind"].startswith("window"), res[0][0]
    for k, (dt, op, count, variant, seed) in enumerate(cases):
        want = oracle.allreduce(inputs_for(n, count, dt, seed, tame=count > 100000), dt, op)
        for r in range(n):
            got = res[r][1][k][0].view(oracle.raw_dtype(dt))
            assert np.array_equal(got, want[r]), (n, dt, op, count, variant, r, res[r][1][k][2])
    assert all(r[2] == 0 for r in res)


@needs2
def test_allreduce_exact_with_small_chunks():
    """HXCCL_IPC_CHUNK bounds the bytes a CTA moves per step, so moderate messages run through
    the many-step pipelines (the reference's HXCCL_IPC_CHUNK=4096 test runs, CMakeLists.txt:98-100).
    One rank asks for a larger chunk: the smallest wish holds for everyone."""
    n = 2
    cases = []
    for dt in (L.FLOAT32, L.BFLOAT16, L.INT32, L.FLOAT8E5M2):
        for op in (L.SUM, L.AVG):
            for count, variant in (((2 << 20) // L.DTYPE_SIZE[dt] + 3, 0), ((2 << 20) // L.DTYPE_SIZE[dt] + 3, 6)):
                cases.append((dt, op, count, variant, 100 + len(cases)))
    cases.append((L.FLOAT32, L.SUM, (5 << 20) // 4 + 1, 0, 99))  # above HXCCL_RING_MIN: the tuner picks the ring
    res = run_ranks(n, _allreduce_body, cases, gpus=True, timeout=120,
                    env={"HXCCL_IPC_CHUNK": "4096", "HXCCL_RING_MIN": str(4 << 20), "HXCCL_TUNE_TABLE": "0"},
                    rank_env={1: {"HXCCL_IPC_CHUNK": "65536"}})
    for k, (dt, op, count, variant, seed) in enumerate(cases):
        want = oracle.allreduce(inputs_for(n, count, dt, seed, tame=True), dt, op)
        for r in range(n):
            got = res[r][1][k][0].view(oracle.raw_dtype(dt))
            assert np.array_equal(got, want[r]), (dt, op, count, variant, r)
            assert res[r][1][k][2] == (6 if variant == 6 or count * L.DTYPE_SIZE[dt] >= (4 << 20) else 2)
    assert all(r[2] == 0 for r in res)


def _nvls_body(comm, rank, n):
    import torch

    info = comm.device_info()
    if "nvls" not in info["kind"]:
        return info, None
    out = {}
    comm.tune(variant=3, exact=False)
    count = 1 << 20
    for name, tdt in (("f32", torch.float32), ("bf16", torch.bfloat16), ("f16", torch.float16)):
        g = torch.Generator().manual_seed(100 + rank)
        x = (torch.rand(count, generator=g) * 2 - 1).to(tdt).cuda()
        y = torch.empty_like(x)
        comm.all_reduce(x, y, op=L.SUM)
        torch.cuda.synchronize()
        out[name] = (y.float().cpu().numpy(), comm.device_info()["variant"])
    xi = torch.from_numpy(np.random.default_rng(rank).integers(-1000, 1001, count).astype(np.int32)).cuda()
    comm.all_reduce(xi, xi, op=L.AVG)
    torch.cuda.synchronize()
    out["i32avg"] = (xi.cpu().numpy(), comm.device_info()["variant"])
    return info, out


@needs2
@pytest.mark.parametrize("n", WORLDS)
def test_allreduce_nvls(n):
    import torch

    res = run_ranks(n, _nvls_body, gpus=True, timeout=120, nvls=True)
    if res[0][1] is None:
        pytest.skip("no NVSwitch multicast on this node: " + res[0][0]["kind"])
    count = 1 << 20
    for name, tdt, tol in (("f32", torch.float32, 1e-5), ("bf16", torch.bfloat16, 5e-2), ("f16", torch.float16, 5e-3)):
        ref = sum((torch.rand(count, generator=torch.Generator().manual_seed(100 + r)) * 2 - 1).to(tdt).double()
                  for r in range(n)).numpy()
        for r in range(n):
            got, variant = res[r][1][name]
            assert variant == 3
            assert np.abs(got - ref).max() <= tol * n, (name, np.abs(got - ref).max())
    tot = sum(np.random.default_rng(r).integers(-1000, 1001, count).astype(np.int64) for r in range(n))
    want = np.trunc(tot / n).astype(np.int32)
    for r in range(n):
        assert res[r][1]["i32avg"][1] == 3 and np.array_equal(res[r][1]["i32avg"][0], want)


def _pipelines_body(comm, rank, n, cases):
    """The large-message role pipelines forced onto small messages: exact two-shot whose results
    go out with multimem.st (variant 4 on a multicast window), and the in-switch reduction
    (variant 5)."""
    import torch

    info = comm.device_info()
    comm.knob("roles_min", 1)
    comm.knob("roles_sub", 8192)
    comm.knob("roles_min_ranks", 2)
    comm.knob("nvls_min", 1)
    outs = []
    for (dt, op, count, exact, seed) in cases:
        comm.tune(variant=0 if not exact else 2, exact=bool(exact))
        x = torch.from_numpy(inputs_for(n, count, dt, seed, tame=True)[rank].view(np.uint8).copy()).cuda()
        y = torch.zeros_like(x)
        comm.all_reduce(x, y, op=op, count=count, dtype=dt)
        comm.all_reduce(x, x, op=op, count=count, dtype=dt)  # in place, the ring buffers in their next cycle
        torch.cuda.synchronize()
        outs.append((y.cpu().numpy(), x.cpu().numpy(), comm.device_info()["variant"]))
    return info, outs, comm.async_error()


@needs2
@pytest.mark.parametrize("n", WORLDS)
def test_allreduce_role_pipelines_with_multicast(n):
    import torch

    cases = []
    for dt, op in ((L.FLOAT32, L.SUM), (L.BFLOAT16, L.AVG), (L.INT32, L.AVG), (L.FLOAT8E4M3, L.SUM), (L.INT64, L.MAX)):
        es = L.DTYPE_SIZE[dt]
        for count in ((3 << 20) // es + 16 // es * 3, (1 << 20) // es):
            cases.append((dt, op, count, 1, len(cases)))            # exact: variant 4
            if dt in (L.INT32, L.INT64):
                cases.append((dt, op, count, 0, len(cases)))        # integers: the switch is exact too
    cases.append((L.FLOAT32, L.SUM, 1 << 20, 0, 77))               # floats through the switch: tolerance
    cases.append((L.BFLOAT16, L.SUM, 1 << 20, 0, 78))
    res = run_ranks(n, _pipelines_body, cases, gpus=True, timeout=180, nvls=True, env={"HXCCL_TUNE_TABLE": "0"})
    nvls = "nvls" in res[0][0]["kind"]
    for k, (dt, op, count, exact, seed) in enumerate(cases):
        xs = inputs_for(n, count, dt, seed, tame=True)
        for r in range(n):
            y, x, variant = res[r][1][k]
            if exact or dt <= L.UINT64:
                want = oracle.allreduce(xs, dt, op, order=0)
                assert np.array_equal(y.view(oracle.raw_dtype(dt)), want[r]), (n, dt, op, count, exact, r, variant)
                assert np.array_equal(x.view(oracle.raw_dtype(dt)), want[r]), ("in place", n, dt, op, count, exact, r, variant)
            else:
                tdt = {L.FLOAT32: torch.float32, L.BFLOAT16: torch.bfloat16}[dt]
                ref = sum(torch.from_numpy(v.copy()).view(tdt).double() for v in xs)
                got = torch.from_numpy(y.copy()).view(tdt).double()
                scale = float(ref.abs().max()) + 1.0
                assert float((got - ref).abs().max()) <= scale * (1e-5 if dt == L.FLOAT32 else 3e-2) * n
            if n > 2 or exact:
                assert variant == (4 if exact else (5 if nvls else 4)), (variant, exact, nvls)
    assert all(r[2] == 0 for r in res)


def _multicast_copy_body(comm, rank, n):
    """AllGather and Broadcast whose pushes go through the multicast alias, sizes from below one
    vector (peer stores only) over odd tails to several pipelined steps; the lines of the small
    AllReduce through the alias too."""
    import torch

    out = {"kind": comm.device_info()["kind"], "ag": [], "bc": [], "ll": []}
    for nb in (8, 16, 1000, 65536 + 24, (5 << 20) + 7):
        x = torch.from_numpy(np.random.default_rng(100 + rank).integers(0, 256, nb, dtype=np.uint8)).cuda()
        ag = torch.zeros(nb * n, dtype=torch.uint8, device="cuda")
        comm.all_gather(x, ag)
        inplace = torch.zeros(nb * n, dtype=torch.uint8, device="cuda")
        inplace[rank * nb:(rank + 1) * nb] = x
        comm.all_gather(inplace[rank * nb:(rank + 1) * nb], inplace)
        for root in (0, n - 1):
            b = x.clone()
            comm.bcast(b, root=root)
            o = torch.zeros_like(x)
            comm.broadcast(x, o, root=root)
            torch.cuda.synchronize()
            want = np.random.default_rng(100 + root).integers(0, 256, nb, dtype=np.uint8)
            out["bc"].append(bool((b.cpu().numpy() == want).all() and (o.cpu().numpy() == want).all()))
        torch.cuda.synchronize()
        want = np.concatenate([np.random.default_rng(100 + r).integers(0, 256, nb, dtype=np.uint8) for r in range(n)])
        out["ag"].append(bool((ag.cpu().numpy() == want).all() and (inplace.cpu().numpy() == want).all()))
    for dt, op, count in ((L.FLOAT32, L.SUM, 1), (L.FLOAT32, L.SUM, 2049), (L.BFLOAT16, L.AVG, 777), (L.INT64, L.MIN, 5),
                          (L.FLOAT8E5M2, L.SUM, 4001)):
        xs = inputs_for(n, count, dt, 900 + count)
        x = torch.from_numpy(xs[rank].view(np.uint8).copy()).cuda()
        for _ in range(3):  # both halves of the line region, and one reuse
            y = torch.zeros_like(x)
            comm.all_reduce(x, y, op=op, count=count, dtype=dt)
        torch.cuda.synchronize()
        out["ll"].append((y.cpu().numpy(), comm.device_info()["variant"]))
    out["err"] = comm.async_error()
    return out


@needs2
@pytest.mark.parametrize("n", WORLDS)
@pytest.mark.parametrize("multicast", [True, False])
def test_multicast_allgather_broadcast_and_lines(n, multicast):
    # the fixed thresholds, not the measured table, so that the variants asserted below are known
    res = run_ranks(n, _multicast_copy_body, gpus=True, timeout=180, nvls=multicast,
                    env={"HXCCL_TUNE_TABLE": "0", "HXCCL_MC_FORCE": "1" if multicast else "0"})
    if multicast and "nvls" not in res[0]["kind"]:
        pytest.skip("no NVSwitch multicast on this node: " + res[0]["kind"])
    cases = ((L.FLOAT32, L.SUM, 1), (L.FLOAT32, L.SUM, 2049), (L.BFLOAT16, L.AVG, 777), (L.INT64, L.MIN, 5),
             (L.FLOAT8E5M2, L.SUM, 4001))
    for r in range(n):
        assert all(res[r]["ag"]) and all(res[r]["bc"]) and res[r]["err"] == 0, (r, res[r]["ag"], res[r]["bc"], res[r]["err"])
        for k, (dt, op, count) in enumerate(cases):
            want = oracle.allreduce(inputs_for(n, count, dt, 900 + count), dt, op)
            got, variant = res[r]["ll"][k]
            assert variant == 7 and np.array_equal(got.view(oracle.raw_dtype(dt)), want[r]), (n, dt, op, count, r, variant)


def _cast_and_ring_rs_body(comm, rank, n):
    import torch

    out = {}
    count = (3 << 20) // 2 + 5
    g = torch.Generator().manual_seed(4242 + rank)
    x = (torch.randn(count, generator=g) * 3).float().cuda()
    y = torch.zeros_like(x)
    comm.all_reduce_cast(x, y, wire_dtype=L.BFLOAT16, op=L.AVG)
    torch.cuda.synchronize()
    out["cast"] = y.cpu().numpy()  # numpy, not a tensor: a tensor's storage would travel by file descriptor
    out["cast_small"] = comm.all_reduce_cast(x[:100], y[:100], wire_dtype=L.BFLOAT16, op=L.AVG, check=False)
    comm.knob("rs_ring_min", 1)
    per = 300001
    xs = inputs_for(n, per * n, L.FLOAT32, 31, tame=True)
    s = torch.from_numpy(xs[rank].view(np.uint8).copy()).cuda()
    r_out = torch.zeros(per * 4, dtype=torch.uint8, device="cuda")
    comm.reduce_scatter(s, r_out, op=L.SUM, count=per, dtype=L.FLOAT32)
    torch.cuda.synchronize()
    out["rs"] = r_out.cpu().numpy().view(np.uint32)
    out["err"] = comm.async_error()
    return out


@needs2
@pytest.mark.parametrize("n", WORLDS)
def test_fused_cast_allreduce_and_ring_reducescatter(n):
    import torch

    res = run_ranks(n, _cast_and_ring_rs_body, gpus=True, timeout=180)
    count = (3 << 20) // 2 + 5
    narrow = [(torch.randn(count, generator=torch.Generator().manual_seed(4242 + r)) * 3).float().to(torch.bfloat16)
              .view(torch.uint16).numpy().copy() for r in range(n)]
    want = oracle.allreduce(narrow, L.BFLOAT16, L.AVG, order=0)
    want_rs = oracle.reducescatter(inputs_for(n, 300001 * n, L.FLOAT32, 31, tame=True), L.FLOAT32, L.SUM)
    for r in range(n):
        w32 = torch.from_numpy(want[r].copy()).view(torch.bfloat16).float()
        assert np.array_equal(res[r]["cast"].view(np.uint32), w32.numpy().view(np.uint32)), r
        assert res[r]["cast_small"] == L.INVALID_USAGE and res[r]["err"] == 0
        assert np.array_equal(res[r]["rs"], want_rs[r]), r


def _crossed_group_body(comm, rank, n):
    """One group over two communicators whose calls name them in opposite order on the two ranks
    (the crossed form of the reference's tests/repro_two_comm_group.cc), with messages far beyond
    what the slot rings hold and several operations per lane: completes only when every rank
    launches the communicators' kernels in the same order."""
    import torch
    import hxccl_b200 as hx

    other = comm.split(0, rank)
    nb = 40 << 20
    peer = 1 - rank
    src = [torch.full((nb,), 10 * rank + k, dtype=torch.uint8, device="cuda") for k in range(3)]
    dst = [torch.zeros(nb, dtype=torch.uint8, device="cuda") for _ in range(3)]
    first, second = (comm, other) if rank == 0 else (other, comm)
    hx.group_start()
    for k in range(3):
        first.send(src[k], peer)
    for k in range(3):
        second.recv(dst[k], peer)
    rc = hx.group_end()
    torch.cuda.synchronize()
    got = [(int(d[0]), int(d[-1])) for d in dst]
    errs = (comm.async_error(), other.async_error())
    other.destroy()
    return rc, got, errs


@needs2
def test_crossed_group_over_two_communicators_with_large_messages():
    res = run_ranks(2, _crossed_group_body, gpus=True, timeout=120)
    for rank, (rc, got, errs) in enumerate(res):
        peer = 1 - rank
        assert rc == 0 and errs == (0, 0), (rank, rc, errs)
        assert got == [(10 * peer + k, 10 * peer + k) for k in range(3)], (rank, got)


def _collectives_body(comm, rank, n):
    import torch
    import hxccl_b200 as hx

    out = {}
    nb = 3 << 20
    x = torch.from_numpy(np.random.default_rng(rank).integers(0, 256, nb, dtype=np.uint8)).cuda()
    ag = torch.zeros(nb * n, dtype=torch.uint8, device="cuda")
    comm.all_gather(x, ag)
    bc = x.clone()
    comm.bcast(bc, root=n - 1)
    a2a = torch.zeros_like(ag)
    comm.all_to_all(ag.clone() + rank, a2a, count=nb, dtype=L.UINT8)
    rs_in = torch.from_numpy(inputs_for(n, 1000 * n, L.FLOAT32, 5)[rank].view(np.uint8).copy()).cuda()
    rs = torch.zeros(4000, dtype=torch.uint8, device="cuda")
    comm.reduce_scatter(rs_in, rs, op=L.SUM, count=1000, dtype=L.FLOAT32)
    # ring shift inside a group, twice (the second launch continues the lane counters)
    got = torch.zeros_like(x)
    for _ in range(2):
        hx.group_start()
        comm.send(x, (rank + 1) % n)
        comm.recv(got, (rank - 1) % n)
        assert hx.group_end() == 0
    torch.cuda.synchronize()
    out["ag"] = bool((ag.cpu().numpy() == np.concatenate([np.random.default_rng(r).integers(0, 256, nb, dtype=np.uint8) for r in range(n)])).all())
    out["bc"] = bool((bc.cpu().numpy() == np.random.default_rng(n - 1).integers(0, 256, nb, dtype=np.uint8)).all())
    out["shift"] = bool((got.cpu().numpy() == np.random.default_rng((rank - 1) % n).integers(0, 256, nb, dtype=np.uint8)).all())
    out["a2a"] = a2a.cpu().numpy()[::nb].tolist()
    out["rs"] = rs.cpu().numpy().view(np.uint32)
    # a buffer on another GPU of this process is refused before anything is launched
    stranger = torch.ones(8, device=f"cuda:{(torch.cuda.current_device() + 1) % torch.cuda.device_count()}")
    out["foreign"] = (comm.all_reduce(stranger, check=False), comm.last_error())
    out["err"] = comm.async_error()
    return out


@needs2
@pytest.mark.parametrize("n", WORLDS)
def test_other_collectives(n):
    res = run_ranks(n, _collectives_body, gpus=True, timeout=120)
    want_rs = oracle.reducescatter(inputs_for(n, 1000 * n, L.FLOAT32, 5), L.FLOAT32, L.SUM)
    for r in range(n):
        assert res[r]["ag"] and res[r]["bc"] and res[r]["shift"] and res[r]["err"] == 0, (r, res[r])
        assert res[r]["foreign"][0] == L.INVALID_ARGUMENT and "lives on CUDA device" in res[r]["foreign"][1]
        assert np.array_equal(res[r]["rs"], want_rs[r])
        first = [int(np.random.default_rng(r).integers(0, 256, 3 << 20, dtype=np.uint8)[0])] * n
        # block j of rank r's result is block r of rank j's send buffer: x_r + j (uint8, wrapping)
        assert res[r]["a2a"] == [(first[0] + i) % 256 for i in range(n)], (r, res[r]["a2a"], first[0])


def _departure_body(comm, rank, n):
    """Rank 1 leaves between two steps (nothing of its in flight); rank 0's next collective must
    end with an error status after the bounded wait, and its CUDA context must stay usable."""
    import time

    import torch

    x = torch.ones(1 << 16, device="cuda")
    comm.all_reduce(x)
    torch.cuda.synchronize()
    assert float(x[0]) == n
    if rank == 1:
        return "left"
    time.sleep(1.0)  # the peer is gone by now (it destroys its communicator when it returns)
    t0 = time.time()
    rc = comm.all_reduce(x, check=False)
    torch.cuda.synchronize()
    waited = time.time() - t0
    err = comm.async_error()
    later = comm.all_reduce(x, check=False)  # the path stays failed: no new launch
    alive = float(torch.ones(8, device="cuda").sum())
    return rc, err, later, comm.last_error(), waited, alive


@needs2
def test_peer_departure_is_reported_not_hung():
    env = {"HXCCL_NVLS": "0", "NCCL_NVLS_ENABLE": "0", "HXCCL_WAIT_LIMIT_MS": "1500"}
    res = run_ranks(2, _departure_body, gpus=True, timeout=120, env=env)
    assert res[1] == "left"
    rc, err, later, msg, waited, alive = res[0]
    assert rc == 0                      # the launch itself succeeds: calls enqueue and return
    assert err == L.TIMEOUT and later == L.TIMEOUT, (err, later, msg)
    assert "ran out of time" in msg and 1.0 < waited < 20.0
    assert alive == 8.0
