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
                    env={"HXCCL_IPC_CHUNK": "4096", "HXCCL_RING_MIN": str(4 << 20)},
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
    out["err"] = comm.async_error()
    return out


@needs2
@pytest.mark.parametrize("n", WORLDS)
def test_other_collectives(n):
    res = run_ranks(n, _collectives_body, gpus=True, timeout=120)
    want_rs = oracle.reducescatter(inputs_for(n, 1000 * n, L.FLOAT32, 5), L.FLOAT32, L.SUM)
    for r in range(n):
        assert res[r]["ag"] and res[r]["bc"] and res[r]["shift"] and res[r]["err"] == 0, (r, res[r])
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
