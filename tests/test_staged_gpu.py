"""The staged device path (device -> host -> host algorithm -> device), which every rank falls
back to together when peer windows cannot be shared. Two ranks on ONE GPU are such a case (kernels
that wait on each other must not share a GPU), so this runs on a single-GPU machine. Mirrors the
reference's staged runs of tests/gpu_allreduce.cc, gpu_collectives.cc and gpu_p2p.cc."""
import numpy as np
import pytest

import hxccl_b200 as hx
from hxccl_b200 import _lib as L
from hxccl_b200.ops import oracle
from hxccl_b200.utils import run_ranks

pytestmark = pytest.mark.gpu


def inputs_for(n, count, dt, seed):
    es = L.DTYPE_SIZE[dt]
    return [np.random.default_rng(seed * 1000 + r).integers(0, 64, count * es, dtype=np.uint8)
            .view(oracle.raw_dtype(dt)) for r in range(n)]


def _body(comm, rank, n, force):
    import torch

    torch.cuda.set_device(0)
    out = {"kind": comm.device_info()["kind"]}
    res = []
    for dt in (L.INT32, L.FLOAT32, L.BFLOAT16, L.FLOAT8E4M3, L.INT64):
        for op in (L.SUM, L.MAX, L.AVG):
            for count in (1, 4097, 300000):
                x = torch.from_numpy(inputs_for(n, count, dt, dt + count)[rank].view(np.uint8).copy()).cuda()
                y = torch.zeros_like(x)
                comm.reset_stats()
                comm.all_reduce(x, y, op=op, count=count, dtype=dt)
                dev_stats = comm.stats()
                xh, yh = x.cpu().numpy(), np.zeros(x.numel(), dtype=np.uint8)
                comm.reset_stats()
                comm.all_reduce(xh, yh, op=op, count=count, dtype=dt)
                res.append((y.cpu().numpy(), yh, dev_stats, comm.stats()))
    out["allreduce"] = res
    a = torch.full((1000,), float(rank + 1), device="cuda")
    ag = torch.zeros(1000 * n, device="cuda")
    comm.all_gather(a, ag)
    out["ag"] = ag.cpu().numpy()[::1000].tolist()
    got = torch.zeros(1000, device="cuda")
    hx.group_start()
    comm.send(a, (rank + 1) % n)
    comm.recv(got, (rank - 1) % n)
    out["group"] = hx.group_end()
    out["shift"] = float(got[0])
    # mixing host and device buffers in one call / one group is refused
    out["mixed_call"] = comm.all_reduce(a, np.zeros(1000, dtype=np.float32), check=False)
    hx.group_start()
    comm.send(a, (rank + 1) % n)
    comm.recv(np.zeros(1000, dtype=np.float32), (rank - 1) % n)
    out["mixed_group"] = hx.group_end()
    return out


@pytest.mark.parametrize("force", [False, True])
def test_staged_path_matches_host_path(force):
    n = 2
    env = {"HXCCL_DEVICE_TRANSPORT": "staged"} if force else {}
    # both ranks on device 0, also on a machine with more GPUs: that is the case under test
    res = run_ranks(n, _body, force, gpus=True, timeout=180, env=env, one_gpu=True)
    k = 0
    for r in range(n):
        assert res[r]["kind"] == "staged", res[r]["kind"]
    for dt in (L.INT32, L.FLOAT32, L.BFLOAT16, L.FLOAT8E4M3, L.INT64):
        for op in (L.SUM, L.MAX, L.AVG):
            for count in (1, 4097, 300000):
                want = oracle.allreduce(inputs_for(n, count, dt, dt + count), dt, op)
                for r in range(n):
                    dev, host, dev_stats, host_stats = res[r]["allreduce"][k]
                    assert np.array_equal(dev.view(oracle.raw_dtype(dt)), want[r]), (dt, op, count, r)
                    assert np.array_equal(dev, host)
                    assert dev_stats == host_stats  # the same call books the same traffic on both paths
                k += 1
    for r in range(n):
        assert res[r]["ag"] == [1.0, 2.0] and res[r]["group"] == 0 and res[r]["shift"] == float((r - 1) % n + 1)
        assert res[r]["mixed_call"] == L.INVALID_ARGUMENT and res[r]["mixed_group"] == L.INVALID_USAGE


def _copy_failure(comm, rank, n):
    import torch

    x = torch.ones(100, device="cuda")
    rc = comm.all_reduce(x, check=False)
    return rc, comm.last_error(), comm.all_reduce(x, check=False)


def test_injected_copy_failure_is_an_error_on_the_failing_rank():
    """Host-side fault injection: the device-to-host copy of rank 0 'fails'."""
    res = run_ranks(2, _copy_failure, gpus=True, timeout=60, env={"HXCCL_NET_TIMEOUT_MS": "3000"},
                    rank_env={0: {"HXCCL_TEST_FAIL_DEVICE_COPY": "1"}}, one_gpu=True)
    rc0, msg0, again0 = res[0]
    assert rc0 == L.UNHANDLED_CUDA and "injected" in msg0 and again0 == L.UNHANDLED_CUDA  # sticky
    assert res[1][0] != 0  # the peer does not hang: its receive times out or sees the closed mesh
