"""The "hxccl" torch.distributed backend on CUDA tensors, one process per GPU: results against
plain arithmetic, asynchronous Work objects, and a DistributedDataParallel step whose gradients
must match an NCCL run of the same model."""
import os

import pytest

from conftest import gpu_count

torch = pytest.importorskip("torch")
import torch.distributed as dist  # noqa: E402
import torch.multiprocessing as mp  # noqa: E402

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
NGPU = gpu_count()
WAIT_LIMIT_MS = 5000


def _worker(rank, world, port, q):
    try:
        import hxccl_b200.parallel as hp
        from hxccl_b200.models import GPT2, GPT2Config
        from torch.nn.parallel import DistributedDataParallel as DDP

        torch.cuda.set_device(rank)
        hp.register()
        # not about multicast: windows stay unbound, and waits are short, so that a rank whose
        # peer failed leaves through its bounded wait instead of being ended from outside
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), HXCCL_NVLS="0",
                          HXCCL_WAIT_LIMIT_MS=str(WAIT_LIMIT_MS))
        dist.init_process_group("hxccl", rank=rank, world_size=world)
        assert hp.device_info()["kind"].startswith("window")
        dev = torch.device("cuda", rank)
        for dtype in (torch.float32, torch.bfloat16, torch.float16, torch.int32, torch.int64):
            x = (torch.arange(100003, device=dev) % 7 + rank).to(dtype)
            dist.all_reduce(x)
            want = (torch.arange(100003, device=dev) % 7).to(torch.float64) * world + sum(range(world))
            assert torch.equal(x.double(), want), dtype
        y = torch.full((1 << 22,), float(rank + 1), device=dev)
        w = dist.all_reduce(y, op=dist.ReduceOp.AVG, async_op=True)
        z = torch.ones(8, device=dev) * 3  # work on the caller's stream while the collective runs
        w.wait()
        assert torch.allclose(y, torch.full_like(y, (world + 1) / 2)) and float(z.sum()) == 24.0
        fut = dist.all_reduce(torch.ones(4, device=dev), async_op=True).get_future()
        assert float(fut.wait()[0].sum()) == 4.0 * world
        out = torch.empty(world * 5, device=dev)
        dist.all_gather_into_tensor(out, torch.full((5,), float(rank), device=dev))
        assert out.tolist() == [float(r) for r in range(world) for _ in range(5)]
        rs = torch.empty(3, device=dev)
        dist.reduce_scatter_tensor(rs, torch.arange(3 * world, dtype=torch.float32, device=dev))
        assert rs.tolist() == [world * (3.0 * rank + k) for k in range(3)]
        b = torch.full((9,), float(rank), device=dev)
        dist.broadcast(b, src=world - 1)
        assert b.tolist() == [float(world - 1)] * 9
        a2a = torch.empty(world * 2, device=dev)
        dist.all_to_all_single(a2a, torch.arange(world * 2, dtype=torch.float32, device=dev) + 100 * rank)
        assert a2a.tolist() == [100.0 * r + 2 * rank + k for r in range(world) for k in range(2)]
        if rank == 0:
            dist.send(torch.tensor([42.0], device=dev), dst=1)
        elif rank == 1:
            t = torch.zeros(1, device=dev)
            dist.recv(t, src=0)
            assert t.item() == 42.0
        # fp32 bucket with bfloat16 on the wire: the one-kernel form against the casts done here
        g32 = torch.randn(300007, device=dev, generator=torch.Generator(device=dev).manual_seed(9 + rank))
        two_pass = g32.to(torch.bfloat16)
        dist.all_reduce(two_pass, op=dist.ReduceOp.AVG)
        fused = g32.clone()
        hp.all_reduce_cast(fused, bf16=True, average=True).wait()
        assert torch.equal(fused.view(torch.int32), two_pass.float().view(torch.int32))
        dist.barrier()
        # DDP: two steps with the fused-average hook; gradients equal the average of the ranks'
        torch.manual_seed(0)
        model = GPT2(GPT2Config.tiny()).to(dev)
        ref = GPT2(GPT2Config.tiny()).to(dev)
        ref.load_state_dict(model.state_dict())
        ddp = DDP(model, device_ids=[rank], bucket_cap_mb=1)
        ddp.register_comm_hook(None, hp.fused_average_hook)
        gen = torch.Generator(device=dev).manual_seed(5 + rank)
        x = torch.randint(0, 512, (4, 65), device=dev, generator=gen)
        ddp(x[:, :-1], x[:, 1:]).backward()
        ref(x[:, :-1], x[:, 1:]).backward()
        for p, rp in zip(model.parameters(), ref.parameters()):
            g = rp.grad.clone()
            dist.all_reduce(g)  # plain sum through the backend, divided here
            assert torch.allclose(p.grad, g / world, rtol=1e-5, atol=1e-7)
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except BaseException as e:  # noqa: BLE001
        import traceback

        q.put((rank, f"{e!r}\n{traceback.format_exc()}"))


@pytest.mark.skipif(NGPU < 2, reason="needs two GPUs")
@pytest.mark.parametrize("world", [n for n in (2, 4) if n <= NGPU])
def test_backend_on_gpus(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, 29680 + world, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = []
    try:
        for _ in range(world):
            got.append(q.get(timeout=240))
            if got[-1][1] != "ok":
                break
    finally:
        # survivors of a failed run leave on their own once their device-side waits run out and
        # their process group is torn down; only after that grace period is a process ended
        import time

        give_up = time.monotonic() + WAIT_LIMIT_MS / 1000.0 + 10.0
        for p in procs:
            p.join(max(0.1, give_up - time.monotonic()))
        for p in procs:
            if p.is_alive():
                p.kill()
    assert len(got) == world and all(m == "ok" for _, m in got), got
