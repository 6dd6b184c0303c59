"""The torch.distributed "hxccl" backend on CPU tensors (host path), against gloo on the same
inputs: the reference's python/tests/test_backend.py:24-77 strategy. The CUDA side of the
backend is exercised by tests/test_torch_backend_gpu.py."""
import os

import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist  # noqa: E402
import torch.multiprocessing as mp  # noqa: E402


def _worker(rank, world, port, q):
    try:
        import hxccl_b200.parallel as hp

        hp.register()
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("hxccl", rank=rank, world_size=world)
        ref = dist.new_group(backend="gloo")
        torch.manual_seed(rank)
        for dtype in (torch.float32, torch.int32, torch.bfloat16, torch.float16):
            for op in (dist.ReduceOp.SUM, dist.ReduceOp.MAX):
                for n in (1, 1000, 100000):
                    x = (torch.rand(n) * 10).to(dtype)
                    a, b = x.clone(), x.clone()
                    dist.all_reduce(a, op=op)
                    dist.all_reduce(b, op=op, group=ref)
                    tol = 0 if dtype in (torch.int32,) or op == dist.ReduceOp.MAX else 2e-2
                    assert torch.allclose(a.float(), b.float(), rtol=tol, atol=tol), (dtype, op, n)
        x = torch.arange(6, dtype=torch.float32) + rank
        y = x.clone()
        dist.all_reduce(y, op=dist.ReduceOp.AVG)
        assert torch.allclose(y, torch.arange(6, dtype=torch.float32) + (world - 1) / 2)
        out = torch.empty(world * 4)
        dist.all_gather_into_tensor(out, torch.full((4,), float(rank)))
        assert out.tolist() == [float(r) for r in range(world) for _ in range(4)]
        outs = [torch.empty(3) for _ in range(world)]
        dist.all_gather(outs, torch.full((3,), float(rank)))
        assert [o[0].item() for o in outs] == [float(r) for r in range(world)]
        rs = torch.empty(5)
        dist.reduce_scatter_tensor(rs, torch.arange(5 * world, dtype=torch.float32))
        assert torch.allclose(rs, world * (torch.arange(5, dtype=torch.float32) + 5 * rank))
        b = torch.full((7,), float(rank))
        dist.broadcast(b, src=world - 1)
        assert b.tolist() == [float(world - 1)] * 7
        a2a = torch.empty(world * 2)
        dist.all_to_all_single(a2a, torch.arange(world * 2, dtype=torch.float32) + 100 * rank)
        assert a2a.tolist() == [100.0 * r + 2 * rank + k for r in range(world) for k in range(2)]
        if rank == 0:
            dist.send(torch.tensor([42.0]), dst=1)
        elif rank == 1:
            t = torch.zeros(1)
            dist.recv(t, src=0)
            assert t.item() == 42.0
        g = [torch.empty(2) for _ in range(world)] if rank == 0 else None
        dist.gather(torch.full((2,), float(rank)), g, dst=0)
        if rank == 0:
            assert [t[0].item() for t in g] == [float(r) for r in range(world)]
        sc = torch.empty(2)
        dist.scatter(sc, [torch.full((2,), float(r)) for r in range(world)] if rank == 0 else None, src=0)
        assert sc.tolist() == [float(rank)] * 2
        # a batch of sends and receives is one hxccl group: a crossed exchange of 8 MiB with both
        # ranks naming the send first runs without either side waiting for the other's order
        nxt, prv = (rank + 1) % world, (rank - 1) % world
        big_out = torch.full((2 << 20,), float(rank))
        big_in, small_in = torch.empty(2 << 20), torch.empty(3)
        works = dist.batch_isend_irecv([dist.P2POp(dist.isend, big_out, nxt),
                                        dist.P2POp(dist.isend, torch.full((3,), rank + 0.5), nxt),
                                        dist.P2POp(dist.irecv, big_in, prv),
                                        dist.P2POp(dist.irecv, small_in, prv)])
        for w in works:
            w.wait()
        assert big_in[0].item() == float(prv) and big_in[-1].item() == float(prv)
        assert small_in.tolist() == [prv + 0.5] * 3
        offered = dist.distributed_c10d._get_default_group()._get_backend(torch.device("cpu")).supports_coalescing
        assert offered == (not torch.cuda.is_available() or os.environ.get("HXCCL_TORCH_COALESCE") == "1")
        if offered:  # several collectives under torch's coalescing manager
            c1, c2 = torch.full((5,), float(rank)), torch.full((70000,), 1.0)
            with dist.distributed_c10d._coalescing_manager(device=torch.device("cpu")):
                dist.all_reduce(c1)
                dist.all_reduce(c2)
            assert c1.tolist() == [float(sum(range(world)))] * 5 and c2[-1].item() == float(world)
        dist.barrier()
        with pytest.raises((ValueError, RuntimeError)):
            dist.all_reduce(torch.zeros(4, 4).t())  # not contiguous
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except BaseException as e:  # noqa: BLE001
        import traceback

        q.put((rank, f"{e!r}\n{traceback.format_exc()}"))


@pytest.mark.parametrize("world", [2, 4])
def test_backend_matches_gloo(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29650 + world
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = [q.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(10)
        if p.is_alive():
            p.kill()
    assert all(m == "ok" for _, m in got), got


def _ddp_worker(rank, world, port, q):
    """Two steps of SGD on a small CPU model under DDP with each hook; every rank must end with the
    weights of a single process that saw the whole batch (exactly for the fp32 hook up to summation
    order, within bfloat16 rounding for the compressing one)."""
    try:
        import hxccl_b200.parallel as hp

        hp.register()
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("hxccl", rank=rank, world_size=world)
        torch.manual_seed(0)
        data, target = torch.randn(world * 8, 16), torch.randn(world * 8, 4)

        def make():
            torch.manual_seed(1)
            return torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.Tanh(), torch.nn.Linear(32, 4))

        def train(model, x, y):
            opt = torch.optim.SGD(model.parameters(), lr=0.1)
            for _ in range(2):
                opt.zero_grad()
                torch.nn.functional.mse_loss(model(x), y).backward()
                opt.step()
            return torch.cat([p.detach().flatten() for p in model.parameters()])

        want = train(make(), data, target)  # the whole batch in one process
        mine = slice(rank * 8, rank * 8 + 8)
        for compress, tol in ((False, 1e-5), (True, 2e-2)):
            got = train(hp.wrap(make(), compress=compress, bucket_cap_mb=1), data[mine], target[mine])
            assert torch.allclose(got, want, rtol=tol, atol=tol), (compress, (got - want).abs().max())
            same = [torch.empty_like(got) for _ in range(world)]
            dist.all_gather(same, got)
            assert all(torch.equal(s, same[0]) for s in same)  # replicas stay identical
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except BaseException as e:  # noqa: BLE001
        import traceback

        q.put((rank, f"{e!r}\n{traceback.format_exc()}"))


def test_ddp_hooks_on_cpu():
    world, ctx = 2, mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_ddp_worker, args=(r, world, 29671, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = [q.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(10)
        if p.is_alive():
            p.kill()
    assert all(m == "ok" for _, m in got), got
