"""DistributedDataParallel glue: gradient buckets are averaged by one AllReduce whose 1/N
scaling happens inside the kernel (hxcclAvg pre-multiplies every rank's input by 1/N as it is
read, so no separate division pass touches the bucket), issued on the backend's communication
stream so that it overlaps the rest of backward.

    model = DDP(model, device_ids=[dev], bucket_cap_mb=25)
    model.register_comm_hook(None, fused_average_hook)
"""
from __future__ import annotations


def fused_average_hook(state, bucket):
    """DDP communication hook: AllReduce(AVG) of the flat bucket, returned as a Future."""
    import torch.distributed as dist  # noqa: PLC0415

    group = state if state is not None else dist.group.WORLD
    buf = bucket.buffer()
    work = dist.all_reduce(buf, op=dist.ReduceOp.AVG, group=group, async_op=True)
    return work.get_future().then(lambda fut: fut.value()[0])


def bf16_compress_average_hook(state, bucket):
    """Like fused_average_hook with half the bytes on the links: the bucket is cast to bfloat16,
    averaged in bfloat16 (each rank's contribution is scaled by 1/N and rounded to bfloat16 before
    the sum, the library's Avg rule) and cast back into the bucket when the collective is done."""
    import torch  # noqa: PLC0415
    import torch.distributed as dist  # noqa: PLC0415

    group = state if state is not None else dist.group.WORLD
    buf = bucket.buffer()
    small = buf.to(torch.bfloat16)
    work = dist.all_reduce(small, op=dist.ReduceOp.AVG, group=group, async_op=True)

    def widen(fut):
        buf.copy_(fut.value()[0])
        return buf

    return work.get_future().then(widen)


def wrap(module, device=None, bucket_cap_mb: int = 25, process_group=None, compress: bool = False, **kw):
    """DDP around `module` with the fused averaging hook installed (`compress=True`: the bfloat16
    variant). `device=None` wraps a CPU module (the backend's host path)."""
    from torch.nn.parallel import DistributedDataParallel as DDP  # noqa: PLC0415

    ddp = DDP(module, device_ids=None if device is None else [device], bucket_cap_mb=bucket_cap_mb,
              process_group=process_group, gradient_as_bucket_view=True, **kw)
    ddp.register_comm_hook(process_group, bf16_compress_average_hook if compress else fused_average_hook)
    return ddp
