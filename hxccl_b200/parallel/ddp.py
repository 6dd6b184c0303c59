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


def wrap(module, device, bucket_cap_mb: int = 25, process_group=None, **kw):
    """DDP around `module` with the fused averaging hook installed."""
    from torch.nn.parallel import DistributedDataParallel as DDP  # noqa: PLC0415

    ddp = DDP(module, device_ids=[device], bucket_cap_mb=bucket_cap_mb, process_group=process_group,
              gradient_as_bucket_view=True, **kw)
    ddp.register_comm_hook(process_group, fused_average_hook)
    return ddp
