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
    """Like fused_average_hook with half the bytes on the links: every gradient is rounded to
    bfloat16, scaled by 1/N and summed in bfloat16 (the library's Avg rule), and the result is
    widened back into the fp32 bucket. On the window device path all of that is one kernel
    (hxcclAllReduceCast: the cast happens as the bucket is read and written); small buckets and
    the other paths cast with tensor ops around an ordinary bfloat16 AllReduce, with the same bits."""
    import torch  # noqa: PLC0415
    import torch.distributed as dist  # noqa: PLC0415

    from . import backend as hb  # noqa: PLC0415

    group = state if state is not None else dist.group.WORLD
    buf = bucket.buffer()
    if (buf.is_cuda and buf.dtype == torch.float32 and buf.numel() * 2 >= 64 * 1024
            and dist.get_world_size(group) > 1 and _fused_cast_ok(group)):
        work = hb.all_reduce_cast(buf, bf16=True, average=True, group=None if state is None else group)
        return work.get_future().then(lambda fut: fut.value()[0])
    small = buf.to(torch.bfloat16)
    work = dist.all_reduce(small, op=dist.ReduceOp.AVG, group=group, async_op=True)

    def widen(fut):
        buf.copy_(fut.value()[0])
        return buf

    return work.get_future().then(widen)


_FUSED_OK: dict = {}


def _fused_cast_ok(group) -> bool:
    """Whether the group's communicator runs on the window device path (asked once per group)."""
    key = id(group)
    if key not in _FUSED_OK:
        from . import backend as hb  # noqa: PLC0415

        try:
            _FUSED_OK[key] = hb.device_info(group).get("kind", "").startswith("window")
        except Exception:  # noqa: BLE001  (another backend behind this group)
            _FUSED_OK[key] = False
    return _FUSED_OK[key]


def wrap(module, device=None, bucket_cap_mb: int = 25, process_group=None, compress: bool = False, **kw):
    """DDP around `module` with the fused averaging hook installed (`compress=True`: the bfloat16
    variant). `device=None` wraps a CPU module (the backend's host path)."""
    from torch.nn.parallel import DistributedDataParallel as DDP  # noqa: PLC0415

    ddp = DDP(module, device_ids=None if device is None else [device], bucket_cap_mb=bucket_cap_mb,
              process_group=process_group, gradient_as_bucket_view=True, **kw)
    ddp.register_comm_hook(process_group, bf16_compress_average_hook if compress else fused_average_hook)
    return ddp
