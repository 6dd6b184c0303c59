"""torch.distributed integration: the "hxccl" backend and DDP helpers."""
from .backend import all_reduce_cast, device_info, extension, register, tune  # noqa: F401
from .ddp import bf16_compress_average_hook, fused_average_hook, wrap  # noqa: F401
