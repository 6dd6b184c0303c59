"""Registration of the "hxccl" torch.distributed backend (C++: hxccl_b200/csrc/backend.cpp).

    import hxccl_b200.parallel            # registers the backend
    dist.init_process_group("hxccl", ...)  # or "cpu:gloo,cuda:hxccl"

CUDA tensors run on the library's kernels, asynchronously on a communication stream; CPU
tensors run on its host path. (Reference: python/hxccl_torch/__init__.py:1-17.)
"""
from __future__ import annotations

import importlib
import importlib.util
from pathlib import Path

_ext = None


def extension():
    """The compiled backend module, built on first use when missing."""
    global _ext
    if _ext is not None:
        return _ext
    import torch  # noqa: F401,PLC0415  (libtorch must be loaded before the extension)

    from .. import _lib  # noqa: PLC0415

    _lib.lib()  # libhxccl.so first: the extension links against it
    so = Path(__file__).resolve().parent.parent / "_hxccl_c10d.so"
    if not so.exists():
        from .. import build  # noqa: PLC0415

        build.build_torch_ext()
    spec = importlib.util.spec_from_file_location("_hxccl_c10d", so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    _ext = mod
    return mod


_registered = False


def register() -> None:
    """Makes `backend="hxccl"` known to torch.distributed (idempotent)."""
    global _registered
    if _registered:
        return
    import torch.distributed as dist  # noqa: PLC0415

    from ..utils.env import fill_env_from_openmpi  # noqa: PLC0415

    fill_env_from_openmpi()  # under mpirun: RANK / WORLD_SIZE / LOCAL_RANK from Open MPI's variables
    ext = extension()
    dist.Backend.register_backend("hxccl", ext.create_backend, devices=["cuda", "cpu"])
    _registered = True


def _backend_of(group=None, device="cuda"):
    import torch  # noqa: PLC0415
    import torch.distributed as dist  # noqa: PLC0415

    pg = group if group is not None else dist.distributed_c10d._get_default_group()
    return pg._get_backend(torch.device(device))


def tune(variant: int = 0, exact: bool = True, max_ctas: int = 0, group=None) -> None:
    """hxcclCommTune for the communicator behind a process group; call on every rank."""
    extension().tune(_backend_of(group), variant, int(exact), max_ctas)


def all_reduce_cast(tensor, bf16: bool = True, average: bool = True, group=None):
    """In-place AllReduce of an fp32 CUDA tensor with bfloat16 (or float16) on the wire, as one
    kernel (hxcclAllReduceCast). Returns the Work object; the tensor needs at least 32 Ki elements."""
    return extension().allreduce_cast(_backend_of(group), tensor, bf16, average)


def device_info(group=None) -> dict:
    kind, variant, launches = extension().device_info(_backend_of(group))
    return {"kind": kind, "variant": variant, "launches": launches}
