"""Launch-environment helpers (reference: python/hxccl_torch/launch.py:4-12)."""
from __future__ import annotations

import os


def fill_env_from_openmpi() -> None:
    """Under mpirun, derive torch.distributed's variables from Open MPI's; set the default
    rendezvous address and port when nothing else did."""
    for ompi, ours in (("OMPI_COMM_WORLD_RANK", "RANK"), ("OMPI_COMM_WORLD_SIZE", "WORLD_SIZE"),
                       ("OMPI_COMM_WORLD_LOCAL_RANK", "LOCAL_RANK")):
        if ompi in os.environ:
            os.environ.setdefault(ours, os.environ[ompi])
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
