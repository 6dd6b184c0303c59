"""hxccl for B200: NCCL-style collectives over NVLink 5 / NVSwitch with hxccl 0.2's C API and
semantics. The native library (C API, host path, sm_100a kernels) is built in-tree by
`python -m hxccl_b200.build`; this package is its Python face:

  hxccl_b200.comm       Communicator over numpy arrays / torch tensors (ctypes)
  hxccl_b200.parallel   torch.distributed "hxccl" backend, DDP gradient hooks
  hxccl_b200.ops        single-GPU elementwise kernels and the world-on-one-GPU harness
  hxccl_b200.models     GPT-2 used by the training benchmark
  hxccl_b200.utils      process launcher, environment helpers
"""
from ._lib import (AVG, BFLOAT16, FLOAT8E4M3, FLOAT8E5M2, FLOAT16, FLOAT32, FLOAT64, INT8, INT32,  # noqa: F401
                   INT64, MAX, MIN, PROD, SUM, UINT8, UINT32, UINT64)
from .comm import Communicator, HxcclError, get_unique_id, get_version, group_end, group_start  # noqa: F401

__version__ = "0.2.0"
