"""ctypes binding of libhxccl.so (include/hxccl.h and include/hxccl_ext.h)."""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent / "lib" / "libhxccl.so"

# result codes / dtypes / ops: NCCL numbering (include/hxccl.h)
SUCCESS, UNHANDLED_CUDA, SYSTEM_ERROR, INTERNAL_ERROR, INVALID_ARGUMENT, INVALID_USAGE, \
    REMOTE_ERROR, IN_PROGRESS, TIMEOUT = range(9)
INT8, UINT8, INT32, UINT32, INT64, UINT64, FLOAT16, FLOAT32, FLOAT64, BFLOAT16, FLOAT8E4M3, \
    FLOAT8E5M2 = range(12)
SUM, PROD, MAX, MIN, AVG = range(5)
NUM_OPS = 5
SCALAR_DEVICE, SCALAR_HOST_IMMEDIATE = 0, 1
SPLIT_NOCOLOR = -1
CONFIG_MAGIC = 0x6878636C
CONFIG_UNDEF_INT = -(2 ** 31)

DTYPE_SIZE = {INT8: 1, UINT8: 1, INT32: 4, UINT32: 4, INT64: 8, UINT64: 8, FLOAT16: 2, FLOAT32: 4,
              FLOAT64: 8, BFLOAT16: 2, FLOAT8E4M3: 1, FLOAT8E5M2: 1}


class UniqueId(C.Structure):
    _fields_ = [("internal", C.c_char * 128)]


class Config(C.Structure):
    _fields_ = [("size", C.c_size_t), ("magic", C.c_uint), ("version", C.c_uint),
                ("blocking", C.c_int), ("commName", C.c_char_p)]

    @classmethod
    def initializer(cls) -> "Config":
        return cls(C.sizeof(cls), CONFIG_MAGIC, 200, CONFIG_UNDEF_INT, None)


_lib = None


def lib() -> C.CDLL:
    """Loads the library, building it first when the shared object is missing."""
    global _lib
    if _lib is not None:
        return _lib
    override = os.environ.get("HXCCL_LIBRARY")  # e.g. the sanitizer build (python -m hxccl_b200.build --sanitize)
    if override:
        path = Path(override)
    else:
        path = _LIB_PATH
    if not path.exists():
        if override or os.environ.get("HXCCL_NO_AUTOBUILD"):
            raise OSError(f"{path} is missing; run `python -m hxccl_b200.build`")
        from . import build  # noqa: PLC0415

        build.build_lib()
    L = C.CDLL(str(path), mode=C.RTLD_GLOBAL)
    vp, sz, i, u64p = C.c_void_p, C.c_size_t, C.c_int, C.POINTER(C.c_uint64)
    szp = C.POINTER(C.c_size_t)
    sig = {
        "hxcclGetVersion": [C.POINTER(i)],
        "hxcclGetUniqueId": [C.POINTER(UniqueId)],
        "hxcclCommInitRank": [C.POINTER(vp), i, UniqueId, i],
        "hxcclCommInitRankConfig": [C.POINTER(vp), i, UniqueId, i, C.POINTER(Config)],
        "hxcclCommDestroy": [vp],
        "hxcclCommSplit": [vp, i, i, C.POINTER(vp), C.POINTER(Config)],
        "hxcclCommShrink": [vp, C.POINTER(i), i, C.POINTER(vp), C.POINTER(Config), i],
        "hxcclCommAbort": [vp],
        "hxcclCommFinalize": [vp],
        "hxcclCommGetAsyncError": [vp, C.POINTER(i)],
        "hxcclCommCount": [vp, C.POINTER(i)],
        "hxcclCommUserRank": [vp, C.POINTER(i)],
        "hxcclAllReduce": [vp, vp, sz, i, i, vp, vp],
        "hxcclAllReduceCast": [vp, vp, sz, i, i, vp, vp],
        "hxcclAllGather": [vp, vp, sz, i, vp, vp],
        "hxcclReduceScatter": [vp, vp, sz, i, i, vp, vp],
        "hxcclBroadcast": [vp, vp, sz, i, i, vp, vp],
        "hxcclReduce": [vp, vp, sz, i, i, i, vp, vp],
        "hxcclBcast": [vp, sz, i, i, vp, vp],
        "hxcclGather": [vp, vp, sz, i, i, vp, vp],
        "hxcclScatter": [vp, vp, sz, i, i, vp, vp],
        "hxcclAlltoAll": [vp, vp, sz, i, vp, vp],
        "hxcclAllToAll": [vp, vp, sz, i, vp, vp],
        "hxcclAllToAllv": [vp, szp, szp, vp, szp, szp, i, vp, vp],
        "hxcclSend": [vp, sz, i, i, vp, vp],
        "hxcclRecv": [vp, sz, i, i, vp, vp],
        "hxcclGroupStart": [],
        "hxcclGroupEnd": [],
        "hxcclRedOpCreatePreMulSum": [C.POINTER(i), vp, i, i, vp],
        "hxcclRedOpDestroy": [i, vp],
        "hxcclCommGetStats": [vp, u64p, u64p],
        "hxcclCommResetStats": [vp],
        # extensions
        "hxcclCommDeviceInfo": [vp, C.c_char_p, sz, C.POINTER(i), C.POINTER(C.c_ulonglong)],
        "hxcclCommTune": [vp, i, i, i],
        "hxcclCommTuneKnob": [vp, C.c_char_p, C.c_long],
        "hxcclCommReadTrace": [vp, C.POINTER(C.c_ulonglong), i],
        "hxcclWorldTuneKnob": [vp, C.c_char_p, C.c_long],
        "hxcclDevReduce": [vp, vp, sz, i, i, vp],
        "hxcclDevScale": [vp, vp, sz, i, vp, vp],
        "hxcclDevDivide": [vp, sz, i, i, vp],
        "hxcclHostReduce": [vp, vp, sz, i, i],
        "hxcclHostScale": [vp, vp, sz, i, vp],
        "hxcclHostDivide": [vp, sz, i, i],
        "hxcclTestFailSends": [vp, C.c_long],
        "hxcclTestSeverPeer": [vp, i],
        "hxcclWorldCreate": [C.POINTER(vp), i, i, i],
        "hxcclWorldDestroy": [vp],
        "hxcclWorldTune": [vp, i, i, i],
        "hxcclWorldAllReduce": [vp, C.POINTER(vp), C.POINTER(vp), sz, i, i, vp, i, vp],
        "hxcclWorldAllReduceCast": [vp, C.POINTER(vp), C.POINTER(vp), sz, i, i, vp],
        "hxcclWorldReduceScatter": [vp, C.POINTER(vp), C.POINTER(vp), sz, i, i, vp, vp],
        "hxcclWorldReduce": [vp, C.POINTER(vp), C.POINTER(vp), sz, i, i, vp, i, vp],
        "hxcclWorldAllGather": [vp, C.POINTER(vp), C.POINTER(vp), sz, vp],
        "hxcclWorldBroadcast": [vp, C.POINTER(vp), C.POINTER(vp), sz, i, vp],
        "hxcclWorldGather": [vp, C.POINTER(vp), C.POINTER(vp), sz, i, vp],
        "hxcclWorldScatter": [vp, C.POINTER(vp), C.POINTER(vp), sz, i, vp],
        "hxcclWorldAllToAllv": [vp, C.POINTER(vp), C.POINTER(vp), szp, szp, szp, vp],
        "hxcclWorldSendRecv": [vp, i, C.POINTER(i), C.POINTER(i), C.POINTER(vp), szp,
                               C.POINTER(vp), szp, vp],
        "hxcclWorldStatus": [vp, i, C.POINTER(C.c_ulonglong), C.POINTER(C.c_ulonglong)],
        "hxcclWorldInfo": [vp, C.POINTER(i), C.POINTER(C.c_ulonglong)],
        "hxcclWorldMute": [vp, i],
    }
    for name, args in sig.items():
        fn = getattr(L, name)
        fn.argtypes = args
        fn.restype = i
    L.hxcclGetErrorString.argtypes = [i]
    L.hxcclGetErrorString.restype = C.c_char_p
    L.hxcclGetLastError.argtypes = [vp]
    L.hxcclGetLastError.restype = C.c_char_p
    L.hxcclWorldLastError.argtypes = []
    L.hxcclWorldLastError.restype = C.c_char_p
    L.hxcclHostEncode.argtypes = [i, C.c_float]
    L.hxcclHostEncode.restype = C.c_uint
    L.hxcclHostDecode.argtypes = [i, C.c_uint]
    L.hxcclHostDecode.restype = C.c_float
    L.hxcclRingBlock.argtypes = [sz, i, i, szp, szp]
    L.hxcclRingBlock.restype = None
    _lib = L
    return L
