"""Python face of the C API: a Communicator whose methods take numpy arrays (host buffers) or
torch tensors (host or CUDA). Device calls enqueue on the given (or current) CUDA stream and
return before the work is done, exactly like the C functions they wrap."""
from __future__ import annotations

import ctypes as C
from typing import Any, Optional, Sequence

import numpy as np

from . import _lib as L


class HxcclError(RuntimeError):
    def __init__(self, code: int, what: str, detail: str = ""):
        self.code = code
        name = L.lib().hxcclGetErrorString(code).decode()
        super().__init__(f"{what}: {name} ({code})" + (f": {detail}" if detail else ""))


_NP_DT = {np.dtype(np.int8): L.INT8, np.dtype(np.uint8): L.UINT8, np.dtype(np.int32): L.INT32,
          np.dtype(np.uint32): L.UINT32, np.dtype(np.int64): L.INT64, np.dtype(np.uint64): L.UINT64,
          np.dtype(np.float16): L.FLOAT16, np.dtype(np.float32): L.FLOAT32,
          np.dtype(np.float64): L.FLOAT64}


_TORCH_DT: dict = {}  # filled on first use: torch is imported only when tensors show up


def _torch_dt(t) -> int:
    if not _TORCH_DT:
        import torch  # noqa: PLC0415

        _TORCH_DT.update({torch.int8: L.INT8, torch.uint8: L.UINT8, torch.int32: L.INT32, torch.int64: L.INT64,
                          torch.float16: L.FLOAT16, torch.float32: L.FLOAT32, torch.float64: L.FLOAT64,
                          torch.bfloat16: L.BFLOAT16, torch.float8_e4m3fn: L.FLOAT8E4M3,
                          torch.float8_e5m2: L.FLOAT8E5M2})
        for name, code in (("uint32", L.UINT32), ("uint64", L.UINT64)):
            if hasattr(torch, name):
                _TORCH_DT[getattr(torch, name)] = code
    return _TORCH_DT[t.dtype]


def ptr(buf: Any) -> Optional[int]:
    """Address of a numpy array / torch tensor / raw integer address; None stays NULL."""
    if buf is None:
        return None
    if isinstance(buf, int):
        return buf
    if isinstance(buf, np.ndarray):
        assert buf.flags["C_CONTIGUOUS"], "buffers must be contiguous"
        return buf.ctypes.data
    assert buf.is_contiguous(), "buffers must be contiguous"
    return buf.data_ptr()


def dtype_of(buf: Any, dtype: Optional[int] = None) -> int:
    if dtype is not None:
        return dtype
    if isinstance(buf, np.ndarray):
        return _NP_DT[buf.dtype]
    return _torch_dt(buf)


def _numel(buf: Any) -> int:
    return int(buf.size) if isinstance(buf, np.ndarray) else int(buf.numel())


def _stream(stream: Any, *bufs: Any) -> Optional[int]:
    if stream is not None:
        return stream if isinstance(stream, int) else stream.cuda_stream
    for b in bufs:
        if b is not None and not isinstance(b, (np.ndarray, int)) and b.is_cuda:
            import torch  # noqa: PLC0415

            return torch.cuda.current_stream(b.device).cuda_stream
    return None


def get_version() -> int:
    v = C.c_int()
    L.lib().hxcclGetVersion(C.byref(v))
    return v.value


def get_unique_id() -> bytes:
    uid = L.UniqueId()
    rc = L.lib().hxcclGetUniqueId(C.byref(uid))
    if rc:
        raise HxcclError(rc, "hxcclGetUniqueId")
    return bytes(uid)


def group_start() -> None:
    L.lib().hxcclGroupStart()


def group_end() -> int:
    return L.lib().hxcclGroupEnd()


class Communicator:
    """One rank's handle. `check=False` methods return the result code instead of raising."""

    def __init__(self, handle: int):
        self._h = C.c_void_p(handle)
        self._ops: list = []

    # ---- construction -------------------------------------------------------------------
    @classmethod
    def init_rank(cls, uid: bytes, nranks: int, rank: int, config: Optional[L.Config] = None):
        u = L.UniqueId.from_buffer_copy(uid)
        h = C.c_void_p()
        if config is None:
            rc = L.lib().hxcclCommInitRank(C.byref(h), nranks, u, rank)
        else:
            rc = L.lib().hxcclCommInitRankConfig(C.byref(h), nranks, u, rank, C.byref(config))
        if rc:
            raise HxcclError(rc, "hxcclCommInitRank")
        return cls(h.value)

    def split(self, color: int, key: int) -> Optional["Communicator"]:
        h = C.c_void_p()
        self._ok(L.lib().hxcclCommSplit(self._h, color, key, C.byref(h), None), "hxcclCommSplit")
        return Communicator(h.value) if h.value else None

    def shrink(self, exclude: Sequence[int]) -> "Communicator":
        arr = (C.c_int * max(1, len(exclude)))(*exclude)
        h = C.c_void_p()
        self._ok(L.lib().hxcclCommShrink(self._h, arr, len(exclude), C.byref(h), None, 0),
                 "hxcclCommShrink")
        return Communicator(h.value)

    def destroy(self) -> None:
        if self._h:
            L.lib().hxcclCommDestroy(self._h)
            self._h = C.c_void_p()

    def abort(self) -> None:
        if self._h:
            L.lib().hxcclCommAbort(self._h)
            self._h = C.c_void_p()

    def finalize(self) -> None:
        self._ok(L.lib().hxcclCommFinalize(self._h), "hxcclCommFinalize")

    # ---- queries ------------------------------------------------------------------------
    @property
    def handle(self) -> int:
        return self._h.value

    @property
    def rank(self) -> int:
        v = C.c_int()
        L.lib().hxcclCommUserRank(self._h, C.byref(v))
        return v.value

    @property
    def size(self) -> int:
        v = C.c_int()
        L.lib().hxcclCommCount(self._h, C.byref(v))
        return v.value

    def last_error(self) -> str:
        return L.lib().hxcclGetLastError(self._h).decode()

    def async_error(self) -> int:
        v = C.c_int()
        L.lib().hxcclCommGetAsyncError(self._h, C.byref(v))
        return v.value

    def stats(self) -> tuple:
        b, m = C.c_uint64(), C.c_uint64()
        L.lib().hxcclCommGetStats(self._h, C.byref(b), C.byref(m))
        return b.value, m.value

    def reset_stats(self) -> None:
        L.lib().hxcclCommResetStats(self._h)

    def device_info(self) -> dict:
        kind = C.create_string_buffer(32)
        var, n = C.c_int(), C.c_ulonglong()
        L.lib().hxcclCommDeviceInfo(self._h, kind, 32, C.byref(var), C.byref(n))
        return {"kind": kind.value.decode(), "variant": var.value, "launches": n.value}

    def tune(self, variant: int = 0, exact: bool = True, max_ctas: int = 0) -> int:
        return L.lib().hxcclCommTune(self._h, variant, int(exact), max_ctas)

    def knob(self, name: str, value: int) -> int:
        """One tuning knob of the device path by name (same call on every rank)."""
        return L.lib().hxcclCommTuneKnob(self._h, name.encode(), value)

    def read_trace(self, max_ctas: int = 512):
        """Phase timers (HXCCL_TRACE=1): array [ctas, 16] of nanosecond sums since the last read."""
        buf = (C.c_ulonglong * (16 * max_ctas))()
        rows = L.lib().hxcclCommReadTrace(self._h, buf, max_ctas)
        return np.frombuffer(buf, dtype=np.uint64).reshape(max_ctas, 16)[:rows].copy()

    def _ok(self, rc: int, what: str, check: bool = True) -> int:
        if rc and check:
            raise HxcclError(rc, what, self.last_error() if self._h else "")
        return rc

    # ---- collectives ----------------------------------------------------------------------
    def all_reduce(self, send, recv=None, op: int = L.SUM, count=None, dtype=None, stream=None,
                   check: bool = True) -> int:
        recv = send if recv is None else recv
        n = _numel(send) if count is None else count
        return self._ok(L.lib().hxcclAllReduce(ptr(send), ptr(recv), n, dtype_of(send, dtype), op,
                                               self._h, _stream(stream, send, recv)),
                        "hxcclAllReduce", check)

    def all_reduce_cast(self, send, recv=None, wire_dtype: int = L.BFLOAT16, op: int = L.SUM, count=None,
                        stream=None, check: bool = True) -> int:
        """AllReduce of fp32 CUDA buffers with fp16 / bf16 on the wire, one kernel
        (hxcclAllReduceCast): the bits of cast, all_reduce in the wire type, cast back."""
        recv = send if recv is None else recv
        n = _numel(send) if count is None else count
        return self._ok(L.lib().hxcclAllReduceCast(ptr(send), ptr(recv), n, wire_dtype, op, self._h,
                                                   _stream(stream, send, recv)), "hxcclAllReduceCast", check)

    def all_gather(self, send, recv, count=None, dtype=None, stream=None, check=True) -> int:
        n = _numel(send) if count is None else count
        return self._ok(L.lib().hxcclAllGather(ptr(send), ptr(recv), n, dtype_of(send, dtype),
                                               self._h, _stream(stream, send, recv)),
                        "hxcclAllGather", check)

    def reduce_scatter(self, send, recv, op: int = L.SUM, count=None, dtype=None, stream=None,
                       check=True) -> int:
        n = _numel(recv) if count is None else count
        return self._ok(L.lib().hxcclReduceScatter(ptr(send), ptr(recv), n, dtype_of(recv, dtype),
                                                   op, self._h, _stream(stream, send, recv)),
                        "hxcclReduceScatter", check)

    def broadcast(self, send, recv, root: int, count=None, dtype=None, stream=None,
                  check=True) -> int:
        ref = recv if recv is not None else send
        n = _numel(ref) if count is None else count
        return self._ok(L.lib().hxcclBroadcast(ptr(send), ptr(recv), n, dtype_of(ref, dtype), root,
                                               self._h, _stream(stream, send, recv)),
                        "hxcclBroadcast", check)

    def bcast(self, buf, root: int, stream=None, check=True) -> int:
        return self._ok(L.lib().hxcclBcast(ptr(buf), _numel(buf), dtype_of(buf), root, self._h,
                                           _stream(stream, buf)), "hxcclBcast", check)

    def reduce(self, send, recv, root: int, op: int = L.SUM, count=None, dtype=None, stream=None,
               check=True) -> int:
        n = _numel(send) if count is None else count
        return self._ok(L.lib().hxcclReduce(ptr(send), ptr(recv), n, dtype_of(send, dtype), op,
                                            root, self._h, _stream(stream, send, recv)),
                        "hxcclReduce", check)

    def gather(self, send, recv, root: int, count=None, dtype=None, stream=None, check=True) -> int:
        n = _numel(send) if count is None else count
        return self._ok(L.lib().hxcclGather(ptr(send), ptr(recv), n, dtype_of(send, dtype), root,
                                            self._h, _stream(stream, send, recv)),
                        "hxcclGather", check)

    def scatter(self, send, recv, root: int, count=None, dtype=None, stream=None, check=True) -> int:
        n = _numel(recv) if count is None else count
        return self._ok(L.lib().hxcclScatter(ptr(send), ptr(recv), n, dtype_of(recv, dtype), root,
                                             self._h, _stream(stream, send, recv)),
                        "hxcclScatter", check)

    def all_to_all(self, send, recv, count=None, dtype=None, stream=None, check=True,
                   rccl_spelling: bool = False) -> int:
        n = _numel(send) // self.size if count is None else count
        fn = L.lib().hxcclAllToAll if rccl_spelling else L.lib().hxcclAlltoAll
        return self._ok(fn(ptr(send), ptr(recv), n, dtype_of(send, dtype), self._h,
                           _stream(stream, send, recv)), "hxcclAlltoAll", check)

    def all_to_allv(self, send, sendcounts, sdispls, recv, recvcounts, rdispls, dtype=None,
                    stream=None, check=True) -> int:
        def arr(x):
            return None if x is None else (C.c_size_t * len(x))(*x)

        ref = send if send is not None else recv
        return self._ok(L.lib().hxcclAllToAllv(ptr(send), arr(sendcounts), arr(sdispls), ptr(recv),
                                               arr(recvcounts), arr(rdispls), dtype_of(ref, dtype),
                                               self._h, _stream(stream, send, recv)),
                        "hxcclAllToAllv", check)

    def send(self, buf, peer: int, count=None, dtype=None, stream=None, check=True) -> int:
        n = _numel(buf) if count is None else count
        return self._ok(L.lib().hxcclSend(ptr(buf), n, dtype_of(buf, dtype), peer, self._h,
                                          _stream(stream, buf)), "hxcclSend", check)

    def recv(self, buf, peer: int, count=None, dtype=None, stream=None, check=True) -> int:
        n = _numel(buf) if count is None else count
        return self._ok(L.lib().hxcclRecv(ptr(buf), n, dtype_of(buf, dtype), peer, self._h,
                                          _stream(stream, buf)), "hxcclRecv", check)

    # ---- PreMulSum ---------------------------------------------------------------------------
    def create_premul_sum(self, scalar, dtype: Optional[int] = None, residence: int = L.SCALAR_HOST_IMMEDIATE,
                          check=True) -> int:
        """`scalar` is a one-element numpy array / tensor (kept alive by this object when its
        address is stored) or a raw address."""
        op = C.c_int()
        self._ops.append(scalar)
        rc = L.lib().hxcclRedOpCreatePreMulSum(C.byref(op), ptr(scalar), dtype_of(scalar, dtype),
                                               residence, self._h)
        self._ok(rc, "hxcclRedOpCreatePreMulSum", check)
        return op.value if rc == 0 else -rc

    def destroy_op(self, op: int, check=True) -> int:
        return self._ok(L.lib().hxcclRedOpDestroy(op, self._h), "hxcclRedOpDestroy", check)
