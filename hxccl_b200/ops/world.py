"""The world-on-one-GPU harness (include/hxccl_ext.h: hxcclWorld*) over torch tensors.

All ranks of a small communicator live on the current CUDA device; one cooperative launch runs
the collective kernel for every rank, so the very kernels of the multi-GPU path can be checked
on a machine with one GPU. Tensors are passed per rank: send[r], recv[r].
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import numpy as np

from .. import _lib as L
from ..comm import HxcclError, ptr


def _ptrs(ts: Optional[Sequence]) -> Optional[C.Array]:
    if ts is None:
        return None
    return (C.c_void_p * len(ts))(*[ptr(t) for t in ts])


def _stream(stream) -> Optional[int]:
    if stream is None:
        import torch  # noqa: PLC0415

        return torch.cuda.current_stream().cuda_stream
    return stream if isinstance(stream, int) else stream.cuda_stream


class World:
    def __init__(self, n: int, window_mb: int = 16, wait_ms: int = 10000):
        self.n = n
        h = C.c_void_p()
        rc = L.lib().hxcclWorldCreate(C.byref(h), n, window_mb, wait_ms)
        if rc:
            raise HxcclError(rc, "hxcclWorldCreate")
        self._h = h

    def close(self) -> None:
        if self._h:
            L.lib().hxcclWorldDestroy(self._h)
            self._h = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def _ok(self, rc: int, what: str) -> None:
        if rc:
            raise HxcclError(rc, what, L.lib().hxcclWorldLastError().decode())

    def tune(self, variant: int = 0, exact: bool = True, max_ctas: int = 0) -> None:
        self._ok(L.lib().hxcclWorldTune(self._h, variant, int(exact), max_ctas), "hxcclWorldTune")

    def knob(self, name: str, value: int) -> None:
        self._ok(L.lib().hxcclWorldTuneKnob(self._h, name.encode(), value), "hxcclWorldTuneKnob")

    def info(self) -> dict:
        v, n = C.c_int(), C.c_ulonglong()
        L.lib().hxcclWorldInfo(self._h, C.byref(v), C.byref(n))
        return {"variant": v.value, "launches": n.value}

    def status(self, rank: int) -> tuple:
        s, soft = C.c_ulonglong(), C.c_ulonglong()
        L.lib().hxcclWorldStatus(self._h, rank, C.byref(s), C.byref(soft))
        return s.value, soft.value

    def mute(self, rank: int) -> None:
        self._ok(L.lib().hxcclWorldMute(self._h, rank), "hxcclWorldMute")

    @staticmethod
    def _scalar(scalar: Optional[np.ndarray]):
        return None if scalar is None else scalar.ctypes.data

    def all_reduce(self, send: List, recv: List, count: int, dt: int, op: int = L.SUM,
                   scalar: Optional[np.ndarray] = None, order: int = -1, stream=None) -> None:
        self._ok(L.lib().hxcclWorldAllReduce(self._h, _ptrs(send), _ptrs(recv), count, dt, op,
                                             self._scalar(scalar), order, _stream(stream)),
                 "hxcclWorldAllReduce")

    def all_reduce_cast(self, send, recv, count: int, wire_dt: int, op: int = L.SUM, stream=None) -> None:
        """fp32 buffers, `wire_dt` (FLOAT16 / BFLOAT16) carried and summed (hxcclAllReduceCast)."""
        self._ok(L.lib().hxcclWorldAllReduceCast(self._h, _ptrs(send), _ptrs(recv), count, wire_dt, op,
                                                 _stream(stream)), "hxcclWorldAllReduceCast")

    def reduce_scatter(self, send, recv, recvcount: int, dt: int, op: int = L.SUM, scalar=None,
                       stream=None) -> None:
        self._ok(L.lib().hxcclWorldReduceScatter(self._h, _ptrs(send), _ptrs(recv), recvcount, dt, op,
                                                 self._scalar(scalar), _stream(stream)),
                 "hxcclWorldReduceScatter")

    def reduce(self, send, recv, count: int, dt: int, root: int, op: int = L.SUM, scalar=None,
               stream=None) -> None:
        self._ok(L.lib().hxcclWorldReduce(self._h, _ptrs(send), _ptrs(recv), count, dt, op,
                                          self._scalar(scalar), root, _stream(stream)),
                 "hxcclWorldReduce")

    def all_gather(self, send, recv, nbytes: int, stream=None) -> None:
        self._ok(L.lib().hxcclWorldAllGather(self._h, _ptrs(send), _ptrs(recv), nbytes, _stream(stream)),
                 "hxcclWorldAllGather")

    def broadcast(self, send, recv, nbytes: int, root: int, stream=None) -> None:
        self._ok(L.lib().hxcclWorldBroadcast(self._h, _ptrs(send), _ptrs(recv), nbytes, root,
                                             _stream(stream)), "hxcclWorldBroadcast")

    def gather(self, send, recv, nbytes: int, root: int, stream=None) -> None:
        self._ok(L.lib().hxcclWorldGather(self._h, _ptrs(send), _ptrs(recv), nbytes, root,
                                          _stream(stream)), "hxcclWorldGather")

    def scatter(self, send, recv, nbytes: int, root: int, stream=None) -> None:
        self._ok(L.lib().hxcclWorldScatter(self._h, _ptrs(send), _ptrs(recv), nbytes, root,
                                           _stream(stream)), "hxcclWorldScatter")

    def all_to_allv(self, send, recv, nbytes, soff, roff, stream=None) -> None:
        """nbytes / soff / roff: n x n nested sequences (see hxcclWorldAllToAllv)."""
        flat = lambda m: (C.c_size_t * (self.n * self.n))(*[int(v) for row in m for v in row])  # noqa: E731
        self._ok(L.lib().hxcclWorldAllToAllv(self._h, _ptrs(send), _ptrs(recv), flat(nbytes), flat(soff),
                                             flat(roff), _stream(stream)), "hxcclWorldAllToAllv")

    def send_recv(self, transfers, stream=None) -> None:
        """transfers: list of (from_rank, to_rank, src_tensor, send_bytes, dst_tensor, room_bytes)."""
        k = len(transfers)
        fr = (C.c_int * k)(*[t[0] for t in transfers])
        to = (C.c_int * k)(*[t[1] for t in transfers])
        src = (C.c_void_p * k)(*[ptr(t[2]) for t in transfers])
        sb = (C.c_size_t * k)(*[t[3] for t in transfers])
        dst = (C.c_void_p * k)(*[ptr(t[4]) for t in transfers])
        rb = (C.c_size_t * k)(*[t[5] for t in transfers])
        self._ok(L.lib().hxcclWorldSendRecv(self._h, k, fr, to, src, sb, dst, rb, _stream(stream)),
                 "hxcclWorldSendRecv")
