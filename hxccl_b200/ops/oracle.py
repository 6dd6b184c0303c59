"""Expected results of the reducing collectives, computed in-process by walking the host
algorithms' message schedules with the library's own host element rules (hxcclHostReduce /
hxcclHostScale / hxcclHostDivide). Buffers are numpy arrays whose dtype has the element's size
(uint8 for fp8, uint16 for fp16/bf16 and so on); values are compared as raw bits.

The schedules are those of src/host/algos.cc (ring, recursive doubling, ring reduce-scatter,
tree / chain reduce); the multi-process CPU tests check that file against this module, the GPU
tests check the kernels against it.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import numpy as np

from .. import _lib as L

DOUBLING_MAX = 64 * 1024
TREE_MAX = 512 * 1024

_RAW = {1: np.uint8, 2: np.uint16, 4: np.uint32, 8: np.uint64}


def raw_dtype(dt: int):
    return _RAW[L.DTYPE_SIZE[dt]]


def combine(a: np.ndarray, b: np.ndarray, dt: int, op: int) -> np.ndarray:
    """a (op) b with `a` as the held value (left operand); returns a new array."""
    out = np.ascontiguousarray(a).copy()
    b = np.ascontiguousarray(b)
    if out.size:
        L.lib().hxcclHostReduce(out.ctypes.data, b.ctypes.data, out.size, dt, op)
    return out


def scaled(x: np.ndarray, dt: int, scalar: np.ndarray) -> np.ndarray:
    out = np.ascontiguousarray(x).copy()
    if out.size:
        L.lib().hxcclHostScale(out.ctypes.data, out.ctypes.data, out.size, dt, scalar.ctypes.data)
    return out


def divided(x: np.ndarray, dt: int, d: int) -> np.ndarray:
    out = np.ascontiguousarray(x).copy()
    if out.size:
        L.lib().hxcclHostDivide(out.ctypes.data, out.size, dt, d)
    return out


def avg_scalar(dt: int, n: int) -> np.ndarray:
    """1/n as the library stores it: double -> float -> dt."""
    f = np.float32(1.0 / n)
    if dt == L.FLOAT64:
        return np.array([1.0 / n], dtype=np.float64).view(np.uint64)
    if dt == L.FLOAT32:
        return np.array([f], dtype=np.float32).view(np.uint32)
    bits = L.lib().hxcclHostEncode(dt, C.c_float(float(f)))
    return np.array([bits], dtype=raw_dtype(dt))


def ring_block(count: int, n: int, i: int):
    off, ln = C.c_size_t(), C.c_size_t()
    L.lib().hxcclRingBlock(count, n, i, C.byref(off), C.byref(ln))
    return off.value, ln.value


def _plan(inputs: List[np.ndarray], dt: int, op: int, scalar: Optional[np.ndarray]):
    """Resolves Avg / PreMulSum into (scaled inputs, base op, post divisor)."""
    n = len(inputs)
    is_int = dt <= L.UINT64
    if scalar is not None:
        return [scaled(x, dt, scalar) for x in inputs], L.SUM, 0
    if op == L.AVG:
        if is_int:
            return inputs, L.SUM, n
        s = avg_scalar(dt, n)
        return [scaled(x, dt, s) for x in inputs], L.SUM, 0
    return inputs, op, 0


def _ring(xs: List[np.ndarray], dt: int, op: int) -> np.ndarray:
    n, count = len(xs), xs[0].size
    out = np.empty_like(xs[0])
    for c in range(n):
        off, ln = ring_block(count, n, c)
        acc = xs[c][off:off + ln]
        for k in range(1, n):
            acc = combine(xs[(c + k) % n][off:off + ln], acc, dt, op)  # newcomer on the left
        out[off:off + ln] = acc
    return out


def _doubling(xs: List[np.ndarray], dt: int, op: int) -> List[np.ndarray]:
    n = len(xs)
    p = 1
    while 2 * p <= n:
        p *= 2
    spare = n - p
    val = [x.copy() for x in xs]
    for r in range(1, 2 * spare, 2):  # odd rank takes in its even neighbour
        val[r] = combine(val[r], val[r - 1], dt, op)

    def real(q):
        return 2 * q + 1 if q < spare else q + spare

    bit = 1
    while bit < p:
        nxt = list(val)
        for q in range(p):
            nxt[real(q)] = combine(val[real(q)], val[real(q ^ bit)], dt, op)
        val = nxt
        bit <<= 1
    for r in range(0, 2 * spare, 2):  # the even rank gets its neighbour's result
        val[r] = val[r + 1].copy()
    return val


def allreduce(inputs: List[np.ndarray], dt: int, op: int, order: int = -1,
              scalar: Optional[np.ndarray] = None) -> List[np.ndarray]:
    """Per-rank results. order 0 ring, 1 recursive doubling, -1 chosen by size like the API."""
    n = len(inputs)
    xs, base, div = _plan(inputs, dt, op, scalar)
    if order < 0:
        order = 1 if inputs[0].size * L.DTYPE_SIZE[dt] < DOUBLING_MAX else 0
    if n == 1 or inputs[0].size == 0:
        outs = [x.copy() for x in xs]
    elif order == 0:
        r = _ring(xs, dt, base)
        outs = [r.copy() for _ in range(n)]
    else:
        outs = _doubling(xs, dt, base)
    return [divided(o, dt, div) for o in outs] if div else outs


def reducescatter(inputs: List[np.ndarray], dt: int, op: int,
                  scalar: Optional[np.ndarray] = None) -> List[np.ndarray]:
    n = len(inputs)
    per = inputs[0].size // n
    xs, base, div = _plan(inputs, dt, op, scalar)
    outs = []
    for b in range(n):
        sl = slice(b * per, (b + 1) * per)
        acc = xs[(b + 1) % n][sl]
        for k in range(2, n + 1):
            acc = combine(xs[(b + k) % n][sl], acc, dt, base)
        acc = acc.copy()
        outs.append(divided(acc, dt, div) if div else acc)
    return outs


def reduce(inputs: List[np.ndarray], dt: int, op: int, root: int,
           scalar: Optional[np.ndarray] = None) -> np.ndarray:
    """The root's result."""
    n = len(inputs)
    xs, base, div = _plan(inputs, dt, op, scalar)
    byv = [xs[(v + root) % n] for v in range(n)]  # by position relative to the root
    nbytes = inputs[0].size * L.DTYPE_SIZE[dt]
    if n == 1 or inputs[0].size == 0:
        acc = byv[0].copy()
    elif nbytes < TREE_MAX:
        val = [x.copy() for x in byv]
        bit = 1
        while bit < n:
            for v in range(0, n, 2 * bit):
                if v + bit < n:
                    val[v] = combine(val[v], val[v + bit], dt, base)
            bit <<= 1
        acc = val[0]
    else:
        acc = byv[n - 1]
        for v in range(n - 2, -1, -1):
            acc = combine(byv[v], acc, dt, base)
    return divided(acc, dt, div) if div else acc
