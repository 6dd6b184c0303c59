"""Element rules and narrow-float conversions on the host (the oracle of every device test).
Mirrors the reference's tests/test_reduce.cc, tests/test_fp.cc and tests/test_fp8_paths.cc:
literal values, exhaustive round trips over all codes, and torch's own converters as an
independent check of rounding."""
import ctypes as C
import math

import numpy as np
import pytest

from hxccl_b200 import _lib as L
from hxccl_b200.ops import oracle

torch = pytest.importorskip("torch")
NARROW = {L.FLOAT16: (16, torch.float16, np.uint16), L.BFLOAT16: (16, torch.bfloat16, np.uint16),
          L.FLOAT8E4M3: (8, torch.float8_e4m3fn, np.uint8), L.FLOAT8E5M2: (8, torch.float8_e5m2, np.uint8)}
CANON_NAN = {L.FLOAT16: 0x7E00, L.BFLOAT16: 0x7FC0, L.FLOAT8E4M3: 0x7F, L.FLOAT8E5M2: 0x7E}


def enc(dt, v):
    return L.lib().hxcclHostEncode(dt, C.c_float(v))


def dec(dt, bits):
    return L.lib().hxcclHostDecode(dt, bits)


def test_sizes_and_ring_blocks():
    assert [L.DTYPE_SIZE[d] for d in range(12)] == [1, 1, 4, 4, 8, 8, 2, 4, 8, 2, 1, 1]
    assert [oracle.ring_block(10, 4, i) for i in range(4)] == [(0, 3), (3, 3), (6, 2), (8, 2)]
    assert [oracle.ring_block(2, 4, i) for i in range(4)] == [(0, 1), (1, 1), (2, 0), (2, 0)]
    assert oracle.ring_block(0, 3, 2) == (0, 0)


@pytest.mark.parametrize("dt", list(NARROW))
def test_decode_matches_torch_and_round_trips(dt):
    bits, tdt, npdt = NARROW[dt]
    codes = np.arange(1 << bits, dtype=np.uint32)
    ours = np.array([dec(dt, int(c)) for c in codes], dtype=np.float32)
    theirs = torch.from_numpy(codes.astype(npdt)).view(tdt).float().numpy()
    nan = np.isnan(theirs)
    assert np.array_equal(np.isnan(ours), nan)
    assert np.array_equal(ours[~nan].view(np.uint32), theirs[~nan].view(np.uint32))  # exact, signed zeros too
    for c in codes[~nan]:
        assert enc(dt, float(ours[c])) == c  # every non-NaN code survives a round trip
    for c in codes[nan]:
        assert enc(dt, float("nan")) == CANON_NAN[dt]


@pytest.mark.parametrize("dt", list(NARROW))
def test_encode_rounding_matches_torch(dt):
    _, tdt, npdt = NARROW[dt]
    rng = np.random.default_rng(dt)
    # random bit patterns (all exponents), values around every representable number and the ties
    # between neighbours
    samples = [rng.integers(0, 1 << 32, 200000, dtype=np.uint64).astype(np.uint32).view(np.float32)]
    codes = np.arange(1 << NARROW[dt][0], dtype=np.uint32).astype(npdt)
    vals = torch.from_numpy(codes).view(tdt).float().numpy()
    vals = np.sort(vals[np.isfinite(vals)])
    mid = (vals[:-1].astype(np.float64) + vals[1:].astype(np.float64)) / 2
    for d in (0.0, 1e-7, -1e-7):
        samples.append((mid * (1 + d)).astype(np.float32))
    samples.append(np.nextafter(vals, np.float32(np.inf)))
    samples.append(np.nextafter(vals, np.float32(-np.inf)))
    x = np.concatenate(samples)
    x = x[np.isfinite(x)]
    ours = np.array([enc(dt, float(v)) for v in x[:60000]], dtype=np.uint32)
    theirs = torch.from_numpy(x[:60000].copy()).to(tdt).view(torch.uint8 if npdt == np.uint8 else torch.int16)
    theirs = theirs.numpy().astype(npdt).astype(np.uint32)
    # torch saturates fp8 NaN/overflow differently only in sign of NaN; compare where both finite
    tf = torch.from_numpy(theirs.astype(npdt)).view(tdt).float().numpy()
    of = np.array([dec(dt, int(c)) for c in ours], dtype=np.float32)
    both = np.isfinite(tf) & np.isfinite(of)
    assert np.array_equal(ours[both], theirs[both])
    assert np.array_equal(np.isfinite(tf), np.isfinite(of)) or dt == L.FLOAT8E4M3


def test_overflow_and_special_codes():
    # e4m3fn: 448 is the largest finite; 464 is the tie that still rounds down; beyond is NaN with sign
    assert enc(L.FLOAT8E4M3, 448.0) == 0x7E and enc(L.FLOAT8E4M3, 464.0) == 0x7E
    assert enc(L.FLOAT8E4M3, 465.0) == 0x7F and enc(L.FLOAT8E4M3, -480.0) == 0xFF
    assert enc(L.FLOAT8E4M3, float("inf")) == 0x7F and enc(L.FLOAT8E4M3, float("-inf")) == 0xFF
    # IEEE-style formats overflow to infinity
    assert enc(L.FLOAT8E5M2, 57344.0) == 0x7B and enc(L.FLOAT8E5M2, 61440.0) == 0x7C
    assert enc(L.FLOAT8E5M2, -1e9) == 0xFC
    assert enc(L.FLOAT16, 65504.0) == 0x7BFF and enc(L.FLOAT16, 65520.0) == 0x7C00
    assert enc(L.BFLOAT16, 3.4e38) == 0x7F80
    # subnormals and ties to even
    assert enc(L.FLOAT16, 2.0 ** -24) == 1 and enc(L.FLOAT16, 2.0 ** -25) == 0 and enc(L.FLOAT16, 1.5 * 2.0 ** -24) == 2
    assert enc(L.FLOAT8E5M2, 2.0 ** -16) == 1 and enc(L.FLOAT8E4M3, 2.0 ** -9) == 1
    assert enc(L.FLOAT16, -0.0) == 0x8000 and math.copysign(1, dec(L.FLOAT16, 0x8000)) == -1


def _reduce(a, b, dt, op):
    return oracle.combine(np.array(a), np.array(b), dt, op)


def test_integer_rules():
    assert _reduce(np.int8([127, -128]), np.int8([1, -1]), L.INT8, L.SUM).tolist() == [-128, 127]  # wraps
    assert _reduce(np.uint8([200]), np.uint8([3]), L.UINT8, L.PROD).tolist() == [600 % 256]
    assert _reduce(np.int64([-5, 7]), np.int64([3, -9]), L.INT64, L.MAX).tolist() == [3, 7]
    assert _reduce(np.uint32([5]), np.uint32([0xFFFFFFFF]), L.UINT32, L.MIN).tolist() == [5]
    # Avg divides in 64 bits toward zero; the divisor need not fit the element type
    assert oracle.divided(np.int8([-7, 7, -128]), L.INT8, 2).tolist() == [-3, 3, -64]
    assert oracle.divided(np.int8([100, -100]), L.INT8, 200).tolist() == [0, 0]
    assert oracle.divided(np.uint64([2 ** 64 - 1]), L.UINT64, 3).tolist() == [(2 ** 64 - 1) // 3]
    assert oracle.divided(np.int32([-9]), L.INT32, 4).tolist() == [-2]


def test_float_nan_and_zero_rules():
    snan_a, nan_b = np.uint32(0x7F800001), np.uint32(0xFFC12345)
    one = np.float32(1).view(np.uint32)
    # the first NaN operand wins, quieted, payload and sign kept
    assert _reduce([snan_a], [nan_b], L.FLOAT32, L.SUM)[0] == 0x7FC00001
    assert _reduce([one], [nan_b], L.FLOAT32, L.PROD)[0] == 0xFFC12345
    # a NaN born from non-NaN operands is the x86 default NaN
    inf, ninf = np.float32(np.inf).view(np.uint32), np.float32(-np.inf).view(np.uint32)
    assert _reduce([inf], [ninf], L.FLOAT32, L.SUM)[0] == 0xFFC00000
    assert _reduce(np.uint64([0x7FF0000000000000]), np.uint64([0]), L.FLOAT64, L.PROD)[0] == 0xFFF8000000000000
    # Max/Min: plain comparisons, so a NaN on either side keeps the held value
    assert _reduce([one], [nan_b], L.FLOAT32, L.MAX)[0] == one and _reduce([nan_b], [one], L.FLOAT32, L.MIN)[0] == nan_b
    pz, nz = np.uint32(0), np.uint32(0x80000000)
    assert _reduce([pz], [nz], L.FLOAT32, L.MAX)[0] == pz and _reduce([nz], [pz], L.FLOAT32, L.MAX)[0] == nz
    # narrow types: a NaN operand yields the other operand; equal values (also +0/-0) yield b
    h = lambda v: np.uint16(enc(L.FLOAT16, v))  # noqa: E731
    assert _reduce([np.uint16(0x7E00)], [h(2.0)], L.FLOAT16, L.MAX)[0] == h(2.0)
    assert _reduce([h(2.0)], [np.uint16(0x7E00)], L.FLOAT16, L.MIN)[0] == h(2.0)
    assert _reduce([np.uint16(0x0000)], [np.uint16(0x8000)], L.FLOAT16, L.MAX)[0] == 0x8000
    assert _reduce([np.uint16(0x7E00)], [h(1.0)], L.FLOAT16, L.SUM)[0] == 0x7E00
    # fp16 Avg of values near 60000 stays near 60000: scaling by 1/n comes first
    s = oracle.avg_scalar(L.FLOAT16, 4)
    x = oracle.scaled(np.uint16([h(60000.0)] * 1), L.FLOAT16, s)
    acc = x
    for _ in range(3):
        acc = oracle.combine(x, acc, L.FLOAT16, L.SUM)
    assert dec(L.FLOAT16, int(acc[0])) == 60000.0


def test_fp8_sum_and_product_same_through_half():
    """For all finite fp8 pairs, widening to float or to half gives the same fp8 result."""
    for dt, tdt in ((L.FLOAT8E4M3, torch.float8_e4m3fn), (L.FLOAT8E5M2, torch.float8_e5m2)):
        codes = torch.arange(256, dtype=torch.int16).to(torch.uint8)
        v = codes.view(tdt).float()
        fin = torch.isfinite(v)
        a, b = v[fin][:, None], v[fin][None, :]
        for f in (torch.add, torch.mul):
            via_float = f(a, b)
            via_half = f(a.half(), b.half()).float()
            ef = np.array([enc(dt, float(x)) for x in via_float.flatten()[::37]])
            eh = np.array([enc(dt, float(x)) for x in via_half.flatten()[::37]])
            assert np.array_equal(ef, eh)


def _host_reduce(dst, src, dt, op, chunk=None):
    """dst = dst (op) src through hxcclHostReduce, whole or in calls of `chunk` elements."""
    lib = L.lib()
    lib.hxcclHostReduce.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_int]
    n, es = dst.size, dst.itemsize
    step = n if chunk is None else chunk
    for i in range(0, n, step):
        k = min(step, n - i)
        assert lib.hxcclHostReduce(dst.ctypes.data + i * es, src.ctypes.data + i * es, k, dt, op) == 0


def test_bulk_paths_equal_the_element_rule():
    """Long vectors take shortcuts on the host (pair tables for the 8-bit floats, the machine's
    half conversions for fp16 sums and products); short ones go element by element through the
    rule. Both must give the same bits: all 65536 pairs of each 8-bit type, and every fp16 code
    against random and special partners."""
    for dt in (L.FLOAT8E4M3, L.FLOAT8E5M2):
        a = np.repeat(np.arange(256, dtype=np.uint8), 256)
        b = np.tile(np.arange(256, dtype=np.uint8), 256)
        for op in (L.SUM, L.PROD, L.MAX, L.MIN):
            bulk, slow = a.copy(), a.copy()
            _host_reduce(bulk, b, dt, op)               # 65536 elements: table
            _host_reduce(slow, b, dt, op, chunk=1024)   # below 4096 per call: rule
            assert np.array_equal(bulk, slow), (dt, op)
    rng = np.random.default_rng(5)
    special = np.array([0x0000, 0x8000, 0x0001, 0x8001, 0x03FF, 0x0400, 0x7BFF, 0xFBFF, 0x7C00, 0xFC00,
                        0x7C01, 0xFE00, 0x7E00, 0x3C00, 0xBC00, 0x3555], dtype=np.uint16)
    a = np.arange(65536, dtype=np.uint16)
    partners = [rng.integers(0, 65536, 65536).astype(np.uint16) for _ in range(3)]
    partners += [np.full(65536, s, dtype=np.uint16) for s in special]
    for op in (L.SUM, L.PROD):
        for b in partners[:6] if op == L.PROD else partners:
            bulk, slow = a.copy(), a.copy()
            _host_reduce(bulk, b, L.FLOAT16, op)
            _host_reduce(slow, b, L.FLOAT16, op, chunk=7)  # fewer than eight per call: rule
            assert np.array_equal(bulk, slow), (op, hex(int(b[0])))


def test_bulk_scaling_equals_the_element_rule():
    """Long vectors of the narrow floats are scaled through a table of all codes; short ones
    element by element. Every code times a few scalars, both ways."""
    lib = L.lib()
    lib.hxcclHostScale.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p]
    for dt, (bits, _, npdt) in NARROW.items():
        codes = np.arange(1 << bits, dtype=npdt)
        src = np.tile(codes, 4)                      # four times the number of codes: table
        for scalar in (0.125, -3.0, 1.0 / 3.0, 0.0, float("inf"), float("nan"), 60000.0):
            k = np.array([enc(dt, scalar)], dtype=npdt)
            bulk, slow = np.zeros_like(src), np.zeros_like(src)
            assert lib.hxcclHostScale(bulk.ctypes.data, src.ctypes.data, src.size, dt, k.ctypes.data) == 0
            for i in range(0, src.size, codes.size):  # below the threshold per call: rule
                assert lib.hxcclHostScale(slow.ctypes.data + i * src.itemsize, src.ctypes.data + i * src.itemsize,
                                          codes.size, dt, k.ctypes.data) == 0
            assert np.array_equal(bulk, slow), (dt, scalar)
