"""Element rules on the device against the host rules, bit for bit: the standalone reduce /
scale / divide kernels for all 12 types on random bytes (NaN, inf, signed zeros and subnormals
included; reference: tests/gpu_reduce.cc:36-81), and the narrow-float converters for every
possible input."""
import ctypes as C

import numpy as np
import pytest

from hxccl_b200 import _lib as L
from hxccl_b200.ops import oracle

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.mark.parametrize("dt", [L.FLOAT16, L.BFLOAT16, L.FLOAT8E4M3, L.FLOAT8E5M2])
def test_converters_match_host_rules_for_every_input(dt):
    bad, first = C.c_ulonglong(1), C.c_uint(0)
    fn = L.lib().hxcclTestNarrowConvert
    fn.argtypes = [C.c_int, C.POINTER(C.c_ulonglong), C.POINTER(C.c_uint)]
    assert fn(dt, C.byref(bad), C.byref(first)) == 0
    assert bad.value == 0, f"{bad.value} inputs differ, first float bits {first.value:#010x}"


@pytest.mark.parametrize("dt", list(range(12)))
def test_elementwise_kernels_match_host(dt):
    lib = L.lib()
    rng = np.random.default_rng(dt)
    es = L.DTYPE_SIZE[dt]
    stream = torch.cuda.current_stream().cuda_stream
    for n in (1, 7, 4097, 1 << 20):
        a = rng.integers(0, 256, n * es, dtype=np.uint8)
        b = rng.integers(0, 256, n * es, dtype=np.uint8)
        for op in (L.SUM, L.PROD, L.MAX, L.MIN):
            da, db = torch.from_numpy(a.copy()).cuda(), torch.from_numpy(b).cuda()
            assert lib.hxcclDevReduce(da.data_ptr(), db.data_ptr(), n, dt, op, stream) == 0
            want = oracle.combine(a.view(oracle.raw_dtype(dt)), b.view(oracle.raw_dtype(dt)), dt, op)
            assert np.array_equal(da.cpu().numpy().view(oracle.raw_dtype(dt)), want), (dt, op, n)
        k = rng.integers(0, 256, es, dtype=np.uint8)
        da, out = torch.from_numpy(a.copy()).cuda(), torch.zeros(n * es, dtype=torch.uint8, device="cuda")
        assert lib.hxcclDevScale(out.data_ptr(), da.data_ptr(), n, dt, k.ctypes.data, stream) == 0
        want = oracle.scaled(a.view(oracle.raw_dtype(dt)), dt, k.view(oracle.raw_dtype(dt)))
        assert np.array_equal(out.cpu().numpy().view(oracle.raw_dtype(dt)), want), ("scale", dt, n)
        if dt <= L.UINT64:
            da = torch.from_numpy(a.copy()).cuda()
            assert lib.hxcclDevDivide(da.data_ptr(), n, dt, 3, stream) == 0
            assert np.array_equal(da.cpu().numpy().view(oracle.raw_dtype(dt)),
                                  oracle.divided(a.view(oracle.raw_dtype(dt)), dt, 3)), ("div", dt, n)
