"""hxcclAllReduceNoAlloc (src/kernels/noalloc.h): the AllReduce entry point for callers that
cannot allocate device memory. It is called through its exported C symbol and must give the
same bits as the existing world entry point, hxcclWorldAllReduce, twice in a row (the second
call finds the scratch array as the first one left it). Collected last on purpose, so that a
run which stops at the first failure has already run every other test."""
import ctypes as C

import numpy as np
import pytest

from hxccl_b200 import _lib as L

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _entry():
    lib = L.lib()
    fn = lib.hxcclAllReduceNoAlloc
    fn.argtypes = [C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_size_t, C.c_int, C.c_int,
                   C.c_void_p]
    fn.restype = C.c_int
    lib.hxcclNoAllocLastError.restype = C.c_char_p
    return lib, fn


def _ptrs(ts):
    return (C.c_void_p * len(ts))(*[t.data_ptr() for t in ts])


@pytest.mark.parametrize("n", [2, 4])
def test_matches_world_allreduce_twice(n):
    from hxccl_b200.ops.world import World

    lib, fn = _entry()
    stream = torch.cuda.current_stream().cuda_stream
    with World(n, window_mb=8, wait_ms=10000) as w:
        w.tune(variant=1, exact=True)
        for round_no in range(2):  # two calls in a row share the static scratch
            for dt, op, nbytes in ((L.FLOAT32, L.SUM, 1 << 20), (L.BFLOAT16, L.AVG, 4096 + 6),
                                   (L.INT32, L.AVG, 40), (L.FLOAT8E4M3, L.MAX, 333)):
                es = L.DTYPE_SIZE[dt]
                count = nbytes // es
                rng = np.random.default_rng(17 * round_no + dt)
                xs = [torch.from_numpy(rng.integers(0, 256, count * es, dtype=np.uint8)).cuda() for _ in range(n)]
                got = [torch.zeros_like(x) for x in xs]
                want = [torch.zeros_like(x) for x in xs]
                rc = fn(n, _ptrs(xs), _ptrs(got), count, dt, op, stream)
                assert rc == 0, lib.hxcclNoAllocLastError().decode()
                w.all_reduce(xs, want, count, dt, op=op)
                torch.cuda.synchronize()
                for r in range(n):
                    assert torch.equal(got[r], want[r]), (n, round_no, dt, op, r)


@pytest.mark.parametrize("n", [1, 2, 3, 4])
def test_matches_the_host_rules(n):
    """An oracle that shares no code with the kernels: the reduction orders and element rules of
    the host path, restated in hxccl_b200/ops/oracle.py. One rank included (its result is its
    input, scaled by 1/1 for a float average)."""
    from hxccl_b200.ops import oracle

    lib, fn = _entry()
    stream = torch.cuda.current_stream().cuda_stream
    for dt, op, count in ((L.FLOAT32, L.SUM, 70001), (L.FLOAT16, L.AVG, 513), (L.INT32, L.AVG, 11),
                          (L.BFLOAT16, L.MAX, 3), (L.FLOAT32, L.SUM, 5)):
        es = L.DTYPE_SIZE[dt]
        xs_np = []
        for r in range(n):
            x = np.random.default_rng(1000 * dt + r).integers(0, 256, count * es, dtype=np.uint8).view(oracle.raw_dtype(dt))
            if dt >= L.FLOAT16:  # moderate magnitudes: clear the top exponent bit
                x &= x.dtype.type(~(1 << (8 * es - 2)) & ((1 << (8 * es)) - 1))
            xs_np.append(x)
        want = oracle.allreduce(xs_np, dt, op)
        xs = [torch.from_numpy(x.view(np.uint8).copy()).cuda() for x in xs_np]
        got = [torch.zeros_like(x) for x in xs]
        rc = fn(n, _ptrs(xs), _ptrs(got), count, dt, op, stream)
        assert rc == 0, lib.hxcclNoAllocLastError().decode()
        for r in range(n):
            assert np.array_equal(got[r].cpu().numpy().view(oracle.raw_dtype(dt)), want[r]), (n, dt, op, count, r)


def test_rejects_what_it_cannot_hold():
    lib, fn = _entry()
    x = [torch.zeros(16, device="cuda") for _ in range(2)]
    too_many = (1 << 20) // 4 + 1
    assert fn(2, _ptrs(x), _ptrs(x), too_many, L.FLOAT32, L.SUM, None) == L.INVALID_ARGUMENT
    assert b"HXCCL_NOALLOC_MAX_BYTES" in lib.hxcclNoAllocLastError()
    assert fn(5, _ptrs(x), _ptrs(x), 4, L.FLOAT32, L.SUM, None) == L.INVALID_ARGUMENT
    assert fn(2, _ptrs(x), _ptrs(x), 4, 99, L.SUM, None) == L.INVALID_ARGUMENT
