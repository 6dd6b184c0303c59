"""The collective kernels, run for every rank of a small world on one GPU and compared bit
for bit with the host schedules (hxccl_b200.ops.oracle). Inputs are random bytes, so NaN, inf,
signed zeros and overflow all occur (the technique of the reference's tests/gpu_reduce.cc:36-81
and tests/gpu_allreduce.cc:39-79)."""
import numpy as np
import pytest

from hxccl_b200 import _lib as L
from hxccl_b200.ops import oracle

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

ALL_DT = list(range(12))
FLOATS = [L.FLOAT16, L.FLOAT32, L.FLOAT64, L.BFLOAT16, L.FLOAT8E4M3, L.FLOAT8E5M2]


def rand_inputs(n, count, dt, seed):
    rng = np.random.default_rng(seed)
    es = L.DTYPE_SIZE[dt]
    return [rng.integers(0, 256, count * es, dtype=np.uint8).view(oracle.raw_dtype(dt)) for _ in range(n)]


def to_dev(a):
    return torch.from_numpy(a.view(np.uint8).copy()).cuda()


def back(t, dt):
    return t.cpu().numpy().view(oracle.raw_dtype(dt))


@pytest.fixture(scope="module")
def worlds():
    from hxccl_b200.ops.world import World

    made = {}

    def get(n):
        if n not in made:
            made[n] = World(n, window_mb=8, wait_ms=20000)
        return made[n]

    yield get
    for w in made.values():
        w.close()


@pytest.mark.parametrize("n", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("variant,order", [(1, 0), (1, 1), (2, 0)])
def test_allreduce_all_types(worlds, n, variant, order):
    w = worlds(n)
    w.tune(variant=variant, exact=True)
    for dt in ALL_DT:
        for op in (L.SUM, L.PROD, L.MAX, L.MIN, L.AVG):
            for count in (1, 7, 4099):
                xs = rand_inputs(n, count, dt, seed=dt * 100 + op * 10 + n)
                send = [to_dev(x) for x in xs]
                recv = [torch.zeros_like(s) for s in send]
                w.all_reduce(send, recv, count, dt, op=op, order=order)
                torch.cuda.synchronize()
                want = oracle.allreduce(xs, dt, op, order=order)
                for r in range(n):
                    got = back(recv[r], dt)
                    assert np.array_equal(got, want[r]), (n, variant, order, dt, op, count, r)
    assert all(w.status(r) == (0, 0) for r in range(n))


@pytest.mark.parametrize("n", [2, 4, 8])
def test_allreduce_large_multistep_inplace(worlds, n):
    """Messages beyond one staging step, in place, both variants; also PreMulSum."""
    w = worlds(n)
    for variant in (1, 2):
        w.tune(variant=variant, exact=True)
        for dt, op, scalar in ((L.FLOAT32, L.SUM, None), (L.BFLOAT16, L.AVG, None), (L.INT32, L.AVG, None),
                               (L.FLOAT16, L.SUM, np.array([0x3000], dtype=np.uint16)),  # x 0.125
                               (L.FLOAT8E4M3, L.SUM, None)):
            count = (3 << 20) // L.DTYPE_SIZE[dt] + 3
            xs = rand_inputs(n, count, dt, seed=7 + dt)
            if dt in FLOATS:  # keep magnitudes moderate so sums are not all NaN/inf
                for x in xs:
                    x &= x.dtype.type(~(1 << (8 * L.DTYPE_SIZE[dt] - 2)) & ((1 << (8 * L.DTYPE_SIZE[dt])) - 1))
            buf = [to_dev(x) for x in xs]
            w.all_reduce(buf, buf, count, dt, op=op, scalar=scalar, order=0)
            torch.cuda.synchronize()
            want = oracle.allreduce(xs, dt, op, order=0, scalar=scalar)
            for r in range(n):
                assert np.array_equal(back(buf[r], dt), want[r]), (n, variant, dt, op, r)
    assert all(w.status(r) == (0, 0) for r in range(n))


@pytest.mark.parametrize("n", [2, 3, 8])
def test_allreduce_three_role_pipeline(worlds, n):
    """The large-message variant (one CTA each for staging in, combining and staging out per
    lane), forced onto small messages: many steps, ring reuse, odd sizes, in place."""
    w = worlds(n)
    w.tune(variant=2, exact=True)
    w.knob("roles_min", 1)
    w.knob("roles_sub", 4096)
    try:
        for dt, op, count in ((L.FLOAT32, L.SUM, (3 << 20) // 4 + 3), (L.BFLOAT16, L.AVG, 700001),
                              (L.INT64, L.MAX, 40001), (L.FLOAT8E5M2, L.SUM, 1 << 20), (L.FLOAT32, L.PROD, 5)):
            xs = rand_inputs(n, count, dt, seed=31 + dt)
            if dt in FLOATS:
                for x in xs:
                    x &= x.dtype.type(~(1 << (8 * L.DTYPE_SIZE[dt] - 2)) & ((1 << (8 * L.DTYPE_SIZE[dt])) - 1))
            buf = [to_dev(x) for x in xs]
            w.all_reduce(buf, buf, count, dt, op=op, order=0)
            torch.cuda.synchronize()
            assert w.info()["variant"] == 4
            want = oracle.allreduce(xs, dt, op, order=0)
            for r in range(n):
                assert np.array_equal(back(buf[r], dt), want[r]), (n, dt, op, count, r)
        assert all(w.status(r) == (0, 0) for r in range(n))
    finally:
        w.knob("roles_min", 96 << 20)
        w.knob("roles_sub", 65536)


@pytest.mark.parametrize("n", [2, 3, 4, 8])
def test_allreduce_neighbour_ring(worlds, n):
    """The ring kernel (every hop a store into the right neighbour's window): every type and
    operator on small counts (blocks of zero and one element included), then many rounds with
    small slots, odd sizes, in place, PreMulSum and both Avg forms."""
    w = worlds(n)
    w.tune(variant=6, exact=True)
    for dt in ALL_DT:
        for op in (L.SUM, L.PROD, L.MAX, L.MIN, L.AVG):
            for count in (1, 7, 4099):
                xs = rand_inputs(n, count, dt, seed=dt * 100 + op * 10 + n + 5)
                send = [to_dev(x) for x in xs]
                recv = [torch.zeros_like(s) for s in send]
                w.all_reduce(send, recv, count, dt, op=op, order=0)
                torch.cuda.synchronize()
                assert w.info()["variant"] == 6
                want = oracle.allreduce(xs, dt, op, order=0)
                for r in range(n):
                    assert np.array_equal(back(recv[r], dt), want[r]), (n, dt, op, count, r)
    w.knob("ring_sub", 4096)
    try:
        for dt, op, scalar, count in ((L.FLOAT32, L.SUM, None, (3 << 20) // 4 + 3), (L.BFLOAT16, L.AVG, None, 700001),
                                      (L.INT32, L.AVG, None, 400003), (L.FLOAT8E4M3, L.SUM, None, 1 << 20),
                                      (L.FLOAT16, L.SUM, np.array([0x3000], dtype=np.uint16), 500000)):
            xs = rand_inputs(n, count, dt, seed=57 + dt)
            if dt in FLOATS:
                for x in xs:
                    x &= x.dtype.type(~(1 << (8 * L.DTYPE_SIZE[dt] - 2)) & ((1 << (8 * L.DTYPE_SIZE[dt])) - 1))
            buf = [to_dev(x) for x in xs]
            w.all_reduce(buf, buf, count, dt, op=op, scalar=scalar, order=0)
            torch.cuda.synchronize()
            want = oracle.allreduce(xs, dt, op, order=0, scalar=scalar)
            for r in range(n):
                assert np.array_equal(back(buf[r], dt), want[r]), (n, dt, op, count, r)
        assert all(w.status(r) == (0, 0) for r in range(n))
    finally:
        w.knob("ring_sub", 512 * 1024)


@pytest.mark.parametrize("n", [2, 3, 4, 8])
def test_allreduce_flag_in_data_lines(worlds, n):
    """The small-message kernel whose 16-byte lines carry their own epoch: every type and
    operator in both operand orders, in place and out of place, sizes from one element to the
    most a slot holds, and back-to-back launches (the halves alternate with the epoch)."""
    w = worlds(n)
    most = ((8 << 20) // 2 // n // 256 * 256) // 2  # payload bytes of one slot
    for order in (1, 0):
        w.tune(variant=7, exact=True)
        for dt in ALL_DT:
            es = L.DTYPE_SIZE[dt]
            for op in (L.SUM, L.PROD, L.MAX, L.MIN, L.AVG):
                for count in (1, 7, 1021) + ((most // es,) if (dt + op) % 5 == 0 else ()):
                    xs = rand_inputs(n, count, dt, seed=dt * 100 + op * 10 + n + 11 * order)
                    send = [to_dev(x) for x in xs]
                    recv = [torch.zeros_like(s) for s in send]
                    w.all_reduce(send, recv, count, dt, op=op, order=order)
                    assert w.info()["variant"] == 7
                    w.all_reduce(send, send, count, dt, op=op, order=order)  # in place, next epoch
                    torch.cuda.synchronize()
                    want = oracle.allreduce(xs, dt, op, order=order)
                    for r in range(n):
                        assert np.array_equal(back(recv[r], dt), want[r]), (n, order, dt, op, count, r)
                        assert np.array_equal(back(send[r], dt), want[r]), ("in place", n, order, dt, op, count, r)
    # left to the tuner, small messages take it and larger ones do not
    w.tune(variant=0, exact=True)
    x = [to_dev(v) for v in rand_inputs(n, 64, L.FLOAT32, 1)]
    w.all_reduce(x, x, 64, L.FLOAT32)
    assert w.info()["variant"] == 7
    y = [to_dev(v) for v in rand_inputs(n, 1 << 18, L.FLOAT32, 2)]
    w.all_reduce(y, y, 1 << 18, L.FLOAT32)
    assert w.info()["variant"] != 7
    # one element more than a slot holds: forcing the variant falls back to the one-shot kernel
    w.tune(variant=7, exact=True)
    big = [to_dev(v) for v in rand_inputs(n, most + 8, L.UINT8, 3)]
    w.all_reduce(big, big, most + 8, L.UINT8)
    torch.cuda.synchronize()
    assert w.info()["variant"] != 7
    w.tune(variant=0, exact=True)
    assert all(w.status(r) == (0, 0) for r in range(n))


@pytest.mark.parametrize("n", [2, 3, 8])
def test_allreduce_with_narrow_wire_type(worlds, n):
    """fp32 buffers with bf16 / fp16 on the wire (hxcclAllReduceCast): the bits of "cast, AllReduce
    in the narrow type, cast back", computed here with torch's casts and the host oracle.
    Single-step and pipelined sizes, odd counts, in place."""
    w = worlds(n)
    w.tune(variant=0, exact=True)
    for wire, tdt in ((L.BFLOAT16, torch.bfloat16), (L.FLOAT16, torch.float16)):
        for op in (L.AVG, L.SUM, L.MAX):
            for count in (32768, 70001, (3 << 20) // 2 + 5):
                g = torch.Generator().manual_seed(count + wire + op)
                xs = [(torch.randn(count, generator=g) * 3).float() for _ in range(n)]
                narrow = [x.to(tdt).view(torch.uint16).numpy().copy() for x in xs]
                want = oracle.allreduce(narrow, wire, op, order=0)
                want32 = [torch.from_numpy(v.copy()).view(tdt).float() for v in want]
                send = [x.cuda() for x in xs]
                recv = [torch.zeros_like(s) for s in send]
                w.all_reduce_cast(send, recv, count, wire, op=op)
                w.all_reduce_cast(send, send, count, wire, op=op)  # in place
                torch.cuda.synchronize()
                for r in range(n):
                    assert torch.equal(recv[r].cpu().view(torch.int32), want32[r].view(torch.int32)), (n, wire, op, count, r)
                    assert torch.equal(send[r].cpu().view(torch.int32), want32[r].view(torch.int32)), ("in place", n, wire, op, count, r)
    assert all(w.status(r) == (0, 0) for r in range(n))


@pytest.mark.parametrize("n", [2, 3, 4, 8])
def test_reducescatter_neighbour_ring(worlds, n):
    """ReduceScatter around the ring (the large-input form) forced onto small inputs: all types,
    blocks of one element, many rounds with small slots (both slot sets), in place."""
    w = worlds(n)
    w.knob("rs_ring_min", 1)
    try:
        for sub in (512 * 1024, 4096):
            w.knob("ring_sub", sub)
            for dt in ALL_DT:
                for op in (L.SUM, L.MAX, L.AVG):
                    for per in ((1, 1031) if sub > 4096 else ((300 * 1024) // L.DTYPE_SIZE[dt] + 3,)):
                        xs = rand_inputs(n, per * n, dt, seed=per + dt + n)
                        if dt in FLOATS and per > 2000:
                            for x in xs:
                                x &= x.dtype.type(~(1 << (8 * L.DTYPE_SIZE[dt] - 2)) & ((1 << (8 * L.DTYPE_SIZE[dt])) - 1))
                        send = [to_dev(x) for x in xs]
                        recv = [torch.zeros(per * L.DTYPE_SIZE[dt], dtype=torch.uint8, device="cuda") for _ in range(n)]
                        before = w.info()["launches"]
                        w.reduce_scatter(send, recv, per, dt, op=op)
                        # in place: recv is the rank's own block of send
                        nb = per * L.DTYPE_SIZE[dt]
                        w.reduce_scatter(send, [send[r][r * nb:(r + 1) * nb] for r in range(n)], per, dt, op=op)
                        torch.cuda.synchronize()
                        assert w.info()["launches"] == before + 2
                        want = oracle.reducescatter(xs, dt, op)
                        for r in range(n):
                            assert np.array_equal(back(recv[r], dt), want[r]), ("ring rs", n, sub, dt, op, per, r)
                            assert np.array_equal(back(send[r][r * nb:(r + 1) * nb].contiguous(), dt), want[r]), ("in place", n, dt, op, r)
        assert all(w.status(r) == (0, 0) for r in range(n))
    finally:
        w.knob("rs_ring_min", 256 << 20)
        w.knob("ring_sub", 512 * 1024)


@pytest.mark.parametrize("n", [2, 3, 8])
def test_reducescatter_and_reduce(worlds, n):
    w = worlds(n)
    for dt in (L.INT8, L.INT64, L.FLOAT32, L.FLOAT64, L.BFLOAT16, L.FLOAT8E5M2):
        for op in (L.SUM, L.MAX, L.AVG):
            for per in (1, 5, 1031):
                xs = rand_inputs(n, per * n, dt, seed=per + dt)
                send = [to_dev(x) for x in xs]
                recv = [torch.zeros(per * L.DTYPE_SIZE[dt], dtype=torch.uint8, device="cuda") for _ in range(n)]
                w.reduce_scatter(send, recv, per, dt, op=op)
                torch.cuda.synchronize()
                want = oracle.reducescatter(xs, dt, op)
                for r in range(n):
                    assert np.array_equal(back(recv[r], dt), want[r]), ("rs", n, dt, op, per, r)
            for count, root in ((9, 0), (2053, n - 1), ((600 * 1024) // L.DTYPE_SIZE[dt] + 1, n // 2)):
                xs = rand_inputs(n, count, dt, seed=count + dt)
                send = [to_dev(x) for x in xs]
                recv = [torch.zeros_like(s) if r == root else None for r, s in enumerate(send)]
                w.reduce(send, recv, count, dt, root, op=op)
                torch.cuda.synchronize()
                want = oracle.reduce(xs, dt, op, root)
                assert np.array_equal(back(recv[root], dt), want), ("reduce", n, dt, op, count, root)
    assert all(w.status(r) == (0, 0) for r in range(n))


@pytest.mark.parametrize("n", [2, 4, 8])
def test_copy_collectives(worlds, n):
    w = worlds(n)
    rng = np.random.default_rng(n)
    for nbytes in (8, 1000, 3 << 20):
        xs = [rng.integers(0, 256, nbytes, dtype=np.uint8) for _ in range(n)]
        send = [torch.from_numpy(x).cuda() for x in xs]
        # AllGather, also in place
        recv = [torch.zeros(nbytes * n, dtype=torch.uint8, device="cuda") for _ in range(n)]
        w.all_gather(send, recv, nbytes)
        inplace = [torch.zeros(nbytes * n, dtype=torch.uint8, device="cuda") for _ in range(n)]
        for r in range(n):
            inplace[r][r * nbytes:(r + 1) * nbytes] = send[r]
        w.all_gather([inplace[r][r * nbytes:(r + 1) * nbytes] for r in range(n)], inplace, nbytes)
        torch.cuda.synchronize()
        want = np.concatenate(xs)
        for r in range(n):
            assert np.array_equal(recv[r].cpu().numpy(), want)
            assert np.array_equal(inplace[r].cpu().numpy(), want)
        # Broadcast / Gather / Scatter from a middle root
        root = n // 2
        out = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(n)]
        w.broadcast(send, out, nbytes, root)
        gat = [torch.zeros(nbytes * n, dtype=torch.uint8, device="cuda") if r == root else None for r in range(n)]
        w.gather(send, gat, nbytes, root)
        big = [torch.from_numpy(want.copy()).cuda() if r == root else None for r in range(n)]
        sca = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(n)]
        w.scatter(big, sca, nbytes, root)
        torch.cuda.synchronize()
        for r in range(n):
            assert np.array_equal(out[r].cpu().numpy(), xs[root])
            assert np.array_equal(sca[r].cpu().numpy(), xs[r])
        assert np.array_equal(gat[root].cpu().numpy(), want)
    assert all(w.status(r) == (0, 0) for r in range(n))


@pytest.mark.parametrize("n", [2, 4, 8])
def test_alltoallv(worlds, n):
    w = worlds(n)
    rng = np.random.default_rng(7)
    for mean in (16, 5000, 400000):
        nb = rng.integers(0, 2 * mean + 1, (n, n))  # nb[r][j]: rank r -> rank j
        soff = np.zeros((n, n), dtype=np.int64)
        roff = np.zeros((n, n), dtype=np.int64)
        for r in range(n):
            soff[r] = np.concatenate([[0], np.cumsum(nb[r] + 3)[:-1]])      # gaps between blocks
            roff[r] = np.concatenate([[0], np.cumsum(nb[:, r] + 5)[:-1]])
        send_np = [rng.integers(0, 256, int(soff[r][-1] + nb[r][-1]) + 8, dtype=np.uint8) for r in range(n)]
        recv_len = [int(roff[r][-1] + nb[n - 1][r]) + 8 for r in range(n)]
        send = [torch.from_numpy(x).cuda() for x in send_np]
        recv = [torch.full((recv_len[r],), 0xEE, dtype=torch.uint8, device="cuda") for r in range(n)]
        w.all_to_allv(send, recv, nb.tolist(), soff.tolist(), roff.tolist())
        torch.cuda.synchronize()
        for r in range(n):
            want = np.full(recv_len[r], 0xEE, dtype=np.uint8)
            for i in range(n):
                want[roff[r][i]:roff[r][i] + nb[i][r]] = send_np[i][soff[i][r]:soff[i][r] + nb[i][r]]
            assert np.array_equal(recv[r].cpu().numpy(), want), (n, mean, r)
    assert all(w.status(r) == (0, 0) for r in range(n))


def test_send_recv_groups(worlds):
    n = 4
    w = worlds(n)
    rng = np.random.default_rng(3)
    sizes = [0, 24, 300000, 5 << 20]
    # ring shift of every size, all in one group, plus two sends to the same peer (order kept)
    src = {(r, s): torch.from_numpy(rng.integers(0, 256, max(s, 1), dtype=np.uint8)).cuda() for r in range(n) for s in sizes}
    dst = {(r, s): torch.zeros(max(s, 1), dtype=torch.uint8, device="cuda") for r in range(n) for s in sizes}
    transfers = [(r, (r + 1) % n, src[(r, s)], s, dst[((r + 1) % n, s)], s) for s in sizes for r in range(n)]
    w.send_recv(transfers)
    torch.cuda.synchronize()
    for s in sizes:
        for r in range(n):
            assert torch.equal(dst[((r + 1) % n, s)][:s], src[(r, s)][:s]), (r, s)
    # a second launch continues the counters; truncation: 1000 bytes into a 600-byte buffer
    a = torch.arange(1000, dtype=torch.int32, device="cuda").to(torch.uint8)
    b = torch.zeros(600, dtype=torch.uint8, device="cuda")
    c = torch.zeros(1000, dtype=torch.uint8, device="cuda")
    w.send_recv([(0, 1, a, 1000, b, 600), (2, 3, a, 1000, c, 1000)])
    torch.cuda.synchronize()
    assert torch.equal(b, a[:600]) and torch.equal(c, a)
    assert w.status(1)[1] >> 56 == 3 and w.status(3) == (0, 0) and w.status(0) == (0, 0)
    # and the lanes still work afterwards
    w.send_recv([(0, 1, a, 1000, c, 1000)])
    torch.cuda.synchronize()
    assert torch.equal(c, a) and w.status(1) == (0, 0)


def test_bounded_wait_reports_timeout():
    """A rank whose flags never arrive: its peers give up after the limit, record a timeout and
    the kernel returns; the CUDA context stays usable."""
    from hxccl_b200.ops.world import World

    with World(2, window_mb=2, wait_ms=300) as w:
        x = [torch.ones(64, dtype=torch.float32, device="cuda") for _ in range(2)]
        w.mute(1)
        w.all_reduce(x, x, 64, L.FLOAT32)
        torch.cuda.synchronize()
        sticky, _ = w.status(0)
        assert sticky >> 56 == 1 and (sticky & 0xffffff) == 1  # timeout, waiting for rank 1
    assert float(torch.ones(4, device="cuda").sum()) == 4.0
