"""Host path across real processes: AllReduce for all 12 element types, five operators, both
algorithms, compared bit for bit with the in-process oracle (every rank's inputs are a
function of its rank, so each test recomputes them: the reference's technique in
tests/test_dtypes.cc:51-88), plus the exact traffic counters (tests/test_allreduce.cc:57-86)."""
import os

import numpy as np
import pytest

from hxccl_b200 import _lib as L
from hxccl_b200.ops import oracle
from hxccl_b200.utils import run_ranks


def inputs_for(n, count, dt, seed):
    es = L.DTYPE_SIZE[dt]
    return [np.random.default_rng(seed * 1000 + r).integers(0, 256, count * es, dtype=np.uint8)
            .view(oracle.raw_dtype(dt)) for r in range(n)]


def _body(comm, rank, n, cases):
    out = []
    for (dt, op, count, algo, seed) in cases:
        if algo:
            os.environ["HXCCL_ALGO"] = algo
        else:
            os.environ.pop("HXCCL_ALGO", None)
        x = inputs_for(n, count, dt, seed)[rank]
        y = np.zeros_like(x)
        comm.reset_stats()
        comm.all_reduce(x, y, op=op, count=count, dtype=dt)
        out.append((y, comm.stats()))
    return out


@pytest.mark.parametrize("n", [1, 2, 3, 4, 5, 8])
def test_allreduce_matches_oracle(n):
    cases = []
    for dt in range(12):
        for op in (L.SUM, L.PROD, L.MAX, L.MIN, L.AVG):
            for count, algo in ((0, None), (1, "ring"), (7, "rd"), (1000, "ring"), (1000, "rd"), (4099, None)):
                cases.append((dt, op, count, algo, len(cases)))
    res = run_ranks(n, _body, cases)
    for k, (dt, op, count, algo, seed) in enumerate(cases):
        order = {"ring": 0, "rd": 1, None: -1}[algo]
        want = oracle.allreduce(inputs_for(n, count, dt, seed), dt, op, order=order)
        for r in range(n):
            assert np.array_equal(res[r][k][0], want[r]), (n, dt, op, count, algo, r)


def _traffic_body(comm, rank, n):
    out = {}
    x = np.ones(1000, dtype=np.float32)
    for algo in ("ring", "rd"):
        os.environ["HXCCL_ALGO"] = algo
        comm.reset_stats()
        comm.all_reduce(x.copy(), op=L.SUM)
        out[algo] = comm.stats()
    os.environ.pop("HXCCL_ALGO")
    comm.reset_stats()
    comm.all_reduce(np.ones(3, dtype=np.float64), op=L.SUM)  # fewer elements than ranks at n > 3
    out["tiny"] = comm.stats()
    return out


@pytest.mark.parametrize("n", [2, 4, 5])
def test_traffic_counters(n):
    res = run_ranks(n, _traffic_body)
    total = 1000 * 4
    for r in range(n):
        # ring: 2(n-1) messages that together carry every block but one, twice
        blocks = [oracle.ring_block(1000, n, i)[1] * 4 for i in range(n)]
        rs = sum(blocks[(r - h) % n] for h in range(n - 1))
        ag = sum(blocks[(r + 1 - h) % n] for h in range(n - 1))
        assert res[r]["ring"] == (rs + ag, 2 * (n - 1))
        p = 1 << (n.bit_length() - 1)
        spare = n - p
        levels = p.bit_length() - 1
        if r < 2 * spare and r % 2 == 0:
            assert res[r]["rd"] == (total, 1)
        elif r < 2 * spare:
            assert res[r]["rd"] == (total * (levels + 1), levels + 1)
        else:
            assert res[r]["rd"] == (total * levels, levels)
        assert res[r]["tiny"][1] > 0


def _plumbing_body(comm, rank, n):
    """The CPU plumbing configuration of the baseline: fp32, 1,048,576 elements of U(-1,1)
    from seed 1234+rank, sum and avg, ring at full size and recursive doubling at 16 KB."""
    x = np.random.default_rng(1234 + rank).uniform(-1.0, 1.0, 1 << 20).astype(np.float32)
    out = {}
    for algo, count in (("ring", 1 << 20), ("rd", 4096)):
        os.environ["HXCCL_ALGO"] = algo
        for name, op in (("sum", L.SUM), ("avg", L.AVG)):
            y = np.zeros(count, dtype=np.float32)
            comm.reset_stats()
            comm.all_reduce(x[:count], y, op=op)
            out[algo, name] = (y, comm.stats())
    os.environ.pop("HXCCL_ALGO")
    return out


def test_cpu_plumbing_config_against_fp64_sum():
    n = 2
    res = run_ranks(n, _plumbing_body, timeout=120)
    xs = [np.random.default_rng(1234 + r).uniform(-1.0, 1.0, 1 << 20).astype(np.float32) for r in range(n)]
    for algo, count in (("ring", 1 << 20), ("rd", 4096)):
        ref = sum(x[:count].astype(np.float64) for x in xs)
        for r in range(n):
            got_sum, stats = res[r][algo, "sum"]
            got_avg, _ = res[r][algo, "avg"]
            assert np.abs(got_sum.astype(np.float64) - ref).max() <= 2.5e-7  # one fp32 rounding of a value below 2
            assert np.abs(got_avg.astype(np.float64) - ref / n).max() <= 2.5e-7
            assert np.array_equal(got_sum, res[0][algo, "sum"][0])  # every rank holds the same bits
            # with two ranks both schedules move the whole vector once: two halves (ring) or one piece (rd)
            assert stats == ((count * 4, 2) if algo == "ring" else (count * 4, 1)), (algo, stats)


def _sliced_body(comm, rank, n):
    out = []
    for dt, op, count in ((L.FLOAT32, L.SUM, 100_003), (L.BFLOAT16, L.AVG, 70_001), (L.INT64, L.MAX, 30_000)):
        x = inputs_for(n, count, dt, 77)[rank]
        y = np.zeros_like(x)
        comm.reset_stats()
        comm.all_reduce(x, y, op=op, count=count, dtype=dt)
        stats = comm.stats()
        z = x.copy()
        comm.all_reduce(z, op=op, count=count, dtype=dt)          # in place
        per = count // n
        rs_in = inputs_for(n, per * n, dt, 78)[rank]
        rs = np.zeros(per * L.DTYPE_SIZE[dt], dtype=np.uint8).view(oracle.raw_dtype(dt))
        comm.reduce_scatter(rs_in, rs, op=op, count=per, dtype=dt)
        ag = np.zeros(per * n * L.DTYPE_SIZE[dt], dtype=np.uint8).view(oracle.raw_dtype(dt))
        comm.all_gather(rs_in[:per], ag, count=per, dtype=dt)
        out.append((y, stats, z, rs, ag))
    return out


@pytest.mark.parametrize("n", [2, 3, 5])
def test_ring_rounds_keep_results_and_message_counts(n):
    """Ring blocks above HXCCL_RING_SLICE_KB (here 16 KiB, so dozens of rounds with a ragged
    last one) travel in rounds; the bits, and the messages counted, are those of whole blocks."""
    res = run_ranks(n, _sliced_body, env={"HXCCL_RING_SLICE_KB": "16"})
    for k, (dt, op, count) in enumerate(((L.FLOAT32, L.SUM, 100_003), (L.BFLOAT16, L.AVG, 70_001), (L.INT64, L.MAX, 30_000))):
        ins = inputs_for(n, count, dt, 77)
        want = oracle.allreduce(ins, dt, op, order=0)
        per = count // n
        rs_ins = inputs_for(n, per * n, dt, 78)
        rs_want = oracle.reducescatter(rs_ins, dt, op) if hasattr(oracle, "reducescatter") else None
        for r in range(n):
            y, stats, z, rs, ag = res[r][k]
            assert np.array_equal(y, want[r]) and np.array_equal(z, want[r]), (n, dt, r)
            assert stats[1] == 2 * (n - 1), stats
            if rs_want is not None:
                assert np.array_equal(rs, rs_want[r]), (n, dt, r)
            assert np.array_equal(ag, np.concatenate([rs_ins[q][:per] for q in range(n)])), (n, dt, r)
