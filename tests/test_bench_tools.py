"""The plotting tool turns benchmark output (JSON lines of bench/sweep.py, tables of
bench/hx_perf) into well-formed SVG."""
import json
import os
import subprocess
import sys
import xml.dom.minidom

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_plot_curves_and_phases(tmp_path):
    src = tmp_path / "rows.jsonl"
    rows = [{"config": c, "bytes": b, "us": 10.0, "busbw_GBps": v,
             "trace_us": {"in": 1, "sigA": 0.5, "waitA": 2, "mid": 3, "sigB": 0.5, "waitB": 1, "out": 2, "all": 10}}
            for c, b, v in (("default", 65536, 5.0), ("default", 1 << 28, 570.0), ("nccl", 65536, 4.0), ("nccl", 1 << 28, 630.0))]
    text = "\n".join(json.dumps(r) for r in rows)
    text += ("\n# hx_perf  op=allreduce type=float red=sum ranks=2 buffers=device path=window iters=20 warmup=5\n"
             "#        bytes        count     time(us)  algbw(GB/s)  busbw(GB/s)\n"
             "         65536        16384        17.07         3.84         3.84\n"
             "       1048576       262144        26.12        40.15        40.15\n")
    src.write_text(text)
    for kind, tag, least in (("curves", "path", 3), ("phases", "rect", 4 * 7)):
        out = tmp_path / f"{kind}.svg"
        subprocess.run([sys.executable, os.path.join(ROOT, "bench", "plot.py"), kind, str(src), "-o", str(out)],
                       check=True, timeout=60)
        doc = xml.dom.minidom.parse(str(out))
        assert doc.documentElement.tagName == "svg"
        assert len(doc.getElementsByTagName(tag)) >= least


def test_torch_allreduce_bench_on_cpu():
    """bench/torch_allreduce.py as two CPU ranks: one JSON line per backend and size."""
    import socket

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", str(port),
                          os.path.join(ROOT, "bench", "torch_allreduce.py"), "--device", "cpu",
                          "--backends", "hxccl,gloo", "--sizes", "4K,256K", "--iters", "3", "--warmup", "1"],
                         capture_output=True, text=True, timeout=240)
    assert res.returncode == 0, res.stderr[-2000:]
    rows = [json.loads(line) for line in res.stdout.splitlines() if line.startswith("{")]
    assert [(r["backend"], r["bytes"]) for r in rows] == [("hxccl", 4096), ("hxccl", 262144), ("gloo", 4096), ("gloo", 262144)]
    assert all(r["us"] > 0 and r["ranks"] == 2 for r in rows)


def test_c_example_builds_as_c99_and_runs(tmp_path):
    """The public headers are plain C; examples/allreduce.c runs three ranks over the socket bootstrap."""
    from hxccl_b200 import _lib

    _lib.lib()  # builds the library when it is missing
    libdir = os.path.join(ROOT, "hxccl_b200", "lib")
    exe = tmp_path / "allreduce"
    subprocess.run(["gcc", "-std=c99", "-D_POSIX_C_SOURCE=200809L", "-Wall", "-Wextra", "-pedantic", "-Werror",
                    "-I" + os.path.join(ROOT, "include"), os.path.join(ROOT, "examples", "allreduce.c"),
                    "-L" + libdir, "-lhxccl", "-Wl,-rpath," + libdir, "-o", str(exe)], check=True, timeout=120)
    res = subprocess.run([str(exe), "3"], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0 and "3 ranks: average 2, ring shift ok" in res.stdout, (res.stdout, res.stderr)


def test_mpi_entry_point_compiles_against_an_mpi_header():
    """hxcclCommInitMPI is only built where MPI exists; the stand-in header of the reference arm is
    enough to check that it still compiles together with the public header's MPI section."""
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    subprocess.run(["g++", "-std=c++17", "-fsyntax-only", "-Wall", "-Wextra", "-Werror", "-DHXCCL_HAVE_MPI",
                    "-I" + os.path.join(ROOT, "baseline", "mpi_stub"), "-I" + os.path.join(ROOT, "include"),
                    "-I" + os.path.join(ROOT, "src"), "-I" + os.path.join(cuda, "include"),
                    os.path.join(ROOT, "src", "core", "comm_mpi.cc")], check=True, timeout=120)


def test_launch_environment_from_openmpi(monkeypatch):
    from hxccl_b200.utils.env import fill_env_from_openmpi

    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT"):
        monkeypatch.delenv(k, raising=False)
    monkeypatch.setenv("OMPI_COMM_WORLD_RANK", "3")
    monkeypatch.setenv("OMPI_COMM_WORLD_SIZE", "8")
    monkeypatch.setenv("OMPI_COMM_WORLD_LOCAL_RANK", "1")
    monkeypatch.setenv("MASTER_PORT", "12345")  # what the user set stays
    fill_env_from_openmpi()
    assert (os.environ["RANK"], os.environ["WORLD_SIZE"], os.environ["LOCAL_RANK"]) == ("3", "8", "1")
    assert os.environ["MASTER_ADDR"] == "127.0.0.1" and os.environ["MASTER_PORT"] == "12345"


def test_measurement_session_on_host_buffers(tmp_path):
    """bench/measure.py in host mode (no GPU): one table per (collective, rank count), a session record,
    and tables the plotting tool can read."""
    out = tmp_path / "res"
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench", "measure.py"), "--out", str(out), "--ranks", "2,3",
                          "--modes", "host", "--ops", "allreduce,sendrecv", "--min-bytes", "1024", "--max-bytes", "65536",
                          "--factor", "8", "--iters", "3"], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    session = json.loads((out / "session.json").read_text())
    assert [r["file"] for r in session["runs"]] == ["allreduce_np2_host.txt", "sendrecv_np2_host.txt",
                                                    "allreduce_np3_host.txt", "sendrecv_np3_host.txt"]
    assert all(r["rc"] == 0 for r in session["runs"])
    table = (out / "allreduce_np3_host.txt").read_text()
    assert "# hx_perf  op=allreduce" in table and "ranks=3" in table and table.count("\n") >= 5
    svg = tmp_path / "c.svg"
    subprocess.run([sys.executable, os.path.join(ROOT, "bench", "plot.py"), "curves", str(out / "allreduce_np2_host.txt"),
                    str(out / "allreduce_np3_host.txt"), "-o", str(svg)], check=True, timeout=60)
    assert len(xml.dom.minidom.parse(str(svg)).getElementsByTagName("path")) == 2


def test_gpu_numa_cpus_reads_sysfs(tmp_path):
    """The NUMA helper of the launcher against a made-up sysfs tree."""
    from hxccl_b200.utils.env import _parse_cpulist, gpu_numa_cpus

    dev = tmp_path / "bus/pci/devices/0000:1b:00.0"
    dev.mkdir(parents=True)
    (dev / "numa_node").write_text("1\n")
    node = tmp_path / "devices/system/node/node1"
    node.mkdir(parents=True)
    (node / "cpulist").write_text("32-47,96-99\n")
    assert gpu_numa_cpus("0000:1B:00.0", sysfs=str(tmp_path)) == set(range(32, 48)) | set(range(96, 100))
    (dev / "numa_node").write_text("-1\n")
    assert gpu_numa_cpus("0000:1b:00.0", sysfs=str(tmp_path)) == set()
    assert gpu_numa_cpus("0000:ff:00.0", sysfs=str(tmp_path)) == set()
    assert _parse_cpulist("0,2-3") == {0, 2, 3}


def test_host_benchmark_against_the_reference_runs():
    """bench/host_vs_reference.py: one JSON line per size, with the reference's columns filled
    when the reference library has been built (baseline/build_ref.py)."""
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench", "host_vs_reference.py"), "--ranks", "2",
                          "--iters", "3", "--rounds", "1", "--coll", "allgather", "--sizes", "256,70000"],
                         capture_output=True, text=True, timeout=300, check=True)
    rows = [json.loads(ln) for ln in out.stdout.splitlines() if ln.startswith("{")]
    assert [r["bytes"] for r in rows] == [256, 70000] and all(r["coll"] == "allgather" for r in rows)
    assert all(r["hxccl_us"] > 0 and r["hxccl_busbw_GBps"] >= 0 for r in rows)
    built = os.path.exists(os.path.join(ROOT, "baseline", "_ref", "libhxccl_ref.so"))
    assert all((r["reference_us"] is not None) == built for r in rows)


@pytest.mark.parametrize("extra", [[], ["--compress"]])
def test_ddp_example_trains_on_two_cpu_ranks(extra):
    """examples/ddp_train.py through torchrun: the loss falls and all ranks end with the same weights."""
    import socket

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", str(port),
                          os.path.join(ROOT, "examples", "ddp_train.py"), "--cpu", "--steps", "12", *extra],
                         capture_output=True, text=True, timeout=240)
    assert res.returncode == 0, (res.stdout[-1000:], res.stderr[-2000:])
    assert "weights identical on all 2 ranks: True" in res.stdout


@pytest.mark.parametrize("ranks", [2, 3])
def test_parallel_patterns_example_on_cpu_ranks(ranks):
    """examples/parallel_patterns.py: tensor, pipeline, sequence and expert parallel data movement
    on the backend's primitives, each checked against the single-rank computation."""
    import socket

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(ranks),
                          "--master-addr", "127.0.0.1", "--master-port", str(port),
                          os.path.join(ROOT, "examples", "parallel_patterns.py"), "--cpu"],
                         capture_output=True, text=True, timeout=240)
    assert res.returncode == 0, (res.stdout[-1000:], res.stderr[-2000:])
    assert "all ranks agree: True" in res.stdout
