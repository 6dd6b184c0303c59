#!/usr/bin/env python
"""Builds the reference library (Thisish3/hxccl) from its unmodified sources into
baseline/_ref/libhxccl_ref.so, for the reference arm of bench.py.

The reference needs MPI at compile time (include/hxccl.h includes <mpi.h>) and no MPI is
installed here, so it is compiled against baseline/mpi_stub/mpi.h, a stand-in whose functions
all fail; the reference arm only uses the reference's socket bootstrap (hxcclGetUniqueId /
hxcclCommInitRank), which never calls MPI. The reference's CMakeLists.txt targets sm_86; here
its one kernel file is compiled for sm_100a. No reference source file is changed or copied
into this repository: the sources are read from --src (or $HXCCL_REFERENCE_SRC).
"""
import argparse
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--src", default=os.environ.get("HXCCL_REFERENCE_SRC", os.path.join(os.sep, "root", "reference")))
    args = ap.parse_args()
    src = Path(args.src)
    out = HERE / "_ref"
    obj = out / "obj"
    obj.mkdir(parents=True, exist_ok=True)
    cuda = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
    inc = [f"-I{HERE / 'mpi_stub'}", f"-I{src / 'include'}", f"-I{src / 'src'}", f"-I{cuda / 'include'}"]
    objs = []
    for f in sorted((src / "src").glob("*.cc")):
        if f.name == "memspace.cc":  # the CPU-only variant, replaced by memspace_cuda.cc (as in its CMakeLists)
            continue
        o = obj / (f.name + ".o")
        subprocess.check_call(["g++", "-std=c++17", "-O2", "-fPIC", "-DHXCCL_CUDA=1", *inc, "-c", str(f), "-o", str(o)])
        objs.append(o)
    for f in sorted((src / "src").glob("*.cu")):
        o = obj / (f.name + ".o")
        subprocess.check_call([str(cuda / "bin" / "nvcc"), "-std=c++17", "-O3", "-DHXCCL_CUDA=1",
                               "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC", *inc,
                               "-c", str(f), "-o", str(o)])
        objs.append(o)
    stub = obj / "mpi_stub.o"
    subprocess.check_call(["gcc", "-O2", "-fPIC", f"-I{HERE / 'mpi_stub'}", "-c", str(HERE / "mpi_stub" / "mpi_stub.c"),
                           "-o", str(stub)])
    lib = out / "libhxccl_ref.so"
    subprocess.check_call([str(cuda / "bin" / "nvcc"), "-shared", "-cudart", "static", "-o", str(lib), *map(str, objs), str(stub),
                           f"-L{cuda / 'lib64' / 'stubs'}", "-lcuda", "-Xcompiler", "-pthread"])
    print(lib)
    return 0


if __name__ == "__main__":
    sys.exit(main())
