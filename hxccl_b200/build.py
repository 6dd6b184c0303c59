"""Builds the native parts in-tree: libhxccl.so (C API, host path, sm_100a kernels) and, on
request, the torch.distributed backend extension.

    python -m hxccl_b200.build            # library
    python -m hxccl_b200.build --torch    # library + torch backend
    python -m hxccl_b200.build --sanitize # build/libhxccl_san.so: host code under ASan + UBSan

The sanitizer build compiles every host source (.cc) with -fsanitize=address,undefined and links
it with the ordinary kernel objects. Run the CPU tests against it with

    HXCCL_LIBRARY=build/libhxccl_san.so LD_PRELOAD=$(g++ -print-file-name=libasan.so) \
        ASAN_OPTIONS=detect_leaks=0 python -m pytest tests -q -m "not gpu" --deselect tests/test_torch_backend.py \
        --deselect tests/test_bench_tools.py

`python -m hxccl_b200.build --tsan` builds the host sources under ThreadSanitizer together with
build/ranks_as_threads (tests/tsan/ranks_as_threads.cc: the ranks of a communicator as threads of one
process); run `build/ranks_as_threads 4`.

(the interpreter itself is not instrumented, hence the preload and no leak report; the torch
backend test is left out because libtorch throws C++ exceptions before the preloaded ASan has
found the real __cxa_throw, which ends the process with an ASan CHECK that is not about this code).

The CUDA sources are compiled for sm_100a only (-gencode arch=compute_100a,code=sm_100a);
nvcc cross-compiles, so no GPU is needed to build. Objects land in build/ (ignored by git),
the shared objects next to this file so that they travel with the source tree.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
SRC = ROOT / "src"
OBJ = ROOT / "build" / "obj"
LIB_DIR = Path(__file__).resolve().parent / "lib"
LIB = LIB_DIR / "libhxccl.so"
CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
NVCC = str(CUDA_HOME / "bin" / "nvcc")

INCLUDES = [f"-I{ROOT / 'include'}", f"-I{SRC}", f"-I{CUDA_HOME / 'include'}"]
CXXFLAGS = ["-std=c++17", "-O2", "-fPIC", "-ffp-contract=off", "-Wall", "-Wextra", "-pthread"]
NVCCFLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC", "-fmad=false",
]


def _newest_header() -> float:
    hdrs = (list(SRC.rglob("*.h")) + list(SRC.rglob("*.cuh")) + list(SRC.rglob("*.inc"))
            + list((ROOT / "include").glob("*.h")))
    return max(p.stat().st_mtime for p in hdrs)


SANFLAGS = ["-fsanitize=address,undefined", "-fno-omit-frame-pointer", "-g", "-O1"]
TSANFLAGS = ["-fsanitize=thread", "-fno-omit-frame-pointer", "-g", "-O1"]


_TSAN_CXX: list = []


def _tsan_cxx() -> str:
    """A host compiler that can link its ThreadSanitizer runtime (not every installed one ships it)."""
    if not _TSAN_CXX:
        probe = ROOT / "build" / "tsan_probe.cc"
        probe.parent.mkdir(parents=True, exist_ok=True)
        probe.write_text("int main() { return 0; }\n")
        for cxx in dict.fromkeys([os.environ.get("CXX", "g++"), "g++", "/usr/bin/g++", "c++"]):
            try:
                ok = subprocess.run([cxx, "-fsanitize=thread", str(probe), "-o", str(probe.with_suffix(""))],
                                    capture_output=True).returncode == 0
            except OSError:
                ok = False
            if ok:
                _TSAN_CXX.append(cxx)
                break
        else:
            raise RuntimeError("no host compiler here can link -fsanitize=thread")
    return _TSAN_CXX[0]


def _compile(src: Path, hdr_time: float, verbose: bool, sanitize=False) -> Path:
    """`sanitize`: False, True (ASan + UBSan) or "thread" (TSan); host sources only."""
    sanitize = sanitize if src.suffix != ".cu" else False
    suffix = {False: ".o", True: ".san.o", "thread": ".tsan.o"}[sanitize]
    obj = OBJ / (str(src.relative_to(SRC)).replace("/", "_") + suffix)
    if obj.exists() and obj.stat().st_mtime > max(src.stat().st_mtime, hdr_time):
        return obj
    if src.suffix == ".cu":
        cmd = [NVCC, *NVCCFLAGS, *INCLUDES, "-c", str(src), "-o", str(obj)]
    else:
        extra = {False: [], True: SANFLAGS, "thread": TSANFLAGS}[sanitize]
        cxx = _tsan_cxx() if sanitize == "thread" else os.environ.get("CXX", "g++")
        cmd = [cxx, *CXXFLAGS, *extra, *INCLUDES, "-c", str(src), "-o", str(obj)]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"compiling {src} failed:\n{res.stdout}\n{res.stderr}")
    return obj


def build_lib(verbose: bool = False, jobs: int | None = None) -> Path:
    """Compiles every source under src/ and links hxccl_b200/lib/libhxccl.so."""
    OBJ.mkdir(parents=True, exist_ok=True)
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    sources = sorted(SRC.rglob("*.cc")) + sorted(SRC.rglob("*.cu"))
    hdr_time = _newest_header()
    jobs = jobs or max(1, (os.cpu_count() or 2))
    with ThreadPoolExecutor(max_workers=jobs) as pool:
        objs = list(pool.map(lambda s: _compile(s, hdr_time, verbose), sources))
    if LIB.exists() and all(LIB.stat().st_mtime > o.stat().st_mtime for o in objs):
        return LIB
    cmd = [NVCC, "-shared", "-cudart", "static", "-o", str(LIB), *map(str, objs),
           "-Xcompiler", "-pthread", "-ldl", "-lrt"]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"linking libhxccl.so failed:\n{res.stdout}\n{res.stderr}")
    return LIB


def build_sanitized(verbose: bool = False, jobs: int | None = None) -> Path:
    """Links build/libhxccl_san.so: host sources under ASan + UBSan, kernels as in the normal build."""
    build_lib(verbose, jobs)  # the kernel objects
    sources = sorted(SRC.rglob("*.cc")) + sorted(SRC.rglob("*.cu"))
    hdr_time = _newest_header()
    with ThreadPoolExecutor(max_workers=jobs or max(1, (os.cpu_count() or 2))) as pool:
        objs = list(pool.map(lambda s: _compile(s, hdr_time, verbose, sanitize=True), sources))
    out = ROOT / "build" / "libhxccl_san.so"
    cmd = [NVCC, "-shared", "-cudart", "static", "-o", str(out), *map(str, objs),
           "-Xcompiler", "-pthread", "-Xcompiler", "-fsanitize=address", "-Xcompiler", "-fsanitize=undefined",
           "-ldl", "-lrt"]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"linking libhxccl_san.so failed:\n{res.stdout}\n{res.stderr}")
    return out


def build_tsan(verbose: bool = False, jobs: int | None = None) -> Path:
    """Links build/libhxccl_tsan.so (host sources under ThreadSanitizer) and build/ranks_as_threads,
    the program of tests/tsan/ranks_as_threads.cc that runs the ranks of a communicator as threads of
    one process, so that the sanitizer sees both ends of every hand-over."""
    build_lib(verbose, jobs)
    sources = sorted(SRC.rglob("*.cc")) + sorted(SRC.rglob("*.cu"))
    hdr_time = _newest_header()
    with ThreadPoolExecutor(max_workers=jobs or max(1, (os.cpu_count() or 2))) as pool:
        objs = list(pool.map(lambda s: _compile(s, hdr_time, verbose, sanitize="thread"), sources))
    out = ROOT / "build" / "libhxccl_tsan.so"
    cxx = _tsan_cxx()  # the host compiler links: it knows where its TSan runtime is
    steps = [[cxx, "-shared", "-fsanitize=thread", "-o", str(out), *map(str, objs), f"-L{CUDA_HOME / 'lib64'}",
              "-lcudart_static", "-pthread", "-ldl", "-lrt"],
             [cxx, "-std=c++17", *TSANFLAGS, *INCLUDES,
              str(ROOT / "tests" / "tsan" / "ranks_as_threads.cc"), "-o", str(ROOT / "build" / "ranks_as_threads"),
              f"-L{ROOT / 'build'}", "-lhxccl_tsan", f"-Wl,-rpath,{ROOT / 'build'}", "-pthread"]]
    for cmd in steps:
        if verbose:
            print(" ".join(cmd), flush=True)
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"{cmd[0]} failed:\n{res.stdout}\n{res.stderr}")
    return out


def build_perf(verbose: bool = False) -> Path:
    """Builds bench/hx_perf, the native sweep tool, against libhxccl.so."""
    build_lib(verbose)
    src = ROOT / "bench" / "hx_perf.cc"
    out = ROOT / "bench" / "hx_perf"
    if out.exists() and out.stat().st_mtime > max(src.stat().st_mtime, LIB.stat().st_mtime):
        return out
    cmd = [NVCC, "-std=c++17", "-O2", *INCLUDES, str(src), "-o", str(out), f"-L{LIB_DIR}", "-lhxccl",
           "-Xlinker", f"-rpath={LIB_DIR}", "-Xlinker", "-rpath=$ORIGIN/../hxccl_b200/lib", "-cudart", "static", "-ldl"]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"building hx_perf failed:\n{res.stdout}\n{res.stderr}")
    return out


def build_torch_ext(verbose: bool = False) -> Path:
    """Builds hxccl_b200/_hxccl_c10d.so, the torch.distributed backend, against libhxccl.so."""
    build_lib(verbose)
    from torch.utils import cpp_extension  # noqa: PLC0415  (import torch only when asked)

    pkg = Path(__file__).resolve().parent
    src = pkg / "csrc" / "backend.cpp"
    out = pkg / "_hxccl_c10d.so"
    if out.exists() and out.stat().st_mtime > max(src.stat().st_mtime, LIB.stat().st_mtime):
        return out
    build_dir = ROOT / "build" / "torch_ext"
    build_dir.mkdir(parents=True, exist_ok=True)
    cpp_extension.load(
        name="_hxccl_c10d",
        sources=[str(src)],
        extra_include_paths=[str(ROOT / "include"), str(CUDA_HOME / "include")],
        extra_cflags=["-O2", "-std=c++17"],
        extra_ldflags=[f"-L{LIB_DIR}", "-lhxccl", f"-Wl,-rpath,{LIB_DIR}", "-Wl,-rpath,$ORIGIN/lib",
                       f"-L{CUDA_HOME / 'lib64'}", "-lcudart"],
        build_directory=str(build_dir),
        with_cuda=True,
        is_python_module=False,
        verbose=verbose,
    )
    shutil.copy2(build_dir / "_hxccl_c10d.so", out)
    return out


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--torch", action="store_true", help="also build the torch.distributed backend")
    ap.add_argument("--perf", action="store_true", help="also build bench/hx_perf")
    ap.add_argument("--sanitize", action="store_true", help="also build build/libhxccl_san.so (ASan + UBSan)")
    ap.add_argument("--tsan", action="store_true", help="also build build/libhxccl_tsan.so and build/ranks_as_threads")
    ap.add_argument("-v", "--verbose", action="store_true")
    ap.add_argument("-j", "--jobs", type=int, default=None)
    args = ap.parse_args()
    print(build_lib(args.verbose, args.jobs))
    if args.torch:
        print(build_torch_ext(args.verbose))
    if args.perf:
        print(build_perf(args.verbose))
    if args.sanitize:
        print(build_sanitized(args.verbose, args.jobs))
    if args.tsan:
        print(build_tsan(args.verbose, args.jobs))


if __name__ == "__main__":
    sys.exit(main())
