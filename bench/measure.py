#!/usr/bin/env python
"""One measurement session: the standard sweeps of bench/hx_perf for a set of rank counts and
transports, each into its own text file, with the GPU clocks logged alongside.

    python bench/measure.py --out results/ --ranks 2,4,8 --modes device,staged,host \
        --ops allreduce,allgather,reducescatter,alltoall,broadcast,sendrecv

Modes: `device` (peer windows / NVLS, the default path), `staged` (HXCCL_DEVICE_TRANSPORT=staged:
device -> host -> host algorithm -> device), `host` (host buffers over the socket mesh). Files:
<out>/<op>_np<N>_<mode>.txt (the hx_perf table), <out>/clocks.csv (nvidia-smi samples every 200 ms
while the sweeps run; only read, never set) and <out>/session.json (commands, exit codes, duration).
`bench/plot.py curves <out>/*.txt` draws the tables. Takes the place of the reference's
scripts/measure_b.sh:1-30 and scripts/measure_e.sh (sweeps np 2/4 x host/device/socket/staged with a
clock log).
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CLOCK_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
               "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
               "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--out", default="results")
    ap.add_argument("--ranks", default="2")
    ap.add_argument("--modes", default="device")
    ap.add_argument("--ops", default="allreduce")
    ap.add_argument("--min-bytes", default="8")
    ap.add_argument("--max-bytes", default=str(256 << 20))
    ap.add_argument("--factor", default="4")
    ap.add_argument("--iters", default="20")
    ap.add_argument("--dtype", default="float")
    ap.add_argument("--red", default="sum")
    ap.add_argument("--timeout", type=float, default=600.0, help="seconds per sweep")
    args = ap.parse_args()

    perf = ROOT / "bench" / "hx_perf"
    if not perf.exists():
        sys.path.insert(0, str(ROOT))
        from hxccl_b200 import build  # noqa: PLC0415

        build.build_perf()
    out = Path(args.out)
    out.mkdir(parents=True, exist_ok=True)
    modes = args.modes.split(",")
    sampler = None
    if shutil.which("nvidia-smi") and any(m != "host" for m in modes):
        sampler = subprocess.Popen(["nvidia-smi", f"--query-gpu={CLOCK_QUERY}", "--format=csv", "-lms", "200"],
                                   stdout=open(out / "clocks.csv", "w"), stderr=subprocess.DEVNULL)
    session, t0 = [], time.time()
    try:
        for n in (int(x) for x in args.ranks.split(",")):
            for mode in modes:
                for op in args.ops.split(","):
                    cmd = [str(perf), "-g", str(n), "-o", op, "-b", args.min_bytes, "-e", args.max_bytes,
                           "-f", args.factor, "-n", args.iters, "-t", args.dtype, "-r", args.red]
                    env = dict(os.environ)
                    if mode == "host":
                        cmd.append("-H")
                    elif mode == "staged":
                        env["HXCCL_DEVICE_TRANSPORT"] = "staged"
                    elif mode != "device":
                        raise SystemExit(f"unknown mode {mode}")
                    path = out / f"{op}_np{n}_{mode}.txt"
                    started = time.time()
                    try:
                        res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=args.timeout)
                        rc, text = res.returncode, res.stdout + (("\n# stderr:\n" + res.stderr) if res.stderr else "")
                    except subprocess.TimeoutExpired as e:
                        rc, text = -1, (e.stdout or "") + f"\n# gave up after {args.timeout} s\n"
                    path.write_text(text)
                    session.append({"file": path.name, "cmd": " ".join(cmd[1:]), "mode": mode, "rc": rc,
                                    "seconds": round(time.time() - started, 1)})
                    print(f"{path.name}: rc {rc}", flush=True)
    finally:
        if sampler is not None:
            sampler.terminate()
            sampler.wait(10)
    (out / "session.json").write_text(json.dumps({"seconds": round(time.time() - t0, 1), "runs": session}, indent=1))
    return 0 if all(r["rc"] == 0 for r in session) else 1


if __name__ == "__main__":
    sys.exit(main())
