"""Profiling helpers: per-step CUDA-event timers, NVTX ranges, torch.profiler traces and an `ncu` command builder.

Counterpart of the reference's `mamba2/run_profile.py` (a CLI around `neuron-profile capture/view` on a compiled
NEFF, :16-60) and of its `--debug`/`--profile` switches (train.py:295-298, mamba2/mamba2_kernel.py:543,598-600):
on B200 the tools are Nsight Compute for single kernels and CUDA events / torch.profiler for whole steps.

    python -m state_space_models_neuron_b200.utils.profiling ncu --kernel gemm_bf16_tcgen05 --launches 3 -- \
        python bench.py --small --steps 1 --warmup 1 --no_e2e
    python -m state_space_models_neuron_b200.utils.profiling summarize report.ncu-rep

prints (or runs, with --run) the `ncu --set full --clock-control none` command, and turns a report into the
short text summary kept under `profiles/`.
"""
from __future__ import annotations

import argparse
import contextlib
import json
import os
import shlex
import subprocess
import sys
import time
from typing import Dict, List, Optional

import torch

KEY_METRICS = [
    "gpu__time_duration.sum", "dram__bytes_read.sum", "dram__bytes_write.sum", "gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed",
    "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active", "sm__warps_active.avg.pct_of_peak_sustained_active",
    "launch__registers_per_thread", "sm__throughput.avg.pct_of_peak_sustained_elapsed",
]


@contextlib.contextmanager
def nvtx_range(name: str):
    if torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if torch.cuda.is_available():
            torch.cuda.nvtx.range_pop()


class CudaTimer:
    """Accumulates device time of named regions with CUDA events (no synchronisation until `summary`)."""

    def __init__(self):
        self.events: Dict[str, List] = {}

    @contextlib.contextmanager
    def region(self, name: str):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        try:
            yield
        finally:
            b.record()
            self.events.setdefault(name, []).append((a, b))

    def summary(self) -> Dict[str, float]:
        torch.cuda.synchronize()
        return {k: sum(a.elapsed_time(b) for a, b in v) for k, v in self.events.items()}


class StepProfiler:
    """torch.profiler trace of a few optimizer steps, written under `output_dir/profile` (train.py --profile)."""

    def __init__(self, output_dir: str, wait: int = 2, active: int = 2):
        from torch.profiler import ProfilerActivity, profile, schedule
        self.dir = os.path.join(output_dir, "profile")
        os.makedirs(self.dir, exist_ok=True)
        self.prof = profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA],
                            schedule=schedule(wait=wait, warmup=1, active=active, repeat=1),
                            on_trace_ready=self._done)
        self.prof.start()

    def _done(self, prof):
        prof.export_chrome_trace(os.path.join(self.dir, f"trace_{int(time.time())}.json"))
        with open(os.path.join(self.dir, "kernels.txt"), "w") as f:
            f.write(prof.key_averages().table(sort_by="cuda_time_total", row_limit=40))

    def step(self):
        self.prof.step()


def ncu_command(cmd: List[str], kernel: Optional[str], launches: int = 3, skip: int = 0, out: str = "profiles_raw/prof",
                full: bool = True) -> List[str]:
    """`ncu` invocation for one kernel of a small case; always with `--clock-control none`."""
    base = ["ncu", "--clock-control", "none"]
    base += ["--set", "full"] if full else ["--metrics", "gpu__time_duration.sum"]
    if kernel:
        base += ["-k", f"regex:{kernel}"]
    base += ["-s", str(skip), "-c", str(launches), "-o", out]
    return base + cmd


def summarize_report(path: str) -> str:
    """Key metrics of an .ncu-rep as text (runs `ncu -i ... --page raw --csv`, no GPU needed)."""
    r = subprocess.run(["ncu", "-i", path, "--page", "raw", "--csv"], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(r.stderr)
    import csv
    rows = list(csv.reader(r.stdout.splitlines()))
    header, units, data = rows[0], rows[1], rows[2:]
    lines = []
    want = [i for i, h in enumerate(header) if any(h.startswith(k.split(".")[0]) for k in KEY_METRICS) or h in ("Kernel Name", "Grid Size", "Block Size")]
    for row in data:
        lines.append("; ".join(f"{header[i]}={row[i]}{(' ' + units[i]) if units[i] else ''}" for i in want))
    return "\n".join(lines)


def main(argv=None):
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    a = sub.add_parser("ncu")
    a.add_argument("--kernel", default=None)
    a.add_argument("--launches", type=int, default=3)
    a.add_argument("--skip", type=int, default=0)
    a.add_argument("--out", default="profiles_raw/prof")
    a.add_argument("--run", action="store_true")
    a.add_argument("rest", nargs=argparse.REMAINDER)
    b = sub.add_parser("summarize")
    b.add_argument("report")
    args = ap.parse_args(argv)
    if args.cmd == "ncu":
        rest = [x for x in args.rest if x != "--"]
        cmd = ncu_command(rest, args.kernel, args.launches, args.skip, args.out)
        print(" ".join(shlex.quote(c) for c in cmd))
        if args.run:
            sys.exit(subprocess.call(cmd))
    else:
        print(summarize_report(args.report))


if __name__ == "__main__":
    main()
