"""Choice between the fused GEMM + collective kernels and the library collective + plain GEMM, by measurement.

Whether `ag_gemm` (all-gather inside the GEMM) and `gemm_rs` (reduce-scatter inside the GEMM) beat NCCL followed by
the same GEMM kernel depends on the number of ranks and the per-rank shapes, and timing the ops in isolation does not
settle it: inside a step the ranks arrive skewed and a fused op also saves a launch.  `pick_fastest` therefore times
the caller's WHOLE step under each of the four on/off combinations and leaves the fastest one switched on.  Every rank
takes the same decision because the times are reduced with MAX over the ranks first.

The reference has no counterpart (its collectives are chosen by the Neuron compiler).
"""
from __future__ import annotations

from typing import Callable, Dict, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from . import fused

class CandidateFailed(RuntimeError):
    """A candidate ran but the caller's health check failed afterwards (e.g. a bounded wait of a fused kernel ran
    out on some rank).  The symmetric workspace may be inconsistent between ranks then, so the tuner stops instead of
    trying further candidates; the caller should switch the fused collectives off altogether."""


COMBOS: Tuple[Tuple[bool, bool], ...] = ((True, True), (False, True), (True, False), (False, False))


def combo_name(ag: bool, rs: bool) -> str:
    return f"ag_gemm={'fused' if ag else 'nccl'},gemm_rs={'fused' if rs else 'nccl'}"


def _max_over_ranks(ms: float, device) -> float:
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())
    return ms


def time_steps(run: Callable[[], object], reps: int, device) -> float:
    """Milliseconds per call of `run`, max over ranks: CUDA events on the current stream for a CUDA device, the host
    clock otherwise (gloo ranks on CPU)."""
    import time
    dev = torch.device(device)
    multi = dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1
    if dev.type != "cuda":
        if multi:
            dist.barrier()
        t0 = time.perf_counter()
        for _ in range(reps):
            run()
        return _max_over_ranks((time.perf_counter() - t0) * 1e3 / reps, dev)
    torch.cuda.synchronize(dev)
    if multi:
        dist.barrier()
        torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        run()
    e1.record()
    torch.cuda.synchronize(dev)
    return _max_over_ranks(e0.elapsed_time(e1) / reps, dev)


def pick_fastest(build: Callable[[], Optional[Callable[[], object]]], device, reps: int = 3,
                 combos: Sequence[Tuple[bool, bool]] = COMBOS, release: Optional[Callable[[object], None]] = None,
                 healthy: Optional[Callable[[], bool]] = None) -> Dict:
    """`build()` prepares the step under the CURRENT switch settings (e.g. captures it into a CUDA graph) and returns
    a zero-argument callable that runs one step, or None when that combination cannot run.  Each candidate is
    released (`release(step)`, then the caching allocator is emptied) before the next one is built, so only one
    captured step is alive at a time; the winner is built again at the end.  Returns {"chosen": name,
    "ms": {name: ms per step}, "step": the winner's callable}; the switches are left on the choice.  `healthy()`, if
    given, is called after every candidate's timed calls and must return the same answer on every rank; False raises
    `CandidateFailed` (after releasing the candidate)."""
    report: Dict = {"ms": {}, "chosen": None, "step": None}
    best = None
    for ag, rs in combos:
        fused.set_kernel("ag_gemm", ag)
        fused.set_kernel("gemm_rs", rs)
        name = combo_name(ag, rs)
        step = build()
        if step is None:
            report["ms"][name] = None
            continue
        step()                                        # one untimed call
        ms = time_steps(step, reps, device)
        report["ms"][name] = round(ms, 3)
        ok = healthy() if healthy is not None else True
        if ok and (best is None or ms < best[0]):
            best = (ms, ag, rs)
        if release is not None:
            release(step)
        del step
        if torch.cuda.is_available():
            torch.cuda.empty_cache()
        if not ok:
            raise CandidateFailed(f"health check failed after the timed steps of {name}")
    if best is None:
        raise RuntimeError("no combination of the fused collective kernels could run")
    _, ag, rs = best
    fused.set_kernel("ag_gemm", ag)
    fused.set_kernel("gemm_rs", rs)
    report["chosen"], report["step"] = combo_name(ag, rs), build()
    return report
