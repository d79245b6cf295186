"""Debug aids that stand in for a race detector / memory checker (the reference has none beyond the NKI CPU
simulator its tests use, tests/mamba2_kernel_test_no_tp.py:48):

  * `CanaryBuffer`: allocate a tensor with guard words on both sides and verify them afterwards; finds kernels
    that write outside their output.
  * `assert_deterministic`: run a callable twice on cloned inputs and require bit-identical results; flag/semaphore
    protocol races and uninitialised reads show up as run-to-run differences.
  * `check_finite`: NaN/Inf check with a named error (the reference's decode script does this by hand,
    mamba2_inference_no_tp.py:104-106).
  * `tile_schedule_is_permutation`: host-side check of the GEMM tile visiting order used by the fused
    collectives (every tile visited exactly once for every rank rotation).
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch

_CANARY = 0x5A


class CanaryBuffer:
    def __init__(self, shape, dtype, device, guard_bytes: int = 4096):
        self.numel = 1
        for s in shape:
            self.numel *= int(s)
        self.item = torch.empty((), dtype=dtype).element_size()
        self.guard = guard_bytes
        self.raw = torch.full((self.numel * self.item + 2 * guard_bytes,), _CANARY, dtype=torch.uint8, device=device)
        self.tensor = self.raw[guard_bytes:guard_bytes + self.numel * self.item].view(dtype).view(*shape)

    def intact(self) -> bool:
        g = self.guard
        return bool((self.raw[:g] == _CANARY).all() and (self.raw[-g:] == _CANARY).all())


def assert_deterministic(fn: Callable, inputs: Sequence[torch.Tensor]) -> None:
    outs = []
    for _ in range(2):
        res = fn(*[t.clone() for t in inputs])
        res = res if isinstance(res, (tuple, list)) else (res,)
        outs.append([r.clone() for r in res if isinstance(r, torch.Tensor)])
    for a, b in zip(*outs):
        if not torch.equal(a, b):
            raise AssertionError(f"non-deterministic result: max diff {(a.float() - b.float()).abs().max().item():.3e}")


def check_finite(t: torch.Tensor, name: str = "tensor") -> None:
    if not torch.isfinite(t).all():
        bad = (~torch.isfinite(t)).sum().item()
        raise FloatingPointError(f"{name} has {bad} non-finite values")


def rotate_m(tm: int, tiles_m: int, tiles_per_block: int, first_block: int) -> int:
    """Host copy of the device tile rotation (ops/csrc/gemm.cu `rotate_m`)."""
    v = tm + first_block * tiles_per_block
    return v - tiles_m if v >= tiles_m else v


def tile_schedule_is_permutation(tiles_m: int, tiles_n: int, nranks: int, ctas: int) -> bool:
    per = tiles_m // nranks
    for me in range(nranks):
        seen = set()
        for cta in range(ctas):
            for tile in range(cta, tiles_m * tiles_n, ctas):
                seen.add((rotate_m(tile % tiles_m, tiles_m, per, me), tile // tiles_m))
        if len(seen) != tiles_m * tiles_n:
            return False
    return True
