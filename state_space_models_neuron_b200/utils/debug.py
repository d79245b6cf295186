"""Debug aids that stand in for a race detector / memory checker (the reference has none beyond the NKI CPU
simulator its tests use, tests/mamba2_kernel_test_no_tp.py:48):

  * `CanaryBuffer`: allocate a tensor with guard words on both sides and verify them afterwards; finds kernels
    that write outside their output.
  * `assert_deterministic`: run a callable twice on cloned inputs and require bit-identical results; flag/semaphore
    protocol races and uninitialised reads show up as run-to-run differences.
  * `check_finite`: NaN/Inf check with a named error (the reference's decode script does this by hand,
    mamba2_inference_no_tp.py:104-106).
  * `tile_schedule_is_permutation`, `gemm_schedule_covers_once`: host-side models of the GEMM's tile visiting
    order under the fused collectives' rotations and of its full-wave / K-split tail work distribution, for
    property tests of the index arithmetic (every tile and k-block computed exactly once).
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


def collective_tile_origin(tile: int, tiles_n: int, tiles_per_block: int, nranks: int, first_block: int):
    """Host copy of the tile order of the GEMMs fused with a collective (ops/csrc/gemm.cu `tile_origin`): tiles are
    visited block by block (a block = the rows of one shard / owner, `tiles_per_block` m-tiles), starting with
    `first_block` and going round the ranks; returns (m-tile, n-tile)."""
    per_block = tiles_per_block * tiles_n
    bi, within = divmod(tile, per_block)
    block = (first_block + bi) % nranks
    tn, tm_in = divmod(within, tiles_per_block)
    return block * tiles_per_block + tm_in, tn


def gemm_tile_cost_kb(bn: int, pair: bool) -> float:
    """Host copy of `tile_cost_kb` in ops/csrc/gemm.cu: cost of one tile per k-block relative to the single-CTA
    128 x 256 tile."""
    if pair:
        return 0.68 if bn == 256 else 0.52
    return 1.00 if bn == 256 else 0.80


def gemm_plan(M: int, N: int, K: int, accumulate: bool = False, allow_pair: bool = True):
    """What `ssm_gemm_plan` of the native library answers for a plain GEMM of this shape: a dict with the tile width
    `bn`, `pair`, `tiles_m`, `tiles_n`, `units`, `full_tiles`, `rem`, `split`.  Works without a GPU (148 SMs assumed)."""
    import ctypes
    from ..ops import native
    out = (ctypes.c_int * 8)()
    code = native.lib().ssm_gemm_plan(int(M), int(N), int(K), 2 if accumulate else 0, int(allow_pair), out)
    if code != 0:
        raise ValueError(f"ssm_gemm_plan({M}, {N}, {K}) returned {code}")
    keys = ("bn", "pair", "tiles_m", "tiles_n", "units", "full_tiles", "rem", "split")
    return dict(zip(keys, [int(v) for v in out]))


def gemm_tail_split(rem: int, units: int, kblocks: int, accumulate: bool = False, pair: bool = False,
                    cost_kb: float = 1.0, always: bool = False) -> int:
    """Host copy of `tail_split` in ops/csrc/gemm.cu: K slices per tail tile.  The split is taken only where the
    saved share of the main loop exceeds the exchange of partial sums (22 k-block units for a pair tile, 12 for a
    single-CTA tile, 4 in accumulate mode) unless `always`."""
    if rem <= 0:
        return 1
    split = min(units // rem, 8 if accumulate else 4, kblocks // 4)
    if split <= 1:
        return 1
    exch = 4.0 if accumulate else (22.0 if pair else 12.0)
    if not always and (1.0 - 1.0 / split) * kblocks * cost_kb <= exch:
        return 1
    return split


def gemm_schedule(tiles: int, max_units: int, kblocks: int, accumulate: bool = False, split_enabled: bool = True,
                  pair: bool = False, cost_kb: float = 1.0, always_split: bool = True):
    """Host copy of the GEMM's work distribution (ops/csrc/gemm.cu `launch_gemm` + `get_work`): returns
    (units, [(unit, tile, kb0, kb1, slice, nslices)]).  Whole tiles go round-robin over the units for as many full
    waves as there are; the tiles of the last partial wave are cut into K slices, one per otherwise idle unit
    (`always_split=False` applies the kernel's pay-off rule, see `gemm_tail_split`)."""
    units = min(tiles, max_units)
    full = (tiles // units) * units
    rem = tiles - full
    split = 1
    if split_enabled and (rem > 0 or tiles < max_units):
        if tiles < max_units:
            units, full, rem = max_units, 0, tiles
        split = gemm_tail_split(rem, units, kblocks, accumulate, pair, cost_kb, always_split)
        if tiles < max_units:
            units = rem * split
    work = []
    for unit in range(units):
        it = 0
        while True:
            idx = unit + it * units
            if idx < full:
                work.append((unit, idx, 0, kblocks, 0, 1))
            elif it == full // units and unit < rem * split:
                tail = unit // split
                sl = unit - tail * split
                work.append((unit, full + tail, sl * kblocks // split, (sl + 1) * kblocks // split, sl, split))
            else:
                break
            it += 1
    return units, work


def gemm_schedule_covers_once(tiles: int, max_units: int, kblocks: int, accumulate: bool = False) -> bool:
    """Every (tile, k-block) is computed exactly once, no unit gets two pieces of the tail, and no slice is empty."""
    units, work = gemm_schedule(tiles, max_units, kblocks, accumulate)
    seen = {}
    tail_units = set()
    for unit, tile, kb0, kb1, sl, n in work:
        if kb1 <= kb0 or unit >= units:
            return False
        if n > 1:
            if unit in tail_units:
                return False
            tail_units.add(unit)
        for kb in range(kb0, kb1):
            if (tile, kb) in seen:
                return False
            seen[(tile, kb)] = unit
    return len(seen) == tiles * kblocks


def tile_schedule_is_permutation(tiles_m: int, tiles_n: int, nranks: int, ctas: int) -> bool:
    """The block-major tile order of the fused collectives (local shard first for the all-gather, next rank's rows
    first for the reduce-scatter) visits every tile exactly once for every rank, and a rank's first
    `tiles_per_block * tiles_n` tiles are exactly the rows of its first block."""
    per = tiles_m // nranks
    for me in range(nranks):
        for first in (me, (me + 1) % nranks):
            seen = []
            for cta in range(ctas):
                for tile in range(cta, tiles_m * tiles_n, ctas):
                    seen.append((tile, collective_tile_origin(tile, tiles_n, per, nranks, first)))
            if len({o for _, o in seen}) != tiles_m * tiles_n or len(seen) != tiles_m * tiles_n:
                return False
            if any(tm // per != first for tile, (tm, tn) in seen if tile < per * tiles_n):
                return False
    return True


def ag_push_plan(rows_per_shard: int, K: int, n_sms: int = 148, max_groups: int = 4):
    """Host copy of how the all-gather GEMM cuts the local shard into push boxes (ops/csrc/gemm.cu, host side):
    box height 128, halved down to 32 while there are fewer than 3 boxes per SM; up to `max_groups` column groups of
    whole 64-column blocks.  Returns (push_rows, col_blocks, group_kb, ngroups, staging slots per CTA)."""
    col_blocks = -(-K // 64)
    push_rows = 128
    while push_rows > 32 and (rows_per_shard // push_rows) * col_blocks < 3 * n_sms:
        push_rows //= 2
    group_kb = -(-col_blocks // max_groups)
    ngroups = -(-col_blocks // group_kb)
    nslots = (2 * 128 * 64 * 2) // (push_rows * 128)
    return push_rows, col_blocks, group_kb, ngroups, nslots


def ag_push_boxes(grid: int, rows_per_shard: int, push_rows: int, col_blocks: int, group_kb: int):
    """Host copy of the dealing of push boxes over the CTAs of the grid (the push loop of `gemm_bf16_tcgen05`):
    returns per CTA the list of (group, first row, first column) it moves, in issue order.  Groups are dealt
    round-robin, each group continuing where the previous one stopped."""
    row_blocks = rows_per_shard // push_rows
    ngroups = -(-col_blocks // group_kb)
    per_cta = [[] for _ in range(grid)]
    for cta in range(grid):
        dealt = 0
        for g in range(ngroups):
            cols_g = min(group_kb, col_blocks - g * group_kb)
            boxes_g = cols_g * row_blocks
            start = (cta - dealt % grid + grid) % grid
            dealt += boxes_g
            for b in range(start, boxes_g, grid):
                per_cta[cta].append((g, (b // cols_g) * push_rows, (g * group_kb + b % cols_g) * 64))
    return per_cta
