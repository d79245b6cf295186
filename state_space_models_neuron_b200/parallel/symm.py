"""Symmetric (peer-mapped) workspace of a tensor-parallel group.

Every rank allocates the same layout through `torch.distributed._symmetric_memory` and learns the device
addresses of all peers' copies; the fused kernels take those addresses and move data with P2P stores over
NVLink.  Layout (per rank):

    flags    int32 [4 kinds][2 parities][8 sources]   published sequence numbers (all-gather, reduce-scatter,
                                                       small all-reduce, embedding); monotonically increasing
    gather   2 x [rows_total, cols] bf16              all-gather destinations, alternating by call parity
    land     2 x [nranks][rows_per_owner, cols] bf16  reduce-scatter landing zones, alternating by call parity
    slots    2 x [nranks][n_max] fp32                 small all-reduce staging
    embed    2 x [rows_total / nranks, cols] bf16      vocabulary-parallel embedding landing buffer

Two alternating buffers are enough because a rank can be at most one fused call of a kind ahead of its peers:
each call needs data that every peer only produces after finishing its own previous call of that kind.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

KIND_AG, KIND_RS, KIND_AR, KIND_EMB = 0, 1, 2, 3
MAX_RANKS = 8
SMALL_N_MAX = 16384


def _ptr_array(ptrs: List[int]):
    arr = (ctypes.c_void_p * MAX_RANKS)()
    for i, p in enumerate(ptrs):
        arr[i] = p
    return arr


class SymmWorkspace:
    def __init__(self, group, nranks: int, me: int, rows_total: int, cols: int, device):
        import torch.distributed._symmetric_memory as symm_mem
        if nranks > MAX_RANKS:
            raise ValueError(f"fused collectives support up to {MAX_RANKS} ranks per TP group")
        self.group, self.nranks, self.me = group, nranks, me
        self.rows_total, self.cols = rows_total, cols
        self.device = torch.device(device)
        self.seq = 0
        elems = rows_total * cols
        self.gather_bytes = elems * 2
        self.flags_bytes = 4096
        self.slots_bytes = 2 * MAX_RANKS * SMALL_N_MAX * 4
        self.embed_bytes = (-(-elems // nranks) * 2 + 255) // 256 * 256
        total = self.flags_bytes + 4 * self.gather_bytes + self.slots_bytes + 2 * self.embed_bytes
        self.buf = symm_mem.empty(total, dtype=torch.uint8, device=self.device)
        self.handle = symm_mem.rendezvous(self.buf, group)
        self.base_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.buf.zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)
        self.counters = torch.zeros(64, dtype=torch.int32, device=self.device)   # local, not shared
        # sequence number of a fused call = seq_base (device, advanced once per training step) + its position in
        # the step (host); the device part keeps the numbers growing when a captured CUDA graph is replayed
        self.seq_base = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.flag_ptr_array = _ptr_array(self.base_ptrs)
        self._keep = []

    # ---- addresses -------------------------------------------------------------------------
    def flag_base(self, kind: int, parity: int) -> int:
        return (kind * 2 + parity) * MAX_RANKS

    def gather_offset(self, parity: int) -> int:
        return self.flags_bytes + parity * self.gather_bytes

    def land_offset(self, parity: int) -> int:
        return self.flags_bytes + (2 + parity) * self.gather_bytes

    def slots_offset(self, parity: int) -> int:
        return self.flags_bytes + 4 * self.gather_bytes + parity * MAX_RANKS * SMALL_N_MAX * 4

    def embed_offset(self, parity: int) -> int:
        return self.flags_bytes + 4 * self.gather_bytes + self.slots_bytes + parity * self.embed_bytes

    def peer_ptrs(self, byte_offset: int):
        return _ptr_array([p + byte_offset for p in self.base_ptrs])

    def local_view(self, byte_offset: int, rows: int, cols: int, dtype=torch.bfloat16) -> torch.Tensor:
        n = rows * cols * torch.empty((), dtype=dtype).element_size()
        return self.buf[byte_offset:byte_offset + n].view(dtype).view(rows, cols)

    def fits(self, rows: int, cols: int) -> bool:
        return rows * cols <= self.rows_total * self.cols

    STEP_STRIDE = 1 << 16    # host positions stay below this; the base is advanced before they reach it

    def next_seq(self) -> int:
        """Position of the next fused call since the last advance (parity selects the double buffers).  Long runs
        of calls without an optimizer step (gradient accumulation over many micro-steps) advance the base on their
        own; every rank makes the same calls in the same order, so all ranks do this at the same call."""
        if self.seq + 1 >= self.STEP_STRIDE - 2:
            self.advance_step()
        self.seq += 1
        return self.seq

    def advance_step(self, compact: bool = False) -> None:
        """Start a new block of sequence numbers: bump the device-side base by STEP_STRIDE (a kernel on the current
        stream, so it is captured into CUDA graphs) and restart the host-side position.  The numbers are 31-bit:
        32767 advances (optimizer steps, plus one per ~65k fused calls under gradient accumulation) fit before
        they would wrap; a wrap-safe comparison in the waiting kernels is the planned follow-up.
        `compact` advances by the number of calls actually made (rounded up to even) instead: for callers that
        advance very often (one graph replay per micro-step)."""
        from ..ops.cuda_ops import _P, _run, _st
        amount = (self.seq + 2) // 2 * 2 if compact else self.STEP_STRIDE
        _run("ssm_advance_counter", _P(self.seq_base), amount, _st())
        self.seq = 0
        self.advances = getattr(self, "advances", 0) + 1
        if self.advances == 30000:
            import warnings
            warnings.warn("fused-collective sequence numbers are close to their 31-bit limit; restart the job from a "
                          "checkpoint before ~32000 advances")

    def counter_ptr(self, index: int) -> int:
        return self.counters.data_ptr() + 4 * index


_WS: Optional[SymmWorkspace] = None


def get_workspace(rows_total: int, cols: int, device) -> Optional[SymmWorkspace]:
    """Workspace of the current TP group, created on first use (collective: all ranks of the group must call
    this at the same point of the program)."""
    global _WS
    from . import state as ps
    if _WS is not None and _WS.group is ps.get_tensor_model_parallel_group() and _WS.fits(rows_total, cols):
        return _WS
    if _WS is not None and _WS.group is ps.get_tensor_model_parallel_group():
        return None   # does not fit: caller falls back to library collectives
    _WS = SymmWorkspace(ps.get_tensor_model_parallel_group(), ps.get_tensor_model_parallel_size(),
                        ps.get_tensor_model_parallel_rank(), rows_total, cols, device)
    return _WS


def advance_step(compact: bool = False) -> None:
    if _WS is not None:
        _WS.advance_step(compact)


def reset_workspace() -> None:
    global _WS
    _WS = None
