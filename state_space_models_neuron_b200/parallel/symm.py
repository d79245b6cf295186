"""Symmetric (peer-mapped) workspace of a tensor-parallel group.

Every rank allocates the same layout through `torch.distributed._symmetric_memory` and learns the device
addresses of all peers' copies; the fused kernels take those addresses and move data with P2P stores over
NVLink.  Layout (per rank):

    flags    int32 [4 kinds][2 parities][32 slots]     published sequence numbers.  The all-gather kind uses slot
                                                       source * 4 + column group (a shard becomes consumable group
                                                       by group), the other kinds (reduce-scatter, small all-reduce,
                                                       embedding) use slot = source
    gather   2 x [rows_total, cols] bf16              all-gather destinations, alternating by call parity
    land     2 x [nranks][rows_per_owner, cols] bf16  reduce-scatter landing zones, alternating by call parity
    slots    2 x [nranks][n_max] fp32                 small all-reduce staging
    embed    2 x [rows_total / nranks, cols] bf16      vocabulary-parallel embedding landing buffer

Sequence numbers: a call's number is `seq_base` (device, advanced by a kernel once per step, so replays of a
captured CUDA graph publish fresh numbers) plus the call's position in the step (host).  Numbers wrap modulo 2^32;
the kernels compare them by signed distance and the advance kernel keeps idle flags within range.

Double buffering: each kind alternates between two buffers (and flag sets) by its own call counter, which is never
reset.  Two buffers are enough because a rank cannot start call j of a kind before every peer has finished call
j - 1 of that kind: each call needs data that a peer only sends after completing its previous calls.  The one case
the alternation does not cover by itself is a captured CUDA graph, whose calls keep the parities they had at
capture: a replay can end and the next one start on the same buffer of a kind.  `check_replay_safe` verifies for
the recorded calls that some other collective lies between any two such calls.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

KIND_AG, KIND_RS, KIND_AR, KIND_EMB = 0, 1, 2, 3
N_KINDS = 4
MAX_RANKS = 8
AG_GROUPS = 4                      # column groups per shard with a ready flag of their own (all-gather)
FLAG_SLOTS = MAX_RANKS * AG_GROUPS
N_FLAGS = N_KINDS * 2 * FLAG_SLOTS
SMALL_N_MAX = 16384


def _ptr_array(ptrs: List[int]):
    arr = (ctypes.c_void_p * MAX_RANKS)()
    for i, p in enumerate(ptrs):
        arr[i] = p
    return arr


class SeqCounter:
    """Host side of the sequence-number protocol (no device access: testable on CPU)."""

    STEP_STRIDE = 1 << 16    # host positions stay below this; the base is advanced before they reach it

    def __init__(self):
        self.seq = 0
        self.kind_calls = [0] * N_KINDS
        self.recording: Optional[List[Tuple[int, int]]] = None

    def take(self, kind: int) -> Tuple[int, int, bool]:
        """(position of this call in the current block, parity of the kind's double buffer, advance_first).
        `advance_first`: the caller must advance the device base before using the position (the block is full)."""
        advance = self.seq + 1 >= self.STEP_STRIDE - 2
        if advance:
            self.seq = 0
        self.seq += 1
        par = self.kind_calls[kind] & 1
        self.kind_calls[kind] += 1
        if self.recording is not None:
            self.recording.append((kind, par))
        return self.seq, par, advance

    def advance_amount(self, compact: bool) -> int:
        """Amount to add to the device base: a full stride, or (compact) just past the positions used, kept even."""
        amount = (self.seq + 2) // 2 * 2 if compact else self.STEP_STRIDE
        self.seq = 0
        return amount


def check_replay_safe(calls: List[Tuple[int, int]]) -> None:
    """`calls`: (kind, buffer parity) of fused calls in the order in which captured graphs will replay them (for a
    graph that is replayed back to back: its recording twice).  Two consecutive calls of a kind on the same buffer
    are only safe if another collective lies between them (a rank passes a collective only after every peer has
    finished everything before it, so the buffer's previous readers are done); raise otherwise."""
    last = {}
    for i, (kind, par) in enumerate(calls):
        if kind in last:
            j, prev_par = last[kind]
            if prev_par == par and i == j + 1:
                raise RuntimeError(f"fused calls {j} and {i} of kind {kind} would use the same buffer back to back: a "
                                   "replay could overwrite data that peers still read")
        last[kind] = (i, par)


class SymmWorkspace(SeqCounter):
    def __init__(self, group, nranks: int, me: int, rows_total: int, cols: int, device):
        import torch.distributed._symmetric_memory as symm_mem
        super().__init__()
        if nranks > MAX_RANKS:
            raise ValueError(f"fused collectives support up to {MAX_RANKS} ranks per TP group")
        self.group, self.nranks, self.me = group, nranks, me
        self.rows_total, self.cols = rows_total, cols
        self.device = torch.device(device)
        elems = rows_total * cols
        self.gather_bytes = (elems * 2 + 1023) // 1024 * 1024
        self.flags_bytes = 4096
        assert N_FLAGS * 4 <= self.flags_bytes
        self.slots_bytes = 2 * MAX_RANKS * SMALL_N_MAX * 4
        self.embed_bytes = (-(-elems // nranks) * 2 + 1023) // 1024 * 1024
        total = self.flags_bytes + 4 * self.gather_bytes + self.slots_bytes + 2 * self.embed_bytes
        self.buf = symm_mem.empty(total, dtype=torch.uint8, device=self.device)
        self.handle = symm_mem.rendezvous(self.buf, group)
        self.base_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.buf.zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)
        self.counters = torch.zeros(64, dtype=torch.int32, device=self.device)   # local, not shared
        self.seq_base = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.flag_ptr_array = _ptr_array(self.base_ptrs)
        self._keep = []

    # ---- addresses -------------------------------------------------------------------------
    def flag_base(self, kind: int, parity: int) -> int:
        return (kind * 2 + parity) * FLAG_SLOTS

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

    def local_ptr(self, byte_offset: int) -> int:
        return self.base_ptrs[self.me] + byte_offset

    def local_view(self, byte_offset: int, rows: int, cols: int, dtype=torch.bfloat16) -> torch.Tensor:
        n = rows * cols * torch.empty((), dtype=dtype).element_size()
        return self.buf[byte_offset:byte_offset + n].view(dtype).view(rows, cols)

    def fits(self, rows: int, cols: int) -> bool:
        return rows * cols <= self.rows_total * self.cols

    # ---- sequence numbers ------------------------------------------------------------------
    def next_seq(self, kind: int) -> Tuple[int, int]:
        """(sequence position, buffer parity) of the next fused call of `kind`.  Long runs of calls without an
        optimizer step (gradient accumulation over many micro-steps) advance the base on their own; every rank
        makes the same calls in the same order, so all ranks do this at the same call."""
        seq, par, advance = self.take(kind)
        if advance:
            self._advance_device(self.STEP_STRIDE)
        return seq, par

    def _advance_device(self, amount: int) -> None:
        from ..ops.cuda_ops import _P, _run, _st
        _run("ssm_advance_counter", _P(self.seq_base), int(amount), ctypes.c_void_p(self.base_ptrs[self.me]), N_FLAGS,
             _st())

    def advance_step(self, compact: bool = False) -> None:
        """Start a new block of sequence numbers: bump the device-side base (a kernel on the current stream, so it
        is captured into CUDA graphs) and restart the host-side position.  `compact` advances by the number of
        calls actually made instead of a full stride: for callers that advance very often (one decode token, one
        graph replay per micro-step)."""
        self._advance_device(self.advance_amount(compact))

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


def start_recording() -> None:
    """Begin recording (kind, buffer parity) of the fused calls (used while a step is captured into a CUDA graph)."""
    if _WS is not None:
        _WS.recording = []


def stop_recording() -> List[Tuple[int, int]]:
    if _WS is None or _WS.recording is None:
        return []
    rec, _WS.recording = _WS.recording, None
    return rec


def reset_workspace() -> None:
    global _WS
    _WS = None
