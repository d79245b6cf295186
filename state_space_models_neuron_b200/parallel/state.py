"""Process-group bookkeeping: world = data-parallel x tensor-parallel, TP ranks contiguous.

Replaces the `neuronx_distributed.parallel_layers.parallel_state` surface the reference calls
(mamba2/mamba2_mixer.py:64-65,193-194; mamba2/conv1d_grouped.py:324-325; train.py:80,86-87,150-151;
mamba2hybrid/mamba2hybrid_attn.py:358-362).  Works without torch.distributed (single process:
TP=DP=1) so models can be built and run on one device with no launcher.
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass, field
from typing import List, Optional

import torch
import torch.distributed as dist


@dataclass
class _State:
    initialized: bool = False
    tp_size: int = 1
    dp_size: int = 1
    tp_rank: int = 0
    dp_rank: int = 0
    world_size: int = 1
    rank: int = 0
    tp_group: Optional[object] = None
    dp_group: Optional[object] = None
    tp_ranks: List[List[int]] = field(default_factory=lambda: [[0]])
    dp_ranks: List[List[int]] = field(default_factory=lambda: [[0]])


_S = _State()


def initialize_model_parallel(tensor_model_parallel_size: int = 1, backend: Optional[str] = None,
                              timeout_s: Optional[float] = None) -> None:
    """Create TP and DP groups.  TP group i holds ranks [i*tp, (i+1)*tp); DP group j holds
    ranks {j, j+tp, j+2tp, ...}.  Calls dist.init_process_group from the torchrun environment
    when the default group does not exist yet and WORLD_SIZE > 1."""
    global _S
    tp = int(tensor_model_parallel_size)
    env_world = int(os.environ.get("WORLD_SIZE", "1"))
    if not dist.is_initialized() and env_world > 1:
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        kw = {}
        if timeout_s is not None:
            kw["timeout"] = datetime.timedelta(seconds=timeout_s)
        if backend == "nccl":
            local = int(os.environ.get("LOCAL_RANK", "0"))
            torch.cuda.set_device(local)
            kw["device_id"] = torch.device("cuda", local)
        dist.init_process_group(backend=backend, **kw)
    if dist.is_initialized():
        world, rank = dist.get_world_size(), dist.get_rank()
    else:
        world, rank = 1, 0
    if world % tp != 0:
        raise ValueError(f"world size {world} is not divisible by tensor parallel size {tp}")
    dp = world // tp
    st = _State(initialized=True, tp_size=tp, dp_size=dp, world_size=world, rank=rank,
                tp_rank=rank % tp, dp_rank=rank // tp)
    st.tp_ranks = [list(range(i * tp, (i + 1) * tp)) for i in range(dp)]
    st.dp_ranks = [list(range(j, world, tp)) for j in range(tp)]
    if dist.is_initialized() and world > 1:
        kw = {}
        if timeout_s is not None:
            kw["timeout"] = datetime.timedelta(seconds=timeout_s)
        for ranks in st.tp_ranks:
            g = dist.new_group(ranks, **kw) if tp > 1 else None
            if rank in ranks:
                st.tp_group = g
        for ranks in st.dp_ranks:
            g = dist.new_group(ranks, **kw) if dp > 1 else None
            if rank in ranks:
                st.dp_group = g
    _S = st


def destroy_model_parallel() -> None:
    global _S
    _S = _State()


def model_parallel_is_initialized() -> bool:
    return _S.initialized


def get_tensor_model_parallel_size() -> int:
    return _S.tp_size


def get_tensor_model_parallel_rank() -> int:
    return _S.tp_rank


def get_data_parallel_size() -> int:
    return _S.dp_size


def get_data_parallel_rank() -> int:
    return _S.dp_rank


def get_tensor_model_parallel_group(as_list: bool = False):
    return _S.tp_ranks if as_list else _S.tp_group


def get_data_parallel_group(as_list: bool = False):
    return _S.dp_ranks if as_list else _S.dp_group


def get_world_size() -> int:
    return _S.world_size


def get_rank() -> int:
    return _S.rank


def is_master() -> bool:
    return _S.rank == 0


def barrier() -> None:
    if dist.is_initialized() and _S.world_size > 1:
        dist.barrier()
