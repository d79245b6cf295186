"""Tensor-parallel layers: column/row parallel linear, vocab-parallel embedding.

Own implementation of the `neuronx_distributed.parallel_layers` classes the reference builds its
models from (mamba2/mamba2_mixer.py:156-158,186-188; mamba2/modeling_mamba2.py:225,367-376;
mamba2hybrid/mamba2hybrid_attn.py:305-357; mamba2hybrid/mamba2hybrid_mlp.py:79-99).

Conventions (same as the reference's call sites): activations are batch-first `[B, L, D]`, the
sequence dimension is 1, weights are `[out, in]`.  With sequence parallelism the input of a
column-parallel layer is the rank's `[B, L/TP, D]` slice and the output of a row-parallel layer
is reduce-scattered back to that shape.

Initialisation is drawn for the *global* tensor from a seed that depends only on the order of
layer construction and then sliced, so a model is bit-identical for every TP degree.
"""
from __future__ import annotations

import math
from typing import Callable, Optional, Sequence

import torch
import torch.nn as nn

from . import mappings as mp
from . import state as ps
from .. import ops

_INIT_SEED = [1234]
_INIT_COUNTER = [0]


def set_init_seed(seed: int) -> None:
    """Reset the stream of per-layer init seeds (call before building a model)."""
    _INIT_SEED[0] = int(seed)
    _INIT_COUNTER[0] = 0


def _next_generator(device) -> torch.Generator:
    _INIT_COUNTER[0] += 1
    g = torch.Generator(device=device)
    g.manual_seed((_INIT_SEED[0] * 1000003 + _INIT_COUNTER[0] * 7919) % (2 ** 31 - 1))
    return g


def default_linear_init(w: torch.Tensor, generator=None) -> None:
    bound = 1.0 / math.sqrt(w.shape[1])
    w.uniform_(-bound, bound, generator=generator)


def normal_init(std: float) -> Callable:
    def f(w: torch.Tensor, generator=None):
        w.normal_(0.0, std, generator=generator)
    return f


def shard_rows(full: torch.Tensor, segments: Optional[Sequence[int]], rank: int, size: int) -> torch.Tensor:
    """Rows of `full` owned by `rank`: every segment is split evenly, the rank's pieces are
    concatenated in segment order (the `z|x|B|C|dt` layout of mamba2/mamba2_mixer.py:192-206 and
    merge_tp_checkpoints.py:36-65)."""
    if size == 1:
        return full
    if segments is None:
        segments = [full.shape[0]]
    assert sum(segments) == full.shape[0], (segments, full.shape)
    out, off = [], 0
    for s in segments:
        if s % size:
            raise ValueError(f"segment of {s} rows is not divisible by TP size {size}")
        per = s // size
        out.append(full[off + rank * per: off + (rank + 1) * per])
        off += s
    return torch.cat(out, dim=0)


def unshard_rows(shards: Sequence[torch.Tensor], segments: Optional[Sequence[int]]) -> torch.Tensor:
    """Inverse of `shard_rows` over all ranks."""
    size = len(shards)
    if size == 1:
        return shards[0]
    if segments is None:
        return torch.cat(list(shards), dim=0)
    out = []
    off = 0
    for s in segments:
        per = s // size
        for sh in shards:
            out.append(sh[off:off + per])
        off += per
    return torch.cat(out, dim=0)


def _mark(p: nn.Parameter, dim: int, segments=None) -> None:
    p.tensor_model_parallel = True
    p.partition_dim = dim
    p.partition_segments = None if segments is None else tuple(segments)


class ColumnParallelLinear(nn.Module):
    """Y = X W^T with W split along its output rows.

    forward: (SP) all-gather X along the sequence, GEMM -> `[B, L, out/TP]`.
    backward: dX is reduce-scattered (SP) or all-reduced; dW is local.
    `segments` gives the sizes of row blocks of the global weight that are sharded separately.
    """

    def __init__(self, input_size: int, output_size: int, bias: bool = False, gather_output: bool = False,
                 init_method: Optional[Callable] = None, dtype: torch.dtype = torch.float32,
                 sequence_parallel_enabled: bool = False, sequence_dimension: int = 1,
                 segments: Optional[Sequence[int]] = None, device=None, stride: int = 1):
        super().__init__()
        assert sequence_dimension == 1
        tp, r = ps.get_tensor_model_parallel_size(), ps.get_tensor_model_parallel_rank()
        self.input_size, self.output_size = input_size, output_size
        self.gather_output = gather_output
        self.sequence_parallel_enabled = sequence_parallel_enabled and tp > 1
        if segments is None and stride > 1:
            segments = [output_size // stride] * stride
        self.segments = None if segments is None else tuple(segments)
        if output_size % tp:
            raise ValueError(f"output size {output_size} not divisible by TP size {tp}")
        self.output_size_per_partition = output_size // tp
        gen = _next_generator(device if device is not None else "cpu")
        full = torch.empty(output_size, input_size, dtype=torch.float32, device=device)
        (init_method or default_linear_init)(full, generator=gen)
        self.weight = nn.Parameter(shard_rows(full, self.segments, r, tp).to(dtype).contiguous())
        _mark(self.weight, 0, self.segments)
        if bias:
            self.bias = nn.Parameter(torch.zeros(self.output_size_per_partition, dtype=dtype, device=device))
            _mark(self.bias, 0, self.segments)
        else:
            self.register_parameter("bias", None)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.sequence_parallel_enabled:
            from . import fused
            if fused.enabled_for(x):
                y = fused.all_gather_linear(x, self.weight, self.bias)
            else:
                y = ops.linear(mp.gather_from_sequence_parallel_region(x, True), self.weight, self.bias)
        else:
            y = ops.linear(mp.copy_to_tensor_parallel_region(x), self.weight, self.bias)
        if self.gather_output and ps.get_tensor_model_parallel_size() > 1:
            parts = [torch.empty_like(y) for _ in range(ps.get_tensor_model_parallel_size())]
            torch.distributed.all_gather(parts, y.contiguous(), group=ps.get_tensor_model_parallel_group())
            y = torch.cat(parts, dim=-1)
        return y


class RowParallelLinear(nn.Module):
    """Y = X W^T with W split along its input columns; X arrives already split on its last dim.

    forward: GEMM on the local slice -> reduce-scatter along the sequence (SP) or all-reduce.
    backward: all-gather dY (SP); dW local.
    """

    def __init__(self, input_size: int, output_size: int, bias: bool = False, input_is_parallel: bool = True,
                 init_method: Optional[Callable] = None, dtype: torch.dtype = torch.float32,
                 sequence_parallel_enabled: bool = False, sequence_dimension: int = 1, device=None):
        super().__init__()
        assert sequence_dimension == 1 and input_is_parallel
        tp, r = ps.get_tensor_model_parallel_size(), ps.get_tensor_model_parallel_rank()
        if input_size % tp:
            raise ValueError(f"input size {input_size} not divisible by TP size {tp}")
        self.input_size, self.output_size = input_size, output_size
        self.input_size_per_partition = input_size // tp
        self.sequence_parallel_enabled = sequence_parallel_enabled and tp > 1
        gen = _next_generator(device if device is not None else "cpu")
        full = torch.empty(output_size, input_size, dtype=torch.float32, device=device)
        (init_method or default_linear_init)(full, generator=gen)
        per = self.input_size_per_partition
        self.weight = nn.Parameter(full[:, r * per:(r + 1) * per].to(dtype).contiguous())
        _mark(self.weight, 1)
        if bias:
            self.bias = nn.Parameter(torch.zeros(output_size, dtype=dtype, device=device))
            if self.sequence_parallel_enabled:
                self.bias.sequence_parallel_enabled = True
        else:
            self.register_parameter("bias", None)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.sequence_parallel_enabled:
            from . import fused
            if fused.enabled_for(x):
                y = fused.linear_reduce_scatter(x, self.weight)
            else:
                y = mp.reduce_scatter_to_sequence_parallel_region(ops.linear(x, self.weight, None))
        else:
            y = mp.reduce_from_tensor_parallel_region(ops.linear(x, self.weight, None))
        if self.bias is not None:
            y = y + self.bias
        return y


class _VocabParallelLookup(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, weight, vocab_start):
        local = ids - vocab_start
        inside = (local >= 0) & (local < weight.shape[0])
        idx = torch.where(inside, local, torch.zeros_like(local))
        out = weight[idx] * inside[..., None].to(weight.dtype)
        ctx.save_for_backward(idx, inside)
        ctx.shape = weight.shape
        return out

    @staticmethod
    def backward(ctx, g):
        idx, inside = ctx.saved_tensors
        gw = torch.zeros(ctx.shape, dtype=torch.float32, device=g.device)
        gm = (g * inside[..., None].to(g.dtype)).reshape(-1, g.shape[-1]).float()
        gw.index_add_(0, idx.reshape(-1), gm)
        return None, gw.to(g.dtype), None


class ParallelEmbedding(nn.Module):
    """Vocabulary-sharded embedding `[V/TP, D]`; ids outside the shard contribute zeros and the
    partial results are summed over the TP group (all-reduce, or reduce-scatter along the
    sequence when `scatter_to_sequence_parallel` is set, which fuses the reference's
    all-reduce + `scatter_to_sequence_parallel_region`, mamba2/modeling_mamba2.py:276,300-301)."""

    def __init__(self, num_embeddings: int, embedding_dim: int, init_method: Optional[Callable] = None,
                 dtype: torch.dtype = torch.float32, device=None):
        super().__init__()
        tp, r = ps.get_tensor_model_parallel_size(), ps.get_tensor_model_parallel_rank()
        if num_embeddings % tp:
            raise ValueError(f"vocab size {num_embeddings} not divisible by TP size {tp}")
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        per = num_embeddings // tp
        self.vocab_start, self.vocab_end = r * per, (r + 1) * per
        gen = _next_generator(device if device is not None else "cpu")
        full = torch.empty(num_embeddings, embedding_dim, dtype=torch.float32, device=device)
        (init_method or normal_init(1.0))(full, generator=gen)
        self.weight = nn.Parameter(full[self.vocab_start:self.vocab_end].to(dtype).contiguous())
        _mark(self.weight, 0)

    def forward(self, ids: torch.Tensor, scatter_to_sequence_parallel: bool = False) -> torch.Tensor:
        tp = ps.get_tensor_model_parallel_size()
        from .. import ops
        if tp == 1:
            if self.weight.is_cuda:
                return ops.embedding(ids, self.weight, 0)
            return torch.nn.functional.embedding(ids, self.weight)
        if scatter_to_sequence_parallel and self.weight.is_cuda:
            from . import fused
            out = fused.vocab_embed_scatter(ids, self.weight, self.vocab_start)
            if out is not None:
                return out
        if self.weight.is_cuda:
            part = ops.embedding(ids, self.weight, self.vocab_start)
        else:
            part = _VocabParallelLookup.apply(ids, self.weight, self.vocab_start)
        if scatter_to_sequence_parallel:
            return mp.reduce_scatter_to_sequence_parallel_region(part)
        return mp.reduce_from_tensor_parallel_region(part)
