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

    def forward(self, x: torch.Tensor, ce_labels: Optional[torch.Tensor] = None):
        """`ce_labels` (global ids, one per output row of the full sequence; negative = ignored) turns the layer into
        an LM head that also returns the cross-entropy statistics of its logits, taken in the GEMM epilogue where
        the kernels support it: the result is then `(y, statistics or None)`."""
        if ce_labels is not None:
            if self.bias is not None or self.gather_output:
                raise ValueError("cross-entropy statistics need a bias-free layer without gathered output")
            vocab_start = ps.get_tensor_model_parallel_rank() * self.output_size_per_partition
            if self.sequence_parallel_enabled:
                from . import fused
                if fused.enabled_for(x):
                    return fused.all_gather_linear(x, self.weight, None, ce=(ce_labels, vocab_start))
                xg = mp.gather_from_sequence_parallel_region(x, True)
            else:
                xg = mp.copy_to_tensor_parallel_region(x)
            return ops.linear_ce(xg, self.weight, ce_labels, vocab_start)
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


class _ReplicaGradSync(torch.autograd.Function):
    """Identity whose gradient is summed over the ranks that hold copies of the same weight rows."""

    @staticmethod
    def forward(ctx, w, group):
        ctx.group = group
        return w.view_as(w)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        torch.distributed.all_reduce(g, group=ctx.group)
        return g, None


_KV_REPLICA_GROUPS = {}


def _kv_replica_group(multiplier: int):
    """Process group of the `multiplier` consecutive TP ranks that share one replicated KV head block.  Created
    collectively (every rank creates every group, in the same order) on first use."""
    if multiplier == 1 or not torch.distributed.is_initialized():
        return None
    key = (multiplier, id(ps.get_tensor_model_parallel_group()))
    if key not in _KV_REPLICA_GROUPS:
        world = torch.distributed.get_world_size()
        tp = ps.get_tensor_model_parallel_size()
        mine = None
        for base in range(0, world, tp):                 # every TP group of the job
            for j in range(0, tp, multiplier):
                ranks = list(range(base + j, base + j + multiplier))
                grp = torch.distributed.new_group(ranks)
                if torch.distributed.get_rank() in ranks:
                    mine = grp
        _KV_REPLICA_GROUPS[key] = mine
    return _KV_REPLICA_GROUPS[key]


class GQAQKVColumnParallelLinear(nn.Module):
    """Query / key / value projections of grouped-query attention as one column-parallel layer that returns
    `(q, k, v)` (neuronx-distributed's GQAQKVColumnParallelLinear as the reference would use it when
    `config.qkv_linear` is set, mamba2hybrid/mamba2hybrid_attn.py:291-303; the hybrid presets leave it off).

    `output_sizes = [q_size, kv_size]`.  Parameters: `weight_q [q_size/TP, in]`, `weight_k`, `weight_v`
    `[kv_size * kv_size_multiplier / TP, in]`.  `kv_size_multiplier` > 1 replicates every KV head that many times
    (adjacent copies, so query head h still meets the copy of its original KV head) which lets TP exceed the number
    of KV heads; the copies start equal and stay equal because their gradients are summed over the ranks that hold
    them.  All three projections share one sequence all-gather (the fused all-gather GEMM on the GPU path)."""

    def __init__(self, input_size: int, output_sizes: Sequence[int], bias: bool = False, gather_output: bool = False,
                 init_method: Optional[Callable] = None, dtype: torch.dtype = torch.float32,
                 sequence_parallel_enabled: bool = False, sequence_dimension: int = 1, kv_size_multiplier: int = 1,
                 fuse_qkv: bool = False, head_dim: Optional[int] = None, device=None):
        super().__init__()
        assert sequence_dimension == 1 and not gather_output
        tp, r = ps.get_tensor_model_parallel_size(), ps.get_tensor_model_parallel_rank()
        q_size, kv_size = int(output_sizes[0]), int(output_sizes[1])
        m = int(kv_size_multiplier)
        if q_size % tp or (kv_size * m) % tp:
            raise ValueError("q size and kv size * kv_size_multiplier must be divisible by the TP size")
        if m > 1 and (tp % m or head_dim is None or kv_size % head_dim):
            raise ValueError("kv_size_multiplier > 1 needs head_dim and a TP size that is a multiple of it")
        self.input_size, self.q_size, self.kv_size, self.kv_size_multiplier = input_size, q_size, kv_size, m
        self.sequence_parallel_enabled = sequence_parallel_enabled and tp > 1
        self.fuse_qkv = fuse_qkv       # accepted for API parity; the three GEMMs already share the all-gather
        init = init_method or default_linear_init
        gen = _next_generator(device if device is not None else "cpu")

        def make(rows, replicate):
            full = torch.empty(rows, input_size, dtype=torch.float32, device=device)
            init(full, generator=gen)
            if replicate > 1:      # copy whole heads, copies adjacent
                full = full.view(rows // head_dim, 1, head_dim, input_size).expand(-1, replicate, -1, -1) \
                           .reshape(rows * replicate, input_size)
            p = nn.Parameter(shard_rows(full, None, r, tp).to(dtype).contiguous())
            _mark(p, 0)
            return p

        self.weight_q = make(q_size, 1)
        self.weight_k = make(kv_size, m)
        self.weight_v = make(kv_size, m)
        if bias:
            self.bias_q = nn.Parameter(torch.zeros(self.weight_q.shape[0], dtype=dtype, device=device))
            self.bias_k = nn.Parameter(torch.zeros(self.weight_k.shape[0], dtype=dtype, device=device))
            self.bias_v = nn.Parameter(torch.zeros(self.weight_v.shape[0], dtype=dtype, device=device))
            for b in (self.bias_q, self.bias_k, self.bias_v):
                _mark(b, 0)
        else:
            self.bias_q = self.bias_k = self.bias_v = None
        self._replica_group = _kv_replica_group(m) if tp > 1 else None

    def forward(self, x: torch.Tensor):
        wq, wk, wv = self.weight_q, self.weight_k, self.weight_v
        bk, bv = self.bias_k, self.bias_v
        if self._replica_group is not None:
            wk, wv = _ReplicaGradSync.apply(wk, self._replica_group), _ReplicaGradSync.apply(wv, self._replica_group)
            if bk is not None:
                bk, bv = _ReplicaGradSync.apply(bk, self._replica_group), _ReplicaGradSync.apply(bv, self._replica_group)
        if self.sequence_parallel_enabled:
            from . import fused
            if self.bias_q is None and self._replica_group is None and fused.enabled_for(x):
                out = fused.all_gather_multi_linear(x, (wq, wk, wv))
                if out is not None:
                    return out
            xg = mp.gather_from_sequence_parallel_region(x, True)
        else:
            xg = mp.copy_to_tensor_parallel_region(x)
        return ops.linear(xg, wq, self.bias_q), ops.linear(xg, wk, bk), ops.linear(xg, wv, bv)


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
        # the embedding gradient is scatter-added (and, when tied, lands on top of the LM head's): its share of the
        # gradient norm is always taken from the buffer, never from a GEMM epilogue
        self.weight.no_norm_tracking = True

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
