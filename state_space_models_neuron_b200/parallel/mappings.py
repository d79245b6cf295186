"""Differentiable tensor-/sequence-parallel region mappings (library collectives).

This is the NCCL (or gloo on CPU ranks) implementation of the mappings the reference gets from
`neuronx_distributed.parallel_layers.mappings` (mamba2/modeling_mamba2.py:300-301,
mamba2hybrid/modeling_mamba2hybrid.py:417-418) and of the collectives implied by its column/row
parallel layers with `sequence_dimension=1` (mamba2/mamba2_mixer.py:156-158,186-188).  Activations
are batch-first, the sequence dimension is 1.  The kernels in `parallel/fused.py` replace the
collective+GEMM pairs on GPUs; these functions stay as the baseline and as the CPU-rank path.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import state as ps

SEQ_DIM = 1


def _tp():
    return ps.get_tensor_model_parallel_size(), ps.get_tensor_model_parallel_group()


def all_reduce_tp(x: torch.Tensor) -> torch.Tensor:
    n, g = _tp()
    if n > 1:
        dist.all_reduce(x, group=g)
    return x


def all_gather_seq(x: torch.Tensor) -> torch.Tensor:
    n, g = _tp()
    if n == 1:
        return x
    x = x.contiguous()
    if x.shape[0] == 1 and dist.get_backend(g) != "gloo":       # batch 1: the gathered tensor is one flat buffer
        out = torch.empty(1, n * x.shape[1], *x.shape[2:], dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x, group=g)
        return out
    parts = [torch.empty_like(x) for _ in range(n)]
    dist.all_gather(parts, x, group=g)
    return torch.cat(parts, dim=SEQ_DIM)


def reduce_scatter_seq(x: torch.Tensor) -> torch.Tensor:
    n, g = _tp()
    if n == 1:
        return x
    if x.shape[SEQ_DIM] % n:
        raise ValueError(f"sequence length {x.shape[SEQ_DIM]} is not divisible by TP size {n}")
    if x.shape[0] == 1 and dist.get_backend(g) != "gloo":
        x = x.contiguous()
        out = torch.empty(1, x.shape[1] // n, *x.shape[2:], dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x, group=g)
        return out
    parts = [p.contiguous() for p in x.chunk(n, dim=SEQ_DIM)]
    out = torch.empty_like(parts[0])
    if dist.get_backend(g) == "gloo":
        # gloo has no reduce_scatter: all-reduce then slice
        full = x.contiguous().clone()
        dist.all_reduce(full, group=g)
        return full.chunk(n, dim=SEQ_DIM)[ps.get_tensor_model_parallel_rank()].contiguous()
    dist.reduce_scatter(out, parts, group=g)
    return out


def split_seq(x: torch.Tensor) -> torch.Tensor:
    n, _ = _tp()
    if n == 1:
        return x
    if x.shape[SEQ_DIM] % n:
        raise ValueError(f"sequence length {x.shape[SEQ_DIM]} is not divisible by TP size {n}")
    return x.chunk(n, dim=SEQ_DIM)[ps.get_tensor_model_parallel_rank()].contiguous()


class _CopyToTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return x

    @staticmethod
    def backward(ctx, g):
        return all_reduce_tp(g.contiguous().clone())


class _ReduceFromTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return all_reduce_tp(x.contiguous().clone())

    @staticmethod
    def backward(ctx, g):
        return g


class _ScatterToSP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return split_seq(x)

    @staticmethod
    def backward(ctx, g):
        return all_gather_seq(g)


class _GatherFromSP(torch.autograd.Function):
    """all-gather along the sequence; gradient is reduce-scattered (the input feeds a
    column-parallel GEMM, so every rank holds a partial sum of dX)."""

    @staticmethod
    def forward(ctx, x, reduce_grad):
        ctx.reduce_grad = reduce_grad
        return all_gather_seq(x)

    @staticmethod
    def backward(ctx, g):
        if ctx.reduce_grad:
            return reduce_scatter_seq(g), None
        return split_seq(g), None


class _ReduceScatterToSP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return reduce_scatter_seq(x)

    @staticmethod
    def backward(ctx, g):
        return all_gather_seq(g)


def copy_to_tensor_parallel_region(x):
    return x if ps.get_tensor_model_parallel_size() == 1 else _CopyToTP.apply(x)


def reduce_from_tensor_parallel_region(x):
    if ps.get_tensor_model_parallel_size() == 1:
        return x
    if x.is_cuda and not (torch.is_grad_enabled() and x.requires_grad):
        from . import fused
        y = fused.allreduce_bf16(x)
        if y is not None:
            return y
    return _ReduceFromTP.apply(x)


def scatter_to_sequence_parallel_region(x, dim: int = SEQ_DIM):
    assert dim == SEQ_DIM, "activations are batch-first; the sequence dimension is 1"
    return x if ps.get_tensor_model_parallel_size() == 1 else _ScatterToSP.apply(x)


def gather_from_sequence_parallel_region(x, reduce_grad: bool = True):
    return x if ps.get_tensor_model_parallel_size() == 1 else _GatherFromSP.apply(x, reduce_grad)


def reduce_scatter_to_sequence_parallel_region(x):
    return x if ps.get_tensor_model_parallel_size() == 1 else _ReduceScatterToSP.apply(x)
