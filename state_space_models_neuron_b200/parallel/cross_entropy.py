"""Vocabulary-parallel cross entropy.

Semantics of `neuronx_distributed.parallel_layers.loss_functions.parallel_cross_entropy` as the
reference uses it (mamba2/modeling_mamba2.py:505-510): logits are `[..., V/TP]` shards, the
per-row maximum, the sum of exponentials and the target logit are combined across the TP group,
the backward pass is (softmax - onehot) on the local shard.  The three reductions of the
reference are packed into two collectives (one MAX, one SUM over a packed [sum-exp, target] pair).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import state as ps
from .. import ops


class _ParallelCrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, labels, vocab_start, ignore_index, m=None, s=None, tgt=None):
        shape = logits.shape
        V = shape[-1]
        lg = logits.reshape(-1, V) if logits.dim() != 2 else logits
        if lg.dim() == 2 and lg.stride(1) != 1:
            lg = lg.contiguous()
        lb = labels.reshape(-1)
        tp, grp = ps.get_tensor_model_parallel_size(), ps.get_tensor_model_parallel_group()
        if m is None:          # statistics not delivered by the producer of the logits: one pass over them here
            m, s, tgt = ops.ce_partials(lg, lb, vocab_start)
        if tp > 1:
            from . import fused
            gm = m.clone()
            if not fused.small_allreduce(gm, "max"):
                dist.all_reduce(gm, op=dist.ReduceOp.MAX, group=grp)
            packed = torch.stack([s * torch.exp(m - gm), tgt], dim=0).contiguous()
            if not fused.small_allreduce(packed.view(-1), "sum"):
                dist.all_reduce(packed, group=grp)
            s, tgt, m = packed[0], packed[1], gm
        valid = lb != ignore_index
        loss = torch.where(valid, torch.log(s) + m - tgt, torch.zeros_like(s))
        ctx.save_for_backward(lg, lb, m, s)
        ctx.vocab_start, ctx.ignore_index, ctx.shape = vocab_start, ignore_index, shape
        return loss.reshape(shape[:-1])

    @staticmethod
    def backward(ctx, g):
        lg, lb, m, s = ctx.saved_tensors
        grad = ops.ce_backward(lg, lb, m, s, g.reshape(-1), ctx.vocab_start, ctx.ignore_index)
        return grad.reshape(ctx.shape), None, None, None, None, None, None


def parallel_cross_entropy(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100,
                           stats=None) -> torch.Tensor:
    """Per-token loss (no reduction) for vocab-sharded logits and global label ids.  `stats` = (row max, row
    sum of exp(x - max), target logit or 0) of the local shard when the GEMM that produced the logits already
    computed them (`ColumnParallelLinear.forward(..., ce_labels=...)`); labels must then be the ones given there."""
    tp, r = ps.get_tensor_model_parallel_size(), ps.get_tensor_model_parallel_rank()
    vocab_start = r * logits.shape[-1] if tp > 1 else 0
    if stats is not None:
        return _ParallelCrossEntropy.apply(logits, labels, vocab_start, ignore_index, *stats)
    return _ParallelCrossEntropy.apply(logits, labels, vocab_start, ignore_index)


@torch.no_grad()
def parallel_argmax(logits: torch.Tensor) -> torch.Tensor:
    """Greedy token over vocabulary-sharded logits `[..., V/TP]`: global index of the maximum (lowest index on
    ties), identical on every TP rank.  Two tiny all-reduces (max of the values, then max of the negated
    candidate index), through the fused small all-reduce when it is available."""
    tp, r = ps.get_tensor_model_parallel_size(), ps.get_tensor_model_parallel_rank()
    val, idx = logits.float().max(dim=-1)
    if tp == 1:
        return idx
    from . import fused
    grp = ps.get_tensor_model_parallel_group()
    shape = val.shape
    gmax = val.reshape(-1).contiguous().clone()
    if not fused.small_allreduce(gmax, "max"):
        dist.all_reduce(gmax, op=dist.ReduceOp.MAX, group=grp)
    cand = torch.where(val.reshape(-1) == gmax, -(idx.reshape(-1) + r * logits.shape[-1]).float(),
                       torch.full_like(gmax, -float(1 << 24))).contiguous()
    if not fused.small_allreduce(cand, "max"):
        dist.all_reduce(cand, op=dist.ReduceOp.MAX, group=grp)
    return (-cand).long().reshape(shape)
