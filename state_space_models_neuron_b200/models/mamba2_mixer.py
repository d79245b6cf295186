"""Mamba-2 mixer block: in_proj -> conv/SiLU -> SSD scan -> gated norm -> out_proj.

Parameter names, shapes and the tensor-parallel slicing follow the reference
(mamba2/mamba2_mixer.py:116-206, mamba2/conv1d_grouped.py:295-334): `in_proj.weight` rows are
`z | x | B | C | dt`, `conv1d.weight` rows `x | B | C`, each block sharded separately; heads,
groups and `A_log/D/dt_bias/norm.weight` are sliced by TP rank.  Unlike the reference the full
forward also works in eval mode, with batch > 1, and can hand its final conv/SSM state to the
decode path.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn

from .. import ops
from ..parallel import state as ps
from ..parallel.layers import (ColumnParallelLinear, RowParallelLinear, _mark, _next_generator, shard_rows)
from .cache import Mamba2Cache


class MambaRMSNormGated(nn.Module):
    """Gated RMSNorm weight holder (mamba2/mamba2_mixer.py:45-105).

    `rmsnorm_within_groups=True` normalises each of the rank's `n_groups/TP` groups on its own;
    False normalises over the rank-local `d_inner/TP` slice (no collective), which is what the
    reference's training kernel does when n_groups == TP (mamba2/fused_kernel.py:255,280).
    """

    def __init__(self, d: int, eps: float = 1e-5, n_groups: int = 1, rmsnorm_within_groups: bool = True,
                 dtype=torch.float32, device=None):
        super().__init__()
        tp, r = ps.get_tensor_model_parallel_size(), ps.get_tensor_model_parallel_rank()
        assert d % tp == 0 and n_groups % tp == 0
        self.eps = eps
        self.d_local = d // tp
        self.n_groups_local = n_groups // tp
        self.rmsnorm_within_groups = rmsnorm_within_groups
        self.weight = nn.Parameter(torch.ones(self.d_local, dtype=dtype, device=device))
        _mark(self.weight, 0)

    @property
    def group_size(self) -> int:
        return self.d_local // self.n_groups_local if self.rmsnorm_within_groups else self.d_local

    def forward(self, hidden_states, gate=None):
        return ops.gated_rmsnorm(hidden_states, gate, self.weight, self.eps, self.group_size)


class DepthwiseConv1d(nn.Module):
    """Parameters of the causal depthwise conv, `weight [C/TP, 1, K]`, `bias [C/TP]`, initialised
    like `nn.Conv1d` on the global tensor and sliced per `x | B | C` block
    (mamba2/conv1d_grouped.py:318-331)."""

    def __init__(self, channels: int, kernel_size: int, bias: bool, segments, dtype=torch.float32, device=None):
        super().__init__()
        tp, r = ps.get_tensor_model_parallel_size(), ps.get_tensor_model_parallel_rank()
        gen = _next_generator(device if device is not None else "cpu")
        bound = 1.0 / math.sqrt(kernel_size)
        w = torch.empty(channels, 1, kernel_size, dtype=torch.float32, device=device).uniform_(-bound, bound, generator=gen)
        self.weight = nn.Parameter(shard_rows(w, segments, r, tp).to(dtype).contiguous())
        _mark(self.weight, 0, segments)
        if bias:
            b = torch.empty(channels, dtype=torch.float32, device=device).uniform_(-bound, bound, generator=gen)
            self.bias = nn.Parameter(shard_rows(b, segments, r, tp).to(dtype).contiguous())
            _mark(self.bias, 0, segments)
        else:
            self.register_parameter("bias", None)
        self.kernel_size = kernel_size


class Mamba2Mixer(nn.Module):
    def __init__(self, config, layer_idx: int, device=None):
        super().__init__()
        tp, r = ps.get_tensor_model_parallel_size(), ps.get_tensor_model_parallel_rank()
        self.config = config
        self.layer_idx = layer_idx
        self.hidden_size = config.hidden_size
        self.num_heads = config.num_heads
        self.head_dim = config.head_dim
        self.ssm_state_size = config.state_size
        self.n_groups = config.n_groups
        self.conv_kernel_size = config.conv_kernel
        self.intermediate_size = int(config.expand * config.hidden_size)
        self.chunk_size = 128  # kernels are written for 128-token chunks (mamba2/mamba2_kernel.py:78)
        self.layer_norm_epsilon = config.layer_norm_epsilon
        if self.intermediate_size != self.num_heads * self.head_dim:
            raise ValueError("expand * hidden_size must equal num_heads * head_dim")
        if self.intermediate_size % tp or self.n_groups % tp or self.num_heads % tp:
            raise ValueError("d_inner, n_groups and num_heads must be divisible by the TP size")
        if config.hidden_act not in ("silu", "swish"):
            raise ValueError("only SiLU activation is supported")
        gn = self.n_groups * self.ssm_state_size
        self.conv_dim = self.intermediate_size + 2 * gn
        self.intermediate_size_tp = self.intermediate_size // tp
        self.n_groups_tp = self.n_groups // tp
        self.num_heads_tp = self.num_heads // tp
        self.conv_dim_tp = self.conv_dim // tp
        dtype = config.dtype or torch.float32

        self.conv1d = DepthwiseConv1d(self.conv_dim, config.conv_kernel, config.use_conv_bias,
                                      segments=(self.intermediate_size, gn, gn), dtype=dtype, device=device)
        self.in_proj = ColumnParallelLinear(
            self.hidden_size, self.intermediate_size + self.conv_dim + self.num_heads, bias=config.use_bias,
            dtype=dtype, sequence_parallel_enabled=config.sequence_parallel_enabled, device=device,
            segments=(self.intermediate_size, self.intermediate_size, gn, gn, self.num_heads))

        gen = _next_generator(device if device is not None else "cpu")
        u = torch.rand(self.num_heads, generator=gen, device=device)
        dt = torch.exp(u * (math.log(config.time_step_max) - math.log(config.time_step_min))
                       + math.log(config.time_step_min)).clamp(min=config.time_step_floor)
        heads = slice(self.num_heads_tp * r, self.num_heads_tp * (r + 1))
        self.dt_bias = nn.Parameter(ops.oracle.inverse_softplus(dt)[heads].clone())
        self.dt_bias._no_reinit = True
        if getattr(config, "a_log_init", "arange") == "uniform":
            A = torch.empty(self.num_heads, device=device).uniform_(1.0, 16.0, generator=gen)
        else:
            A = torch.arange(1, self.num_heads + 1, dtype=torch.float32, device=device)
        self.A_log = nn.Parameter(torch.log(A)[heads].clone())
        self.A_log._no_weight_decay = True
        self.D = nn.Parameter(torch.ones(self.num_heads_tp, device=device))
        self.D._no_weight_decay = True
        for p in (self.dt_bias, self.A_log, self.D):
            _mark(p, 0)
        self.norm = MambaRMSNormGated(self.intermediate_size, eps=self.layer_norm_epsilon, n_groups=self.n_groups,
                                      rmsnorm_within_groups=config.rmsnorm_within_groups, dtype=dtype, device=device)
        out_init = None
        if getattr(config, "rescale_prenorm_residual", False):
            # GPT-2 style: residual-branch output projections are drawn as usual and scaled by 1/sqrt(n_layers)
            # (mamba2/modeling_mamba2.py:172-187 of the reference)
            from ..parallel.layers import default_linear_init
            scale = 1.0 / math.sqrt(config.num_hidden_layers)

            def out_init(w, generator=None):
                default_linear_init(w, generator=generator)
                w.mul_(scale)
        self.out_proj = RowParallelLinear(self.intermediate_size, self.hidden_size, bias=config.use_bias,
                                          init_method=out_init, dtype=dtype,
                                          sequence_parallel_enabled=config.sequence_parallel_enabled, device=device)

    def _core_kwargs(self):
        return dict(d_inner=self.intermediate_size_tp, n_groups=self.n_groups_tp, d_state=self.ssm_state_size,
                    head_dim=self.head_dim, eps=self.layer_norm_epsilon, norm_group_size=self.norm.group_size)

    def forward(self, hidden_states: torch.Tensor, cache_params: Optional[Mamba2Cache] = None,
                cache_position=None, attention_mask=None) -> torch.Tensor:
        """Full-sequence path.  With `cache_params` the final conv window and SSM state are stored
        in the cache (prefill), ready for `step`."""
        if attention_mask is not None:
            raise NotImplementedError("attention masks are not supported; left-pad to a chunk multiple")
        zxBCdt = self.in_proj(hidden_states)
        if zxBCdt.shape[1] % self.chunk_size:
            raise ValueError(f"sequence length {zxBCdt.shape[1]} must be a multiple of {self.chunk_size}")
        kw = self._core_kwargs()
        if cache_params is not None:
            y, (conv_state, ssm_state) = ops.mamba2_mixer_core(
                zxBCdt, self.conv1d.weight, self.conv1d.bias, self.dt_bias, self.A_log, self.D, self.norm.weight,
                chunk_size=self.chunk_size, return_final_states=True, **kw)
            cache_params.update_conv_state(self.layer_idx, conv_state)
            cache_params.update_ssm_state(self.layer_idx, ssm_state)
        else:
            y = ops.mamba2_mixer_core(
                zxBCdt, self.conv1d.weight, self.conv1d.bias, self.dt_bias, self.A_log, self.D, self.norm.weight,
                chunk_size=self.chunk_size, recompute=getattr(self.config, "b200_recompute_mixer", False), **kw)
        return self.out_proj(y)

    @torch.no_grad()
    def step(self, hidden_states: torch.Tensor, cache_params: Mamba2Cache) -> torch.Tensor:
        """Single-token decode; hidden_states [B, 1, D] (mamba2/mamba2_mixer.py:248-282)."""
        assert hidden_states.shape[1] == 1, "step() takes one token at a time"
        if self.in_proj.sequence_parallel_enabled:
            raise RuntimeError("decode runs without sequence parallelism; build the model with it disabled")
        zxBCdt = self.in_proj(hidden_states)[:, 0]
        y = ops.ssm_decode_step(zxBCdt, cache_params.conv_states[self.layer_idx],
                                cache_params.ssm_states[self.layer_idx], self.conv1d.weight, self.conv1d.bias,
                                self.dt_bias, self.A_log, self.D, self.norm.weight, **self._core_kwargs())
        return self.out_proj(y[:, None, :])
