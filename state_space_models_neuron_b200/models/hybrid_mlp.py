"""MLP block of the hybrid model: `gate_up_proj` (column parallel) -> activation -> `down_proj`
(row parallel).  Default is the reference's ungated GELU MLP (mamba2hybrid/mamba2hybrid_mlp.py:
118-134,152-165); `gated_linear_unit=True` doubles `gate_up_proj` into `gate | up` blocks and
multiplies act(gate) * up.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..parallel import state as ps
from ..parallel.layers import ColumnParallelLinear, RowParallelLinear, normal_init


class Mamba2HybridMLP(nn.Module):
    def __init__(self, config, layer_idx: int, device=None):
        super().__init__()
        tp = ps.get_tensor_model_parallel_size()
        self.layer_idx = layer_idx
        self.hidden_size = config.hidden_size
        self.intermediate_size = config.mlp_hidden_size
        self.gated = bool(getattr(config, "gated_linear_unit", False))
        self.act_name = config.mlp_hidden_act
        if self.intermediate_size % tp:
            raise ValueError("mlp_hidden_size must be divisible by the TP size")
        self.split_size = self.intermediate_size // tp
        dtype = config.dtype or torch.float32
        init = normal_init(config.initializer_range)
        stride = 2 if self.gated else 1
        self.gate_up_proj = ColumnParallelLinear(
            self.hidden_size, stride * self.intermediate_size, bias=False, init_method=init, dtype=dtype,
            sequence_parallel_enabled=config.sequence_parallel_enabled, stride=stride, device=device)
        self.down_proj = RowParallelLinear(
            self.intermediate_size, self.hidden_size, bias=False, init_method=init, dtype=dtype,
            sequence_parallel_enabled=config.sequence_parallel_enabled, device=device)

    def _act(self, x):
        if self.act_name == "gelu":
            return ops.gelu(x)
        if self.act_name in ("silu", "swish"):
            return F.silu(x)
        if self.act_name == "relu":
            return F.relu(x)
        raise ValueError(f"unsupported activation {self.act_name}")

    def forward(self, hidden_states: torch.Tensor, cache_params=None) -> torch.Tensor:
        h = self.gate_up_proj(hidden_states)
        if self.gated:
            if self.act_name in ("gelu", "silu", "swish", "relu"):
                h = ops.glu(h, self.act_name)           # act(gate) * up in one kernel on the GPU path
            else:
                gate, up = h.split(self.split_size, dim=-1)
                h = self._act(gate) * up
        else:
            h = self._act(h)
        return self.down_proj(h)
