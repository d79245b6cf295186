"""Decode cache: per layer a rolling conv window and the SSM state.

Field names and shapes follow the `Mamba2Cache` of transformers 4.46 that the reference imports
(mamba2/mamba2_mixer.py:23) and the layouts its decode kernel uses
(mamba2/mamba2_kernel_inference.py:36-43): `conv_states[layer]` is `[B, conv_dim, K]` (oldest token
first), `ssm_states[layer]` is `[B, H, P, N]`; sizes are per tensor-parallel rank.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..parallel import state as ps


class Mamba2Cache:
    def __init__(self, config, batch_size: int, dtype: torch.dtype = torch.float16,
                 device: Optional[torch.device] = None, ssm_dtype: torch.dtype = torch.float32,
                 layer_indices=None):
        tp = ps.get_tensor_model_parallel_size()
        self.dtype = dtype
        self.seqlen_offset = 0
        self.conv_kernel_size = config.conv_kernel
        conv_dim = (config.intermediate_size + 2 * config.n_groups * config.state_size) // tp
        heads = config.num_heads // tp
        layers = range(config.num_hidden_layers) if layer_indices is None else layer_indices
        self.conv_states = {i: torch.zeros(batch_size, conv_dim, config.conv_kernel, device=device, dtype=dtype)
                            for i in layers}
        self.ssm_states = {i: torch.zeros(batch_size, heads, config.head_dim, config.state_size,
                                          device=device, dtype=ssm_dtype) for i in layers}

    def update_conv_state(self, layer_idx: int, new_conv_state: torch.Tensor) -> torch.Tensor:
        self.conv_states[layer_idx].copy_(new_conv_state.to(self.conv_states[layer_idx].dtype))
        return self.conv_states[layer_idx]

    def update_ssm_state(self, layer_idx: int, new_ssm_state: torch.Tensor) -> torch.Tensor:
        self.ssm_states[layer_idx].copy_(new_ssm_state.to(self.ssm_states[layer_idx].dtype))
        return self.ssm_states[layer_idx]

    def reset(self) -> None:
        self.seqlen_offset = 0
        for t in list(self.conv_states.values()) + list(self.ssm_states.values()):
            t.zero_()
