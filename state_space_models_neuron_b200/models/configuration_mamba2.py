"""Mamba-2 model configuration (HuggingFace `PretrainedConfig`, `model_type = "mamba2"`).

Field names, defaults and the three additions over the HuggingFace class
(`rmsnorm_within_groups`, `sequence_parallel_enabled`, `dtype`) follow the reference
(mamba2/configuration_mamba2.py:112-189) so that `config.json` files are interchangeable.
Framework-only knobs are prefixed `b200_` and have defaults that do nothing.
"""
from __future__ import annotations

import math

import torch
from transformers import PretrainedConfig


def _dtype_from(value):
    if isinstance(value, torch.dtype) or value is None:
        return value
    name = str(value).replace("torch.", "")
    return getattr(torch, name)


class Mamba2Config(PretrainedConfig):
    model_type = "mamba2"

    def __init__(
        self,
        num_heads: int = 128,
        head_dim: int = 64,
        vocab_size: int = 32768,
        hidden_size: int = 4096,
        state_size: int = 128,
        num_hidden_layers: int = 64,
        layer_norm_epsilon: float = 1e-5,
        pad_token_id: int = 1,
        bos_token_id: int = 0,
        eos_token_id: int = 2,
        expand: int = 2,
        conv_kernel: int = 4,
        n_groups: int = 8,
        use_bias: bool = False,
        use_conv_bias: bool = True,
        hidden_act: str = "silu",
        initializer_range: float = 0.1,
        residual_in_fp32: bool = False,
        time_step_rank="auto",
        time_step_min: float = 0.001,
        time_step_max: float = 0.1,
        time_step_floor: float = 1e-4,
        time_step_limit=(0.0, float("inf")),
        rescale_prenorm_residual: bool = False,
        use_cache: bool = False,
        rms_norm: bool = True,
        rmsnorm_within_groups: bool = True,
        chunk_size: int = 256,
        tie_word_embeddings: bool = False,
        sequence_parallel_enabled: bool = False,
        dtype=torch.float32,
        a_log_init: str = "arange",
        b200_recompute_mixer: bool = False,
        **kwargs,
    ):
        self.num_heads = num_heads
        self.head_dim = head_dim
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.state_size = state_size
        self.num_hidden_layers = num_hidden_layers
        self.layer_norm_epsilon = layer_norm_epsilon
        self.expand = expand
        self.conv_kernel = conv_kernel
        self.n_groups = n_groups
        self.use_bias = use_bias
        self.use_conv_bias = use_conv_bias
        self.hidden_act = hidden_act
        self.initializer_range = initializer_range
        self.residual_in_fp32 = residual_in_fp32
        self.time_step_rank = math.ceil(hidden_size / 16) if time_step_rank == "auto" else time_step_rank
        self.time_step_min = time_step_min
        self.time_step_max = time_step_max
        self.time_step_floor = time_step_floor
        self.time_step_limit = tuple(time_step_limit)
        self.rescale_prenorm_residual = rescale_prenorm_residual
        self.use_cache = use_cache
        self.rms_norm = rms_norm
        self.rmsnorm_within_groups = rmsnorm_within_groups
        self.chunk_size = chunk_size
        self.sequence_parallel_enabled = sequence_parallel_enabled
        # "arange": A_log = log(1..H) (mamba2/mamba2_mixer.py:172-174); "uniform": log(U[1,16])
        self.a_log_init = a_log_init
        self.b200_recompute_mixer = b200_recompute_mixer
        super().__init__(
            bos_token_id=bos_token_id,
            eos_token_id=eos_token_id,
            pad_token_id=pad_token_id,
            tie_word_embeddings=tie_word_embeddings,
            dtype=_dtype_from(dtype),
            **kwargs,
        )

    # derived sizes -------------------------------------------------------------------------
    @property
    def intermediate_size(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def conv_dim(self) -> int:
        return self.intermediate_size + 2 * self.n_groups * self.state_size

    @property
    def in_proj_size(self) -> int:
        return self.intermediate_size + self.conv_dim + self.num_heads
