"""Mamba-2 hybrid (Mamba + attention + MLP layers) configuration, `model_type = "mamba2hybrid"`.

Defaults follow the reference (mamba2hybrid/configuration_mamba2hybrid.py:130-231).  Two switches
cover variants the reference's hybrid never turns on but whose code it carries
(mamba2hybrid/mamba2hybrid_attn.py:500-503, mamba2hybrid/mamba2hybrid_mlp.py:155-165):
`rotary_emb_dim`/`rope_theta` (rotary position embedding in attention; None = off) and
`gated_linear_unit` (SwiGLU-style gated MLP; False = plain GELU MLP).
"""
from __future__ import annotations

import torch

from .configuration_mamba2 import Mamba2Config


class Mamba2HybridConfig(Mamba2Config):
    model_type = "mamba2hybrid"

    def __init__(
        self,
        vocab_size: int = 256000,
        num_hidden_layers: int = 56,
        pad_token_id: int = 0,
        unk_token_id: int = 1,
        bos_token_id: int = 2,
        eos_token_id: int = 3,
        residual_in_fp32: bool = True,
        time_step_rank=256,
        chunk_size: int = 128,
        hybrid_attention_ratio: float = 0.08,
        hybrid_mlp_ratio: float = 0.5,
        hybrid_override_pattern=None,
        attn_num_heads: int = 32,
        attn_head_dim: int = 128,
        attn_key_value_heads: int = 8,
        kv_channels: int = 128,
        mlp_hidden_size: int = 16384,
        mlp_hidden_act: str = "gelu",
        gated_linear_unit: bool = False,
        rotary_emb_dim=None,
        rope_theta: float = 10000.0,
        max_position_embeddings: int = 8192,
        dtype=torch.bfloat16,
        **kwargs,
    ):
        self.unk_token_id = unk_token_id
        self.hybrid_attention_ratio = hybrid_attention_ratio
        self.hybrid_mlp_ratio = hybrid_mlp_ratio
        self.hybrid_override_pattern = hybrid_override_pattern
        self.attn_num_heads = attn_num_heads
        self.attn_head_dim = attn_head_dim
        self.attn_key_value_heads = attn_key_value_heads
        self.kv_channels = kv_channels
        self.mlp_hidden_size = mlp_hidden_size
        self.mlp_hidden_act = mlp_hidden_act
        self.gated_linear_unit = gated_linear_unit
        self.rotary_emb_dim = rotary_emb_dim
        self.rope_theta = rope_theta
        self.max_position_embeddings = max_position_embeddings
        super().__init__(
            vocab_size=vocab_size,
            num_hidden_layers=num_hidden_layers,
            pad_token_id=pad_token_id,
            bos_token_id=bos_token_id,
            eos_token_id=eos_token_id,
            residual_in_fp32=residual_in_fp32,
            time_step_rank=time_step_rank,
            chunk_size=chunk_size,
            dtype=dtype,
            **kwargs,
        )
