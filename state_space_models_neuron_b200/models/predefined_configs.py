"""Named model sizes -> configs (predefined_configs.py:10-85 of the reference).

`get_config` keeps the reference's behaviour (head_dim 128 for the Mamba presets, num_heads =
2*d_model/head_dim, tied embeddings, token ids 0, use_cache off) and adds optional overrides for
`head_dim`, `state_size` and arbitrary config fields, because checkpoints published for Mamba-2 and the
benchmark configurations use head_dim 64.
"""
from __future__ import annotations

from dataclasses import astuple, dataclass
from typing import Dict, Optional

import torch

from .configuration_mamba2 import Mamba2Config
from .configuration_mamba2hybrid import Mamba2HybridConfig


@dataclass
class ConfParams:
    d_model: int
    n_layers: int
    head_dim: int = 128


MAMBA2_CONFIGS_KWARGS: Dict[str, ConfParams] = {
    "Mamba130M": ConfParams(768, 24),
    "Mamba370M": ConfParams(1024, 48),
    "Mamba780M": ConfParams(1536, 48),
    "Mamba1B": ConfParams(2048, 48),
    "Mamba3B": ConfParams(2560, 64),
    "Mamba7B": ConfParams(4096, 64),
}
MAMBA2HYBRID_CONFIGS_KWARGS: Dict[str, ConfParams] = {
    "Mamba2Hybrid800M": ConfParams(1024, 48, head_dim=64),
    "Mamba2Hybrid8B": ConfParams(4096, 56, head_dim=128),
}
CONFIGS_KWARGS: Dict[str, ConfParams] = {**MAMBA2_CONFIGS_KWARGS, **MAMBA2HYBRID_CONFIGS_KWARGS}


def get_config(name: str, vocab_size: int, rmsnorm_within_groups: bool = True, n_groups: int = 8,
               sequence_parallel_enabled: bool = False, dtype=torch.float32,
               head_dim: Optional[int] = None, **overrides):
    if name not in CONFIGS_KWARGS:
        raise ValueError(f"Unrecognized config name: {name}")
    d_model, n_layers, preset_head_dim = astuple(CONFIGS_KWARGS[name])
    hd = head_dim or preset_head_dim
    common = dict(
        vocab_size=vocab_size, hidden_size=d_model, head_dim=hd, num_heads=(2 * d_model) // hd,
        num_hidden_layers=n_layers, tie_word_embeddings=True, use_cache=False, n_groups=n_groups,
        bos_token_id=0, eos_token_id=0, pad_token_id=0, rmsnorm_within_groups=rmsnorm_within_groups,
        sequence_parallel_enabled=sequence_parallel_enabled, dtype=dtype,
    )
    common.update(overrides)
    if name in MAMBA2_CONFIGS_KWARGS:
        return Mamba2Config(**common)
    return Mamba2HybridConfig(**common)
