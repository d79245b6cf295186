"""How every parameter of the Mamba-2 / hybrid models is split over tensor-parallel ranks, and the
exact inverses `shard_state_dict` / `merge_state_dicts`.

The rules are those of the reference's TP slicing (mamba2/mamba2_mixer.py:192-206,63-86;
mamba2/conv1d_grouped.py:323-331) and of its merge tool (merge_tp_checkpoints.py:6-72), generalised
from that tool's hard-coded 7B / TP=8 / head_dim=128 / one-group-per-rank case to any config and TP:

    in_proj.weight      rows   z | x | B | C | dt   each block split evenly, rank pieces concatenated
    conv1d.weight/bias  rows   x | B | C            same
    out_proj / o_proj / down_proj weight            split on columns (dim 1)
    A_log, D, dt_bias, mixer norm.weight, embeddings, lm_head, q/k/v, gate_up (per gate/up block)   dim 0
    layer norms, norm_f                              replicated
"""
from __future__ import annotations

import re
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .layers import shard_rows, unshard_rows

Rule = Tuple[Optional[int], Optional[Tuple[int, ...]]]  # (partition dim or None, row segments or None)


def _cfg(config, name, default=None):
    return config.get(name, default) if isinstance(config, dict) else getattr(config, name, default)


def partition_rule(key: str, config) -> Rule:
    d_inner = _cfg(config, "num_heads") * _cfg(config, "head_dim")
    gn = _cfg(config, "n_groups") * _cfg(config, "state_size")
    heads = _cfg(config, "num_heads")
    if key.endswith("in_proj.weight") or key.endswith("in_proj.bias"):
        return 0, (d_inner, d_inner, gn, gn, heads)
    if key.endswith("conv1d.weight") or key.endswith("conv1d.bias"):
        return 0, (d_inner, gn, gn)
    if re.search(r"(out_proj|o_proj|down_proj)\.weight$", key):
        return 1, None
    if re.search(r"(out_proj|o_proj|down_proj)\.bias$", key):
        return None, None
    if key.endswith("gate_up_proj.weight"):
        if _cfg(config, "gated_linear_unit", False):
            h = _cfg(config, "mlp_hidden_size")
            return 0, (h, h)
        return 0, None
    if re.search(r"\.(mixer|layer)\.(A_log|D|dt_bias|norm\.weight)$", key):
        return 0, None
    if re.search(r"(embeddings|embedding|lm_head|q_proj|k_proj|v_proj)\.weight$", key):
        return 0, None
    if re.search(r"qkv_proj\.(weight|bias)_[qkv]$", key):      # kv_size_multiplier 1 only (no replicated heads)
        return 0, None
    return None, None  # block norms, norm_f: replicated


def shard_state_dict(full: Dict[str, torch.Tensor], config, tp_size: int, tp_rank: int) -> Dict[str, torch.Tensor]:
    """HF/global state dict -> the state dict of one TP rank."""
    out = {}
    for k, v in full.items():
        dim, segs = partition_rule(k, config)
        if dim is None or tp_size == 1:
            out[k] = v.clone()
        elif dim == 0:
            out[k] = shard_rows(v, segs, tp_rank, tp_size).clone()
        else:
            per = v.shape[1] // tp_size
            out[k] = v[:, tp_rank * per:(tp_rank + 1) * per].clone()
    return out


def merge_state_dicts(shards: Sequence[Dict[str, torch.Tensor]], config) -> Dict[str, torch.Tensor]:
    """State dicts of TP ranks 0..T-1 -> HF/global state dict (inverse of `shard_state_dict`)."""
    out = {}
    for k in shards[0].keys():
        dim, segs = partition_rule(k, config)
        parts = [s[k] for s in shards]
        if dim is None or len(shards) == 1:
            out[k] = parts[0].clone()
        elif dim == 0:
            out[k] = unshard_rows(parts, segs).clone()
        else:
            out[k] = torch.cat(parts, dim=1)
    return out
