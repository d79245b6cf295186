"""Causal grouped-query self-attention block of the hybrid model.

Parameters `q_proj/k_proj/v_proj` (column parallel) and `o_proj` (row parallel), no biases, no
dropout, per-rank heads = attn_num_heads/TP and kv heads = attn_key_value_heads/TP
(mamba2hybrid/mamba2hybrid_attn.py:305-362,491-514).  The three projections share one sequence
all-gather, K/V heads are never replicated in memory (the kernel indexes kv head = q head // ratio,
where the reference materialises `repeat_kv`, mamba2hybrid_attn.py:440-447), and rotary embedding (its own
kernel, forward and backward, with cached tables) is an option that is off by default as in the reference
hybrid (mamba2hybrid_attn.py:500-503).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import ops
from ..parallel import mappings as mp
from ..parallel import state as ps
from ..parallel.layers import ColumnParallelLinear, GQAQKVColumnParallelLinear, RowParallelLinear, normal_init


class Mamba2HybridAttention(nn.Module):
    def __init__(self, config, layer_idx: int, device=None):
        super().__init__()
        tp = ps.get_tensor_model_parallel_size()
        self.layer_idx = layer_idx
        self.hidden_size = config.hidden_size
        self.total_heads = config.attn_num_heads
        self.total_kv_heads = config.attn_key_value_heads
        self.head_dim = config.attn_head_dim
        self.qkv_linear = bool(getattr(config, "qkv_linear", False))
        kv_mult = int(getattr(config, "kv_shared_group_size", 1)) if self.qkv_linear else 1
        if self.total_heads % tp or (self.total_kv_heads * kv_mult) % tp:
            raise ValueError("attention heads and kv heads (times kv_shared_group_size) must be divisible by the TP size")
        self.num_heads = self.total_heads // tp
        self.num_kv_heads = self.total_kv_heads * kv_mult // tp
        self.sequence_parallel_enabled = config.sequence_parallel_enabled and tp > 1
        self.rotary_emb_dim = getattr(config, "rotary_emb_dim", None)
        self.rope_theta = getattr(config, "rope_theta", 10000.0)
        dtype = config.dtype or torch.float32
        init = normal_init(config.initializer_range)
        kw = dict(bias=False, init_method=init, dtype=dtype, device=device,
                  sequence_parallel_enabled=config.sequence_parallel_enabled)
        if self.qkv_linear:
            # one layer for q, k, v with optional KV-head replication (mamba2hybrid_attn.py:291-303 of the reference)
            self.qkv_proj = GQAQKVColumnParallelLinear(
                self.hidden_size, [self.total_heads * self.head_dim, self.total_kv_heads * self.head_dim],
                kv_size_multiplier=kv_mult, fuse_qkv=bool(getattr(config, "fuse_qkv", False)), head_dim=self.head_dim, **kw)
        else:
            self.q_proj = ColumnParallelLinear(self.hidden_size, self.total_heads * self.head_dim, **kw)
            self.k_proj = ColumnParallelLinear(self.hidden_size, self.total_kv_heads * self.head_dim, **kw)
            self.v_proj = ColumnParallelLinear(self.hidden_size, self.total_kv_heads * self.head_dim, **kw)
        self.o_proj = RowParallelLinear(self.total_heads * self.head_dim, self.hidden_size, bias=False,
                                        init_method=init, dtype=dtype, device=device,
                                        sequence_parallel_enabled=config.sequence_parallel_enabled)

    def forward(self, hidden_states: torch.Tensor, cache_params=None) -> torch.Tensor:
        qkv = None
        if self.qkv_linear:
            qkv = self.qkv_proj(hidden_states)
        elif self.sequence_parallel_enabled:
            from ..parallel import fused
            if fused.enabled_for(hidden_states):
                qkv = fused.all_gather_multi_linear(
                    hidden_states, (self.q_proj.weight, self.k_proj.weight, self.v_proj.weight))
            if qkv is None:
                x = mp.gather_from_sequence_parallel_region(hidden_states, True)
        else:
            x = mp.copy_to_tensor_parallel_region(hidden_states)
        if qkv is None:
            qkv = (ops.linear(x, self.q_proj.weight), ops.linear(x, self.k_proj.weight),
                   ops.linear(x, self.v_proj.weight))
        B, L = qkv[0].shape[0], qkv[0].shape[1]
        q = qkv[0].view(B, L, self.num_heads, self.head_dim)
        k = qkv[1].view(B, L, self.num_kv_heads, self.head_dim)
        v = qkv[2].view(B, L, self.num_kv_heads, self.head_dim)
        if self.rotary_emb_dim is not None:
            cos, sin = ops.rotary_tables(L, self.rotary_emb_dim, self.rope_theta, device=q.device)
            q = ops.apply_rotary(q, cos, sin)
            k = ops.apply_rotary(k, cos, sin)
        o = ops.attention(q, k, v, causal=True)
        return self.o_proj(o.reshape(B, L, self.num_heads * self.head_dim))
