"""Mamba-2 hybrid language model: a stack whose layers are Mamba-2 mixers, GQA attention or MLPs
according to `allocate_layers`, each wrapped as `norm + layer + residual`.

State-dict keys follow the reference (mamba2hybrid/modeling_mamba2hybrid.py:116-161,325-345,
462-478): `backbone.layers.{i}.norm.weight`, `backbone.layers.{i}.layer.*`.
"""
from __future__ import annotations

import logging
from typing import Optional

import torch
import torch.nn as nn
from transformers import GenerationMixin

from ..parallel import mappings as mp
from ..parallel import state as ps
from ..parallel.cross_entropy import parallel_cross_entropy
from ..parallel.layers import ColumnParallelLinear, ParallelEmbedding, normal_init
from .cache import Mamba2Cache
from .configuration_mamba2hybrid import Mamba2HybridConfig
from .hybrid_attn import Mamba2HybridAttention
from .hybrid_mlp import Mamba2HybridMLP
from .layer_allocation import ATTENTION, MAMBA, MLP, allocate_layers
from .mamba2_mixer import Mamba2Mixer
from .modeling_mamba2 import (Mamba2CausalLMOutput, Mamba2ForCausalLM, Mamba2Output, Mamba2PreTrainedModel,
                              Mamba2RMSNorm, _rename_legacy_keys)

log = logging.getLogger(__name__)


class Mamba2HybridBlock(nn.Module):
    def __init__(self, config, layer_idx: int, layer_type: str, device=None):
        super().__init__()
        self.layer_idx, self.layer_type = layer_idx, layer_type
        self.residual_in_fp32 = config.residual_in_fp32
        self.norm = Mamba2RMSNorm(config.hidden_size, eps=config.layer_norm_epsilon,
                                  sequence_parallel_enabled=config.sequence_parallel_enabled,
                                  dtype=config.dtype or torch.float32, device=device)
        if layer_type == MAMBA:
            self.layer = Mamba2Mixer(config, layer_idx=layer_idx, device=device)
        elif layer_type == ATTENTION:
            self.layer = Mamba2HybridAttention(config, layer_idx=layer_idx, device=device)
        elif layer_type == MLP:
            self.layer = Mamba2HybridMLP(config, layer_idx=layer_idx, device=device)
        else:
            raise ValueError(f"unknown layer type {layer_type!r}")

    def forward(self, hidden_states, residual=None, cache_params=None):
        rd = torch.float32 if self.residual_in_fp32 else None
        normed, residual = self.norm.forward_add(hidden_states, residual, rd)
        return self.layer(normed, cache_params=cache_params), residual


class Mamba2HybridPreTrainedModel(Mamba2PreTrainedModel):
    config_class = Mamba2HybridConfig
    _no_split_modules = ["Mamba2HybridBlock"]


class Mamba2HybridModel(Mamba2HybridPreTrainedModel):
    def __init__(self, config, device=None):
        super().__init__(config)
        dtype = config.dtype or torch.float32
        self.embeddings = ParallelEmbedding(config.vocab_size, config.hidden_size,
                                            init_method=normal_init(config.initializer_range), dtype=dtype, device=device)
        self.layer_types = allocate_layers(config.num_hidden_layers, config.hybrid_attention_ratio,
                                           config.hybrid_mlp_ratio, config.hybrid_override_pattern,
                                           verbose=ps.is_master())
        self.layers = nn.ModuleList([Mamba2HybridBlock(config, i, t, device=device)
                                     for i, t in enumerate(self.layer_types)])
        self.sequence_parallel_enabled = config.sequence_parallel_enabled and ps.get_tensor_model_parallel_size() > 1
        self.norm_f = Mamba2RMSNorm(config.hidden_size, eps=config.layer_norm_epsilon,
                                    sequence_parallel_enabled=config.sequence_parallel_enabled, dtype=dtype, device=device)
        self._register_load_state_dict_pre_hook(_rename_legacy_keys)
        self.post_init()

    def get_input_embeddings(self):
        return self.embeddings

    def set_input_embeddings(self, new_embeddings):
        self.embeddings = new_embeddings

    def forward(self, input_ids=None, inputs_embeds=None, output_hidden_states: Optional[bool] = None,
                return_dict: Optional[bool] = None, **kwargs):
        if (input_ids is None) == (inputs_embeds is None):
            raise ValueError("pass exactly one of input_ids and inputs_embeds")
        sp = self.sequence_parallel_enabled
        if inputs_embeds is None:
            hidden = self.embeddings(input_ids, scatter_to_sequence_parallel=sp)
        else:
            hidden = mp.scatter_to_sequence_parallel_region(inputs_embeds) if sp else inputs_embeds
        all_hidden = () if output_hidden_states else None
        residual = None
        for block in self.layers:
            hidden, residual = block(hidden, residual)
            if output_hidden_states:
                all_hidden = all_hidden + ((hidden + residual).to(hidden.dtype),)
        rd = torch.float32 if self.config.residual_in_fp32 else None
        hidden, _ = self.norm_f.forward_add(hidden, residual, rd)
        if return_dict is False:
            return tuple(v for v in (hidden, all_hidden) if v is not None)
        return Mamba2Output(last_hidden_state=hidden, hidden_states=all_hidden)


class Mamba2HybridForCausalLM(Mamba2HybridPreTrainedModel, GenerationMixin):
    _tied_weights_keys = {"lm_head.weight": "backbone.embeddings.weight"}

    def __init__(self, config, device=None):
        super().__init__(config)
        dtype = config.dtype or torch.float32
        self.backbone = Mamba2HybridModel(config, device=device)
        self.lm_head = ColumnParallelLinear(config.hidden_size, config.vocab_size, bias=False,
                                            init_method=normal_init(config.initializer_range), dtype=dtype,
                                            sequence_parallel_enabled=config.sequence_parallel_enabled, device=device)
        self.post_init()
        if config.tie_word_embeddings:
            self.lm_head.weight = self.backbone.embeddings.weight

    def get_output_embeddings(self):
        return self.lm_head

    def set_output_embeddings(self, new_embeddings):
        self.lm_head = new_embeddings

    def get_input_embeddings(self):
        return self.backbone.get_input_embeddings()

    def set_input_embeddings(self, new_embeddings):
        return self.backbone.set_input_embeddings(new_embeddings)

    loss_from_hidden = Mamba2ForCausalLM.loss_from_hidden

    def forward(self, input_ids=None, inputs_embeds=None, labels=None, output_hidden_states=None,
                return_dict=None, **kwargs):
        out = self.backbone(input_ids=input_ids, inputs_embeds=inputs_embeds,
                            output_hidden_states=output_hidden_states, return_dict=True)
        hidden = out.last_hidden_state
        loss, logits = None, None
        if labels is not None and not kwargs.get("return_logits", True):
            loss = self.loss_from_hidden(hidden, labels)
        else:
            logits = self.lm_head(hidden).float()
            if labels is not None:
                loss = parallel_cross_entropy(logits[:, :-1, :], labels[:, 1:].to(logits.device)).mean()
        if return_dict is False:
            return tuple(v for v in (loss, logits, out.hidden_states) if v is not None)
        return Mamba2CausalLMOutput(loss=loss, logits=logits, hidden_states=out.hidden_states)
