"""Mamba-2 language model, HuggingFace `PreTrainedModel` compatible.

Module tree and state-dict keys match the reference (mamba2/modeling_mamba2.py:106-140,220-350,
359-531): `backbone.embeddings`, `backbone.layers.{i}.norm`, `backbone.layers.{i}.mixer.*`,
`backbone.norm_f`, `lm_head`.  Differences that matter to users: the full forward also serves
as decode prefill (fills a `Mamba2Cache`), `step()` works after it, and the pre-norm residual
add and RMSNorm of consecutive blocks run as one fused kernel on GPUs.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn as nn
from transformers import GenerationMixin, PreTrainedModel
from transformers.utils import ModelOutput

from .. import ops
from ..parallel import mappings as mp
from ..parallel import state as ps
from ..parallel.cross_entropy import parallel_argmax, parallel_cross_entropy
from ..parallel.layers import ColumnParallelLinear, ParallelEmbedding, normal_init
from .cache import Mamba2Cache
from .configuration_mamba2 import Mamba2Config
from .mamba2_mixer import Mamba2Mixer


class Mamba2RMSNorm(nn.Module):
    """fp32 RMSNorm.  Under sequence parallelism the weight only sees a slice of the sequence,
    so it is tagged and its gradient is summed over the TP group before the optimizer step
    (mamba2/modeling_mamba2.py:86-103)."""

    def __init__(self, hidden_size: int, eps: float = 1e-6, sequence_parallel_enabled: bool = False,
                 dtype=torch.float32, device=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size, dtype=dtype, device=device))
        self.variance_epsilon = eps
        if sequence_parallel_enabled:
            self.weight.sequence_parallel_enabled = True

    def forward(self, hidden_states):
        return ops.rmsnorm(hidden_states, self.weight, self.variance_epsilon)

    def forward_add(self, hidden_states, residual, residual_dtype=None):
        """(normed(residual + hidden_states), residual + hidden_states)"""
        return ops.add_rmsnorm(hidden_states, residual, self.weight, self.variance_epsilon, residual_dtype)


class Mamba2Block(nn.Module):
    """Pre-norm residual block: h <- h + mixer(norm(h)).

    `forward(hidden, residual)` takes the previous block's branch output and the running
    residual stream and returns (this block's branch output, updated residual), so the add and
    the next norm fuse; the sum of the two is the block output of the reference
    (mamba2/modeling_mamba2.py:115-131)."""

    def __init__(self, config, layer_idx: int, device=None):
        super().__init__()
        self.config = config
        self.layer_idx = layer_idx
        self.residual_in_fp32 = config.residual_in_fp32
        self.norm = Mamba2RMSNorm(config.hidden_size, eps=config.layer_norm_epsilon,
                                  sequence_parallel_enabled=config.sequence_parallel_enabled,
                                  dtype=config.dtype or torch.float32, device=device)
        self.mixer = Mamba2Mixer(config, layer_idx=layer_idx, device=device)

    def forward(self, hidden_states, residual=None, cache_params=None):
        rd = torch.float32 if self.residual_in_fp32 else None
        normed, residual = self.norm.forward_add(hidden_states, residual, rd)
        return self.mixer(normed, cache_params=cache_params), residual

    def step(self, hidden_states, residual, cache_params):
        rd = torch.float32 if self.residual_in_fp32 else None
        normed, residual = self.norm.forward_add(hidden_states, residual, rd)
        return self.mixer.step(normed, cache_params), residual


@dataclass
class Mamba2Output(ModelOutput):
    last_hidden_state: Optional[torch.FloatTensor] = None
    cache_params: Optional[Mamba2Cache] = None
    hidden_states: Optional[Tuple[torch.FloatTensor]] = None


@dataclass
class Mamba2CausalLMOutput(ModelOutput):
    loss: Optional[torch.FloatTensor] = None
    logits: Optional[torch.FloatTensor] = None
    cache_params: Optional[Mamba2Cache] = None
    hidden_states: Optional[Tuple[torch.FloatTensor]] = None


class Mamba2PreTrainedModel(PreTrainedModel):
    config_class = Mamba2Config
    base_model_prefix = "backbone"
    _no_split_modules = ["Mamba2Block"]
    # per-head SSM parameters are created in fp32 whatever the model dtype: loading must not round them
    _keep_in_fp32_modules_strict = ["dt_bias", "A_log", "D"]
    supports_gradient_checkpointing = False
    _is_stateful = True

    def _init_weights(self, module):
        # parameters are drawn in the layer constructors (TP-consistent global draw, then slice)
        return


def _rename_legacy_keys(state_dict, prefix, *args):
    """Accept `embedding.` for `embeddings.` (mamba2/modeling_mamba2.py:236-240)."""
    for k in list(state_dict.keys()):
        if "embedding." in k:
            state_dict[k.replace("embedding.", "embeddings.")] = state_dict.pop(k)


class Mamba2Model(Mamba2PreTrainedModel):
    def __init__(self, config, device=None):
        super().__init__(config)
        dtype = config.dtype or torch.float32
        self.embeddings = ParallelEmbedding(config.vocab_size, config.hidden_size,
                                            init_method=normal_init(config.initializer_range), dtype=dtype, device=device)
        self.layers = nn.ModuleList([Mamba2Block(config, layer_idx=i, device=device)
                                     for i in range(config.num_hidden_layers)])
        self.sequence_parallel_enabled = config.sequence_parallel_enabled and ps.get_tensor_model_parallel_size() > 1
        self.norm_f = Mamba2RMSNorm(config.hidden_size, eps=config.layer_norm_epsilon,
                                    sequence_parallel_enabled=config.sequence_parallel_enabled, dtype=dtype, device=device)
        self.gradient_checkpointing = False
        self._register_load_state_dict_pre_hook(_rename_legacy_keys)
        self.post_init()

    def get_input_embeddings(self):
        return self.embeddings

    def set_input_embeddings(self, new_embeddings):
        self.embeddings = new_embeddings

    def forward(self, input_ids=None, inputs_embeds=None, cache_params: Optional[Mamba2Cache] = None,
                use_cache: Optional[bool] = None, output_hidden_states: Optional[bool] = None,
                return_dict: Optional[bool] = None, **kwargs):
        if (input_ids is None) == (inputs_embeds is None):
            raise ValueError("pass exactly one of input_ids and inputs_embeds")
        sp = self.sequence_parallel_enabled
        if inputs_embeds is None:
            hidden = self.embeddings(input_ids, scatter_to_sequence_parallel=sp)
        else:
            hidden = mp.scatter_to_sequence_parallel_region(inputs_embeds) if sp else inputs_embeds
        if use_cache and cache_params is None:
            cache_params = Mamba2Cache(self.config, hidden.shape[0], dtype=hidden.dtype, device=hidden.device)
        if use_cache and cache_params.seqlen_offset > 0 and hidden.shape[1] == 1 and not self.training:
            # incremental decoding (what `generate()` does after the prompt): one token over the cached states
            residual = None
            for block in self.layers:
                hidden, residual = block.step(hidden, residual, cache_params)
            rd = torch.float32 if self.config.residual_in_fp32 else None
            hidden, _ = self.norm_f.forward_add(hidden, residual, rd)
            cache_params.seqlen_offset += 1
            return Mamba2Output(last_hidden_state=hidden, cache_params=cache_params)
        all_hidden = () if output_hidden_states else None
        residual = None
        for block in self.layers:
            hidden, residual = block(hidden, residual, cache_params=cache_params if use_cache else None)
            if output_hidden_states:
                all_hidden = all_hidden + ((hidden + residual).to(hidden.dtype),)
        rd = torch.float32 if self.config.residual_in_fp32 else None
        hidden, _ = self.norm_f.forward_add(hidden, residual, rd)
        if use_cache:
            cache_params.seqlen_offset += (input_ids if input_ids is not None else inputs_embeds).shape[1]
        if return_dict is False:
            return tuple(v for v in (hidden, cache_params, all_hidden) if v is not None)
        return Mamba2Output(last_hidden_state=hidden, cache_params=cache_params if use_cache else None,
                            hidden_states=all_hidden)

    @torch.no_grad()
    def step(self, input_ids, cache_params: Mamba2Cache):
        """One decode token through all blocks (mamba2/modeling_mamba2.py:337-350)."""
        if ps.get_tensor_model_parallel_size() > 1 and input_ids.is_cuda:
            from ..parallel import symm
            symm.advance_step(compact=True)      # fresh sequence numbers for this token's fused collectives
        hidden = self.embeddings(input_ids)
        residual = None
        for block in self.layers:
            hidden, residual = block.step(hidden, residual, cache_params)
        rd = torch.float32 if self.config.residual_in_fp32 else None
        hidden, _ = self.norm_f.forward_add(hidden, residual, rd)
        cache_params.seqlen_offset += 1
        return hidden


class Mamba2ForCausalLM(Mamba2PreTrainedModel, GenerationMixin):
    _tied_weights_keys = {"lm_head.weight": "backbone.embeddings.weight"}

    def __init__(self, config, device=None):
        super().__init__(config)
        dtype = config.dtype or torch.float32
        self.backbone = Mamba2Model(config, device=device)
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

    def prepare_inputs_for_generation(self, input_ids, inputs_embeds=None, use_cache=None,
                                      cache_params: Optional[Mamba2Cache] = None, **kwargs):
        if cache_params is not None and cache_params.seqlen_offset > 0:
            input_ids = input_ids[:, -1:]
        model_inputs = {"input_ids": input_ids} if inputs_embeds is None or cache_params is not None \
            else {"inputs_embeds": inputs_embeds}
        model_inputs.update({"cache_params": cache_params, "use_cache": use_cache})
        return model_inputs

    def forward(self, input_ids=None, inputs_embeds=None, cache_params: Optional[Mamba2Cache] = None,
                labels=None, output_hidden_states=None, return_dict=None, use_cache=None, **kwargs):
        """Logits are `[B, L, V/TP]` fp32 (the local vocabulary shard under TP); the loss is the
        mean vocab-parallel cross entropy of logits[:, :-1] against labels[:, 1:]
        (mamba2/modeling_mamba2.py:498-510)."""
        out = self.backbone(input_ids=input_ids, inputs_embeds=inputs_embeds, cache_params=cache_params,
                            use_cache=use_cache, output_hidden_states=output_hidden_states, return_dict=True)
        hidden = out.last_hidden_state
        loss, logits = None, None
        if labels is not None and not kwargs.get("return_logits", True):
            loss = self.loss_from_hidden(hidden, labels)
        else:
            logits = self.lm_head(hidden).float()
            if labels is not None:
                shift_logits = logits[:, :-1, :]
                shift_labels = labels[:, 1:].to(logits.device)
                loss = parallel_cross_entropy(shift_logits, shift_labels).mean()
        if return_dict is False:
            return tuple(v for v in (loss, logits, out.cache_params, out.hidden_states) if v is not None)
        return Mamba2CausalLMOutput(loss=loss, logits=logits, cache_params=out.cache_params,
                                    hidden_states=out.hidden_states)

    def loss_from_hidden(self, hidden, labels):
        """Loss without materialising fp32 logits for the caller: labels are shifted instead of
        the logits (position L-1 is ignored), the mean runs over the B*(L-1) real targets."""
        shifted = torch.full_like(labels, -100)
        shifted[:, :-1] = labels[:, 1:]
        shifted = shifted.to(hidden.device)
        logits, stats = self.lm_head(hidden, ce_labels=shifted)
        per_tok = parallel_cross_entropy(logits, shifted, stats=stats)
        return per_tok.sum() / (labels.shape[0] * (labels.shape[1] - 1))

    @torch.no_grad()
    def prefill(self, input_ids, cache_params: Optional[Mamba2Cache] = None):
        """Run the chunked scan over a prompt, fill the cache, return last-token logits."""
        if cache_params is None:
            p = next(self.parameters())
            cache_params = Mamba2Cache(self.config, input_ids.shape[0], dtype=p.dtype, device=p.device)
        out = self.backbone(input_ids=input_ids, cache_params=cache_params, use_cache=True)
        return self.lm_head(out.last_hidden_state[:, -1:, :]).float(), cache_params

    @torch.no_grad()
    def generate(self, inputs=None, max_new_tokens: Optional[int] = None, max_length: Optional[int] = None,
                 do_sample: bool = False, temperature: float = 1.0, top_k: Optional[int] = None,
                 eos_token_id: Optional[int] = None, input_ids=None, generator=None, **unused):
        """`GenerationMixin.generate`-style entry point on top of `generate_tokens` (the framework's own conv/SSM
        cache drives decoding; HuggingFace's generic loop would hand the model a KV cache object it cannot use).
        Supports greedy decoding and temperature / top-k sampling; other generation options are not implemented."""
        ids = inputs if inputs is not None else input_ids
        if ids is None:
            raise ValueError("generate() needs input ids")
        if unused:
            ignored = sorted(k for k in unused if unused[k] is not None)
            if ignored:
                import logging
                logging.getLogger(__name__).warning("generate(): ignoring unsupported options %s", ignored)
        if max_new_tokens is None:
            max_new_tokens = max(0, (max_length or ids.shape[1] + 20) - ids.shape[1])
        if eos_token_id is None:
            eos_token_id = getattr(self.generation_config, "eos_token_id", None) if hasattr(self, "generation_config") else None
            if isinstance(eos_token_id, (list, tuple)):
                eos_token_id = eos_token_id[0] if eos_token_id else None
        return self.generate_tokens(ids, max_new_tokens, temperature=temperature if do_sample else 0.0, top_k=top_k,
                                    eos_token_id=eos_token_id, generator=generator)

    @torch.no_grad()
    def generate_tokens(self, input_ids, max_new_tokens: int, temperature: float = 0.0, top_k: Optional[int] = None,
                        eos_token_id: Optional[int] = None, generator=None):
        """Prompt -> continuation with the cached decode path: the longest 128-multiple prefix of the prompt goes
        through the chunked scan (prefill), the rest of the prompt and every new token through `step`.
        temperature 0 = greedy.  Returns [B, L + new] token ids.  (HuggingFace's `generate()` plumbing is kept for
        API compatibility, but like in the reference it does not drive this cache.)"""
        B, L = input_ids.shape
        p = next(self.parameters())
        cache = Mamba2Cache(self.config, B, dtype=p.dtype, device=p.device)
        chunk = 128
        Lp = (L // chunk) * chunk
        logits = None
        if Lp:
            logits, cache = self.prefill(input_ids[:, :Lp], cache)
        for t in range(Lp, L):
            logits = self.step(input_ids[:, t:t + 1], cache)
        out = [input_ids]
        done = torch.zeros(B, dtype=torch.bool, device=input_ids.device)
        for _ in range(max_new_tokens):
            last = logits[:, -1].float()
            if temperature and temperature > 0:
                if ps.get_tensor_model_parallel_size() > 1:      # sampling needs the whole vocabulary
                    parts = [torch.empty_like(last) for _ in range(ps.get_tensor_model_parallel_size())]
                    torch.distributed.all_gather(parts, last.contiguous(), group=ps.get_tensor_model_parallel_group())
                    last = torch.cat(parts, dim=-1)
                last = last / temperature
                if top_k:
                    kth = torch.topk(last, top_k, dim=-1).values[:, -1:]
                    last = last.masked_fill(last < kth, float("-inf"))
                nxt = torch.multinomial(torch.softmax(last, -1), 1, generator=generator)
            else:
                nxt = parallel_argmax(last).unsqueeze(-1)
            out.append(nxt)
            if eos_token_id is not None:
                done |= nxt[:, 0] == eos_token_id
                if bool(done.all()):
                    break
            logits = self.step(nxt, cache)
        return torch.cat(out, dim=1)

    @torch.no_grad()
    def step(self, input_ids, cache_params: Mamba2Cache):
        """Single-token decode: logits for the next token (mamba2/modeling_mamba2.py:523-531)."""
        hidden = self.backbone.step(input_ids, cache_params)
        return self.lm_head(hidden).float()
