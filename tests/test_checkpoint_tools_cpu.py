"""Checkpoint formats on CPU: shard/merge are exact inverses for several TP degrees and layouts, the merge CLI
produces a directory HuggingFace's own Mamba2 class loads, the state-spaces converter round-trips, presets and the
hybrid layer allocation match the reference."""
import json
import os
import tempfile

import pytest
import torch

from state_space_models_neuron_b200.models import (Mamba2Config, Mamba2ForCausalLM, Mamba2HybridConfig,
                                                   Mamba2HybridForCausalLM, allocate_layers, get_config)
from state_space_models_neuron_b200.parallel.layers import set_init_seed
from state_space_models_neuron_b200.parallel.layout import merge_state_dicts, shard_state_dict


def _small(head_dim=64, n_groups=8, hybrid=False, gated=False):
    kw = dict(num_heads=1024 // head_dim, head_dim=head_dim, vocab_size=512, hidden_size=512, state_size=16,
              num_hidden_layers=2, n_groups=n_groups, tie_word_embeddings=True)
    if hybrid:
        return Mamba2HybridConfig(**{**kw, "num_hidden_layers": 4}, attn_num_heads=8, attn_head_dim=16,
                                  attn_key_value_heads=8, mlp_hidden_size=256, hybrid_attention_ratio=0.25,
                                  hybrid_mlp_ratio=0.25, gated_linear_unit=gated, dtype=torch.float32)
    return Mamba2Config(**kw)


@pytest.mark.parametrize("tp", [1, 2, 4, 8])
@pytest.mark.parametrize("head_dim,n_groups", [(64, 8), (128, 8), (64, 1)])
def test_shard_then_merge_is_identity(tp, head_dim, n_groups):
    if n_groups % tp:
        pytest.skip("n_groups must be divisible by TP")
    set_init_seed(1)
    cfg = _small(head_dim, n_groups)
    sd = Mamba2ForCausalLM(cfg).state_dict()
    shards = [shard_state_dict(sd, cfg, tp, r) for r in range(tp)]
    in_proj = "backbone.layers.0.mixer.in_proj.weight"
    assert shards[0][in_proj].shape[0] == sd[in_proj].shape[0] // tp
    merged = merge_state_dicts(shards, cfg)
    assert merged.keys() == sd.keys()
    for k in sd:
        assert torch.equal(merged[k], sd[k]), k


@pytest.mark.parametrize("gated", [False, True])
def test_hybrid_shard_merge_identity(gated):
    set_init_seed(2)
    cfg = _small(hybrid=True, gated=gated)
    sd = Mamba2HybridForCausalLM(cfg).state_dict()
    for tp in (2, 4):
        merged = merge_state_dicts([shard_state_dict(sd, cfg, tp, r) for r in range(tp)], cfg)
        for k in sd:
            assert torch.equal(merged[k], sd[k]), k


def test_merge_cli_output_loads_in_huggingface_mamba2():
    import merge_tp_checkpoints
    import shard_hf_checkpoint
    from transformers import Mamba2ForCausalLM as HFModel
    set_init_seed(3)
    cfg = _small(64, 8)
    cfg.chunk_size = 128
    cfg.rmsnorm_within_groups = False   # HuggingFace's gated norm spans all groups; ours does so with this flag
    model = Mamba2ForCausalLM(cfg).eval()
    with tempfile.TemporaryDirectory() as d:
        hf_dir, ck, out = os.path.join(d, "hf"), os.path.join(d, "ck"), os.path.join(d, "out")
        model.save_pretrained(hf_dir)
        shard_hf_checkpoint.main(["--input_dir", hf_dir, "--output_dir", ck, "--tag", "t", "--tp", "4"])
        assert sorted(os.listdir(os.path.join(ck, "t", "model"))) == [
            f"dp_rank_00_tp_rank_{r:02d}_pp_rank_00.pt" for r in range(4)]
        merge_tp_checkpoints.main(["--mamba2_checkpoint_directory", os.path.join(ck, "t", "model"), "--output_dir", out,
                                   "--safetensors"])
        ours = Mamba2ForCausalLM.from_pretrained(out).eval()
        ids = torch.randint(0, 512, (1, 128))
        with torch.no_grad():
            ref = model(input_ids=ids).logits
            assert torch.allclose(ours(input_ids=ids).logits, ref, atol=1e-5)
            with open(os.path.join(out, "config.json")) as f:
                c = json.load(f)
            hf = HFModel.from_pretrained(out).eval()
            assert c["model_type"] == "mamba2"
            assert torch.allclose(hf(input_ids=ids).logits, ref, atol=2e-4, rtol=1e-3)


def test_convert_state_spaces_checkpoint():
    import convert_mamba2_ssm_checkpoint as conv
    set_init_seed(4)
    cfg = Mamba2Config(num_heads=8, head_dim=64, vocab_size=1008, hidden_size=256, state_size=128,
                       num_hidden_layers=2, n_groups=1, tie_word_embeddings=True)
    src = Mamba2ForCausalLM(cfg)
    sd = {k.replace("backbone.embeddings.", "backbone.embedding."): v for k, v in src.state_dict().items()}
    with tempfile.TemporaryDirectory() as d:
        os.makedirs(os.path.join(d, "in"))
        torch.save(sd, os.path.join(d, "in", "pytorch_model.bin"))
        with open(os.path.join(d, "in", "config.json"), "w") as f:
            json.dump({"d_model": 256, "n_layer": 2, "vocab_size": 1000, "pad_vocab_size_multiple": 16,
                       "tie_embeddings": True, "ssm_cfg": {}}, f)
        conv.main(["-i", os.path.join(d, "in"), "-m", "mamba_ssm", "-p", "fp32", "-o", os.path.join(d, "out")])
        loaded = Mamba2ForCausalLM.from_pretrained(os.path.join(d, "out"))
        assert loaded.config.vocab_size == 1008      # 1000 padded up to a multiple of 16
        for k, v in src.state_dict().items():
            assert torch.equal(loaded.state_dict()[k], v), k


def test_presets_and_allocation_match_reference():
    c = get_config("Mamba7B", 50288)
    assert (c.hidden_size, c.num_hidden_layers, c.head_dim, c.num_heads) == (4096, 64, 128, 64)
    assert c.tie_word_embeddings and not c.use_cache and c.pad_token_id == 0
    c64 = get_config("Mamba7B", 50288, head_dim=64)
    assert c64.num_heads == 128
    h = get_config("Mamba2Hybrid8B", 50288, dtype=torch.bfloat16)
    assert (h.num_hidden_layers, h.attn_num_heads, h.attn_key_value_heads, h.mlp_hidden_size) == (56, 32, 8, 16384)
    pattern = "".join(allocate_layers(56, 0.08, 0.5))
    assert pattern == "M-M-M--M-M*-M-M-M-M--M*-M-M-M-M-M*--M-M-M-M-M*-M--M-M-M-"
    assert (pattern.count("M"), pattern.count("*"), pattern.count("-")) == (24, 4, 28)
    with pytest.raises(ValueError):
        allocate_layers(4, 0.5, 0.5, override_pattern="MMX-")
    assert "".join(allocate_layers(4, 0.0, 0.0, override_pattern="M*-M")) == "M*-M"
    with tempfile.TemporaryDirectory() as d:
        h.save_pretrained(d)
        back = Mamba2HybridConfig.from_pretrained(d)
        assert back.hybrid_attention_ratio == 0.08 and back.model_type == "mamba2hybrid"


@pytest.mark.parametrize("hybrid", [False, True])
def test_save_pretrained_from_pretrained_round_trip_keeps_values_and_dtypes(hybrid):
    """HuggingFace save/load of a bf16 model restores every tensor exactly; the fp32 per-head SSM parameters
    (dt_bias, A_log, D) are not rounded to the model dtype on the way."""
    import tempfile
    from state_space_models_neuron_b200.models import (Mamba2Config, Mamba2ForCausalLM, Mamba2HybridConfig,
                                                       Mamba2HybridForCausalLM)
    from state_space_models_neuron_b200.parallel import state as ps
    ps.initialize_model_parallel(1)
    kw = dict(num_heads=4, head_dim=32, vocab_size=64, hidden_size=64, state_size=32, n_groups=2, dtype=torch.bfloat16)
    if hybrid:
        cls, cfg = Mamba2HybridForCausalLM, Mamba2HybridConfig(
            **kw, num_hidden_layers=4, attn_num_heads=4, attn_head_dim=16, attn_key_value_heads=2, mlp_hidden_size=128,
            hybrid_attention_ratio=0.25, hybrid_mlp_ratio=0.25)
    else:
        cls, cfg = Mamba2ForCausalLM, Mamba2Config(**kw, num_hidden_layers=2)
    m = cls(cfg).eval()
    with tempfile.TemporaryDirectory() as d:
        m.save_pretrained(d)
        again = cls.from_pretrained(d).eval()
    a, b = m.state_dict(), again.state_dict()
    assert a.keys() == b.keys()
    for k in a:
        assert a[k].dtype == b[k].dtype and torch.equal(a[k], b[k]), k
    assert any(v.dtype == torch.float32 for v in b.values()) and any(v.dtype == torch.bfloat16 for v in b.values())
