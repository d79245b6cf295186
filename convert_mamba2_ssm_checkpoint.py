"""Convert a `state-spaces/mamba2-*` (mamba_ssm) or Codestral Mamba checkpoint to the HuggingFace layout
this framework loads with `Mamba2ForCausalLM.from_pretrained`.

    python convert_mamba2_ssm_checkpoint.py -i IN_DIR -m mamba_ssm|codestral -p fp32|fp16|bf16 -o OUT_DIR

Same options as the reference converter (convert_mamba2_ssm_checkpoint.py:173-226).  Inputs:
`config.json` + `pytorch_model.bin` (mamba_ssm) or `params.json` + `consolidated.safetensors`
(codestral); output `config.json` + `model.safetensors` (+ tokenizer files when they can be built
offline).  `--split_proj/-s` additionally writes the legacy `in_proj_{z,xBC,dt}` split tensors.
"""
from __future__ import annotations

import argparse
import json
import os
from typing import Dict, Optional

import torch

from state_space_models_neuron_b200.models import Mamba2Config, Mamba2ForCausalLM

_SOURCES = {
    "codestral": dict(hidden_size="dim", num_hidden_layers="n_layers", n_groups="n_groups", bos_token_id=0,
                      pad_token_id=1, eos_token_id=2, config_name="params.json", weights="consolidated.safetensors"),
    "mamba_ssm": dict(hidden_size="d_model", num_hidden_layers="n_layer", n_groups="ngroups", bos_token_id=0,
                      pad_token_id=0, eos_token_id=0, config_name="config.json", weights="pytorch_model.bin"),
}


def load_source_state_dict(directory: str, weights: str) -> Dict[str, torch.Tensor]:
    p = os.path.join(directory, weights)
    if weights.endswith(".safetensors"):
        from safetensors import safe_open
        out = {}
        with safe_open(p, framework="pt") as f:
            for k in f.keys():
                out[k[len("model."):] if k.startswith("model.") else k] = f.get_tensor(k).clone()
        return out
    return torch.load(p, map_location="cpu", weights_only=False)


def convert_ssm_config_to_hf_config(config_ssm: dict, source: dict) -> Mamba2Config:
    """mamba_ssm / codestral config -> Mamba2Config; the vocabulary is padded up to
    `pad_vocab_size_multiple` as the original models do."""
    ssm_cfg = config_ssm.get("ssm_cfg", {}) or {}
    hidden = config_ssm[source["hidden_size"]]
    head_dim = ssm_cfg.get("headdim", 64)
    expand = ssm_cfg.get("expand", 2)
    vocab = config_ssm["vocab_size"]
    mult = config_ssm.get("pad_vocab_size_multiple", 1)
    if vocab % mult:
        vocab += mult - vocab % mult
    n_groups = config_ssm.get(source["n_groups"], ssm_cfg.get("ngroups", 1))
    return Mamba2Config(
        hidden_size=hidden, head_dim=head_dim, expand=expand, num_heads=hidden * expand // head_dim,
        num_hidden_layers=config_ssm[source["num_hidden_layers"]], n_groups=n_groups,
        state_size=ssm_cfg.get("d_state", 128), vocab_size=vocab,
        tie_word_embeddings=config_ssm.get("tie_embeddings", True),
        residual_in_fp32=config_ssm.get("residual_in_fp32", False),
        bos_token_id=source["bos_token_id"], pad_token_id=source["pad_token_id"], eos_token_id=source["eos_token_id"])


def rename_keys(sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """mamba_ssm names (`backbone.embedding`) -> this framework's (`backbone.embeddings`)."""
    out = {}
    for k, v in sd.items():
        k = k.replace("backbone.embedding.", "backbone.embeddings.")
        out[k] = v
    return out


def split_projection_matrix(config: Mamba2Config, sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    out = {}
    d_in = config.num_heads * config.head_dim
    conv = d_in + 2 * config.n_groups * config.state_size
    for k, v in sd.items():
        if not k.endswith("in_proj.weight"):
            out[k] = v
            continue
        base = k[: -len(".in_proj.weight")]
        z, xbc, dt = torch.split(v, [d_in, conv, config.num_heads], dim=0)
        out[base + ".in_proj_z.weight"], out[base + ".in_proj_xBC.weight"] = z.clone(), xbc.clone()
        out[base + ".in_proj_dt.weight"] = dt.clone()
    return out


def save_tokenizer(model_type: str, output_dir: str, tokenizer_model_path: Optional[str]) -> bool:
    try:
        if model_type == "codestral" and tokenizer_model_path is not None:
            from transformers import LlamaTokenizerFast
            LlamaTokenizerFast(tokenizer_model_path, legacy=False, from_slow=True).save_pretrained(output_dir)
            return True
        if model_type == "mamba_ssm":
            from transformers import GPTNeoXTokenizerFast
            GPTNeoXTokenizerFast.from_pretrained("state-spaces/mamba-130m-hf", padding_side="left",
                                                 local_files_only=True).save_pretrained(output_dir)
            return True
    except Exception as e:  # no network / tokenizer not cached: weights are still converted
        print(f"tokenizer not saved ({type(e).__name__}: {e})")
    return False


def convert_mamba2_checkpoint_file_to_huggingface_model_file(mamba2_checkpoint_path: str, mamba2_model_type: str,
                                                             precision: str, output_dir: str,
                                                             tokenizer_model_path: Optional[str] = None,
                                                             split_proj: bool = False) -> None:
    source = _SOURCES[mamba2_model_type]
    with open(os.path.join(mamba2_checkpoint_path, source["config_name"]), encoding="utf-8") as f:
        config_ssm = json.load(f)
    hf_config = convert_ssm_config_to_hf_config(config_ssm, source)
    os.makedirs(output_dir, exist_ok=True)
    sd = rename_keys(load_source_state_dict(mamba2_checkpoint_path, source["weights"]))
    hf_config.dtype = torch.float32
    model = Mamba2ForCausalLM(hf_config)
    missing, unexpected = model.load_state_dict(sd, strict=False)
    missing = [m for m in missing if not (m == "lm_head.weight" and hf_config.tie_word_embeddings)]
    if missing or unexpected:
        raise RuntimeError(f"conversion mismatch: missing {missing}, unexpected {unexpected}")
    dtype = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}[precision]
    model = model.to(dtype)
    hf_config.dtype = dtype
    hf_config.save_pretrained(output_dir)
    from safetensors.torch import save_file, save_model
    if split_proj:
        tensors = split_projection_matrix(hf_config, model.state_dict())
        if hf_config.tie_word_embeddings:
            tensors.pop("lm_head.weight", None)
        save_file({k: v.contiguous() for k, v in tensors.items()}, os.path.join(output_dir, "model.safetensors"),
                  metadata={"format": "pt"})
    else:
        save_model(model, os.path.join(output_dir, "model.safetensors"), metadata={"format": "pt"})
    save_tokenizer(mamba2_model_type, output_dir, tokenizer_model_path)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("-i", "--mamba2_checkpoint_directory", type=str, required=True)
    ap.add_argument("-m", "--mamba2_model_type", type=str, default="mamba_ssm", choices=("codestral", "mamba_ssm"))
    ap.add_argument("-p", "--precision", type=str, default="fp16", choices=("fp32", "fp16", "bf16"))
    ap.add_argument("-o", "--output_dir", type=str, required=True)
    ap.add_argument("-t", "--tokenizer_model_path", type=str, default=None)
    ap.add_argument("-s", "--split_proj", action="store_true")
    a = ap.parse_args(argv)
    convert_mamba2_checkpoint_file_to_huggingface_model_file(
        a.mamba2_checkpoint_directory, a.mamba2_model_type, a.precision, a.output_dir, a.tokenizer_model_path, a.split_proj)


if __name__ == "__main__":
    main()
