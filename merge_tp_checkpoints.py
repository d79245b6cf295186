"""Merge the per-TP-rank model shards of a training checkpoint into one HuggingFace state dict.

    python merge_tp_checkpoints.py --mamba2_checkpoint_directory CKPT/TAG/model --output_dir OUT

Same command line as the reference tool (merge_tp_checkpoints.py:82-101) which only handles
Mamba2-7B at TP=8; this one reads the model config from `TAG/user_content.pt` (or --config) and the
TP degree from the files present, and writes `pytorch_model.bin` (+ `config.json`, and
`model.safetensors` with --safetensors) loadable by `Mamba2ForCausalLM.from_pretrained`.
"""
from __future__ import annotations

import argparse
import glob
import json
import os
import re

import torch

from state_space_models_neuron_b200.models import Mamba2Config, Mamba2HybridConfig
from state_space_models_neuron_b200.parallel.layout import merge_state_dicts


def find_shards(model_dir: str):
    files = glob.glob(os.path.join(model_dir, "dp_rank_00_tp_rank_*_pp_rank_00.pt"))
    by_rank = {int(re.search(r"tp_rank_(\d+)", os.path.basename(f)).group(1)): f for f in files}
    if not by_rank or sorted(by_rank) != list(range(len(by_rank))):
        raise FileNotFoundError(f"expected dp_rank_00_tp_rank_XX_pp_rank_00.pt for ranks 0..T-1 under {model_dir}")
    return [by_rank[r] for r in range(len(by_rank))]


def load_config(model_dir: str, config_path=None):
    if config_path:
        with open(config_path) as f:
            d = json.load(f)
    else:
        uc = os.path.join(os.path.dirname(os.path.normpath(model_dir)), "user_content.pt")
        d = torch.load(uc, map_location="cpu", weights_only=False)["config"]
    d = dict(d)
    cls = Mamba2HybridConfig if d.get("model_type") == "mamba2hybrid" else Mamba2Config
    d.pop("model_type", None)
    return cls(**d)


def merge_tp_ckpts(model_dir: str, config=None, config_path=None):
    config = config or load_config(model_dir, config_path)
    shards = [torch.load(f, map_location="cpu", weights_only=False) for f in find_shards(model_dir)]
    return merge_state_dicts(shards, config), config


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--mamba2_checkpoint_directory", required=True, help=".../TAG/model")
    ap.add_argument("--output_dir", required=True)
    ap.add_argument("--config", default=None, help="config.json (default: TAG/user_content.pt)")
    ap.add_argument("--safetensors", action="store_true")
    args = ap.parse_args(argv)
    merged, config = merge_tp_ckpts(args.mamba2_checkpoint_directory, config_path=args.config)
    os.makedirs(args.output_dir, exist_ok=True)
    config.sequence_parallel_enabled = False
    config.save_pretrained(args.output_dir)
    if config.tie_word_embeddings:
        merged.pop("lm_head.weight", None)
    if args.safetensors:
        from safetensors.torch import save_file
        save_file({k: v.contiguous() for k, v in merged.items()}, os.path.join(args.output_dir, "model.safetensors"),
                  metadata={"format": "pt"})
    else:
        torch.save(merged, os.path.join(args.output_dir, "pytorch_model.bin"))
    print(f"merged {len(merged)} tensors into {args.output_dir}")


if __name__ == "__main__":
    main()
