"""Split a HuggingFace-format Mamba-2 / hybrid checkpoint into per-TP-rank training shards.

    python shard_hf_checkpoint.py --input_dir HF_DIR --output_dir CKPT --tag hf_import --tp 8

Writes `CKPT/TAG/model/dp_rank_00_tp_rank_XX_pp_rank_00.pt`, `user_content.pt` and `newest`, the
inverse of merge_tp_checkpoints.py.  The reference's counterpart is `tp_loader`
(mamba2_inference_no_tp.py:142-165), which targets an older parameter naming and no longer works
with its own mixer.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from state_space_models_neuron_b200.models import Mamba2Config, Mamba2HybridConfig
from state_space_models_neuron_b200.parallel.checkpoint import shard_file_name
from state_space_models_neuron_b200.parallel.layout import shard_state_dict


def load_hf_state_dict(input_dir: str):
    st = os.path.join(input_dir, "model.safetensors")
    if os.path.exists(st):
        from safetensors.torch import load_file
        sd = load_file(st)
    else:
        sd = torch.load(os.path.join(input_dir, "pytorch_model.bin"), map_location="cpu", weights_only=False)
    with open(os.path.join(input_dir, "config.json")) as f:
        d = json.load(f)
    cls = Mamba2HybridConfig if d.get("model_type") == "mamba2hybrid" else Mamba2Config
    d.pop("model_type", None)
    config = cls(**d)
    if "lm_head.weight" not in sd and config.tie_word_embeddings:
        sd["lm_head.weight"] = sd["backbone.embeddings.weight"]
    return sd, config


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--input_dir", required=True)
    ap.add_argument("--output_dir", required=True)
    ap.add_argument("--tag", default="hf_import")
    ap.add_argument("--tp", type=int, required=True)
    args = ap.parse_args(argv)
    sd, config = load_hf_state_dict(args.input_dir)
    root = os.path.join(args.output_dir, args.tag)
    os.makedirs(os.path.join(root, "model"), exist_ok=True)
    for r in range(args.tp):
        torch.save(shard_state_dict(sd, config, args.tp, r), os.path.join(root, "model", shard_file_name(0, r)))
    torch.save({"global_step": 0, "config": config.to_dict()}, os.path.join(root, "user_content.pt"))
    for name, text in (("done", "ok"),):
        with open(os.path.join(root, name), "w") as f:
            f.write(text)
    with open(os.path.join(args.output_dir, "newest"), "w") as f:
        f.write(args.tag)
    print(f"wrote {args.tp} shards under {root}")


if __name__ == "__main__":
    main()
