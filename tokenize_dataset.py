"""Tokenise a text dataset into fixed-length training samples.

    python tokenize_dataset.py --dataset NAME_OR_DIR [--dataset_config CFG] --tokenizer TOK --seq_len 2048 \
        --save_path OUT [--num_proc N] [--dryrun] [--format hf|npy]

Same options as the reference script (tokenize_dataset.py:8-17): documents are tokenised, concatenated and cut
into `seq_len` blocks (tail dropped), `labels` is a copy of `input_ids` (the model shifts them).  Sources: a
HuggingFace hub dataset name, a directory written by `datasets.save_to_disk`, or local `.txt` / `.jsonl` files
(`--dataset path/to/file`), so the script also works without network access.  `--format hf` writes a
`datasets.save_to_disk` directory as the reference does; `--format npy` writes `tokens.npy` (int32
[samples, seq_len]) which `utils.data.TokenArrayDataset` memory-maps.
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np


def load_raw(dataset: str, config, num_proc: int):
    import datasets
    if os.path.isdir(dataset) and os.path.exists(os.path.join(dataset, "dataset_info.json")):
        ds = datasets.load_from_disk(dataset)
        return ds["train"] if isinstance(ds, datasets.DatasetDict) else ds
    if os.path.isfile(dataset):
        if dataset.endswith(".jsonl") or dataset.endswith(".json"):
            with open(dataset) as f:
                rows = [json.loads(line) for line in f if line.strip()]
            key = "text" if "text" in rows[0] else list(rows[0].keys())[0]
            return datasets.Dataset.from_dict({"text": [r[key] for r in rows]})
        with open(dataset) as f:
            return datasets.Dataset.from_dict({"text": [ln for ln in f.read().split("\n\n") if ln.strip()]})
    raw = datasets.load_dataset(dataset, config, num_proc=num_proc if num_proc > 1 else None)
    return raw["train"]


def tokenize_and_pack(train, tokenizer, seq_len: int, num_proc: int = 1):
    from state_space_models_neuron_b200.utils.data import pack_token_lists
    cols = train.column_names
    text_col = "text" if "text" in cols else cols[0]
    tok = train.map(lambda ex: {"input_ids": tokenizer(ex[text_col])["input_ids"]}, batched=True, remove_columns=cols,
                    num_proc=num_proc if num_proc > 1 else None, desc="Running tokenizer on dataset")
    block = min(seq_len, getattr(tokenizer, "model_max_length", seq_len) or seq_len)
    if seq_len > block:
        print("block_size > tokenizer.model_max_length")
    return pack_token_lists(tok["input_ids"], block)


def save(tokens: np.ndarray, save_path: str, fmt: str) -> None:
    os.makedirs(save_path, exist_ok=True)
    if fmt == "npy":
        np.save(os.path.join(save_path, "tokens.npy"), tokens.astype(np.int32))
    else:
        import datasets
        ids = tokens.tolist()
        datasets.Dataset.from_dict({"input_ids": ids, "labels": ids}).save_to_disk(save_path)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--dataset", required=True, help="HF dataset name, save_to_disk directory, or .txt/.jsonl file")
    ap.add_argument("--dataset_config", default=None)
    ap.add_argument("--tokenizer", default="EleutherAI/gpt-neox-20b")
    ap.add_argument("--seq_len", type=int, default=1024)
    ap.add_argument("--save_path", required=True)
    ap.add_argument("--num_proc", type=int, default=1)
    ap.add_argument("--dryrun", action="store_true", help="tokenise only 8192 samples")
    ap.add_argument("--format", default="hf", choices=["hf", "npy"])
    args = ap.parse_args(argv)
    from transformers import AutoTokenizer
    train = load_raw(args.dataset, args.dataset_config, args.num_proc)
    if args.dryrun:
        train = train.shuffle(seed=42).select(range(min(8192, len(train))))
    tokenizer = AutoTokenizer.from_pretrained(args.tokenizer)
    tokens = tokenize_and_pack(train, tokenizer, args.seq_len, args.num_proc)
    print(f"Samples in dataset: {tokens.shape[0]}")
    save(tokens, os.path.expanduser(args.save_path), args.format)


if __name__ == "__main__":
    main()
