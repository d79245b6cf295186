"""Download (or read locally) a small text dataset and tokenise it with default settings; the single-process
convenience wrapper around tokenize_dataset.py that the reference ships as get_dataset.py (default dataset
`stas/openwebtext-10k`, tokenizer `EleutherAI/gpt-neox-20b`, seq_len 1024)."""
from __future__ import annotations

import argparse

import tokenize_dataset


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--dataset", default="stas/openwebtext-10k")
    ap.add_argument("--dataset_config", default=None)
    ap.add_argument("--tokenizer", default="EleutherAI/gpt-neox-20b")
    ap.add_argument("--seq_len", type=int, default=1024)
    ap.add_argument("--save_path", required=True)
    ap.add_argument("--format", default="hf", choices=["hf", "npy"])
    a = ap.parse_args(argv)
    cli = ["--dataset", a.dataset, "--tokenizer", a.tokenizer, "--seq_len", str(a.seq_len), "--save_path", a.save_path,
           "--format", a.format]
    if a.dataset_config:
        cli += ["--dataset_config", a.dataset_config]
    tokenize_dataset.main(cli)


if __name__ == "__main__":
    main()
