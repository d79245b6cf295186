"""Input pipeline: pre-tokenised fixed-length samples -> per-DP-rank batches -> device prefetch.

Covers the reference's data path (nxd_training_utils.py:99-127 `create_llama_pretraining_dataset`,
:29-62 `pack_dataset`, :77-96 weight-decay groups; train.py:147-157 `MpDeviceLoader`):
  * a dataset saved by HuggingFace `datasets.save_to_disk` with `input_ids` and `labels` columns,
    or a directory holding `tokens.npy` (int32 `[samples, seq_len]`, memory mapped),
  * `DistributedSampler(shuffle=False, drop_last=True)` over the data-parallel group,
  * `DeviceLoader`: pinned host batches copied to the GPU on a side stream one batch ahead, the
    CUDA replacement for the XLA `MpDeviceLoader`,
  * `SyntheticDataset`: uniform random token ids for benchmarks.
"""
from __future__ import annotations

import os
import threading
from itertools import chain
from typing import Dict, Iterator, List, Optional

import numpy as np
import torch
from torch.utils.data import DataLoader, Dataset, DistributedSampler


class TokenArrayDataset(Dataset):
    """`tokens.npy` int32 [samples, seq_len]; labels are a copy of the ids (the model shifts)."""

    def __init__(self, path: str):
        f = path if path.endswith(".npy") else os.path.join(path, "tokens.npy")
        self.tokens = np.load(f, mmap_mode="r")

    def __len__(self):
        return self.tokens.shape[0]

    def __getitem__(self, i):
        ids = torch.from_numpy(np.asarray(self.tokens[i], dtype=np.int64))
        return {"input_ids": ids, "labels": ids.clone()}


class SyntheticDataset(Dataset):
    """Uniform random token ids in [0, vocab), deterministic per index."""

    def __init__(self, vocab_size: int, seq_len: int, num_samples: int = 1 << 20, seed: int = 0):
        self.vocab_size, self.seq_len, self.num_samples, self.seed = vocab_size, seq_len, num_samples, seed

    def __len__(self):
        return self.num_samples

    def __getitem__(self, i):
        g = torch.Generator().manual_seed(self.seed * 1000003 + i)
        ids = torch.randint(0, self.vocab_size, (self.seq_len,), generator=g)
        return {"input_ids": ids, "labels": ids.clone()}


def _collate(samples: List[Dict]) -> Dict[str, torch.Tensor]:
    out = {}
    for k in samples[0]:
        out[k] = torch.stack([torch.as_tensor(s[k], dtype=torch.long) for s in samples])
    return out


def load_token_dataset(data_dir: str) -> Dataset:
    if os.path.exists(os.path.join(data_dir, "tokens.npy")) or data_dir.endswith(".npy"):
        return TokenArrayDataset(data_dir)
    import datasets  # HuggingFace datasets, save_to_disk format
    ds = datasets.load_from_disk(data_dir)
    keep = [c for c in ds.column_names if c in ("input_ids", "labels")]
    return ds.with_format("torch", columns=keep)


def create_pretraining_dataset(data_dir: Optional[str], mini_batch_size: int, dp_size: int, dp_rank: int, seed: int,
                               synthetic: Optional[SyntheticDataset] = None):
    """Returns (dataloader, sampler); batches are dicts of pinned int64 tensors `[mbs, seq_len]`."""
    data = synthetic if synthetic is not None else load_token_dataset(data_dir)
    sampler = DistributedSampler(data, num_replicas=dp_size, rank=dp_rank, shuffle=False, drop_last=True)
    g = torch.Generator().manual_seed(seed)
    loader = DataLoader(data, collate_fn=_collate, sampler=sampler, batch_size=mini_batch_size, num_workers=0,
                        drop_last=True, pin_memory=torch.cuda.is_available(), generator=g)
    return loader, sampler


# name used by the reference's train.py
create_llama_pretraining_dataset = create_pretraining_dataset


class DeviceLoader:
    """Iterates a host loader one batch ahead: the next batch's host->device copies are issued on a
    side stream while the current step computes; `__next__` makes the compute stream wait on them."""

    def __init__(self, loader, device):
        self.loader, self.device = loader, torch.device(device)
        self.stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None

    def __len__(self):
        return len(self.loader)

    def _to_device(self, batch):
        if self.stream is None:
            return batch, None
        with torch.cuda.stream(self.stream):
            out = {k: v.to(self.device, non_blocking=True) for k, v in batch.items()}
            ev = torch.cuda.Event()
            ev.record(self.stream)
        return out, ev

    def __iter__(self) -> Iterator[Dict[str, torch.Tensor]]:
        it = iter(self.loader)
        try:
            nxt = self._to_device(next(it))
        except StopIteration:
            return
        while nxt is not None:
            cur, ev = nxt
            try:
                nxt = self._to_device(next(it))
            except StopIteration:
                nxt = None
            if ev is not None:
                torch.cuda.current_stream(self.device).wait_event(ev)
                for v in cur.values():
                    v.record_stream(torch.cuda.current_stream(self.device))
            yield cur


def pack_token_lists(token_lists, chunk_length: int) -> np.ndarray:
    """Concatenate tokenised documents and cut into `chunk_length` blocks, dropping the tail
    (tokenize_dataset.py:52-65 of the reference)."""
    flat = np.fromiter(chain.from_iterable(token_lists), dtype=np.int32)
    n = (flat.shape[0] // chunk_length) * chunk_length
    return flat[:n].reshape(-1, chunk_length)


def get_param_groups_by_weight_decay(model, weight_decay: float = 0.01,
                                     no_decay=("bias", "LayerNorm", "norm", "A", "D")):
    """Two AdamW groups: names containing any `no_decay` substring get weight decay 0
    (train.py:110-121 of the reference: dt_bias, conv1d.bias, every norm, A_log, D)."""
    named = list(model.named_parameters())
    return [
        {"params": [p for n, p in named if not any(nd in n for nd in no_decay)], "weight_decay": weight_decay},
        {"params": [p for n, p in named if any(nd in n for nd in no_decay)], "weight_decay": 0.0},
    ]
