"""Sharded training checkpoints, in the directory layout the reference's tools consume.

    {dir}/{tag}/model/dp_rank_00_tp_rank_{TT}_pp_rank_00.pt     state_dict of TP rank TT (written by DP rank 0)
    {dir}/{tag}/optim/dp_rank_{DD}_tp_rank_{TT}_pp_rank_00.pt   optimizer shard of (DP rank DD, TP rank TT)
    {dir}/{tag}/scheduler.pt, {dir}/{tag}/user_content.pt       written by global rank 0
    {dir}/newest                                                tag of the newest complete checkpoint

(layout: training_utils.py:404-422,508-516,533-540 and merge_tp_checkpoints.py:99 of the reference;
call sites train.py:56-63,163-176).  Every file is written to a temporary name and renamed, `newest`
is updated last, and old tags beyond `num_kept_ckpts` are removed by rank 0, so a crash never leaves a
half-written checkpoint selected.  Unlike the reference's loader this one can also restore optimizer,
scheduler and the step counter.
"""
from __future__ import annotations

import os
import shutil
import threading
from typing import Any, Dict, List, Optional

import torch

from . import state as ps

_async_threads: List[threading.Thread] = []


def shard_file_name(dp_rank: int, tp_rank: int, pp_rank: int = 0) -> str:
    return f"dp_rank_{dp_rank:02d}_tp_rank_{tp_rank:02d}_pp_rank_{pp_rank:02d}.pt"


def _atomic_save(obj: Any, path: str) -> None:
    tmp = path + ".tmp"
    torch.save(obj, tmp)
    os.replace(tmp, path)


def _atomic_write_text(text: str, path: str) -> None:
    tmp = path + ".tmp"
    with open(tmp, "w") as f:
        f.write(text)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)


def _cpu_state_dict(sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    out = {}
    for k, v in sd.items():
        out[k] = v.detach().to("cpu", copy=True) if isinstance(v, torch.Tensor) else v
    return out


def list_tags(checkpoint_dir: str) -> List[str]:
    if not os.path.isdir(checkpoint_dir):
        return []
    tags = [d for d in os.listdir(checkpoint_dir)
            if os.path.isdir(os.path.join(checkpoint_dir, d)) and os.path.exists(os.path.join(checkpoint_dir, d, "done"))]
    tags.sort(key=lambda t: os.path.getmtime(os.path.join(checkpoint_dir, t, "done")))
    return tags


def wait_for_async_saves() -> None:
    while _async_threads:
        _async_threads.pop().join()


def save_checkpoint(checkpoint_dir: str, tag: str, model=None, optimizer=None, scheduler=None,
                    user_content: Optional[dict] = None, num_workers: int = 8, use_xser: bool = False,
                    num_kept_ckpts: Optional[int] = None, async_save: bool = False) -> None:
    """Collective: every rank calls it.  `num_workers` and `use_xser` are accepted for call
    compatibility (train.py:163-176 of the reference) and ignored."""
    wait_for_async_saves()
    root = os.path.join(checkpoint_dir, tag)
    dp, tp = ps.get_data_parallel_rank(), ps.get_tensor_model_parallel_rank()
    os.makedirs(os.path.join(root, "model"), exist_ok=True)
    os.makedirs(os.path.join(root, "optim"), exist_ok=True)
    jobs = []
    if model is not None and dp == 0:
        sd = model if isinstance(model, dict) else model.state_dict()
        jobs.append((_cpu_state_dict(sd), os.path.join(root, "model", shard_file_name(0, tp))))
    if optimizer is not None:
        sharded = getattr(optimizer, "shard", False)
        if sharded or dp == 0:
            osd = optimizer if isinstance(optimizer, dict) else optimizer.state_dict()
            jobs.append((osd, os.path.join(root, "optim", shard_file_name(dp if sharded else 0, tp))))
    if ps.get_rank() == 0:
        if scheduler is not None:
            jobs.append((scheduler.state_dict(), os.path.join(root, "scheduler.pt")))
        if user_content is not None:
            jobs.append((user_content, os.path.join(root, "user_content.pt")))

    def write_files():
        for obj, path in jobs:
            _atomic_save(obj, path)

    def publish():
        _atomic_write_text("ok", os.path.join(root, "done"))
        _atomic_write_text(tag, os.path.join(checkpoint_dir, "newest"))
        if num_kept_ckpts is not None and num_kept_ckpts > 0:
            for old in list_tags(checkpoint_dir)[:-num_kept_ckpts]:
                shutil.rmtree(os.path.join(checkpoint_dir, old), ignore_errors=True)

    if async_save and ps.get_world_size() == 1:
        # tensors were already copied to host memory above; only file IO runs in the thread
        t = threading.Thread(target=lambda: (write_files(), publish()), daemon=False)
        t.start()
        _async_threads.append(t)
        return
    write_files()
    ps.barrier()
    if ps.get_rank() == 0:
        publish()
    ps.barrier()


def newest_tag(checkpoint_dir: str) -> Optional[str]:
    path = os.path.join(checkpoint_dir, "newest")
    if not os.path.exists(path):
        return None
    with open(path) as f:
        return f.read().strip() or None


def load_checkpoint(checkpoint_dir: str, tag: Optional[str] = None, model=None, optimizer=None, scheduler=None,
                    strict: bool = True) -> Optional[dict]:
    """Load this rank's shards; returns user_content (or None).  tag None -> the `newest` file."""
    tag = tag or newest_tag(checkpoint_dir)
    if tag is None:
        raise FileNotFoundError(f"no checkpoint tag given and no 'newest' file under {checkpoint_dir}")
    root = os.path.join(checkpoint_dir, tag)
    dp, tp = ps.get_data_parallel_rank(), ps.get_tensor_model_parallel_rank()
    if model is not None:
        path = os.path.join(root, "model", shard_file_name(0, tp))
        sd = torch.load(path, map_location="cpu", weights_only=False)
        missing, unexpected = model.load_state_dict(sd, strict=False)
        tied = set(getattr(model, "_tied_weights_keys", None) or [])
        missing = [m for m in missing if m not in tied]
        if strict and (missing or unexpected):
            raise RuntimeError(f"checkpoint {path}: missing keys {missing}, unexpected keys {unexpected}")
    if optimizer is not None:
        sharded = getattr(optimizer, "shard", False)
        path = os.path.join(root, "optim", shard_file_name(dp if sharded else 0, tp))
        optimizer.load_state_dict(torch.load(path, map_location="cpu", weights_only=False))
    if scheduler is not None:
        scheduler.load_state_dict(torch.load(os.path.join(root, "scheduler.pt"), map_location="cpu", weights_only=False))
    uc = os.path.join(root, "user_content.pt")
    return torch.load(uc, map_location="cpu", weights_only=False) if os.path.exists(uc) else None
