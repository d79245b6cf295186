"""Top-level runtime API: one config object, model and optimizer factories, checkpoint calls.

The calls mirror how the reference drives `neuronx_distributed` (train.py:71-78,129-138,163-176,56-63):

    cfg = parallel_config(tensor_parallel_size=8, optimizer_config={"zero_one_enabled": True, ...},
                          sequence_parallel=True, mixed_precision_config={...})
    model = initialize_parallel_model(cfg, get_model)
    optim = initialize_parallel_optimizer(cfg, torch.optim.AdamW, param_groups, lr=..., betas=...)
    save_checkpoint(...), load_checkpoint(...)
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

from . import state as ps
from .checkpoint import load_checkpoint, save_checkpoint  # noqa: F401
from .layers import set_init_seed
from .zero1 import Zero1Optimizer


def parallel_config(tensor_parallel_size: int = 1, optimizer_config: Optional[dict] = None,
                    sequence_parallel: bool = False, mixed_precision_config: Optional[dict] = None,
                    model_init_config: Optional[dict] = None, backend: Optional[str] = None,
                    fused_comm: bool = True, init_seed: int = 1234, device: Optional[str] = None) -> dict:
    oc = {"zero_one_enabled": False, "grad_clipping": True, "max_grad_norm": 1.0}
    oc.update(optimizer_config or {})
    mpc = {"use_master_weights": True, "use_fp32_grad_acc": True, "use_master_weights_in_ckpt": False}
    mpc.update(mixed_precision_config or {})
    return {"tensor_parallel_size": int(tensor_parallel_size), "optimizer_config": oc,
            "sequence_parallel": bool(sequence_parallel), "mixed_precision_config": mpc,
            "model_init_config": model_init_config, "backend": backend, "fused_comm": bool(fused_comm),
            "init_seed": int(init_seed), "device": device}


# name used by the reference's scripts
neuronx_distributed_config = parallel_config


def default_device() -> torch.device:
    if torch.cuda.is_available():
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def initialize_parallel_model(cfg: dict, model_fn: Callable[[], torch.nn.Module]) -> torch.nn.Module:
    """Create the process groups (if not done), build the rank's shard of the model and move it
    to the rank's device.  `model_fn` builds the model; the parallel layers inside read the TP
    rank from `parallel.state` and only ever hold their own shard."""
    if not ps.model_parallel_is_initialized() or ps.get_tensor_model_parallel_size() != cfg["tensor_parallel_size"]:
        ps.initialize_model_parallel(cfg["tensor_parallel_size"], backend=cfg.get("backend"))
    set_init_seed(cfg.get("init_seed", 1234))
    from . import fused
    fused.set_enabled(cfg.get("fused_comm", True))
    model = model_fn()
    device = torch.device(cfg["device"]) if cfg.get("device") else default_device()
    model = model.to(device)
    if getattr(model.config, "tie_word_embeddings", False) and hasattr(model, "lm_head"):
        model.lm_head.weight = model.get_input_embeddings().weight
    return model


def initialize_parallel_optimizer(cfg: dict, optimizer_cls, param_groups, lr: float, betas=(0.9, 0.999),
                                  eps: float = 1e-8, weight_decay: float = 0.0) -> Zero1Optimizer:
    """AdamW over flat buffers with (ZeRO-1) or without sharding of the state over DP.  Only AdamW
    semantics are implemented; `optimizer_cls` is inspected for the reference's choice between
    fp32 optimizer parameters (`AdamW_FP32OptimParams`, default) and plain low-precision AdamW
    (`--no_optimizer_fp32`, train.py:123-126)."""
    oc, mpc = cfg["optimizer_config"], cfg["mixed_precision_config"]
    name = getattr(optimizer_cls, "__name__", str(optimizer_cls))
    fp32_master = mpc.get("use_master_weights", True) and "LowPrecision" not in name
    first = next(iter(param_groups))
    p0 = first["params"][0] if isinstance(first, dict) else first
    master_dtype = torch.float32 if fp32_master else p0.dtype
    return Zero1Optimizer(param_groups, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                          shard=oc.get("zero_one_enabled", False),
                          max_grad_norm=oc.get("max_grad_norm", 1.0) if oc.get("grad_clipping", True) else None,
                          master_dtype=master_dtype)


class AdamW_FP32OptimParams:  # marker classes for the optimizer_cls argument
    """AdamW with fp32 master weights and moments (the default)."""


class AdamW_LowPrecision:
    """AdamW with state in the parameter dtype (`--no_optimizer_fp32`)."""
