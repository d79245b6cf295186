"""The measured baseline: the same model, parallel layout and optimizer semantics run with library kernels only.

`enable()` switches every op of the framework to plain PyTorch on the GPU (cuBLAS GEMMs through `F.linear`, cuDNN /
ATen kernels for conv, norms, cross entropy and AdamW) and the tensor-parallel collectives to NCCL all-gather /
reduce-scatter / all-reduce, unfused.  The mixer core is `baseline/torch_mixer.py`: the block-decomposed SSD scan
written with `einsum` (bf16 operands for the large contractions, fp32 decays), differentiated by autograd, without
activation checkpointing.  `checkpoint_mixer=True` wraps the mixer core in `torch.utils.checkpoint` for runs whose
activations would not fit otherwise (the 7B model on ONE GPU: 126 GB of weights, gradients and optimizer state leave
too little room for 64 layers of saved scan intermediates).  This is what `bench.py --impl baseline` times; the
reference itself cannot run on a B200 (Trainium-only dependencies).
"""
from __future__ import annotations

import torch
import torch.utils.checkpoint


def enable(checkpoint_mixer: bool = False) -> None:
    from state_space_models_neuron_b200.ops import functional
    from state_space_models_neuron_b200.parallel import fused
    from . import torch_mixer
    functional._BASELINE[0] = True
    fused.set_enabled(False)
    fallback = functional.mamba2_mixer_core

    def core(*args, **kwargs):
        if kwargs.get("return_final_states") or not args[0].is_cuda:
            return fallback(*args, **kwargs)
        kwargs.pop("recompute", None)
        kwargs.pop("return_final_states", None)
        if checkpoint_mixer and torch.is_grad_enabled():
            return torch.utils.checkpoint.checkpoint(lambda *a: torch_mixer.mixer_core(*a, **kwargs), *args,
                                                     use_reentrant=False)
        return torch_mixer.mixer_core(*args, **kwargs)

    import state_space_models_neuron_b200.ops as ops_pkg
    ops_pkg.mamba2_mixer_core = core
