"""The measured baseline: the same model, parallel layout and optimizer semantics run with library kernels only.

`enable()` switches every op of the framework to its plain PyTorch restatement on the GPU (cuBLAS GEMMs through
`F.linear`, ATen elementwise/reduction kernels for conv, scan, norms, cross entropy and AdamW) and the tensor-
parallel collectives to NCCL all-gather / reduce-scatter / all-reduce, unfused.  The SSD scan of the baseline is
the chunked block-decomposition in `ops/oracle.py` under activation checkpointing (its intermediates are
O(L * chunk * heads) per layer).  This is what `bench.py --impl baseline` times; the reference itself cannot run
on a B200 (Trainium-only dependencies).
"""
from __future__ import annotations

import torch
import torch.utils.checkpoint


def enable() -> None:
    from state_space_models_neuron_b200.ops import functional
    from state_space_models_neuron_b200.parallel import fused
    functional._BASELINE[0] = True
    fused.set_enabled(False)
    core = functional.mamba2_mixer_core

    def checkpointed_core(*args, **kwargs):
        if kwargs.get("return_final_states") or not torch.is_grad_enabled():
            return core(*args, **kwargs)
        return torch.utils.checkpoint.checkpoint(lambda *a: core(*a, **kwargs), *args, use_reentrant=False)

    import state_space_models_neuron_b200.ops as ops_pkg
    ops_pkg.mamba2_mixer_core = checkpointed_core
