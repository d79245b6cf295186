"""Ops: CUDA kernels for sm_100a on GPU tensors, the PyTorch oracle on CPU tensors."""
from . import oracle  # noqa: F401
from .functional import (  # noqa: F401
    add_rmsnorm, apply_rotary, attention, causal_conv1d_silu, ce_backward, ce_partials, embedding, gated_rmsnorm, gelu, glu, linear, linear_ce,
    mamba2_mixer_core, rmsnorm, rotary_tables, ssd_chunk_scan, ssm_decode_step,
)
