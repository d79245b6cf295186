"""Public op entry points.

Every function takes torch tensors.  CUDA tensors go to the hand-written sm_100a kernels in
`ops/csrc` (through `ops/cuda_ops.py`; a missing native library is an error there, never a silent
fallback).  CPU tensors run the plain PyTorch restatement in `ops/oracle.py`, differentiated by
autograd, which is also what the kernel tests compare against.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import oracle


# Measurement switch used only by `baseline/nccl_cublas.py`: run the PyTorch/cuBLAS restatement on GPU tensors.
_BASELINE = [False]


def _cuda():
    from . import cuda_ops
    return cuda_ops


def _native(t) -> bool:
    return t.is_cuda and not _BASELINE[0]


# ---- GEMM ---------------------------------------------------------------------------------
def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x @ weight^T (+ bias); weight is [out, in]."""
    if _native(x):
        return _cuda().linear(x, weight, bias)
    return F.linear(x, weight, bias)


def linear_ce(x: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, vocab_start: int = 0):
    """(x @ weight^T, statistics): on the GPU path the GEMM epilogue also delivers the per-row cross-entropy
    statistics (max, sum-exp, target logit) of this vocabulary shard; elsewhere statistics is None and the
    cross entropy computes them itself."""
    if _native(x) and x.dtype == torch.bfloat16:
        return _cuda().linear_ce(x, weight, labels, vocab_start)
    return F.linear(x, weight), None


def rotary_tables(seq_len: int, dim: int, theta: float, device=None, offset: int = 0):
    """cos / sin tables [seq_len, dim / 2] in fp32 (cached on the GPU path)."""
    if device is not None and torch.device(device).type == "cuda" and not _BASELINE[0]:
        return _cuda().rotary_tables(seq_len, dim, theta, device, offset)
    return oracle.rotary_tables(seq_len, dim, theta, device=device, offset=offset)


def apply_rotary(x, cos, sin):
    """Rotary position embedding (rotate-half) on the leading channels of every head of x [B, L, H, Dh]."""
    if _native(x) and x.dtype == torch.bfloat16:
        return _cuda().apply_rotary(x, cos, sin)
    return oracle.apply_rotary(x, cos, sin)


# ---- conv ---------------------------------------------------------------------------------
def causal_conv1d_silu(x, weight, bias, initial_state=None):
    """Depthwise causal conv (taps = weight.shape[-1]) + SiLU on channels-last x [B,L,C]."""
    if _native(x):
        return _cuda().causal_conv1d_silu(x, weight, bias, initial_state)
    return oracle.causal_conv1d_silu(x, weight, bias, initial_state)


# ---- norms --------------------------------------------------------------------------------
def gated_rmsnorm(y, z, weight, eps: float, group_size: Optional[int] = None):
    if _native(y):
        return _cuda().gated_rmsnorm(y, z, weight, eps, group_size)
    return oracle.gated_rmsnorm(y, z, weight, eps, group_size)


def rmsnorm(x, weight, eps: float):
    if _native(x):
        return _cuda().rmsnorm(x, weight, eps)
    return oracle.rmsnorm(x, weight, eps)


def add_rmsnorm(x, residual, weight, eps: float, residual_dtype=None):
    """(residual + x) -> (normed in x.dtype, new residual).  residual may be None."""
    if _native(x):
        return _cuda().add_rmsnorm(x, residual, weight, eps, residual_dtype)
    rd = residual_dtype or x.dtype
    r = x.to(rd) if residual is None else residual.to(rd) + x.to(rd)
    return oracle.rmsnorm(r, weight, eps).to(x.dtype), r


# ---- SSD scan -----------------------------------------------------------------------------
def ssd_chunk_scan(x, dt_raw, A, Bm, Cm, D, dt_bias, chunk_size: int = 128,
                   initial_state=None, return_final_state: bool = False):
    """y = SSD(x, softplus(dt_raw + dt_bias), A, B, C) + D x.

    x [B,L,H,P]; dt_raw [B,L,H]; A,D,dt_bias [H]; Bm,Cm [B,L,G,N].  Returns y (x's dtype) and, if
    asked, the final state [B,H,P,N] in fp32.
    """
    if _native(x):
        return _cuda().ssd_chunk_scan(x, dt_raw, A, Bm, Cm, D, dt_bias, chunk_size,
                                      initial_state, return_final_state)
    dt = oracle.softplus(dt_raw.float() + dt_bias.float())
    y, S = oracle.ssd_chunked(x, dt, A, Bm, Cm, D, chunk_size, initial_state)
    y = y.to(x.dtype)
    return (y, S) if return_final_state else y


def mamba2_mixer_core(zxBCdt, conv_w, conv_b, dt_bias, A_log, D, norm_w, *, d_inner: int,
                      n_groups: int, d_state: int, head_dim: int, eps: float,
                      norm_group_size: Optional[int], chunk_size: int = 128,
                      recompute: bool = False, return_final_states: bool = False):
    """Everything between in_proj and out_proj of a Mamba-2 mixer.

    zxBCdt [B, L, d_inner + (d_inner + 2 G N) + H] is split into z | xBC | dt; then
    conv+SiLU -> softplus(dt + bias) -> SSD scan -> gated group RMSNorm.
    The counterpart of the reference's fused driver kernels (mamba2/fused_kernel.py:251-282 fwd,
    285-420 bwd); `recompute` chooses between its two autograd variants (fused_kernel.py:423-471):
    keep the intermediates of the forward pass, or rebuild them from zxBCdt in backward.
    Returns out [B,L,d_inner] and optionally (conv_state [B,C,K], ssm_state [B,H,P,N]).
    """
    if _native(zxBCdt):
        return _cuda().mamba2_mixer_core(zxBCdt, conv_w, conv_b, dt_bias, A_log, D, norm_w, d_inner,
                                         n_groups, d_state, head_dim, eps, norm_group_size, chunk_size,
                                         recompute, return_final_states)
    Bsz, L, _ = zxBCdt.shape
    conv_dim = d_inner + 2 * n_groups * d_state
    H = d_inner // head_dim
    z = zxBCdt[..., :d_inner]
    xBC = zxBCdt[..., d_inner:d_inner + conv_dim]
    dt_raw = zxBCdt[..., d_inner + conv_dim:]
    K = conv_w.shape[-1]
    act = oracle.causal_conv1d_silu(xBC, conv_w.reshape(conv_dim, K), conv_b)
    x = act[..., :d_inner].reshape(Bsz, L, H, head_dim)
    Bm = act[..., d_inner:d_inner + n_groups * d_state].reshape(Bsz, L, n_groups, d_state)
    Cm = act[..., d_inner + n_groups * d_state:].reshape(Bsz, L, n_groups, d_state)
    A = -torch.exp(A_log.float())
    dt = oracle.softplus(dt_raw.float() + dt_bias.float())
    y, S = oracle.ssd_chunked(x, dt, A, Bm, Cm, D, chunk_size)
    y = y.reshape(Bsz, L, d_inner).to(zxBCdt.dtype)
    out = oracle.gated_rmsnorm(y, z, norm_w, eps, norm_group_size)
    if return_final_states:
        tail = xBC[:, -K:, :] if L >= K else torch.cat(
            [xBC.new_zeros(Bsz, K - L, conv_dim), xBC], dim=1)
        return out, (tail.transpose(1, 2).contiguous(), S)
    return out


# ---- decode -------------------------------------------------------------------------------
def ssm_decode_step(zxBCdt, conv_state, ssm_state, conv_w, conv_b, dt_bias, A_log, D, norm_w, *,
                    d_inner: int, n_groups: int, d_state: int, head_dim: int, eps: float,
                    norm_group_size: Optional[int]):
    """One token through conv state roll, SSM state update and the gated norm.

    zxBCdt [B, d_inner + C + H]; conv_state [B,C,K] and ssm_state [B,H,P,N] are updated in place.
    Fuses what the reference does in three places: the decode kernel
    (mamba2/mamba2_kernel_inference.py:26-104), softplus in torch (mamba2/mamba2_mixer.py:267) and the
    torch gated norm (mamba2/mamba2_mixer.py:279).
    """
    if _native(zxBCdt):
        return _cuda().ssm_decode_step(zxBCdt, conv_state, ssm_state, conv_w, conv_b, dt_bias, A_log, D,
                                       norm_w, d_inner, n_groups, d_state, head_dim, eps, norm_group_size)
    conv_dim = d_inner + 2 * n_groups * d_state
    z = zxBCdt[:, :d_inner]
    xBC = zxBCdt[:, d_inner:d_inner + conv_dim]
    dt_raw = zxBCdt[:, d_inner + conv_dim:]
    A = -torch.exp(A_log.float())
    y = oracle.decode_step(xBC, dt_raw, conv_state, ssm_state, conv_w, conv_b, dt_bias, A, D,
                           d_inner, n_groups, d_state, head_dim)
    return oracle.gated_rmsnorm(y.to(zxBCdt.dtype), z, norm_w, eps, norm_group_size)


# ---- attention ----------------------------------------------------------------------------
def attention(q, k, v, causal: bool = True):
    """GQA flash attention; q [B,L,Hq,Dh], k/v [B,L,Hkv,Dh]."""
    if _native(q):
        return _cuda().attention(q, k, v, causal)
    return oracle.attention(q, k, v, causal)


def gelu(x):
    if _native(x):
        return _cuda().gelu(x)
    return F.gelu(x)


def glu(h, act: str = "silu"):
    """Gated linear unit on h = [gate | up]: act(gate) * up (act gelu or silu)."""
    S = h.shape[-1] // 2
    if _native(h) and h.dtype == torch.bfloat16 and h.shape[-1] % 16 == 0 and act in ("gelu", "silu", "swish"):
        return _cuda().glu(h, act)
    gate, up = h[..., :S], h[..., S:]
    a = F.gelu(gate) if act == "gelu" else F.relu(gate) if act == "relu" else F.silu(gate)
    return a * up


# ---- embedding ----------------------------------------------------------------------------
def embedding(ids, weight, vocab_start: int = 0):
    """Vocabulary-shard lookup: rows `weight[ids - vocab_start]`, zeros for ids outside the shard."""
    if _native(weight):
        return _cuda().embedding(ids, weight, vocab_start)
    local = ids - vocab_start
    inside = (local >= 0) & (local < weight.shape[0])
    return F.embedding(torch.where(inside, local, torch.zeros_like(local)), weight) * inside[..., None].to(weight.dtype)


# ---- cross entropy ------------------------------------------------------------------------
def ce_partials(logits, labels, vocab_start: int):
    if _native(logits):
        return _cuda().ce_partials(logits, labels, vocab_start)
    return oracle.ce_partials(logits, labels, vocab_start)


def ce_backward(logits, labels, row_max, row_sum, grad_rows, vocab_start: int, ignore_index: int):
    """d loss / d logits for the local vocab shard: (softmax - onehot) * grad_rows."""
    if _native(logits):
        return _cuda().ce_backward(logits, labels, row_max, row_sum, grad_rows, vocab_start, ignore_index)
    lf = logits.float()
    p = torch.exp(lf - row_max[:, None]) / row_sum[:, None]
    local = labels - vocab_start
    inside = (local >= 0) & (local < logits.shape[-1])
    idx = torch.where(inside, local, torch.zeros_like(local))
    p.scatter_add_(1, idx[:, None], -inside.to(p.dtype)[:, None])
    g = torch.where(labels != ignore_index, grad_rows.float(), torch.zeros_like(grad_rows, dtype=torch.float32))
    return (p * g[:, None]).to(logits.dtype)
