"""Plain PyTorch restatement of every op in the framework.

These functions are the numerical ground truth for the CUDA kernels (tests compare each
kernel against the fp32 version of the same function) and they are also the execution path
on CPU tensors, where autograd differentiates them directly.

Math follows the reference kernels:
  * chunked SSD scan             mamba2/mamba2_kernel.py:15-62,138-169
  * causal depthwise conv + SiLU mamba2/conv1d_grouped.py:53-61,113-124
  * gated group RMSNorm          mamba2/fused_kernel.py:88-102, mamba2/mamba2_mixer.py:88-105
  * single-token decode          mamba2/mamba2_kernel_inference.py:13-23,68-104
  * softplus with threshold      mamba2/mamba2_mixer.py:36-38
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F


def softplus(x: torch.Tensor, threshold: float = 20.0) -> torch.Tensor:
    """log(1+exp(x)) with the identity above `threshold` (finite in fp32)."""
    return torch.where(x < threshold, torch.log1p(torch.exp(torch.clamp(x, max=threshold))), x)


def inverse_softplus(dt: torch.Tensor) -> torch.Tensor:
    """y with softplus(y) == dt, used to initialise dt_bias (mamba2/mamba2_mixer.py:160-168)."""
    return dt + torch.log(-torch.expm1(-dt))


# --------------------------------------------------------------------------------------
# causal depthwise conv1d + SiLU, channels-last
# --------------------------------------------------------------------------------------
def causal_conv1d_silu(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                       initial_state: Optional[torch.Tensor] = None,
                       activation: bool = True) -> torch.Tensor:
    """x [B, L, C]; weight [C, K] (tap K-1 multiplies the current token); bias [C] or None.

    `initial_state` [B, K-1, C] holds the K-1 tokens that precede x (zeros when None).
    Output has x's dtype; arithmetic is done in fp32.
    """
    Bsz, L, C = x.shape
    K = weight.shape[-1]
    xf = x.float()
    if initial_state is None:
        pad = xf.new_zeros(Bsz, K - 1, C)
    else:
        pad = initial_state.float()
    xp = torch.cat([pad, xf], dim=1)  # [B, L+K-1, C]
    w = weight.float().reshape(C, K)
    out = xf.new_zeros(Bsz, L, C)
    for i in range(K):
        out = out + xp[:, i:i + L, :] * w[:, i]
    if bias is not None:
        out = out + bias.float()
    if activation:
        out = F.silu(out)
    return out.to(x.dtype)


# --------------------------------------------------------------------------------------
# SSD scan
# --------------------------------------------------------------------------------------
def _expand_groups(t: torch.Tensor, n_heads: int) -> torch.Tensor:
    """[B, L, G, N] -> [B, L, H, N] by repeating each group for its heads."""
    G = t.shape[2]
    return t.repeat_interleave(n_heads // G, dim=2)


def ssd_recurrence(x, dt, A, Bm, Cm, D, initial_state=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Naive sequential recurrence, fp32.

    x [B,L,H,P], dt [B,L,H] (already positive), A [H] (negative), Bm/Cm [B,L,G,N], D [H].
    State layout is [B,H,P,N] like the decode cache.  Returns (y [B,L,H,P], final state).
      h_t = exp(A dt_t) h_{t-1} + dt_t x_t (x) B_t ;  y_t = h_t C_t + D x_t
    """
    Bsz, L, H, P = x.shape
    N = Bm.shape[-1]
    xf, dtf = x.float(), dt.float()
    Bh = _expand_groups(Bm.float(), H)
    Ch = _expand_groups(Cm.float(), H)
    Af, Df = A.float(), D.float()
    h = xf.new_zeros(Bsz, H, P, N) if initial_state is None else initial_state.float().clone()
    ys = []
    for t in range(L):
        decay = torch.exp(Af * dtf[:, t])  # [B,H]
        h = h * decay[:, :, None, None] + (dtf[:, t, :, None] * xf[:, t])[..., None] * Bh[:, t, :, None, :]
        y = torch.einsum("bhpn,bhn->bhp", h, Ch[:, t]) + Df[None, :, None] * xf[:, t]
        ys.append(y)
    return torch.stack(ys, dim=1), h


def ssd_chunked(x, dt, A, Bm, Cm, D, chunk_size: int = 128, initial_state=None,
                return_chunk_states: bool = False):
    """Chunked (block-decomposed) SSD scan in fp32: the algorithm the CUDA kernels implement.

    Same arguments and results as `ssd_recurrence`; L must be a multiple of chunk_size.
    With return_chunk_states also returns the state entering every chunk [B,H,nc,P,N].
    """
    Bsz, L, H, P = x.shape
    N = Bm.shape[-1]
    T = chunk_size
    assert L % T == 0, "sequence length must be a multiple of the chunk size"
    nc = L // T
    xf = x.float().reshape(Bsz, nc, T, H, P)
    dtf = dt.float().reshape(Bsz, nc, T, H)
    Bh = _expand_groups(Bm.float(), H).reshape(Bsz, nc, T, H, N)
    Ch = _expand_groups(Cm.float(), H).reshape(Bsz, nc, T, H, N)
    a = A.float() * dtf                         # [B,nc,T,H] log decay per step
    l = torch.cumsum(a, dim=2)                  # inclusive cumsum within chunk
    l_last = l[:, :, -1]                        # [B,nc,H]
    # intra-chunk (diagonal blocks)
    diff = l[:, :, :, None, :] - l[:, :, None, :, :]          # [B,nc,i,j,H]
    causal = torch.tril(torch.ones(T, T, dtype=torch.bool, device=x.device))
    Lmat = torch.where(causal[None, None, :, :, None], torch.exp(torch.where(
        causal[None, None, :, :, None], diff, torch.zeros_like(diff))), torch.zeros_like(diff))
    CB = torch.einsum("bcihn,bcjhn->bcijh", Ch, Bh)
    M = CB * Lmat * dtf[:, :, None, :, :]
    y_diag = torch.einsum("bcijh,bcjhp->bcihp", M, xf)
    # chunk-local end states
    a_right = torch.exp(l_last[:, :, None] - l)               # [B,nc,T,H]
    S_local = torch.einsum("bcjh,bcjhn,bcjhp->bchpn", a_right * dtf, Bh, xf)
    # inter-chunk recurrence
    S = xf.new_zeros(Bsz, H, P, N) if initial_state is None else initial_state.float()
    S_in = []
    a_center = torch.exp(l_last)                              # [B,nc,H]
    for c in range(nc):
        S_in.append(S)
        S = S * a_center[:, c, :, None, None] + S_local[:, c]
    S_in = torch.stack(S_in, dim=2)                           # [B,H,nc,P,N]
    a_left = torch.exp(l)
    y_off = torch.einsum("bcihn,bhcpn->bcihp", Ch, S_in) * a_left[..., None]
    y = y_diag + y_off + D.float()[None, None, None, :, None] * xf
    y = y.reshape(Bsz, L, H, P)
    if return_chunk_states:
        return y, S, S_in
    return y, S


# --------------------------------------------------------------------------------------
# norms
# --------------------------------------------------------------------------------------
def gated_rmsnorm(y: torch.Tensor, z: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                  group_size: Optional[int] = None, out_dtype=None) -> torch.Tensor:
    """out = w * h * rsqrt(mean_group(h^2) + eps),  h = y * silu(z).

    group_size None normalises over the whole last dimension.
    """
    d = y.shape[-1]
    h = y.float()
    if z is not None:
        h = h * F.silu(z.float())
    gs = d if group_size is None else group_size
    hg = h.reshape(*h.shape[:-1], d // gs, gs)
    hg = hg * torch.rsqrt(hg.pow(2).mean(-1, keepdim=True) + eps)
    out = hg.reshape(h.shape) * weight.float()
    return out.to(out_dtype if out_dtype is not None else y.dtype)


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """fp32 RMSNorm times weight, cast back (mamba2/modeling_mamba2.py:94-103)."""
    xf = x.float()
    xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (weight.float() * xf).to(x.dtype)


# --------------------------------------------------------------------------------------
# attention (GQA, causal) and rotary embedding
# --------------------------------------------------------------------------------------
def rotary_tables(seq_len: int, dim: int, theta: float, device=None, offset: int = 0):
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, device=device, dtype=torch.float32) / dim))
    t = torch.arange(offset, offset + seq_len, device=device, dtype=torch.float32)
    fr = torch.outer(t, inv)
    return torch.cos(fr), torch.sin(fr)  # [L, dim/2]


def apply_rotary(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half convention on the first 2*cos.shape[-1] channels of x [B,L,H,Dh]."""
    rd = cos.shape[-1] * 2
    xr, xp = x[..., :rd].float(), x[..., rd:]
    x1, x2 = xr[..., : rd // 2], xr[..., rd // 2:]
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    out = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)
    return torch.cat([out, xp], dim=-1)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True,
              scale: Optional[float] = None) -> torch.Tensor:
    """q [B,L,Hq,Dh], k/v [B,L,Hkv,Dh] -> [B,L,Hq,Dh]; query head h reads kv head h // (Hq/Hkv)."""
    Bsz, L, Hq, Dh = q.shape
    Hkv = k.shape[2]
    rep = Hq // Hkv
    scale = 1.0 / math.sqrt(Dh) if scale is None else scale
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        Lk = k.shape[1]
        mask = torch.ones(L, Lk, dtype=torch.bool, device=q.device).tril(Lk - L)
        s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    o = torch.matmul(p, vf)
    return o.permute(0, 2, 1, 3).to(q.dtype)


# --------------------------------------------------------------------------------------
# cross entropy over a (possibly sharded) vocabulary: the three per-row statistics
# --------------------------------------------------------------------------------------
def ce_partials(logits: torch.Tensor, labels: torch.Tensor, vocab_start: int):
    """Per-row (max, sum exp(l-max), target logit or 0) of a vocabulary shard.

    logits [R, Vs]; labels [R] global ids, -100 = ignored.
    """
    lf = logits.float()
    m = lf.max(dim=-1).values
    s = torch.exp(lf - m[:, None]).sum(-1)
    local = labels - vocab_start
    inside = (local >= 0) & (local < logits.shape[-1])
    idx = torch.where(inside, local, torch.zeros_like(local))
    tgt = torch.where(inside, lf.gather(1, idx[:, None])[:, 0], torch.zeros_like(m))
    return m, s, tgt


# --------------------------------------------------------------------------------------
# single-token decode over cached states
# --------------------------------------------------------------------------------------
def decode_step(xBC_new, dt_raw, conv_state, ssm_state, conv_w, conv_b, dt_bias, A, D,
                d_inner: int, n_groups: int, d_state: int, head_dim: int):
    """One autoregressive step of the mixer core.

    xBC_new [B, C]; dt_raw [B, H]; conv_state [B, C, K] (oldest first, updated in place);
    ssm_state [B, H, P, N] (updated in place).  Returns y [B, H*P] in fp32.
    """
    Bsz, Cdim = xBC_new.shape
    K = conv_w.shape[-1]
    H = dt_raw.shape[-1]
    conv_state.copy_(torch.cat([conv_state[:, :, 1:], xBC_new[:, :, None].to(conv_state.dtype)], dim=-1))
    pre = (conv_state.float() * conv_w.float().reshape(Cdim, K)).sum(-1)
    if conv_b is not None:
        pre = pre + conv_b.float()
    act = F.silu(pre)
    x = act[:, :d_inner].reshape(Bsz, H, head_dim)
    Bv = act[:, d_inner:d_inner + n_groups * d_state].reshape(Bsz, n_groups, d_state)
    Cv = act[:, d_inner + n_groups * d_state:].reshape(Bsz, n_groups, d_state)
    Bh = Bv.repeat_interleave(H // n_groups, dim=1)
    Ch = Cv.repeat_interleave(H // n_groups, dim=1)
    dt = softplus(dt_raw.float() + dt_bias.float())
    decay = torch.exp(A.float() * dt)
    S = ssm_state.float() * decay[:, :, None, None] + (dt[:, :, None] * x)[..., None] * Bh[:, :, None, :]
    ssm_state.copy_(S.to(ssm_state.dtype))
    y = torch.einsum("bhpn,bhn->bhp", S, Ch) + D.float()[None, :, None] * x
    return y.reshape(Bsz, H * head_dim)
