"""Mixer core of the PyTorch + cuBLAS baseline arm: what a user gets from plain PyTorch on a GPU, written the way the
public Mamba-2 reference implementation in PyTorch is written (block decomposition of the SSD scan with `einsum`,
bf16 operands for the large contractions so that cuBLAS runs them on tensor cores, fp32 for decays and
normalisation, cuDNN depthwise convolution), differentiated by autograd.  No hand-written kernel is involved.

Same math as `ops/oracle.py` (which computes everything in fp32 and is the numerical ground truth); this version is
the one that is timed as the baseline, so it is written for speed: no fp32 copies of the big operands, no masked
`where` chains, no activation checkpointing unless asked for.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def _segsum(a: torch.Tensor) -> torch.Tensor:
    """a [..., T] -> [..., T, T] with out[i, j] = sum_{j < k <= i} a[k] for i >= j, -inf above the diagonal."""
    T = a.shape[-1]
    cs = torch.cumsum(a, dim=-1)
    d = cs[..., :, None] - cs[..., None, :]
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool, device=a.device))
    return d.masked_fill(~mask, float("-inf"))


def ssd_minimal(x, dt, A, Bm, Cm, D, chunk: int = 128):
    """x [B,L,H,P] (bf16), dt [B,L,H] fp32 (positive), A [H] fp32 (negative), Bm/Cm [B,L,G,N] (bf16), D [H].
    Returns y [B,L,H,P] in x's dtype."""
    Bsz, L, H, P = x.shape
    G, N = Bm.shape[2], Bm.shape[3]
    nc = L // chunk
    lp = x.dtype
    rep = H // G
    xd = (x.float() * dt[..., None]).to(lp).reshape(Bsz, nc, chunk, H, P)
    Bh = Bm.reshape(Bsz, nc, chunk, G, N)
    Ch = Cm.reshape(Bsz, nc, chunk, G, N)
    a = (A[None, None, :] * dt).reshape(Bsz, nc, chunk, H).permute(0, 3, 1, 2)           # [B,H,nc,T] fp32
    a_cs = torch.cumsum(a, dim=-1)
    # 1. diagonal blocks: (C B^T) per group, decay matrix per head
    CB = torch.einsum("bclgn,bcsgn->bcgls", Ch, Bh)                                       # [B,nc,G,T,T] bf16 GEMMs
    Lm = torch.exp(_segsum(a)).to(lp)                                                     # [B,H,nc,T,T]
    M = CB.repeat_interleave(rep, dim=2).permute(0, 2, 1, 3, 4) * Lm                     # [B,H,nc,T,T]
    y_diag = torch.einsum("bhcls,bcshp->bclhp", M, xd)
    # 2. chunk-local end states
    decay_states = torch.exp(a_cs[..., -1:] - a_cs).to(lp)                                # [B,H,nc,T]
    xw = xd * decay_states.permute(0, 2, 3, 1)[..., None]                                 # [B,nc,T,H,P]
    states = torch.einsum("bclgn,bclgrp->bcgrpn", Bh, xw.reshape(Bsz, nc, chunk, G, rep, P)).reshape(Bsz, nc, H, P, N)
    # 3. inter-chunk recurrence (fp32, nc x nc per head)
    states = torch.cat([torch.zeros_like(states[:, :1]), states], dim=1).float()
    decay_chunk = torch.exp(_segsum(F.pad(a_cs[..., -1], (1, 0))))                         # [B,H,nc+1,nc+1]
    new_states = torch.einsum("bhzc,bchpn->bzhpn", decay_chunk, states)[:, :-1].to(lp)    # state entering each chunk
    # 4. contribution of the carried state
    out_decay = torch.exp(a_cs).to(lp)                                                    # [B,H,nc,T]
    y_off = torch.einsum("bclgn,bcgrpn->bclgrp", Ch, new_states.reshape(Bsz, nc, G, rep, P, N)).reshape(
        Bsz, nc, chunk, H, P) * out_decay.permute(0, 2, 3, 1)[..., None]
    y = (y_diag + y_off).reshape(Bsz, L, H, P) + x * D.to(lp)[None, None, :, None]
    return y.to(lp)


def mixer_core(zxBCdt, conv_w, conv_b, dt_bias, A_log, D, norm_w, *, d_inner, n_groups, d_state, head_dim, eps,
               norm_group_size, chunk_size=128, **unused):
    Bsz, L, _ = zxBCdt.shape
    conv_dim = d_inner + 2 * n_groups * d_state
    H = d_inner // head_dim
    z = zxBCdt[..., :d_inner]
    xBC = zxBCdt[..., d_inner:d_inner + conv_dim]
    dt_raw = zxBCdt[..., d_inner + conv_dim:]
    K = conv_w.shape[-1]
    act = F.silu(F.conv1d(xBC.transpose(1, 2), conv_w.reshape(conv_dim, 1, K), conv_b, padding=K - 1,
                          groups=conv_dim)[..., :L]).transpose(1, 2)
    x = act[..., :d_inner].reshape(Bsz, L, H, head_dim)
    Bm = act[..., d_inner:d_inner + n_groups * d_state].reshape(Bsz, L, n_groups, d_state)
    Cm = act[..., d_inner + n_groups * d_state:].reshape(Bsz, L, n_groups, d_state)
    A = -torch.exp(A_log.float())
    dt = F.softplus(dt_raw.float() + dt_bias.float())
    y = ssd_minimal(x, dt, A, Bm, Cm, D.float(), chunk_size).reshape(Bsz, L, d_inner)
    h = y.float() * F.silu(z.float())
    gs = d_inner if norm_group_size is None else norm_group_size
    hg = h.reshape(Bsz, L, d_inner // gs, gs)
    hg = hg * torch.rsqrt(hg.pow(2).mean(-1, keepdim=True) + eps)
    return (hg.reshape(Bsz, L, d_inner) * norm_w.float()).to(zxBCdt.dtype)
