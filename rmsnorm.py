"""Stand-alone check of the RMSNorm kernels against a plain PyTorch restatement.

Counterpart of the reference's demo script (rmsnorm.py:9-30 torch reference, :33-94 kernel, :97-117 self-check):
builds random inputs, runs the gated group RMSNorm and the plain (residual-add) RMSNorm through the framework's
ops (CUDA kernels on a GPU, the PyTorch oracle on CPU) and prints the largest deviation from an fp32 formula
written out here.  Exit code 0 when both agree.
"""
from __future__ import annotations

import argparse
import sys

import torch

from state_space_models_neuron_b200 import ops


def gated_rmsnorm_reference(y, z, weight, eps, group_size):
    x = y.float() * torch.nn.functional.silu(z.float())
    g = x.view(*x.shape[:-1], -1, group_size)
    g = g * torch.rsqrt(g.pow(2).mean(-1, keepdim=True) + eps)
    return (g.view_as(x) * weight.float()).to(y.dtype)


def rmsnorm_reference(x, weight, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()).to(x.dtype)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=300)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--group_size", type=int, default=512)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    dev = torch.device(a.device)
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    g = torch.Generator().manual_seed(0)
    y = torch.randn(1, a.rows, a.hidden, generator=g).to(dev, dtype)
    z = torch.randn(1, a.rows, a.hidden, generator=g).to(dev, dtype)
    w = (1 + 0.1 * torch.randn(a.hidden, generator=g)).to(dev, dtype)
    tol = 3e-2 if dtype == torch.bfloat16 else 1e-5
    got = ops.gated_rmsnorm(y, z, w, 1e-5, a.group_size)
    e1 = (got.float() - gated_rmsnorm_reference(y, z, w, 1e-5, a.group_size).float()).abs().max().item()
    got2 = ops.rmsnorm(y, w, 1e-5)
    e2 = (got2.float() - rmsnorm_reference(y, w, 1e-5).float()).abs().max().item()
    print(f"gated group RMSNorm max abs err {e1:.3e}; RMSNorm max abs err {e2:.3e}; tolerance {tol:.0e} ({dtype})")
    return 0 if e1 <= tol * 4 and e2 <= tol * 4 else 1


if __name__ == "__main__":
    sys.exit(main())
