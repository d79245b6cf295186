"""Autograd wrappers around the native sm_100a kernels (GPU path of `ops.functional`).

Tensors are passed to the C ABI as raw device pointers on the current CUDA stream.  The kernels
report asynchronous failures (a bounded wait that ran out) through a device status word; `check_status()`
reads it (this synchronises) and raises.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import native

_c = ctypes
_status = {}
_launches = [0]


def launch_count() -> int:
    """Number of native kernel launches issued by this process so far."""
    return _launches[0]


def _lib():
    return native.lib()


class _P:
    """Pointer argument that keeps its tensor alive until the launch call has returned: a temporary
    (`x.float()`, `.contiguous()`) must not be freed, and its block handed to the next temporary in the
    same argument list, before the kernel is enqueued."""
    __slots__ = ("t", "_as_parameter_")

    def __init__(self, t):
        self.t = t
        self._as_parameter_ = _c.c_void_p(0 if t is None else t.data_ptr())


def _p(t: Optional[torch.Tensor]):
    return _P(t)


def _st():
    return _c.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ll(v):
    return _c.c_longlong(int(v))


def status_tensor(device=None) -> torch.Tensor:
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if device not in _status:
        _status[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[device]


def check_status() -> None:
    for dev, t in _status.items():
        code = int(t.item())
        if code != 0:
            t.zero_()
            raise RuntimeError(f"native kernel reported status {code} on {dev} "
                               "(1: mbarrier wait timed out, 2: flag wait timed out, 3: bad argument)")


def _run(name: str, *args):
    fn = getattr(_lib(), name)
    fn.restype = _c.c_int
    code = fn(*args)
    _launches[0] += 1
    if code != 0:
        raise RuntimeError(f"{name} failed with code {code} (negative: argument check, positive: cudaError_t)")


def _require_bf16(*ts):
    for t in ts:
        if t is not None and t.dtype != torch.bfloat16:
            raise TypeError(f"GPU kernels take bfloat16 activations/weights, got {t.dtype}")


def _ceil8(n: int) -> int:
    return (n + 7) // 8 * 8


# ======================================================================================
# GEMM
# ======================================================================================
def _as_operand(t: torch.Tensor) -> torch.Tensor:
    """2D, unit inner stride, row stride % 8 == 0, 16-byte aligned base (TMA requirements)."""
    if t.dim() != 2:
        raise ValueError("GEMM operands are 2D")
    if t.stride(1) != 1 or t.stride(0) % 8 or t.data_ptr() % 16:
        cols = _ceil8(t.shape[1])
        buf = torch.zeros(t.shape[0], cols, dtype=t.dtype, device=t.device) if cols != t.shape[1] else \
            torch.empty(t.shape[0], cols, dtype=t.dtype, device=t.device)
        buf[:, :t.shape[1]].copy_(t)
        return buf[:, :t.shape[1]]
    return t


def gemm(a: torch.Tensor, b: torch.Tensor, a_mn: bool = False, b_mn: bool = False, out: Optional[torch.Tensor] = None,
         out_dtype=torch.bfloat16, accumulate: bool = False, bias: Optional[torch.Tensor] = None,
         gelu: bool = False, sumsq: Optional[torch.Tensor] = None) -> torch.Tensor:
    """C[M,N] = A B on tcgen05.  a is [M,K] (or [K,M] when a_mn), b is [N,K] (or [K,N] when b_mn).
    out: bf16 (fresh, row stride padded to 8) or fp32 (`accumulate` adds into `out`).
    sumsq (fp32 scalar tensor, fp32 store only): the kernel adds sum(C^2) to it."""
    _require_bf16(a, b, bias)
    a, b = _as_operand(a), _as_operand(b)
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    if K != Kb:
        raise ValueError(f"GEMM inner dimensions differ: {K} vs {Kb}")
    if out is None:
        if out_dtype == torch.bfloat16:
            out = torch.empty(M, _ceil8(N), dtype=torch.bfloat16, device=a.device)[:, :N]
        else:
            out = torch.empty(M, (N + 3) // 4 * 4, dtype=torch.float32, device=a.device)[:, :N]
    if out.dtype == torch.float32 and (out.stride(0) % 4 or out.data_ptr() % 16) and out.stride(1) == 1:
        # TMA needs 16-byte aligned rows: go through a padded temporary
        tmp = gemm(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32, sumsq=sumsq)
        if accumulate:
            out.add_(tmp)
        else:
            out.copy_(tmp)
        return out
    if out.dtype == torch.bfloat16:
        mode = 0
        if out.stride(1) != 1 or out.stride(0) % 8 or out.data_ptr() % 16:
            raise ValueError("bf16 GEMM output needs unit inner stride, row stride % 8 == 0, 16-byte base")
    else:
        mode = 2 if accumulate else 1
        if out.stride(1) != 1:
            raise ValueError("fp32 GEMM output needs unit inner stride")
    if sumsq is not None:
        if mode != 1 or sumsq.dtype != torch.float32:
            raise ValueError("sumsq needs an fp32 output that is stored, not accumulated")
        _run("ssm_gemm_bf16_ex", _p(a), _p(b), _p(out), M, N, K, _ll(a.stride(0)), _ll(b.stride(0)), _ll(out.stride(0)),
             int(a_mn), int(b_mn), mode, _p(bias), int(gelu), _p(status_tensor(a.device)), _st(), _p(sumsq))
        return out
    _run("ssm_gemm_bf16", _p(a), _p(b), _p(out), M, N, K, _ll(a.stride(0)), _ll(b.stride(0)), _ll(out.stride(0)),
         int(a_mn), int(b_mn), mode, _p(bias), int(gelu), _p(status_tensor(a.device)), _st())
    return out


def ce_epilogue_buffers(M: int, N: int, K: int, labels: torch.Tensor, vocab_start: int, rows_per_shard: int = 0):
    """Buffers for a GEMM whose epilogue emits cross-entropy statistics of its [M, N] output (the LM head):
    (arguments for the kernel, number of column tiles).  `labels` [M] int64 global ids, negative = ignored;
    `rows_per_shard`: shard rows when the GEMM is the all-gather variant (it decides the tile shape), else 0."""
    fn = _lib().ssm_gemm_ce_tiles
    fn.restype = _c.c_int
    tiles = int(fn(int(M), int(N), int(K), int(rows_per_shard)))
    dev = labels.device
    lab = labels.reshape(-1).contiguous()
    if lab.numel() != M or lab.dtype != torch.int64:
        raise ValueError("labels must be int64 with one entry per output row")
    return dict(labels=lab, vocab_start=int(vocab_start),
                tmax=torch.empty(tiles, M, dtype=torch.float32, device=dev),
                tsum=torch.empty(tiles, M, dtype=torch.float32, device=dev),
                tgt=torch.zeros(M, dtype=torch.float32, device=dev)), tiles


def ce_merge(ced, tiles: int):
    """Per-tile statistics -> (row max, row sum of exp(x - max), target logit or 0) for this vocabulary shard."""
    M = ced["tgt"].numel()
    m = torch.empty(M, dtype=torch.float32, device=ced["tgt"].device)
    s = torch.empty_like(m)
    _run("ssm_ce_merge_tiles", _p(ced["tmax"]), _p(ced["tsum"]), int(tiles), _ll(M), _p(m), _p(s), _st())
    return m, s, ced["tgt"]


def gemm_ce(a: torch.Tensor, b: torch.Tensor, labels: torch.Tensor, vocab_start: int):
    """y = a b^T (bf16, [M, N]) together with the cross-entropy statistics of its rows, produced by the GEMM
    epilogue (no second pass over the logits): returns (y, (max, sumexp, target))."""
    _require_bf16(a, b)
    a, b = _as_operand(a), _as_operand(b)
    M, K = a.shape
    N = b.shape[0]
    out = torch.empty(M, _ceil8(N), dtype=torch.bfloat16, device=a.device)[:, :N]
    ced, tiles = ce_epilogue_buffers(M, N, K, labels, vocab_start)
    _run("ssm_gemm_bf16_ce", _p(a), _p(b), _p(out), M, N, K, _ll(a.stride(0)), _ll(b.stride(0)), _ll(out.stride(0)),
         _p(status_tensor(a.device)), _st(), _p(ced["labels"]), _ll(ced["vocab_start"]), _p(ced["tmax"]),
         _p(ced["tsum"]), _p(ced["tgt"]))
    return out, ce_merge(ced, tiles)


def wgrad_to_main_grad(dy2: torch.Tensor, x2: torch.Tensor, w) -> bool:
    """dW = dY^T X written straight into the optimizer's fp32 `w.main_grad`: stored on the first contribution of a
    step (lazy zeroing), added afterwards.  When the optimizer has given the weight a norm accumulator (`w.norm_acc`)
    a stored gradient also adds its sum of squares to it (`w.norm_tracked` tells the optimizer that this weight's
    share of the gradient norm is already there).  False: no fp32 main_grad, the caller returns dW through autograd."""
    mg = getattr(w, "main_grad", None)
    if mg is None or mg.dtype != torch.float32:
        return False
    stale = getattr(w, "grad_stale", False)
    acc = getattr(w, "norm_acc", None) if stale else None
    if not stale:
        untrack_norm(w)
    gemm(dy2, x2, a_mn=True, b_mn=True, out=mg, accumulate=not stale, sumsq=acc)
    w.grad_stale = False
    if acc is not None:
        w.norm_tracked = True
    return True


def untrack_norm(w) -> None:
    """The gradient of `w` is about to change after a GEMM may already have added its sum of squares to the norm
    accumulator: mark the weight so that the optimizer recomputes the norm from the buffers this step."""
    if getattr(w, "norm_tracked", False):
        w.norm_tracked = False
        w.norm_dirty = True


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, ce_labels=None, ce_vocab_start=0):
        K = x.shape[-1]
        x2 = x.reshape(-1, K)
        ctx.save_for_backward(x2, w)
        ctx.has_bias = bias is not None
        ctx.xshape = x.shape
        if ce_labels is not None:
            y, stats = gemm_ce(x2, w, ce_labels, ce_vocab_start)
            ctx.mark_non_differentiable(*stats)
            return (y.reshape(*x.shape[:-1], w.shape[0]),) + tuple(stats)
        y = gemm(x2, w, bias=bias)
        return y.reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy, *unused):
        x2, w = ctx.saved_tensors
        N = w.shape[0]
        dy2 = dy.reshape(-1, N)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, b_mn=True).reshape(ctx.xshape)          # dX = dY W
        if ctx.needs_input_grad[1]:
            if not wgrad_to_main_grad(dy2, x2, w):                       # main_grad (+)= dY^T X
                dw = gemm(dy2, x2, a_mn=True, b_mn=True)
                if not dw.is_contiguous():
                    dw = dw.contiguous()
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy.dtype)
        return dx, dw, db, None, None


def linear(x, w, bias=None):
    _require_bf16(x, w)
    return _Linear.apply(x, w, bias)


def linear_ce(x, w, labels, vocab_start: int = 0):
    """(x w^T, (row max, row sum-exp, target logit)): the LM head with the cross-entropy statistics taken in the
    GEMM epilogue (mamba2/modeling_mamba2.py:498-510 computes them in separate passes over fp32 logits)."""
    _require_bf16(x, w)
    out = _Linear.apply(x, w, None, labels, int(vocab_start))
    return out[0], tuple(out[1:])


# ======================================================================================
# conv
# ======================================================================================
def _conv_fwd(xBC, w2, bias, init, out=None):
    B, L, C = xBC.shape
    assert xBC.stride(2) == 1 and xBC.stride(0) == L * xBC.stride(1)
    if out is None:
        out = torch.empty(B, L, C, dtype=xBC.dtype, device=xBC.device)
    _run("ssm_conv1d_silu_fwd", _p(xBC), _ll(xBC.stride(1)), _p(w2), _p(bias), _p(init), _p(out), _ll(out.stride(1)),
         B, L, C, _st())
    return out


def _conv_bwd(xBC, w2, bias, dy16, dy32, c_split, dx_out, raw=False):
    """dx_out [B,L,C] view (row stride may exceed C); returns (dw [C,K], db [C]) fp32, or the per-tile partial
    buffer [tiles, C, 5] when `raw`."""
    B, L, C = xBC.shape
    tile = _lib().ssm_conv_bwd_tok_tile(B, L, C)
    ntile = (L + tile - 1) // tile
    part = torch.empty(B * ntile, C, 5, dtype=torch.float32, device=xBC.device)
    _run("ssm_conv1d_silu_bwd", _p(xBC), _ll(xBC.stride(1)), _p(w2), _p(bias), _p(dy16),
         _ll(dy16.stride(1) if dy16 is not None else 0), _p(dy32), _ll(dy32.stride(1) if dy32 is not None else 0),
         int(c_split), _p(dx_out), _ll(dx_out.stride(1)), _p(part), B, L, C, _st())
    if raw:
        return part
    s = part.sum(0)
    return s[:, :4], s[:, 4]


class _Conv(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, init):
        C = x.shape[-1]
        w2 = w.reshape(C, -1).contiguous()
        if not (x.stride(2) == 1 and x.stride(0) == x.shape[1] * x.stride(1) and x.stride(1) % 8 == 0):
            x = x.contiguous()
        init3 = None if init is None else init[:, -3:, :].contiguous()
        out = _conv_fwd(x, w2, bias, init3)
        ctx.save_for_backward(x, w2, bias)
        ctx.wshape = w.shape
        return out

    @staticmethod
    def backward(ctx, dy):
        x, w2, bias = ctx.saved_tensors
        dy = dy.contiguous()
        dx = torch.empty(x.shape, dtype=x.dtype, device=x.device)
        dw, db = _conv_bwd(x, w2, bias, dy, None, x.shape[-1], dx)
        return dx, dw.to(w2.dtype).reshape(ctx.wshape), (None if bias is None else db.to(bias.dtype)), None


def causal_conv1d_silu(x, weight, bias, initial_state=None):
    _require_bf16(x, weight, bias)
    if weight.shape[-1] != 4:
        raise ValueError("the conv kernel is written for 4 taps")
    return _Conv.apply(x, weight, bias, initial_state)


# ======================================================================================
# norms
# ======================================================================================
_ROW_SLICES = 296


def _gated_fwd(y2, z2, w, eps, gs, out=None):
    rows, d = y2.shape
    if out is None:
        out = torch.empty(rows, d, dtype=y2.dtype, device=y2.device)
    _run("ssm_gated_rmsnorm_fwd", _p(y2), _ll(y2.stride(0)), _p(z2), _ll(z2.stride(0) if z2 is not None else 0), _p(w),
         _p(out), _ll(out.stride(0)), _ll(rows), d, gs, _c.c_float(eps), _st())
    return out


def _gated_bwd(y2, z2, w, dout2, eps, gs, dy_out, dz_out, raw=False):
    rows, d = y2.shape
    slices = int(min(rows, _ROW_SLICES))
    part = torch.empty(slices, d, dtype=torch.float32, device=y2.device)
    _run("ssm_gated_rmsnorm_bwd", _p(y2), _ll(y2.stride(0)), _p(z2), _ll(z2.stride(0) if z2 is not None else 0), _p(w),
         _p(dout2), _ll(dout2.stride(0)), _p(dy_out), _ll(dy_out.stride(0)), _p(dz_out),
         _ll(dz_out.stride(0) if dz_out is not None else 0), _p(part), slices, _ll(rows), d, gs, _c.c_float(eps), _st())
    return part if raw else part.sum(0)


def _rows(t):
    """[..., d] -> 2D view with unit inner stride (copy only if needed)."""
    d = t.shape[-1]
    if t.dim() == 2 and t.stride(1) == 1:
        return t
    if t.stride(-1) == 1 and t.dim() == 3 and t.stride(0) == t.shape[1] * t.stride(1):
        return t.as_strided((t.shape[0] * t.shape[1], d), (t.stride(1), 1), t.storage_offset())
    return t.reshape(-1, d).contiguous()


class _GatedNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, z, w, eps, gs):
        y2, z2 = _rows(y), (None if z is None else _rows(z))
        out = _gated_fwd(y2, z2, w, eps, gs)
        ctx.save_for_backward(y2, z2, w)
        ctx.eps, ctx.gs, ctx.shape = eps, gs, y.shape
        return out.reshape(y.shape)

    @staticmethod
    def backward(ctx, dout):
        y2, z2, w = ctx.saved_tensors
        d2 = _rows(dout.contiguous())
        dy = torch.empty(y2.shape, dtype=y2.dtype, device=y2.device)
        dz = None if z2 is None else torch.empty(y2.shape, dtype=y2.dtype, device=y2.device)
        dw = _gated_bwd(y2, z2, w, d2, ctx.eps, ctx.gs, dy, dz)
        return dy.reshape(ctx.shape), (None if dz is None else dz.reshape(ctx.shape)), dw.to(w.dtype), None, None


def gated_rmsnorm(y, z, w, eps, group_size=None):
    _require_bf16(y, z, w)
    gs = y.shape[-1] if group_size is None else group_size
    return _GatedNorm.apply(y, z, w, eps, gs)


class _AddRMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, w, eps, res_dtype):
        D = x.shape[-1]
        x2 = x.reshape(-1, D).contiguous()
        rows = x2.shape[0]
        r2 = None if residual is None else residual.reshape(-1, D).contiguous()
        out = torch.empty_like(x2)
        res_out = torch.empty(rows, D, dtype=res_dtype, device=x.device)
        if r2 is not None and r2.dtype != res_dtype:
            r2 = r2.to(res_dtype)
        _run("ssm_add_rmsnorm_fwd", _p(x2), _p(r2), _p(w), _p(out), _p(res_out), _ll(rows), D, _c.c_float(eps),
             int(res_dtype == torch.float32), _st())
        ctx.save_for_backward(res_out, w)
        ctx.eps, ctx.shape, ctx.has_res = eps, x.shape, residual is not None
        ctx.x_dtype = x.dtype
        return out.reshape(x.shape), res_out.reshape(x.shape)

    @staticmethod
    def backward(ctx, dout, dres):
        res_out, w = ctx.saved_tensors
        rows, D = res_out.shape
        d2 = dout.reshape(rows, D).contiguous()
        dr2 = None if dres is None else dres.reshape(rows, D).contiguous()
        dsum = torch.empty_like(res_out)
        slices = int(min(rows, _ROW_SLICES))
        part = torch.empty(slices, D, dtype=torch.float32, device=res_out.device)
        _run("ssm_add_rmsnorm_bwd", _p(res_out), _p(w), _p(d2), _p(dr2), _p(dsum), _p(part), slices, _ll(rows), D,
             _c.c_float(ctx.eps), int(res_out.dtype == torch.float32), _st())
        dsum = dsum.reshape(ctx.shape)
        dx = dsum if dsum.dtype == ctx.x_dtype else dsum.to(ctx.x_dtype)
        mg = getattr(w, "main_grad", None)
        if mg is not None and mg.dtype == torch.float32 and w.is_leaf:
            _run("ssm_colsum", _p(part), slices, D, _p(mg), int(not getattr(w, "grad_stale", False)), _st())
            w.grad_stale = False
            return dx, (dsum if ctx.has_res else None), None, None, None
        return dx, (dsum if ctx.has_res else None), part.sum(0).to(w.dtype), None, None


def add_rmsnorm(x, residual, w, eps, residual_dtype=None):
    _require_bf16(x, w)
    rd = residual_dtype or x.dtype
    return _AddRMSNorm.apply(x, residual, w, eps, rd)


def rmsnorm(x, w, eps):
    return add_rmsnorm(x, None, w, eps)[0]


# ======================================================================================
# GELU
# ======================================================================================
class _Gelu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        xc = x.contiguous()
        y = torch.empty_like(xc)
        _run("ssm_gelu_fwd", _p(xc), _p(y), _ll(xc.numel()), _st())
        ctx.save_for_backward(xc)
        return y

    @staticmethod
    def backward(ctx, dy):
        (xc,) = ctx.saved_tensors
        dx = torch.empty_like(xc)
        _run("ssm_gelu_bwd", _p(xc), _p(dy.contiguous()), _p(dx), _ll(xc.numel()), _st())
        return dx


def gelu(x):
    _require_bf16(x)
    if x.numel() % 8:
        return torch.nn.functional.gelu(x)
    return _Gelu.apply(x)


class _Glu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, act):
        S = h.shape[-1] // 2
        h2 = h.reshape(-1, 2 * S)
        if h2.stride(1) != 1 or h2.stride(0) % 8 or h2.data_ptr() % 16:
            h2 = h2.contiguous()
        out = torch.empty(h2.shape[0], S, dtype=h.dtype, device=h.device)
        _run("ssm_glu_fwd", _p(h2), _ll(h2.stride(0)), _p(out), _ll(h2.shape[0]), S, act, _st())
        ctx.save_for_backward(h2)
        ctx.act, ctx.shape = act, h.shape
        return out.reshape(*h.shape[:-1], S)

    @staticmethod
    def backward(ctx, dout):
        (h2,) = ctx.saved_tensors
        S = h2.shape[1] // 2
        d2 = dout.reshape(-1, S).contiguous()
        dh = torch.empty(h2.shape[0], 2 * S, dtype=h2.dtype, device=h2.device)
        _run("ssm_glu_bwd", _p(h2), _ll(h2.stride(0)), _p(d2), _p(dh), _ll(h2.shape[0]), S, ctx.act, _st())
        return dh.reshape(ctx.shape), None


def glu(h, act: str = "silu"):
    """act(h[..., :S]) * h[..., S:] for h = [gate | up] in one kernel (forward and backward); act gelu or silu."""
    _require_bf16(h)
    if h.shape[-1] % 16 or act not in ("gelu", "silu", "swish"):
        raise ValueError("glu kernel needs an even split into multiples of 8 columns and act in {gelu, silu}")
    return _Glu.apply(h, 0 if act == "gelu" else 1)


# ======================================================================================
# embedding
# ======================================================================================
def embed_grad_target(w):
    """(fp32 [V, D] buffer to accumulate into, direct).  With an optimizer-owned `main_grad` the embedding backward
    adds into it in place (after the tied LM-head wgrad, which ran earlier in the backward pass)."""
    mg = getattr(w, "main_grad", None)
    if mg is not None and mg.dtype == torch.float32 and mg.is_contiguous():
        if getattr(w, "grad_stale", False):
            mg.zero_()
            w.grad_stale = False
        untrack_norm(w)                 # scatter-added rows change the norm of a gradient a GEMM may have stored
        return mg, True
    return torch.zeros(w.shape, dtype=torch.float32, device=w.device), False


class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, w, vocab_start):
        ids_c = ids.contiguous()
        out = torch.empty(*ids.shape, w.shape[1], dtype=w.dtype, device=w.device)
        _run("ssm_embed_lookup", _P(ids_c), _P(w), _ll(vocab_start), _ll(w.shape[0]), _P(out), _ll(ids_c.numel()),
             w.shape[1], _st())
        ctx.save_for_backward(ids_c)
        ctx.w, ctx.vocab_start = w, vocab_start
        return out

    @staticmethod
    def backward(ctx, g):
        (ids,), w = ctx.saved_tensors, ctx.w
        D = w.shape[1]
        g2 = g.reshape(-1, D)
        if g2.stride(1) != 1 or g2.stride(0) % 4:
            g2 = g2.contiguous()
        tgt, direct = embed_grad_target(w)
        n = ids.numel()
        _run("ssm_embed_bwd", _P(ids), _P(g2), _ll(g2.stride(0)), _P(tgt), _ll(ctx.vocab_start), _ll(w.shape[0]), 1, n, n,
             D, 1, None, 0, 0, None, _P(status_tensor(w.device)), _st())
        return None, (None if direct else tgt.to(w.dtype)), None


def embedding(ids, w, vocab_start: int = 0):
    """Rows `w[ids - vocab_start]`, zeros for ids outside the local shard; the gradient is scatter-added in fp32."""
    if w.dtype != torch.bfloat16 or ids.dtype != torch.int64 or w.shape[1] % 8 or not w.is_contiguous():
        local = ids - vocab_start
        inside = (local >= 0) & (local < w.shape[0])
        return torch.nn.functional.embedding(torch.where(inside, local, torch.zeros_like(local)), w) \
            * inside[..., None].to(w.dtype)
    return _Embedding.apply(ids, w, int(vocab_start))


# ======================================================================================
# cross entropy
# ======================================================================================
def ce_partials(logits, labels, vocab_start):
    rows, V = logits.shape
    assert logits.stride(1) == 1
    m = torch.empty(rows, dtype=torch.float32, device=logits.device)
    s, t = torch.empty_like(m), torch.empty_like(m)
    _run("ssm_ce_partials", _p(logits), _ll(logits.stride(0)), int(logits.dtype == torch.float32),
         _p(labels.contiguous()), _ll(rows), V, int(vocab_start), _p(m), _p(s), _p(t), _st())
    return m, s, t


def ce_backward(logits, labels, row_max, row_sum, grad_rows, vocab_start, ignore_index):
    rows, V = logits.shape
    ld = _ceil8(V)
    grad = torch.empty(rows, ld, dtype=logits.dtype, device=logits.device)[:, :V]
    if ld != V:
        grad.as_strided((rows, ld - V), (ld, 1), V).zero_()
    _run("ssm_ce_backward", _p(logits), _ll(logits.stride(0)), int(logits.dtype == torch.float32),
         _p(labels.contiguous()), _ll(rows), V, int(vocab_start), _ll(ignore_index), _p(row_max), _p(row_sum),
         _p(grad_rows.float().contiguous()), _p(grad), _ll(ld), _st())
    return grad


# ======================================================================================
# optimizer
# ======================================================================================
def adamw_step(master, m, v, g, out, clip, lr, b1, b2, eps, wd, step, lr_dev=None, step_dev=None):
    """lr_dev (fp32 [1]) / step_dev (int32 [1]): device-resident values that override `lr` / `step`."""
    if master.dtype != torch.float32:
        raise TypeError("the fused AdamW keeps fp32 state")
    out16 = out if out.dtype == torch.bfloat16 else None
    out32 = out if out.dtype == torch.float32 else None
    _run("ssm_adamw", _p(master), _p(m), _p(v), _p(g), int(g.dtype == torch.float32), _p(out16), _p(out32),
         _ll(master.numel()), _p(clip), _c.c_float(lr), _c.c_float(b1), _c.c_float(b2), _c.c_float(eps),
         _c.c_float(wd), int(step), _p(lr_dev), _p(step_dev), _st())


def sumsq_accumulate(g, total):
    _run("ssm_sumsq", _p(g), int(g.dtype == torch.float32), _ll(g.numel()), _p(total), _st())


# ======================================================================================
# SSD scan and the fused mixer core
# ======================================================================================
_CT = 128


def _ssd_dims(d_inner, head_dim, n_groups, d_state):
    if d_state != 128:
        raise ValueError("the GPU SSD kernels are written for d_state = 128")
    if head_dim % 64:
        raise ValueError("the GPU SSD kernels need head_dim to be a multiple of 64")
    H = d_inner // head_dim
    psplit = head_dim // 64
    if H % n_groups:
        raise ValueError("heads must be divisible by groups")
    return H, psplit, H * psplit


def _ssd_forward(conv_out, dt_raw2, dt_raw_stride, A, D, dt_bias, B, L, d_inner, G, H, Hv, init_state=None,
                 want_final=False):
    """conv_out [B*L, C] bf16 contiguous.  Returns y [B*L, d_inner], dt, l, S_in, final (or None)."""
    dev = conv_out.device
    C = conv_out.shape[1]
    nc = L // _CT
    st = status_tensor(dev)
    dt = torch.empty(B, H, L, dtype=torch.float32, device=dev)
    l = torch.empty_like(dt)
    _run("ssm_ssd_dt_prep", _p(dt_raw2), _ll(dt_raw_stride), _p(dt_bias), _p(A), _p(dt), _p(l), B, L, H, _st())
    s_local = torch.empty(B, Hv, nc, 128, 64, dtype=torch.float32, device=dev)
    _run("ssm_ssd_chunk_state", _p(conv_out), _ll(C), C, d_inner, _p(conv_out), _ll(C), _p(dt), _p(l), _p(s_local),
         B, L, H, Hv, G, 0, _p(st), _st())
    s_in = torch.empty(B, Hv, nc, 128, 64, dtype=torch.bfloat16, device=dev)
    final = torch.empty(B, Hv, 128, 64, dtype=torch.float32, device=dev) if want_final else None
    _run("ssm_ssd_state_pass", _p(s_local), _p(l), _p(init_state), _p(s_in), _p(final), B, L, H, Hv, 0, _st())
    y = torch.empty(B * L, d_inner, dtype=torch.bfloat16, device=dev)
    _run("ssm_ssd_chunk_scan_fwd", _p(conv_out), _ll(C), C, _p(s_in), _p(y), _ll(d_inner), _p(dt), _p(l), _p(D),
         B, L, H, Hv, G, d_inner, _p(st), _st())
    return y, dt, l, s_in, final


def _pick_hpc(hv_per_group, nc, G, B, target=296):
    best = hv_per_group
    for splits in range(1, hv_per_group + 1):
        if hv_per_group % splits:
            continue
        best = hv_per_group // splits
        if nc * G * B * splits >= target:
            break
    return best


def _ssd_backward(conv_out, dy2, y2, dt, l, s_in, dt_raw2, dt_raw_stride, A, D, dt_bias, ddt_out, ddt_stride,
                  B, L, d_inner, G, H, Hv, raw=False):
    """Returns dx [B*L, d_inner] bf16, dBC fp32 [B*L, 2*G*128], dA, dD, d_dt_bias (fp32 [H]);
    d(dt_raw) goes to ddt_out (bf16, row stride ddt_stride, column h)."""
    dev = conv_out.device
    C = conv_out.shape[1]
    nc = L // _CT
    st = status_tensor(dev)
    psplit = Hv // H
    ds_local = torch.empty(B, Hv, nc, 128, 64, dtype=torch.float32, device=dev)
    _run("ssm_ssd_chunk_state", _p(conv_out), _ll(C), C, d_inner + G * 128, _p(dy2), _ll(dy2.stride(0)), _p(dt), _p(l),
         _p(ds_local), B, L, H, Hv, G, 1, _p(st), _st())
    ds_out = torch.empty(B, Hv, nc, 128, 64, dtype=torch.bfloat16, device=dev)
    _run("ssm_ssd_state_pass", _p(ds_local), _p(l), _p(None), _p(ds_out), _p(None), B, L, H, Hv, 1, _st())
    dx = torch.empty(B * L, d_inner, dtype=torch.bfloat16, device=dev)
    dBC = torch.zeros(B * L, 2 * G * 128, dtype=torch.float32, device=dev)
    hpart = torch.empty(B * nc, Hv, 3, dtype=torch.float32, device=dev)
    ddt32 = torch.empty(B, Hv, L, dtype=torch.float32, device=dev) if psplit > 1 else None
    hpc = _pick_hpc(Hv // G, nc, G, B)
    _run("ssm_ssd_chunk_scan_bwd", _p(conv_out), _ll(C), C, _p(dy2), _ll(dy2.stride(0)),
         _p(s_in), _p(ds_out), _p(dx), _ll(d_inner), _p(dBC), _p(hpart), _p(ddt_out), _ll(ddt_stride), _p(ddt32),
         _p(dt_raw2), _ll(dt_raw_stride), _p(dt_bias), _p(A), _p(dt), _p(l), _p(D), B, L, H, Hv, G, d_inner, hpc,
         _p(st), _st())
    if ddt32 is not None:
        summed = ddt32.reshape(B, H, psplit, L).sum(2).transpose(1, 2)           # [B, L, H]
        ddt_out.as_strided((B, L, H), (L * ddt_stride, ddt_stride, 1)).copy_(summed)
    if raw:
        return dx, dBC, hpart
    hp = hpart.sum(0).reshape(H, psplit, 3).sum(1)
    return dx, dBC, hp[:, 0], hp[:, 1], hp[:, 2]


def _final_states(final, xBC, H, psplit, K):
    """kernel state layout [B,Hv,128 n,64 p] -> cache layout [B,H,P,N]; conv window [B,C,K]."""
    B = final.shape[0]
    ssm = final.reshape(B, H, psplit, 128, 64).permute(0, 1, 2, 4, 3).reshape(B, H, psplit * 64, 128).contiguous()
    L = xBC.shape[1]
    tail = xBC[:, -K:, :] if L >= K else torch.cat([xBC.new_zeros(B, K - L, xBC.shape[2]), xBC], dim=1)
    return tail.transpose(1, 2).contiguous(), ssm


def _mixer_params_fp32(A_log, D, dt_bias):
    """(-exp(A_log), D, dt_bias) as fp32 [H] views of one buffer, one launch."""
    H = A_log.numel()
    ok = all(t.dtype in (torch.bfloat16, torch.float32) and t.is_contiguous() and t.numel() == H
             for t in (A_log, D, dt_bias))
    if not ok:
        return -torch.exp(A_log.float()), D.float(), dt_bias.float()
    out = torch.empty(3, H, dtype=torch.float32, device=A_log.device)
    mask = sum(1 << i for i, t in enumerate((A_log, D, dt_bias)) if t.dtype == torch.bfloat16)
    _run("ssm_mixer_param_prep", _P(A_log), _P(D), _P(dt_bias), mask, H, _P(out), _st())
    return out[0], out[1], out[2]


class _MixerCore(torch.autograd.Function):
    @staticmethod
    def forward(ctx, zxBCdt, conv_w, conv_b, dt_bias, A_log, D, norm_w, d_inner, G, N, P, eps, gs, recompute,
                want_final):
        _require_bf16(zxBCdt, conv_w, conv_b, norm_w)
        H, psplit, Hv = _ssd_dims(d_inner, P, G, N)
        B, L, W = zxBCdt.shape
        C = d_inner + 2 * G * N
        if W != d_inner + C + H or L % _CT or d_inner % 8 or (G * N) % 8:
            raise ValueError("bad zxBCdt shape for the mixer core")
        # rows may carry padding (row stride ld >= W, multiple of 8): that is how the GEMM epilogue writes them
        if (zxBCdt.stride(2) != 1 or zxBCdt.stride(1) % 8 or zxBCdt.stride(0) != L * zxBCdt.stride(1)
                or zxBCdt.data_ptr() % 16):
            buf = torch.empty(B * L, _ceil8(W), dtype=zxBCdt.dtype, device=zxBCdt.device)[:, :W]
            buf.copy_(zxBCdt.reshape(B * L, W))
            zxBCdt = buf.as_strided((B, L, W), (L * buf.stride(0), buf.stride(0), 1))
        ld = zxBCdt.stride(1)
        flat = zxBCdt.as_strided((B * L, W), (ld, 1))
        z2, xBC, dt_raw2 = flat[:, :d_inner], zxBCdt[..., d_inner:d_inner + C], flat[:, d_inner + C:]
        w2 = conv_w.reshape(C, -1).contiguous()
        conv_out = _conv_fwd(xBC, w2, conv_b, None).view(B * L, C)
        A, Df, bf = _mixer_params_fp32(A_log, D, dt_bias)
        y, dt, l, s_in, final = _ssd_forward(conv_out, dt_raw2, ld, A, Df, bf, B, L, d_inner, G, H, Hv,
                                             want_final=want_final)
        out = _gated_fwd(y, z2, norm_w, eps, gs)
        ctx.dims = (B, L, W, C, d_inner, G, N, P, H, Hv, eps, gs, recompute)
        if recompute:
            ctx.save_for_backward(zxBCdt, w2, conv_b, dt_bias, A_log, D, norm_w, A, Df, bf)
        else:
            ctx.save_for_backward(zxBCdt, w2, conv_b, dt_bias, A_log, D, norm_w, A, Df, bf, conv_out, y, dt, l, s_in)
        ctx.conv_w_shape = conv_w.shape
        ctx.conv_w_param = conv_w if conv_w.is_leaf else None
        out = out.view(B, L, d_inner)
        if want_final:
            conv_state, ssm_state = _final_states(final, xBC, H, psplit, w2.shape[1])
            ctx.mark_non_differentiable(conv_state, ssm_state)
            return out, conv_state, ssm_state
        return out

    @staticmethod
    def backward(ctx, dout, *unused):
        B, L, W, C, d_inner, G, N, P, H, Hv, eps, gs, recompute = ctx.dims
        saved = ctx.saved_tensors
        zxBCdt, w2, conv_b, dt_bias, A_log, D, norm_w, A, Df, bf = saved[:10]
        ld = zxBCdt.stride(1)
        flat = zxBCdt.as_strided((B * L, W), (ld, 1))
        z2, xBC, dt_raw2 = flat[:, :d_inner], zxBCdt[..., d_inner:d_inner + C], flat[:, d_inner + C:]
        if recompute:
            conv_out = _conv_fwd(xBC, w2, conv_b, None).view(B * L, C)
            y, dt, l, s_in, _ = _ssd_forward(conv_out, dt_raw2, ld, A, Df, bf, B, L, d_inner, G, H, Hv)
        else:
            conv_out, y, dt, l, s_in = saved[10:]
        dflat = torch.empty(B * L, ld, dtype=zxBCdt.dtype, device=zxBCdt.device)[:, :W]
        d_zx = dflat.as_strided((B, L, W), (L * ld, ld, 1))
        dout2 = dout.reshape(B * L, d_inner)
        if not dout2.is_contiguous():
            dout2 = dout2.contiguous()
        dy = torch.empty(B * L, d_inner, dtype=torch.bfloat16, device=dout.device)
        small = [ctx.conv_w_param, conv_b, norm_w, A_log, D, dt_bias]
        direct = all(p is None or (getattr(p, "main_grad", None) is not None and p.main_grad.dtype == torch.float32
                                   and p.main_grad.is_contiguous()) for p in small) and ctx.conv_w_param is not None
        if direct:
            # partial sums go straight into the fp32 main-gradient buffers with one finalisation kernel
            gpart = _gated_bwd(y, z2, norm_w, dout2, eps, gs, dy, dflat[:, :d_inner], raw=True)
            dx, dBC, hpart = _ssd_backward(conv_out, dy, y, dt, l, s_in, dt_raw2, ld, A, Df, bf,
                                           dflat[:, d_inner + C:], ld, B, L, d_inner, G, H, Hv, raw=True)
            cpart = _conv_bwd(xBC, w2, conv_b, dx.view(B, L, d_inner), dBC.view(B, L, 2 * G * N), d_inner,
                              d_zx[..., d_inner:d_inner + C], raw=True)
            mask = 0
            for bit, p in enumerate(small):
                if p is not None:
                    if not getattr(p, "grad_stale", False):
                        mask |= 1 << bit
                    p.grad_stale = False
            mg = [None if p is None else p.main_grad for p in small]
            _run("ssm_mixer_small_grads", _p(cpart), cpart.shape[0], C, _p(gpart), gpart.shape[0], d_inner, _p(hpart),
                 hpart.shape[0], Hv, H, _p(A), _p(mg[0]), _p(mg[1]), _p(mg[2]), _p(mg[3]), _p(mg[4]), _p(mg[5]),
                 mask, _st())
            return (d_zx,) + (None,) * 14
        dnorm_w = _gated_bwd(y, z2, norm_w, dout2, eps, gs, dy, dflat[:, :d_inner])
        dx, dBC, dA, dD, dbias = _ssd_backward(conv_out, dy, y, dt, l, s_in, dt_raw2, ld, A, Df, bf,
                                               dflat[:, d_inner + C:], ld, B, L, d_inner, G, H, Hv)
        dw, db = _conv_bwd(xBC, w2, conv_b, dx.view(B, L, d_inner), dBC.view(B, L, 2 * G * N), d_inner,
                           d_zx[..., d_inner:d_inner + C])
        dA_log = (dA * A).to(A_log.dtype)
        return (d_zx, dw.to(w2.dtype).reshape(ctx.conv_w_shape), None if conv_b is None else db.to(conv_b.dtype),
                dbias.to(dt_bias.dtype), dA_log, dD.to(D.dtype), dnorm_w.to(norm_w.dtype),
                None, None, None, None, None, None, None, None)


def mamba2_mixer_core(zxBCdt, conv_w, conv_b, dt_bias, A_log, D, norm_w, d_inner, n_groups, d_state, head_dim, eps,
                      norm_group_size, chunk_size, recompute, return_final_states):
    if chunk_size != _CT:
        raise ValueError("the GPU kernels use 128-token chunks")
    gs = d_inner if norm_group_size is None else norm_group_size
    res = _MixerCore.apply(zxBCdt, conv_w, conv_b, dt_bias, A_log, D, norm_w, d_inner, n_groups, d_state, head_dim,
                           eps, gs, recompute, return_final_states)
    if return_final_states:
        return res[0], (res[1], res[2])
    return res


class _SSDScan(torch.autograd.Function):
    """Stand-alone scan op (tests, custom models): packs x|B|C into the layout the kernels read."""

    @staticmethod
    def forward(ctx, x, dt_raw, A, Bm, Cm, D, dt_bias, want_final, init_state):
        _require_bf16(x, Bm, Cm)
        Bsz, L, H, P = x.shape
        G, N = Bm.shape[2], Bm.shape[3]
        d_inner = H * P
        _, psplit, Hv = _ssd_dims(d_inner, P, G, N)
        conv_out = torch.cat([x.reshape(Bsz, L, d_inner), Bm.reshape(Bsz, L, G * N), Cm.reshape(Bsz, L, G * N)],
                             dim=-1).reshape(Bsz * L, -1).contiguous()
        Hp = _ceil8(H)
        dtr = torch.zeros(Bsz * L, Hp, dtype=torch.bfloat16, device=x.device)
        dtr[:, :H] = dt_raw.reshape(Bsz * L, H).to(torch.bfloat16)
        Af, Df, bf = A.float().contiguous(), D.float().contiguous(), dt_bias.float().contiguous()
        init = None
        if init_state is not None:   # [B,H,P,N] -> [B,Hv,128,64]
            init = init_state.float().reshape(Bsz, H, psplit, 64, N).permute(0, 1, 2, 4, 3).reshape(
                Bsz, Hv, N, 64).contiguous()
        y, dt, l, s_in, final = _ssd_forward(conv_out, dtr, Hp, Af, Df, bf, Bsz, L, d_inner, G, H, Hv, init,
                                             want_final)
        ctx.save_for_backward(conv_out, y, dt, l, s_in, dtr, Af, Df, bf)
        ctx.dims = (Bsz, L, H, P, G, N, Hv, Hp)
        ctx.in_dtypes = (dt_raw.dtype, A.dtype, D.dtype, dt_bias.dtype)
        yv = y.view(Bsz, L, H, P)
        if want_final:
            fin = final.reshape(Bsz, H, psplit, N, 64).permute(0, 1, 2, 4, 3).reshape(Bsz, H, P, N).contiguous()
            ctx.mark_non_differentiable(fin)
            return yv, fin
        return yv

    @staticmethod
    def backward(ctx, dy, *unused):
        conv_out, y, dt, l, s_in, dtr, Af, Df, bf = ctx.saved_tensors
        Bsz, L, H, P, G, N, Hv, Hp = ctx.dims
        d_inner = H * P
        dy2 = dy.reshape(Bsz * L, d_inner).contiguous()
        ddt = torch.zeros(Bsz * L, Hp, dtype=torch.bfloat16, device=dy.device)
        dx, dBC, dA, dD, dbias = _ssd_backward(conv_out, dy2, y, dt, l, s_in, dtr, Hp, Af, Df, bf, ddt, Hp,
                                               Bsz, L, d_inner, G, H, Hv)
        t0, t1, t2, t3 = ctx.in_dtypes
        return (dx.view(Bsz, L, H, P), ddt[:, :H].reshape(Bsz, L, H).to(t0), dA.to(t1),
                dBC[:, :G * N].reshape(Bsz, L, G, N).to(dy.dtype), dBC[:, G * N:].reshape(Bsz, L, G, N).to(dy.dtype),
                dD.to(t2), dbias.to(t3), None, None)


def ssd_chunk_scan(x, dt_raw, A, Bm, Cm, D, dt_bias, chunk_size, initial_state, return_final_state):
    if chunk_size != _CT:
        raise ValueError("the GPU kernels use 128-token chunks")
    return _SSDScan.apply(x, dt_raw, A, Bm, Cm, D, dt_bias, return_final_state, initial_state)


# ======================================================================================
# decode
# ======================================================================================
_DECODE_PARAMS = {}


def _decode_params_fp32(A_log, D, dt_bias):
    """(-exp(A_log), D, dt_bias) in fp32 for the decode kernel, prepared once per parameter version instead of three
    casts per layer and token (inference leaves the parameters untouched, so this is once per model)."""
    key = (A_log.data_ptr(), D.data_ptr(), dt_bias.data_ptr())
    ver = (A_log._version, D._version, dt_bias._version)
    hit = _DECODE_PARAMS.get(key)
    if hit is None or hit[0] != ver:
        hit = (ver, _mixer_params_fp32(A_log.detach(), D.detach(), dt_bias.detach()))
        _DECODE_PARAMS[key] = hit
    return hit[1]


@torch.no_grad()
def ssm_decode_step(zxBCdt, conv_state, ssm_state, conv_w, conv_b, dt_bias, A_log, D, norm_w, d_inner, n_groups,
                    d_state, head_dim, eps, norm_group_size):
    _require_bf16(zxBCdt, conv_state, conv_w, norm_w)
    if ssm_state.dtype != torch.float32:
        raise TypeError("the decode kernel keeps the SSM state in fp32")
    B, W = zxBCdt.shape
    C = d_inner + 2 * n_groups * d_state
    H = d_inner // head_dim
    if conv_state.shape[-1] != 4 or not conv_state.is_contiguous() or not ssm_state.is_contiguous():
        raise ValueError("decode needs contiguous states and a 4-tap conv window")
    if zxBCdt.stride(1) != 1:
        zxBCdt = zxBCdt.contiguous()
    dev = zxBCdt.device
    act = torch.empty(B, C, dtype=torch.float32, device=dev)
    xBC = zxBCdt[:, d_inner:d_inner + C]
    _run("ssm_decode_conv_step", _p(xBC), _ll(zxBCdt.stride(0)), _p(conv_state), _p(conv_w.reshape(C, 4).contiguous()),
         _p(conv_b), _p(act), B, C, _st())
    y = torch.empty(B, d_inner, dtype=torch.bfloat16, device=dev)
    A, Df, bf = _decode_params_fp32(A_log, D, dt_bias)
    _run("ssm_decode_ssm_step", _p(act), _p(zxBCdt[:, d_inner + C:]), _ll(zxBCdt.stride(0)), _p(bf),
         _p(A), _p(Df), _p(ssm_state), _p(y), B, C, H, head_dim, d_state, n_groups, d_inner, _st())
    gs = d_inner if norm_group_size is None else norm_group_size
    return _gated_fwd(y, zxBCdt[:, :d_inner], norm_w, eps, gs)


# ======================================================================================
# rotary position embedding
# ======================================================================================
_ROPE_TABLES = {}


def rotary_tables(seq_len: int, dim: int, theta: float, device, offset: int = 0):
    """fp32 cos / sin tables [seq_len, dim / 2], built once per (length, dim, theta, offset, device) and kept."""
    key = (int(seq_len), int(dim), float(theta), int(offset), str(device))
    if key not in _ROPE_TABLES:
        from . import oracle
        cos, sin = oracle.rotary_tables(seq_len, dim, theta, device=device, offset=offset)
        _ROPE_TABLES[key] = (cos.contiguous(), sin.contiguous())
    return _ROPE_TABLES[key]


def _rope_launch(x, cos, sin, inverse: bool):
    B, L, H, Dh = x.shape
    rd = cos.shape[-1] * 2
    x3 = x if (x.stride(3) == 1 and x.stride(2) == Dh and x.stride(0) == L * x.stride(1)) else x.contiguous()
    out = torch.empty(B, L, H, Dh, dtype=x.dtype, device=x.device)
    _run("ssm_rope", _p(x3), _ll(x3.stride(1)), _p(out), _ll(H * Dh), _p(cos), _p(sin), _ll(B * L), L, H, Dh, rd,
         int(inverse), _st())
    return out


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin):
        ctx.save_for_backward(cos, sin)
        return _rope_launch(x, cos, sin, False)

    @staticmethod
    def backward(ctx, dy):
        cos, sin = ctx.saved_tensors
        return _rope_launch(dy, cos, sin, True), None, None


def apply_rotary(x, cos, sin):
    """Rotate-half rotary embedding on the first 2 * cos.shape[-1] channels of x [B, L, H, Dh] (bf16); cos / sin fp32
    [L, rd / 2].  The backward pass is the same kernel with the angle negated."""
    _require_bf16(x)
    rd = cos.shape[-1] * 2
    if x.shape[-1] % 8 or rd % 16 or cos.dtype != torch.float32 or cos.shape[0] != x.shape[1]:
        raise ValueError("rotary kernel needs head_dim % 8 == 0, rotary dim % 16 == 0 and fp32 tables of the sequence length")
    return _Rope.apply(x, cos, sin)


# ======================================================================================
# attention
# ======================================================================================
class _Attention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v):
        B, L, Hq, D = q.shape
        Hkv = k.shape[2]
        q2, k2, v2 = q.reshape(B * L, Hq * D), k.reshape(B * L, Hkv * D), v.reshape(B * L, Hkv * D)
        q2, k2, v2 = [t if t.is_contiguous() else t.contiguous() for t in (q2, k2, v2)]
        out = torch.empty_like(q2)
        lse = torch.empty(B, Hq, L, dtype=torch.float32, device=q.device)
        scale = 1.0 / (D ** 0.5)
        _run("ssm_attn_fwd", _p(q2), _p(k2), _p(v2), _p(out), _p(lse), B, L, Hq, Hkv, D, _c.c_float(scale),
             _p(status_tensor(q.device)), _st())
        ctx.save_for_backward(q2, k2, v2, out, lse)
        ctx.dims = (B, L, Hq, Hkv, D, scale)
        return out.view(B, L, Hq, D)

    @staticmethod
    def backward(ctx, dout):
        q2, k2, v2, out, lse = ctx.saved_tensors
        B, L, Hq, Hkv, D, scale = ctx.dims
        do2 = dout.reshape(B * L, Hq * D)
        if not do2.is_contiguous():
            do2 = do2.contiguous()
        delta = (do2.view(B, L, Hq, D).float() * out.view(B, L, Hq, D).float()).sum(-1).permute(0, 2, 1).contiguous()
        dq32 = torch.zeros(B * L, Hq * D, dtype=torch.float32, device=dout.device)
        dk, dv = torch.empty_like(k2), torch.empty_like(v2)
        _run("ssm_attn_bwd", _p(q2), _p(k2), _p(v2), _p(do2), _p(lse), _p(delta), _p(dq32), _p(dk), _p(dv), B, L, Hq, Hkv,
             D, _c.c_float(scale), _p(status_tensor(dout.device)), _st())
        return (dq32.to(torch.bfloat16).view(B, L, Hq, D), dk.view(B, L, Hkv, D), dv.view(B, L, Hkv, D))


def attention(q, k, v, causal=True):
    _require_bf16(q, k, v)
    if not causal:
        raise NotImplementedError("the GPU attention kernel is causal")
    if q.shape[-1] != 128 or q.shape[1] % 128 or q.shape[1] != k.shape[1]:
        raise ValueError("the GPU attention kernel needs head_dim 128 and equal q/k lengths that are multiples of 128")
    return _Attention.apply(q, k, v)
