"""Column-/row-parallel linear layers whose sequence-parallel collective runs inside the GEMM kernel.

    all_gather_linear      y = all_gather_seq(x_shard) W^T     one kernel: one thread per CTA moves boxes of the local
                           shard into every rank's gather buffer (TMA load into the idle epilogue staging buffers,
                           one TMA store per rank) in up to four column groups with a flag per (source, group), while
                           the TMA / MMA warps already compute: the local shard first (read in place), a remote
                           shard's columns as they land
                           backward: dX = reduce_scatter_seq(dY W) (the kernel below); dW += dY^T x_gathered
    linear_reduce_scatter  y_shard = reduce_scatter_seq(x W^T)  one kernel: tiles are walked owner by owner, the
                           epilogue TMA-stores every partial tile into the owning rank's landing slot and reports
                           the owner as soon as its last tile for it has landed; the sum runs in the same kernel
                           (two ranks: in the epilogue of the own-row tiles; more: by all CTAs after their tiles)
                           backward: dX = all_gather_seq(dY_shard) W (the kernel above), dW += dY_full^T x

Either kernel can be switched to "NCCL collective + plain GEMM kernel" (`fused.set_kernel`, `fused_tune.pick_fastest`);
the autograd functions stay the same.

These replace the pairs (all-gather, GEMM) and (GEMM, reduce-scatter) that the reference leaves to
neuronx-distributed's ColumnParallelLinear / RowParallelLinear with sequence parallelism
(mamba2/mamba2_mixer.py:156-158,186-188,228,233).  The library-collective versions in `mappings.py` remain
the measured baseline and the path for shapes the fused kernels do not take (batch > 1, shard rows not a
multiple of 128).
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import fused
from . import state as ps
from . import symm
from ..ops import cuda_ops
from ..ops.cuda_ops import _P, _ceil8, _ll, _run, _st, status_tensor

CALLS = {"ag_gemm": 0, "gemm_rs": 0}     # how many fused kernels this process has launched
_c = ctypes


def _ws_for(rows_total: int, cols: int, device):
    return symm.get_workspace(max(rows_total, 1), max(cols, 1), device)


def ready_for(x: torch.Tensor) -> bool:
    tp = ps.get_tensor_model_parallel_size()
    if tp < 2 or tp > symm.MAX_RANKS or not x.is_cuda or x.dtype != torch.bfloat16 or x.dim() != 3:
        return False
    return x.shape[0] == 1


def _fused_gemm(a, b, out, M, N, K, lda, ldb, ldc, a_mn, b_mn, mode, bias, act, ws, seq, ag=None, rs=None, ce=None):
    null = symm._ptr_array([])
    ag = ag or dict(on=0, rows=0, base=0, src=None, src_ld=0, dst=null, dst_ld=0, counter=0)
    rs = rs or dict(on=0, rows=0, base=0, land=null, ld=0, counters=0, local=0, slot_stride=0, out=None, out_ld=0)
    ce = ce or dict(labels=None, vocab_start=0, tmax=None, tsum=None, tgt=None)
    _run("ssm_gemm_bf16_fused", _P(a), _P(b), _P(out), M, N, K, _ll(lda), _ll(ldb), _ll(ldc), int(a_mn), int(b_mn), mode,
         _P(bias), int(act), _P(status_tensor(ws.device)), _st(), ws.nranks, ws.me, seq, _P(ws.seq_base),
         ws.flag_ptr_array,
         ag["on"], ag["rows"], ag["base"], _P(ag["src"]), _ll(ag["src_ld"]), ag["dst"], _ll(ag["dst_ld"]),
         _c.c_void_p(ag["counter"]),
         rs["on"], rs["rows"], rs["base"], rs["land"], _ll(rs["ld"]), _c.c_void_p(rs["counters"]),
         _c.c_void_p(rs["local"]), _ll(rs["slot_stride"]), _P(rs["out"]), _ll(rs["out_ld"]),
         _P(ce["labels"]), _ll(ce["vocab_start"]), _P(ce["tmax"]), _P(ce["tsum"]), _P(ce["tgt"]))


def _ag_gemm(x_shard2, w, b_mn, bias, ws, act=0, ce=None):
    """gathered [T*Ls, K] (view of the workspace) and y = gathered @ (w^T or w).  `ce` = (labels [T*Ls] int64,
    vocab_start): the epilogue also produces the cross-entropy statistics of the rows of y; returns
    (gathered, y, (row max, row sum-exp, target logit)) then."""
    Ls, K = x_shard2.shape
    T = ws.nranks
    M = T * Ls
    N = w.shape[1] if b_mn else w.shape[0]
    if not fused.kernel_enabled("ag_gemm"):
        # library collective + the plain GEMM kernel (same results, same autograd functions around it)
        gathered = torch.empty(M, K, dtype=x_shard2.dtype, device=x_shard2.device)
        dist.all_gather_into_tensor(gathered, x_shard2.contiguous(), group=ws.group)
        CALLS["ag_gemm_library"] = CALLS.get("ag_gemm_library", 0) + 1
        if ce is not None:
            labels, vocab_start = ce
            y, stats = cuda_ops.gemm_ce(gathered, w, labels, vocab_start)
            return gathered, y, stats
        return gathered, cuda_ops.gemm(gathered, w, b_mn=b_mn, bias=bias, gelu=bool(act))
    CALLS["ag_gemm"] += 1
    seq, par = ws.next_seq(symm.KIND_AG)
    off = ws.gather_offset(par)
    gathered = ws.local_view(off, M, K)
    y = torch.empty(M, _ceil8(N), dtype=torch.bfloat16, device=x_shard2.device)[:, :N]
    if x_shard2.stride(1) != 1 or x_shard2.stride(0) % 8 or x_shard2.data_ptr() % 16:
        x_shard2 = x_shard2.contiguous()
    ced, stats = None, None
    if ce is not None:
        labels, vocab_start = ce
        ced, stats = cuda_ops.ce_epilogue_buffers(M, N, K, labels, vocab_start, rows_per_shard=Ls)
    _fused_gemm(gathered, w, y, M, N, K, K, w.stride(0), y.stride(0), False, b_mn, 0, bias, act, ws, seq,
                ag=dict(on=1, rows=Ls, base=ws.flag_base(symm.KIND_AG, par), src=x_shard2, src_ld=x_shard2.stride(0),
                        dst=ws.peer_ptrs(off), dst_ld=K, counter=ws.counter_ptr(0)), ce=ced)
    if ce is not None:
        return gathered, y, cuda_ops.ce_merge(ced, stats)
    return gathered, y


def _gemm_rs(a2, w, b_mn, ws):
    """reduce_scatter over rows of (a2 @ w^T) (or a2 @ w when b_mn): returns this rank's [Ls, N] block."""
    M, K = a2.shape
    T = ws.nranks
    Ls = M // T
    N = w.shape[1] if b_mn else w.shape[0]
    if not fused.kernel_enabled("gemm_rs"):
        full = cuda_ops.gemm(a2, w, b_mn=b_mn)
        if not full.is_contiguous():
            full = full.contiguous()
        out = torch.empty(Ls, N, dtype=full.dtype, device=full.device)
        dist.reduce_scatter_tensor(out, full, group=ws.group)
        CALLS["gemm_rs_library"] = CALLS.get("gemm_rs_library", 0) + 1
        return out
    CALLS["gemm_rs"] += 1
    seq, par = ws.next_seq(symm.KIND_RS)
    off = ws.land_offset(par)
    slot_bytes = Ls * N * 2
    land = symm._ptr_array([p + off + ws.me * slot_bytes for p in ws.base_ptrs])
    if a2.stride(1) != 1 or a2.stride(0) % 8 or a2.data_ptr() % 16:
        a2 = cuda_ops._as_operand(a2)
    out = torch.empty(Ls, N, dtype=torch.bfloat16, device=a2.device)
    _fused_gemm(a2, w, None, M, N, K, a2.stride(0), w.stride(0), 0, False, b_mn, 3, None, 0, ws, seq,
                rs=dict(on=1, rows=Ls, base=ws.flag_base(symm.KIND_RS, par), land=land, ld=N,
                        counters=ws.counter_ptr(8), local=ws.local_ptr(off), slot_stride=Ls * N, out=out, out_ld=N))
    return out


def small_allreduce(data: torch.Tensor, op: str = "sum") -> bool:
    """In-place all-reduce (sum or max) of a small fp32 vector over the TP group through the symmetric workspace:
    one single-CTA kernel in which every rank stores its vector into every rank's slot, publishes a flag, waits
    (bounded) for the others and reduces locally.  Used for the cross-entropy statistics, sequence-parallel norm
    gradients and the gradient norm instead of three library all-reduces (modeling_mamba2.py:505-510 of the
    reference goes through parallel_cross_entropy).  Returns False (nothing done) when no workspace exists yet or
    the vector does not fit, so the caller can use the library collective."""
    ws = symm._WS
    if (ws is None or ws.group is not ps.get_tensor_model_parallel_group() or not data.is_cuda
            or data.dtype != torch.float32 or not data.is_contiguous() or data.numel() > symm.SMALL_N_MAX):
        return False
    CALLS["small_allreduce"] = CALLS.get("small_allreduce", 0) + 1
    seq, par = ws.next_seq(symm.KIND_AR)
    _run("ssm_small_allreduce", _P(data), data.numel(), symm.SMALL_N_MAX, ws.peer_ptrs(ws.slots_offset(par)),
         ws.flag_ptr_array, ws.flag_base(symm.KIND_AR, par), ws.nranks, ws.me, seq, _P(ws.seq_base),
         0 if op == "sum" else 1, _P(status_tensor(ws.device)), _st())
    return True


def allreduce_bf16(x: torch.Tensor):
    """Sum of a bf16 activation over the TP group in one kernel (stores into every rank's slot, flag, bounded wait,
    fp32 sum): the decode-time replacement of the all-reduce after the row-parallel out_proj
    (mamba2/mamba2_mixer.py:233 with sequence parallelism off).  Returns None when it does not apply."""
    T = ps.get_tensor_model_parallel_size()
    if (T < 2 or T > symm.MAX_RANKS or not x.is_cuda or x.dtype != torch.bfloat16 or x.numel() % 8
            or x.numel() > (1 << 21) or torch.is_grad_enabled() and x.requires_grad):
        return None
    n = x.numel()
    ws = _ws_for(T * max(1, -(-n // x.shape[-1])), x.shape[-1], x.device)
    if ws is None or n * T * 2 > ws.gather_bytes:
        return None
    xc = x.contiguous()
    out = torch.empty_like(xc)
    CALLS["allreduce_bf16"] = CALLS.get("allreduce_bf16", 0) + 1
    seq, par = ws.next_seq(symm.KIND_AG)
    stride = ws.gather_bytes // 2 // T // 8 * 8
    _run("ssm_allreduce_bf16", _P(xc), _P(out), _ll(n), ws.peer_ptrs(ws.gather_offset(par)), _ll(stride), T, ws.me,
         ws.flag_ptr_array, ws.flag_base(symm.KIND_AG, par), seq, _P(ws.seq_base), _c.c_void_p(ws.counter_ptr(34)),
         _P(status_tensor(ws.device)), _st())
    return out


class _VocabEmbedScatter(torch.autograd.Function):
    """Vocabulary-parallel embedding whose output is already scattered along the sequence.  The reference sums
    the T masked partial lookups with an all-reduce and slices (mamba2/modeling_mamba2.py:276,300-301); here the
    rank that holds a token's row stores it into the sequence owner's buffer over NVLink (no reduction needed: one
    rank holds each row).  Backward: the output gradients are pushed to every rank's gather buffer and each rank
    scatter-adds the rows of its own vocabulary range into the fp32 gradient."""

    @staticmethod
    def forward(ctx, ids, w, vocab_start, ws):
        B, L = ids.shape
        T, D = ws.nranks, w.shape[1]
        Ls = L // T
        ids_c = ids.contiguous()
        CALLS["vocab_embed"] = CALLS.get("vocab_embed", 0) + 1
        seq, par = ws.next_seq(symm.KIND_EMB)
        off = ws.embed_offset(par)
        base = ws.flag_base(symm.KIND_EMB, par)
        _run("ssm_vocab_embed_push", _P(ids_c), _P(w), _ll(vocab_start), _ll(w.shape[0]), ws.peer_ptrs(off), B, L, Ls, D,
             T, ws.me, ws.flag_ptr_array, base, seq, _P(ws.seq_base), _c.c_void_p(ws.counter_ptr(32)), _st())
        out = torch.empty(B, Ls, D, dtype=w.dtype, device=w.device)
        _run("ssm_embed_wait_copy", _P(ws.local_view(off, B * Ls, D)), _P(out), _ll(B * Ls * D), T,
             _c.c_void_p(ws.base_ptrs[ws.me]), base, seq, _P(ws.seq_base), _P(status_tensor(ws.device)), _st())
        ctx.save_for_backward(ids_c)
        ctx.w, ctx.ws, ctx.vocab_start = w, ws, vocab_start
        return out

    @staticmethod
    def backward(ctx, g):
        (ids,), w, ws = ctx.saved_tensors, ctx.w, ctx.ws
        B, L = ids.shape
        T, D = ws.nranks, w.shape[1]
        Ls = L // T
        g2 = g.reshape(B * Ls, D)
        if g2.stride(1) != 1 or g2.stride(0) % 8:
            g2 = g2.contiguous()
        seq, par = ws.next_seq(symm.KIND_AG)
        off = ws.gather_offset(par)
        base = ws.flag_base(symm.KIND_AG, par)
        _run("ssm_push_shard", _P(g2), _ll(g2.stride(0)), ws.peer_ptrs(off), _ll(D), _ll(ws.me * B * Ls), B * Ls, D, T,
             ws.me, ws.flag_ptr_array, base, seq, _P(ws.seq_base), _c.c_void_p(ws.counter_ptr(33)),
             min(148, max(1, B * Ls * D // 8 // 256)), _st())
        tgt, direct = cuda_ops.embed_grad_target(w)
        _run("ssm_embed_bwd", _P(ids), _P(ws.local_view(off, B * L, D)), _ll(D), _P(tgt), _ll(ctx.vocab_start),
             _ll(w.shape[0]), B, L, Ls, D, T, _c.c_void_p(ws.base_ptrs[ws.me]), base, seq, _P(ws.seq_base),
             _P(status_tensor(ws.device)), _st())
        return None, (None if direct else tgt.to(w.dtype)), None, None


def vocab_embed_scatter(ids, w, vocab_start):
    """Fused vocabulary-parallel embedding + sequence scatter, or None when the shapes do not fit the kernels."""
    T = ps.get_tensor_model_parallel_size()
    if (T < 2 or T > symm.MAX_RANKS or ids.dim() != 2 or ids.dtype != torch.int64 or w.dtype != torch.bfloat16
            or not w.is_cuda or not w.is_contiguous() or w.shape[1] % 8 or ids.shape[1] % T):
        return None
    B, L = ids.shape
    ws = _ws_for(B * L, w.shape[1], w.device)
    if ws is None or not ws.fits(B * L, w.shape[1]):
        return None
    return _VocabEmbedScatter.apply(ids, w, int(vocab_start), ws)


def _shape_ok(Ls, K, N, ws):
    """Shard rows in whole 128-row tiles; K (the gathered / reduced inner extent that is moved in 16-byte vectors)
    a multiple of 8.  N (output features of an all-gather GEMM) is free: edge tiles are masked, rows are padded to
    a multiple of 8 elements by the callers."""
    return Ls % 128 == 0 and K % 8 == 0 and N >= 1 and ws is not None


class _AllGatherLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, ws, ce_labels=None, ce_vocab_start=0):
        Ls, K = x.shape[1], x.shape[2]
        ce = None if ce_labels is None else (ce_labels, ce_vocab_start)
        res = _ag_gemm(x.reshape(Ls, K), w, False, bias, ws, ce=ce)
        gathered, y = res[0], res[1]
        xg = gathered.clone()                      # kept for dW; the workspace buffer is reused two calls later
        ctx.save_for_backward(xg, w)
        ctx.ws, ctx.has_bias = ws, bias is not None
        y3 = y.as_strided((1, y.shape[0], w.shape[0]), (y.shape[0] * y.stride(0), y.stride(0), 1))
        if ce is not None:
            ctx.mark_non_differentiable(*res[2])
            return (y3,) + tuple(res[2])
        return y3

    @staticmethod
    def backward(ctx, dy, *unused):
        xg, w = ctx.saved_tensors
        ws = ctx.ws
        N = w.shape[0]
        dy2 = dy.reshape(-1, N) if dy.dim() != 2 else dy
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = _gemm_rs(dy2, w, True, ws)         # reduce_scatter(dY W)
            dx = dx.reshape(1, dx.shape[0], dx.shape[1])
        if ctx.needs_input_grad[1]:
            if not cuda_ops.wgrad_to_main_grad(dy2, xg, w):
                dw = cuda_ops.gemm(dy2, xg, a_mn=True, b_mn=True).contiguous()
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy.dtype)
        return dx, dw, db, None, None, None


class _AllGatherMultiLinear(torch.autograd.Function):
    """Several column-parallel projections of the same sequence-parallel input (q, k, v of the hybrid attention,
    mamba2hybrid/mamba2hybrid_attn.py:411-413) behind ONE fused all-gather: the first GEMM carries the push of
    the shard and waits per source, the others read the gathered rows that are then complete.  Backward: one
    GEMM + reduce-scatter over the concatenated output gradients and weights, one wgrad GEMM per weight."""

    @staticmethod
    def forward(ctx, x, ws, *weights):
        Ls, K = x.shape[1], x.shape[2]
        gathered, y0 = _ag_gemm(x.reshape(Ls, K), weights[0], False, None, ws)
        xg = gathered.clone()
        outs = [y0] + [cuda_ops.gemm(xg, w) for w in weights[1:]]
        ctx.save_for_backward(xg, *weights)
        ctx.ws = ws
        return tuple(y.reshape(1, y.shape[0], w.shape[0]) for y, w in zip(outs, weights))

    @staticmethod
    def backward(ctx, *dys):
        xg, *weights = ctx.saved_tensors
        ws = ctx.ws
        dy2 = [dy.reshape(-1, w.shape[0]) for dy, w in zip(dys, weights)]
        dx = None
        if ctx.needs_input_grad[0]:
            dcat = torch.cat(dy2, dim=1)
            wcat = torch.cat(list(weights), dim=0)
            dx = _gemm_rs(dcat, wcat, True, ws)
            dx = dx.reshape(1, dx.shape[0], dx.shape[1])
        dws = []
        for i, (d, w) in enumerate(zip(dy2, weights)):
            if not ctx.needs_input_grad[2 + i]:
                dws.append(None)
                continue
            d = d if d.stride(1) == 1 and d.stride(0) % 8 == 0 else d.contiguous()
            if cuda_ops.wgrad_to_main_grad(d, xg, w):
                dws.append(None)
            else:
                dws.append(cuda_ops.gemm(d, xg, a_mn=True, b_mn=True).contiguous())
        return (dx, None, *dws)


class _LinearReduceScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, ws):
        L, K = x.shape[1], x.shape[2]
        x2 = x.reshape(L, K)
        y = _gemm_rs(x2, w, False, ws)
        ctx.save_for_backward(x2, w)
        ctx.ws = ws
        return y.reshape(1, y.shape[0], y.shape[1])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        ws = ctx.ws
        Ls, N = dy.shape[1], dy.shape[2]
        dyg, dx = _ag_gemm(dy.reshape(Ls, N), w, True, None, ws)      # all_gather(dY) W
        dw = None
        if ctx.needs_input_grad[1]:
            if not cuda_ops.wgrad_to_main_grad(dyg, x2, w):
                dw = cuda_ops.gemm(dyg, x2, a_mn=True, b_mn=True).contiguous()
        return dx.reshape(1, dx.shape[0], dx.shape[1]), dw, None


class _Impl:
    @staticmethod
    def ready_for(x):
        return ready_for(x)

    @staticmethod
    def all_gather_linear(x, w, bias=None, ce=None):
        T = ps.get_tensor_model_parallel_size()
        Ls, K = x.shape[1], x.shape[2]
        ws = _ws_for(T * Ls, K, x.device)
        if not _shape_ok(Ls, K, w.shape[0], ws) or not ws.fits(T * Ls, K):
            from . import mappings as mp
            from .. import ops
            xg = mp.gather_from_sequence_parallel_region(x, True)
            if ce is not None:
                return ops.linear_ce(xg, w, ce[0], ce[1])
            return ops.linear(xg, w, bias)
        if ce is not None:
            out = _AllGatherLinear.apply(x, w, bias, ws, ce[0], int(ce[1]))
            return out[0], tuple(out[1:])
        return _AllGatherLinear.apply(x, w, bias, ws)

    @staticmethod
    def all_gather_multi_linear(x, weights):
        T = ps.get_tensor_model_parallel_size()
        Ls, K = x.shape[1], x.shape[2]
        ws = _ws_for(T * Ls, K, x.device)
        ntot = sum(w.shape[0] for w in weights)
        if (not all(_shape_ok(Ls, K, w.shape[0], ws) for w in weights) or not ws.fits(T * Ls, K)
                or not ws.fits(T * Ls, ntot)):
            return None
        return _AllGatherMultiLinear.apply(x, ws, *weights)

    @staticmethod
    def linear_reduce_scatter(x, w):
        T = ps.get_tensor_model_parallel_size()
        L, K = x.shape[1], x.shape[2]
        N = w.shape[0]
        ws = _ws_for(L, N, x.device)
        if L % T or not _shape_ok(L // T, K, N, ws) or not ws.fits(L, N):
            from . import mappings as mp
            from .. import ops
            return mp.reduce_scatter_to_sequence_parallel_region(ops.linear(x, w, None))
        return _LinearReduceScatter.apply(x, w, ws)


def install() -> None:
    fused.register(_Impl)
