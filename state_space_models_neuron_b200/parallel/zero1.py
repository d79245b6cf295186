"""ZeRO-1 optimizer: optimizer state and fp32 master weights sharded over the data-parallel group.

Replaces what the reference obtains from `nxd.initialize_parallel_optimizer(...)` with
`zero_one_enabled` plus `AdamW_FP32OptimParams` (train.py:71-77,123-138; utils.py:26-33):
  * model parameters live in one flat buffer per rank, gradients accumulate in a flat fp32 buffer
    (`param.main_grad`, fp32 gradient accumulation across micro-steps),
  * step = [TP all-reduce of sequence-parallel-tagged grads] -> DP reduce-scatter (average) ->
    global grad-norm over DP x TP -> clip -> AdamW on the rank's fp32 master shard -> DP all-gather of
    the updated low-precision parameters,
  * with `shard=False` the same code is plain data parallelism (all-reduce, full state everywhere).
The flat layout orders parameters as [TP-sharded | TP-replicated] x [decay | no decay] so that every
rank's shard is a handful of homogeneous segments; the AdamW update and the norm run as one fused
kernel per segment on GPUs (`adamw_kernel` / `sumsq_kernel` in `ops/csrc/elementwise.cu`, the peer-memory
variants `zero1_*` in `ops/csrc/comm.cu`) and as torch ops on CPU.
A step whose gradient norm is not finite is skipped on the device (no host synchronisation): the clip coefficient
becomes negative, the AdamW kernels leave parameters and moments untouched, and `skipped_steps()` counts it.
"""
from __future__ import annotations

import math
import os
from typing import Dict, Iterable, List, Optional, Tuple

import torch
import torch.distributed as dist

from . import state as ps

_ALIGN = 128  # elements; keeps every parameter 256-byte aligned in the bf16 buffer


def _ceil_to(x: int, m: int) -> int:
    return (x + m - 1) // m * m


class Zero1Optimizer(torch.optim.Optimizer):
    def __init__(self, param_groups: Iterable[dict], lr: float = 1e-3, betas: Tuple[float, float] = (0.9, 0.999),
                 eps: float = 1e-8, weight_decay: float = 0.0, shard: bool = True,
                 max_grad_norm: Optional[float] = 1.0, master_dtype: torch.dtype = torch.float32,
                 grad_dtype: torch.dtype = torch.float32):
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        super().__init__(param_groups, defaults)
        self.dp_size = ps.get_data_parallel_size()
        self.dp_rank = ps.get_data_parallel_rank()
        self.dp_group = ps.get_data_parallel_group()
        self.tp_size = ps.get_tensor_model_parallel_size()
        self.tp_rank = ps.get_tensor_model_parallel_rank()
        self.tp_group = ps.get_tensor_model_parallel_group()
        self.shard = bool(shard) and self.dp_size > 1
        self.max_grad_norm = max_grad_norm
        self.master_dtype = master_dtype
        self.grad_dtype = grad_dtype
        self.step_count = 0
        self.last_grad_norm: Optional[torch.Tensor] = None
        # called in step() once the local gradients are final (lazy zeroing finished, sequence-parallel-tagged
        # gradients summed over the TP group), before the data-parallel reduction: per-parameter `main_grad` can be
        # inspected there (gradient statistics, tests); not called while a CUDA graph is being captured
        self.post_reduce_hook = None
        self._build_flat_buffers()

    # ------------------------------------------------------------------------------------
    def _want_fused_dp(self) -> bool:
        """ZeRO-1 collectives inside our own kernels over peer memory (instead of NCCL reduce-scatter/all-gather):
        CUDA, sharded, at most 8 DP ranks, bf16 parameters with fp32 gradients and master weights."""
        from . import fused
        return bool(self.shard and self.device.type == "cuda" and fused.is_enabled() and self.dp_size <= 8
                    and self.param_dtype == torch.bfloat16 and self.grad_dtype == torch.float32
                    and self.master_dtype == torch.float32 and fused.zero1_enabled())

    def _build_flat_buffers(self) -> None:
        entries = []  # (sort key, group index, param)
        seen = set()
        for gi, g in enumerate(self.param_groups):
            for p in g["params"]:
                if id(p) in seen or not p.requires_grad:
                    continue
                seen.add(id(p))
                replicated = not getattr(p, "tensor_model_parallel", False)
                entries.append(((int(replicated), gi), gi, p))
        entries.sort(key=lambda e: e[0])
        if not entries:
            raise ValueError("optimizer got no trainable parameters")
        p0 = entries[0][2]
        self.device, self.param_dtype = p0.device, p0.dtype
        off = 0
        self.layout: List[Tuple[torch.nn.Parameter, int, int, int, bool]] = []  # (p, start, numel, group, replicated)
        for key, gi, p in entries:
            if p.dtype != self.param_dtype or p.device != self.device:
                raise ValueError("all parameters must share one dtype and device")
            self.layout.append((p, off, p.numel(), gi, bool(key[0])))
            off += _ceil_to(p.numel(), _ALIGN)
        unit = _ALIGN * (self.dp_size if self.shard else 1)
        self.total = _ceil_to(off, unit)
        self._fused_dp = self._want_fused_dp()
        if self._fused_dp:
            # flat buffers in symmetric memory of the DP group: peers read gradients and write parameters directly
            import torch.distributed._symmetric_memory as symm_mem
            self.flat_params = symm_mem.empty(self.total, dtype=self.param_dtype, device=self.device)
            self.flat_grads = symm_mem.empty(self.total, dtype=self.grad_dtype, device=self.device)
            self._zflags = symm_mem.empty(64, dtype=torch.int32, device=self.device)
            self.flat_params.zero_(), self.flat_grads.zero_(), self._zflags.zero_()
            hp = symm_mem.rendezvous(self.flat_params, self.dp_group)
            hg = symm_mem.rendezvous(self.flat_grads, self.dp_group)
            hf = symm_mem.rendezvous(self._zflags, self.dp_group)
            self._peer_params = [int(x) for x in hp.buffer_ptrs]
            self._peer_grads = [int(x) for x in hg.buffer_ptrs]
            self._peer_flags = [int(x) for x in hf.buffer_ptrs]
            self._symm_handles = (hp, hg, hf)
            self._zseq_base = torch.zeros(1, dtype=torch.int32, device=self.device)
            self._zcounter = torch.zeros(4, dtype=torch.int32, device=self.device)
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.dp_group)
        else:
            self.flat_params = torch.zeros(self.total, dtype=self.param_dtype, device=self.device)
            self.flat_grads = torch.zeros(self.total, dtype=self.grad_dtype, device=self.device)
        for p, start, n, gi, rep in self.layout:
            self.flat_params[start:start + n].copy_(p.data.reshape(-1))
            p.data = self.flat_params[start:start + n].view(p.shape)
            p.main_grad = self.flat_grads[start:start + n].view(p.shape)
            p.grad = None
            p.register_post_accumulate_grad_hook(self._accumulate_hook)
        self.shard_size = self.total // self.dp_size if self.shard else self.total
        self.shard_start = self.shard_size * self.dp_rank if self.shard else 0
        s, e = self.shard_start, self.shard_start + self.shard_size
        self.master = self.flat_params[s:e].to(self.master_dtype).clone()
        self.exp_avg = torch.zeros_like(self.master)
        self.exp_avg_sq = torch.zeros_like(self.master)
        self.shard_grad = torch.zeros(self.shard_size, dtype=torch.float32, device=self.device) \
            if self.shard else None
        # homogeneous segments of the local shard: (lo, hi, group index, replicated), shard-relative
        segs: List[List] = []
        for p, start, n, gi, rep in self.layout:
            lo, hi = max(start, s), min(start + _ceil_to(n, _ALIGN), e)
            if lo >= hi:
                continue
            if segs and segs[-1][1] == lo - s and segs[-1][2] == gi and segs[-1][3] == rep:
                segs[-1][1] = hi - s
            else:
                segs.append([lo - s, hi - s, gi, rep])
        self.segments = [tuple(x) for x in segs]
        self._norm_buf = torch.zeros(1, dtype=torch.float32, device=self.device)
        self._setup_norm_tracking()
        # device-resident step counter and per-group learning rates (read by the fused AdamW kernel, so a captured
        # CUDA graph of the step keeps working when the scheduler changes the rate)
        self._dev_step = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._dev_skipped = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._dev_lr = torch.zeros(max(1, len(self.param_groups)), dtype=torch.float32, device=self.device)
        self._host_lr = torch.zeros(max(1, len(self.param_groups)), dtype=torch.float32,
                                    pin_memory=self.device.type == "cuda")

    @staticmethod
    def _accumulate_hook(p: torch.nn.Parameter) -> None:
        if p.grad is not None:
            if getattr(p, "norm_tracked", False):
                p.norm_tracked, p.norm_dirty = False, True
            if getattr(p, "grad_stale", False):
                p.main_grad.copy_(p.grad)
                p.grad_stale = False
            else:
                p.main_grad.add_(p.grad.to(p.main_grad.dtype))
            p.grad = None

    # ------------------------------------------------------------------------------------
    def zero_grad(self, set_to_none: bool = True) -> None:
        """Lazy: gradients are not cleared here; every parameter is marked stale and the first
        contribution of the next micro-step overwrites `main_grad` instead of adding to it (the wgrad GEMM
        then stores instead of read-modify-write).  Parameters that receive no gradient are zeroed in
        `step()`.  This saves one full pass over the fp32 gradient buffer per step."""
        for p, *_ in self.layout:
            p.grad = None
            p.grad_stale = True
            p.norm_tracked = p.norm_dirty = False
        if getattr(self, "_norm_acc", None) is not None:
            self._norm_acc.zero_()

    def _finish_lazy_zero(self) -> None:
        for p, *_ in self.layout:
            if getattr(p, "grad_stale", False):
                p.main_grad.zero_()
                p.grad_stale = False

    def _allreduce_sequence_parallel_grads(self) -> None:
        """Sum over the TP group the grads of TP-replicated parameters that only saw a slice of
        the sequence (norm weights), as one flat bucket."""
        if self.tp_size == 1:
            return
        tagged = [p for p, *_ in self.layout if getattr(p, "sequence_parallel_enabled", False)]
        if not tagged:
            return
        rng = self._sp_grad_range()
        # the tagged parameters normally sit next to each other in the flat buffer: reduce that slice in place
        bucket = self.flat_grads[rng[0]:rng[1]] if rng else torch.cat([p.main_grad.reshape(-1) for p in tagged])
        from . import fused
        done = bucket.dtype == torch.float32 and all(
            fused.small_allreduce(bucket[i:i + 16384], "sum") for i in range(0, bucket.numel(), 16384)) \
            if bucket.numel() <= 32 * 16384 else False
        if not done:
            dist.all_reduce(bucket, group=self.tp_group)
        if rng:
            return
        off = 0
        for p in tagged:
            p.main_grad.copy_(bucket[off:off + p.numel()].view(p.shape))
            off += p.numel()

    def _sp_grad_range(self):
        """(lo, hi) of the flat-buffer slice that holds exactly the sequence-parallel-tagged gradients (padding
        between them is zero and stays zero under a sum), or None when other parameters lie in between."""
        if not hasattr(self, "_sp_range"):
            spans = sorted((start, start + _ceil_to(n, _ALIGN), bool(getattr(p, "sequence_parallel_enabled", False)))
                           for p, start, n, gi, rep in self.layout)
            tagged = [(a, b) for a, b, t in spans if t]
            lo, hi = tagged[0][0], tagged[-1][1]
            clean = all(t for a, b, t in spans if a >= lo and b <= hi)
            self._sp_range = (lo, min(hi, self.total)) if clean else None
        return self._sp_range

    def _reduce_gradients(self) -> torch.Tensor:
        """Average over DP; returns this rank's fp32 gradient shard."""
        if self.dp_size == 1:
            return self.flat_grads
        if not self.shard:
            dist.all_reduce(self.flat_grads, group=self.dp_group)
            self.flat_grads.mul_(1.0 / self.dp_size)
            return self.flat_grads
        if dist.get_backend(self.dp_group) == "gloo":
            dist.all_reduce(self.flat_grads, group=self.dp_group)
            self.shard_grad.copy_(self.flat_grads[self.shard_start:self.shard_start + self.shard_size])
        else:
            dist.reduce_scatter_tensor(self.shard_grad, self.flat_grads, group=self.dp_group)
        self.shard_grad.mul_(1.0 / self.dp_size)
        return self.shard_grad

    def _setup_norm_tracking(self) -> None:
        """Let the wgrad GEMMs deliver their share of the gradient norm: every tensor-parallel 2-D weight gets a
        pointer to one fp32 accumulator; a GEMM that STORES the gradient (first contribution of a step) adds its
        sum of squares there.  Only without data-parallel reduction (the local gradient is the final one) and with
        fp32 gradients on a GPU.  SSM_B200_FUSED_NORM=0 turns it off."""
        self._norm_acc = None
        self._norm_ranges = {}
        on = (self.device.type == "cuda" and self.dp_size == 1 and self.grad_dtype == torch.float32
              and os.environ.get("SSM_B200_FUSED_NORM", "1") != "0")
        if on:
            from ..ops.functional import _native
            on = _native(self.flat_grads)
        if not on:
            return
        self._norm_acc = torch.zeros(1, dtype=torch.float32, device=self.device)
        for p, start, n, gi, rep in self.layout:
            if p.dim() == 2 and not rep and not getattr(p, "no_norm_tracking", False):
                p.norm_acc = self._norm_acc

    def _tracked_norm_sq(self, g: torch.Tensor):
        """Gradient norm^2 from the GEMM epilogues plus one multi-range pass over everything they did not cover;
        None when tracking is off or a tracked gradient was modified after its GEMM (then the full pass runs)."""
        if self._norm_acc is None or g is not self.flat_grads:
            return None
        if any(getattr(p, "norm_dirty", False) for p, *_ in self.layout):
            return None
        key = tuple(bool(getattr(p, "norm_tracked", False)) for p, *_ in self.layout)
        if not any(key):
            return None
        if key not in self._norm_ranges:
            spans = []
            for (p, start, n, gi, rep), tracked in zip(self.layout, key):
                if tracked or (rep and self.tp_rank != 0):
                    continue
                lo, hi = start, start + _ceil_to(n, _ALIGN)
                if spans and spans[-1][1] == lo:
                    spans[-1][1] = hi
                else:
                    spans.append([lo, hi])
            flat = [v for sp in spans for v in sp]
            self._norm_ranges[key] = (torch.tensor(flat, dtype=torch.int64, device=self.device), len(spans))
        ranges, n = self._norm_ranges[key]
        total = self._norm_buf.zero_()
        total += self._norm_acc
        if n:
            from ..ops import cuda_ops
            cuda_ops._run("ssm_sumsq_ranges", cuda_ops._P(g), cuda_ops._P(ranges), n, cuda_ops._P(total), cuda_ops._st())
        return total

    def _grad_norm_sq(self, g: torch.Tensor) -> torch.Tensor:
        """Sum of squares over all distinct gradient elements of the whole model."""
        total = self._tracked_norm_sq(g)
        if total is not None:
            if self.tp_size > 1:
                from . import fused
                if not fused.small_allreduce(total, "sum"):
                    dist.all_reduce(total, group=self.tp_group)
            return total
        total = self._norm_buf.zero_()
        for lo, hi, gi, rep in self.segments:
            if rep and self.tp_rank != 0:
                continue
            seg = g[lo:hi]
            from ..ops.functional import _native
            if _native(seg):
                from ..ops import cuda_ops
                cuda_ops.sumsq_accumulate(seg, total)
            else:
                for lo2 in range(0, seg.numel(), 1 << 26):
                    total += seg[lo2:lo2 + (1 << 26)].float().pow(2).sum()
        if self.shard:
            dist.all_reduce(total, group=self.dp_group)
        if self.tp_size > 1:
            from . import fused
            if not fused.small_allreduce(total, "sum"):
                dist.all_reduce(total, group=self.tp_group)
        return total

    @torch.no_grad()
    def upload_learning_rates(self) -> None:
        """Copy the groups' current learning rates to the device (outside any graph capture)."""
        for i, grp in enumerate(self.param_groups):
            self._host_lr[i] = float(grp["lr"])
        self._dev_lr.copy_(self._host_lr, non_blocking=True)

    def step(self, closure=None):
        capturing = self.device.type == "cuda" and torch.cuda.is_current_stream_capturing()
        if not capturing:
            self.upload_learning_rates()
        self._finish_lazy_zero()
        self._allreduce_sequence_parallel_grads()
        if self.post_reduce_hook is not None and not capturing:
            self.post_reduce_hook(self)
        self.step_count += 1
        if self._fused_dp:
            return self._fused_step()
        g = self._reduce_gradients()
        clip = self._clip_coefficient(lambda: self._grad_norm_sq(g))
        from ..ops.functional import _native
        if not _native(self.master) and float(clip) < 0:
            self.step_count -= 1             # non-finite gradients: skip the update (decided on the host here)
            return None
        s = self.shard_start
        out = self.flat_params[s:s + self.shard_size]
        for lo, hi, gi, rep in self.segments:
            grp = self.param_groups[gi]
            b1, b2 = grp["betas"]
            self._adamw(self.master[lo:hi], self.exp_avg[lo:hi], self.exp_avg_sq[lo:hi], g[lo:hi], out[lo:hi],
                        clip, grp["lr"], b1, b2, grp["eps"], grp["weight_decay"], self.step_count,
                        self._dev_lr[gi:gi + 1], self._dev_step)
        if self.shard:
            dist.all_gather_into_tensor(self.flat_params, out.contiguous(), group=self.dp_group) \
                if dist.get_backend(self.dp_group) != "gloo" else self._gloo_all_gather(out)
        if self.tp_size > 1 and self.device.type == "cuda":
            from . import symm
            symm.advance_step()
        return None

    def _clip_coefficient(self, norm_sq_fn) -> torch.Tensor:
        """Clip coefficient min(1, max_norm / norm) as a device scalar; -1 when the norm is not finite, which makes
        the AdamW kernels skip the step.  Also advances the device-side step counter (only for steps that are
        applied, so the bias correction stays exact) and the skipped-step counter."""
        if self.max_grad_norm is None:
            self._dev_step.add_(1)
            return torch.ones(1, dtype=torch.float32, device=self.device)
        norm = torch.sqrt(norm_sq_fn()).reshape(1)
        self.last_grad_norm = norm
        finite = torch.isfinite(norm)
        clip = torch.where(finite, torch.clamp(self.max_grad_norm / (norm + 1e-6), max=1.0), -torch.ones_like(norm))
        self._dev_step.add_(finite.to(torch.int32))
        self._dev_skipped.add_((~finite).to(torch.int32))
        return clip

    def skipped_steps(self) -> int:
        """Optimizer steps skipped so far because the gradient norm was not finite (reads the device counter)."""
        return int(self._dev_skipped.item())

    def _fused_step(self):
        """reduce-scatter(+1/dp, +norm partial) -> clip -> AdamW(+push of bf16 params to every rank) -> wait."""
        import ctypes
        from ..ops.cuda_ops import _P, _ll, _run, _st, status_tensor

        def arr(ptrs):
            a = (ctypes.c_void_p * 8)()
            for i, p in enumerate(ptrs):
                a[i] = p
            return a
        st = status_tensor(self.device)
        g = self.shard_grad
        total = self._norm_buf.zero_()
        fused_norm = self.tp_size == 1 and self.max_grad_norm is not None
        _run("ssm_zero1_reduce", arr(self._peer_grads), _P(g), _ll(self.shard_start), _ll(self.shard_size), self.dp_size,
             self.dp_rank, ctypes.c_float(1.0 / self.dp_size), _P(total if fused_norm else None), arr(self._peer_flags),
             0, 1, _P(self._zseq_base), _P(st), _st())
        def norm_sq():
            if fused_norm:
                dist.all_reduce(total, group=self.dp_group)
                return total
            return self._grad_norm_sq(g)
        clip = self._clip_coefficient(norm_sq)
        if self.max_grad_norm is None:
            dist.barrier(group=self.dp_group)     # peers must finish reading gradients before the next backward
        for k, (lo, hi, gi, rep) in enumerate(self.segments):
            grp = self.param_groups[gi]
            b1, b2 = grp["betas"]
            last = k == len(self.segments) - 1
            _run("ssm_zero1_adamw_push", _P(self.master[lo:hi]), _P(self.exp_avg[lo:hi]), _P(self.exp_avg_sq[lo:hi]),
                 _P(g[lo:hi]), arr(self._peer_params), _ll(self.shard_start + lo), _ll(hi - lo), self.dp_size,
                 self.dp_rank, _P(clip), ctypes.c_float(grp["lr"]), ctypes.c_float(b1), ctypes.c_float(b2),
                 ctypes.c_float(grp["eps"]), ctypes.c_float(grp["weight_decay"]), _P(self._dev_lr[gi:gi + 1]),
                 _P(self._dev_step), int(self.step_count), arr(self._peer_flags), 16, 2, _P(self._zseq_base),
                 _P(self._zcounter), int(last), _st())
        _run("ssm_zero1_wait", ctypes.c_void_p(self._peer_flags[self.dp_rank]), 16, self.dp_size, 2,
             _P(self._zseq_base), _P(st), _st())
        _run("ssm_advance_counter", _P(self._zseq_base), 4, ctypes.c_void_p(self._peer_flags[self.dp_rank]), 64, _st())
        if self.tp_size > 1:
            from . import symm
            symm.advance_step()
        return None

    def _gloo_all_gather(self, out: torch.Tensor) -> None:
        parts = [torch.empty_like(out) for _ in range(self.dp_size)]
        dist.all_gather(parts, out.contiguous(), group=self.dp_group)
        self.flat_params.copy_(torch.cat(parts))

    @staticmethod
    def _adamw(master, m, v, g, out, clip, lr, b1, b2, eps, wd, step, lr_dev=None, step_dev=None) -> None:
        from ..ops.functional import _native
        if _native(master):
            from ..ops import cuda_ops
            cuda_ops.adamw_step(master, m, v, g, out, clip, lr, b1, b2, eps, wd, step, lr_dev, step_dev)
            return
        bc1, bc2 = 1 - b1 ** step, 1 - b2 ** step
        chunk = 1 << 26        # bounded temporaries: the flat buffers hold billions of elements
        for lo in range(0, master.numel(), chunk):
            sl = slice(lo, lo + chunk)
            gf = g[sl].float() * clip
            mf, vf, w = m[sl].float(), v[sl].float(), master[sl].float()
            mf.mul_(b1).add_(gf, alpha=1 - b1)
            vf.mul_(b2).addcmul_(gf, gf, value=1 - b2)
            w.mul_(1 - lr * wd)
            w.addcdiv_(mf / bc1, (vf / bc2).sqrt_().add_(eps), value=-lr)
            m[sl].copy_(mf), v[sl].copy_(vf), master[sl].copy_(w)
            out[sl].copy_(w)

    # ------------------------------------------------------------------------------------
    def state_dict(self) -> Dict:
        """Per-DP-rank shard of the optimizer state (saved one file per DP rank under ZeRO-1)."""
        return {
            "step": self.step_count, "shard_start": self.shard_start, "shard_size": self.shard_size,
            "total": self.total, "dp_size": self.dp_size if self.shard else 1,
            "master": self.master.cpu(), "exp_avg": self.exp_avg.cpu(), "exp_avg_sq": self.exp_avg_sq.cpu(),
            "param_groups": [{k: v for k, v in g.items() if k != "params"} for g in self.param_groups],
        }

    def load_state_dict(self, sd: Dict) -> None:
        if sd["total"] != self.total or sd["shard_size"] != self.shard_size or sd["shard_start"] != self.shard_start:
            raise ValueError("optimizer checkpoint was written with a different parallel layout")
        self.step_count = int(sd["step"])
        self._dev_step.fill_(self.step_count)
        self.master.copy_(sd["master"])
        self.exp_avg.copy_(sd["exp_avg"])
        self.exp_avg_sq.copy_(sd["exp_avg_sq"])
        for g, saved in zip(self.param_groups, sd["param_groups"]):
            g.update(saved)

    def sync_master_from_params(self) -> None:
        """Re-seed the fp32 master shard from the model parameters (after loading a model-only
        checkpoint)."""
        s = self.shard_start
        self.master.copy_(self.flat_params[s:s + self.shard_size].to(self.master_dtype))
