"""Whole-step CUDA graph: forward, backward, gradient reduction, clipping, AdamW and the fused TP collectives
captured once and replayed, which removes the host from the critical path (thousands of launches per step).

What makes the step capturable:
  * every native kernel is launched on the current stream with arguments that do not change between steps;
  * quantities that do change live on the device: the fused collectives' sequence base (advanced by a kernel
    inside the graph), the optimizer step counter and the learning rates (uploaded before each replay);
  * lazy gradient zeroing follows the same store/accumulate pattern every step;
  * no host synchronisation inside the step (the status word is read afterwards).
The reference reaches the same end with XLA's lazy tensor graphs cut at `xm.mark_step()` (train.py:161,191,226).
"""
from __future__ import annotations

from typing import Callable, Dict, Optional

import torch

from .cross_entropy import parallel_argmax


def _require_side_stream_without_warmup(warmup: int) -> None:
    """Capture needs every stream that autograd associates with the parameters to be able to join the capture; the
    legacy default stream cannot.  The warm-up steps of the graph classes run on a side stream for that reason; a
    caller that passes warmup=0 because it has already run real steps must have run them on a side stream too."""
    if warmup == 0 and torch.cuda.current_stream() == torch.cuda.default_stream():
        raise RuntimeError("warmup=0 needs the preceding eager steps (and this call) to run under "
                           "torch.cuda.stream(side_stream), not on the default stream")


class GraphedTrainStep:
    """`warmup` eager optimizer steps on the example batch (on a side stream), then capture.  With warmup=0 the caller
    has already taken real steps itself, on a non-default stream (see train.py)."""

    def __init__(self, model, optimizer, example_batch: Dict[str, torch.Tensor], loss_fn: Optional[Callable] = None,
                 warmup: int = 2, grad_accum_usteps: int = 1):
        _require_side_stream_without_warmup(warmup)
        self.model, self.optimizer = model, optimizer
        self.accum = grad_accum_usteps
        self.static = {k: v.clone() for k, v in example_batch.items()}
        self.loss_fn = loss_fn or (lambda m, b: m(input_ids=b["input_ids"], labels=b["labels"], return_logits=False).loss)
        self.graph = None
        self.static_loss = None
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(warmup):
                self._eager_step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
        self.optimizer.upload_learning_rates()
        from ..ops import cuda_ops
        before = cuda_ops.launch_count()
        from . import symm
        symm.start_recording()
        self.graph = torch.cuda.CUDAGraph()
        # after a caller's own eager steps (warmup=0) the capture runs on the stream those steps ran on: autograd ties
        # every parameter's gradient accumulation to that stream, and a capture on another stream would have to wait
        # on work that is not part of the capture
        cap = dict(stream=torch.cuda.current_stream()) if warmup == 0 else {}
        with torch.cuda.graph(self.graph, **cap):
            self.static_loss = self._eager_step()
        rec = symm.stop_recording()
        symm.check_replay_safe(rec + rec)          # double-buffer parities must survive back-to-back replays
        self.native_launches_per_step = cuda_ops.launch_count() - before   # native kernel nodes in the graph
        self.replays = 0
        self.optimizer.step_count -= 1     # capturing recorded a step without executing it
        self.eager_steps = warmup          # optimizer steps really taken before the first replay

    def _eager_step(self):
        loss = self.loss_fn(self.model, self.static)
        (loss / self.accum).backward()
        self.optimizer.step()
        self.optimizer.zero_grad()
        return loss.detach()

    def __call__(self, batch: Dict[str, torch.Tensor]) -> torch.Tensor:
        """Copies the batch into the captured input buffers (host or device source), replays the step and
        returns the loss tensor (device, overwritten by the next call)."""
        for k, v in batch.items():
            self.static[k].copy_(v, non_blocking=True)
        self.optimizer.upload_learning_rates()
        self.graph.replay()
        self.optimizer.step_count += 1
        self.replays += 1
        return self.static_loss


class GraphedAccumulationStep:
    """Gradient accumulation with CUDA graphs: three graphs instead of one.

        first    forward + backward of a micro-step right after `zero_grad()` (wgrad GEMMs store)
        next     forward + backward of every further micro-step (wgrad GEMMs accumulate)
        update   gradient reduction, clipping, AdamW, `zero_grad()`

    `micro_step(batch)` replays `first` or `next` and returns the micro-step's loss divided by the number of
    micro-steps (device tensor, overwritten by the next call); after `grad_accum_usteps` micro-steps it replays
    `update`.  The reference accumulates the same way with eager XLA steps (train.py:178-232)."""

    def __init__(self, model, optimizer, example_batch: Dict[str, torch.Tensor], grad_accum_usteps: int,
                 loss_fn: Optional[Callable] = None, warmup: int = 1):
        if grad_accum_usteps < 2:
            raise ValueError("use GraphedTrainStep for grad_accum_usteps == 1")
        _require_side_stream_without_warmup(warmup)
        self.model, self.optimizer, self.accum = model, optimizer, grad_accum_usteps
        self.static = {k: v.clone() for k, v in example_batch.items()}
        self.loss_fn = loss_fn or (lambda m, b: m(input_ids=b["input_ids"], labels=b["labels"], return_logits=False).loss)
        self.micro_index = 0
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(warmup):              # real optimizer steps on the example batch (allocator, workspaces)
                for _ in range(self.accum):
                    self._micro()
                self._update()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
        self.optimizer.upload_learning_rates()
        pool = torch.cuda.graph_pool_handle()
        self.g_first, self.g_next, self.g_update = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
        # capture in the order of a real step so that the host-side store/accumulate flags seen by each graph are
        # the ones it will meet at replay: first (gradients stale) -> next (accumulating) -> update
        from . import symm
        kinds = []
        cap = dict(stream=torch.cuda.current_stream()) if warmup == 0 else {}      # see GraphedTrainStep
        for graph, body, name in ((self.g_first, self._micro, "loss_first"), (self.g_next, self._micro, "loss_next"),
                                  (self.g_update, self._update, None)):
            symm.start_recording()
            with torch.cuda.graph(graph, pool=pool, **cap):
                out = body()
            kinds.append(symm.stop_recording())
            if name:
                setattr(self, name, out)
        # replay order: first, next x (accum - 1), update, first, ...: the buffer parities fixed at capture must be
        # safe for every succession that occurs, in particular `next` replayed back to back
        first, nxt, upd = kinds
        symm.check_replay_safe(first + nxt + nxt + upd + first + nxt + upd + first)
        self.optimizer.step_count -= 1           # capturing recorded an optimizer step without executing it
        self.eager_steps = warmup

    def _micro(self):
        loss = self.loss_fn(self.model, self.static) / self.accum
        loss.backward()
        # every replay of a micro-step graph must publish fresh sequence numbers for its fused collectives: the
        # graph ends with a bump of the device-side base by the number of calls it made
        from . import symm
        symm.advance_step(compact=True)
        return loss.detach()

    def _update(self):
        self.optimizer.step()
        self.optimizer.zero_grad()

    def micro_step(self, batch: Dict[str, torch.Tensor]) -> torch.Tensor:
        for k, v in batch.items():
            self.static[k].copy_(v, non_blocking=True)
        first = self.micro_index == 0
        (self.g_first if first else self.g_next).replay()
        self.micro_index += 1
        if self.micro_index == self.accum:
            self.optimizer.upload_learning_rates()
            self.g_update.replay()
            self.optimizer.step_count += 1
            self.micro_index = 0
        return self.loss_first if first else self.loss_next

    @property
    def at_step_boundary(self) -> bool:
        """True right after the micro-step that completed an optimizer step."""
        return self.micro_index == 0


class GraphedDecodeStep:
    """One autoregressive decode step (all layers, LM head, greedy argmax) captured as a CUDA graph.

    The conv/SSM caches are updated in place by the kernels, so replaying the graph advances them; the token
    buffer is static.  Warm-up and capture run on a copy of the cache contents which is restored afterwards, so
    constructing the object does not disturb the decoding state."""

    def __init__(self, model, cache, batch_size: int, warmup: int = 2):
        self.model, self.cache = model, cache
        dev = next(model.parameters()).device
        self.token = torch.zeros(batch_size, 1, dtype=torch.long, device=dev)
        saved = {k: (cache.conv_states[k].clone(), cache.ssm_states[k].clone()) for k in cache.conv_states}
        offset = cache.seqlen_offset
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(warmup):
                model.step(self.token, cache)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.no_grad(), torch.cuda.graph(self.graph):
            self.logits = model.step(self.token, cache)
            self.next_token = parallel_argmax(self.logits[:, -1]).unsqueeze(-1)
        for k, (c, s) in saved.items():
            cache.conv_states[k].copy_(c)
            cache.ssm_states[k].copy_(s)
        cache.seqlen_offset = offset

    @torch.no_grad()
    def __call__(self, token: torch.Tensor) -> torch.Tensor:
        """token [B, 1] -> next greedy token [B, 1] (device tensor, overwritten by the next call); the logits of
        this step are in `self.logits`."""
        self.token.copy_(token, non_blocking=True)
        self.graph.replay()
        self.cache.seqlen_offset += 1
        return self.next_token
