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


class GraphedTrainStep:
    def __init__(self, model, optimizer, example_batch: Dict[str, torch.Tensor], loss_fn: Optional[Callable] = None,
                 warmup: int = 2, grad_accum_usteps: int = 1):
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
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.static_loss = self._eager_step()
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
