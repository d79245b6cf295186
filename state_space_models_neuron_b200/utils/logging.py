"""Training log line, TensorBoard scalars, moving-window throughput and MFU.

Output format and the MFU formula follow the reference (utils.py:36-161): a stdout line starting
with `LOG`, TensorBoard scalars `step loss / learning rate / step time / throughput / MFU`, a
10-step moving window of seq/s, and
    MFU = 3 * layers * batch * (12 L D^2 + 8 L D + 2 L N D) / 1e12 / (peak_TFLOPs * tp) / step_time.
The peak defaults to the bf16 GEMM throughput measured on this machine's B200s when a
`MEASURED_PEAKS.json` sits next to the working directory, else 1590 TFLOP/s (the reference
hard-codes 95 for a Trainium core).  Additions: tokens/s, device-timed step time, JSON-lines
metrics file.
"""
from __future__ import annotations

import collections
import json
import math
import os
import socket
import sys
import time
from dataclasses import astuple
from typing import Optional

import torch

from ..models.predefined_configs import CONFIGS_KWARGS

B200_FALLBACK_TFLOPS = 1590.0


def measured_peak_tflops(default: float = B200_FALLBACK_TFLOPS) -> float:
    for base in (os.getcwd(), os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))):
        path = os.path.join(base, "MEASURED_PEAKS.json")
        if os.path.exists(path):
            try:
                with open(path) as f:
                    return float(json.load(f).get("bf16_tflops_sustained", default))
            except (OSError, ValueError):
                pass
    return default


def dummy_inputs(batch: int, seq_len: int, vocab_size: int, device="cpu", seed: int = 0):
    """Synthetic batch: uniform random ids, labels = ids (the model shifts them)."""
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, vocab_size, (batch, seq_len), generator=g)
    return {"input_ids": ids.to(device), "labels": ids.clone().to(device)}


def get_mixed_precision_config(use_master_weights: bool = True) -> dict:
    """fp32 master weights + fp32 gradient accumulation (utils.py:26-33 of the reference, which
    effectively always enables both)."""
    on = bool(use_master_weights)
    return {"use_master_weights": on, "use_fp32_grad_acc": on, "use_master_weights_in_ckpt": False}


class Logger:
    def __init__(self, args, model_dtype, world_size: Optional[int] = None, tensorboard: bool = True):
        if world_size is None:
            world_size = torch.distributed.get_world_size() if torch.distributed.is_initialized() else 1
        run = (f"b200_tblogs_{time.strftime('%m%d%y_%H%M')}_{args.model}_{model_dtype}_w{world_size}"
               f"_lr{args.lr}_bs{args.batch}_acc{args.grad_accum_usteps}_max{args.max_steps}_{self.get_instance_type()}")
        self.run_dir = os.path.join(args.output_dir, run)
        os.makedirs(self.run_dir, exist_ok=True)
        self.tb = None
        if tensorboard:
            try:
                from torch.utils.tensorboard import SummaryWriter
                self.tb = SummaryWriter(self.run_dir)
                self.tb.add_text("command", " ".join(sys.argv), 0)
            except Exception:  # tensorboard is optional
                self.tb = None
        self.jsonl = open(os.path.join(self.run_dir, "metrics.jsonl"), "a")

    @staticmethod
    def get_instance_type() -> str:
        name = torch.cuda.get_device_name(0).replace(" ", "-") if torch.cuda.is_available() else "cpu"
        return f"{name}_{os.environ.get('HOSTNAME', socket.gethostname())}"

    def log(self, step, step_loss, learning_rate, step_time=None, throughput=None, MFU=None,
            tokens_per_s=None, device_step_time=None, grad_norm=None):
        msg = (f"LOG {time.asctime()} - step: {step}, step_loss : {step_loss:.8f} "
               f"learning_rate : {learning_rate:.2e} ")
        if step_time:
            msg += f"step time : {step_time:.4f} s  "
        if throughput:
            msg += f"throughput : {throughput:.4f} seq/s  "
        if MFU:
            msg += f"MFU : {MFU:.4f}  "
        if tokens_per_s:
            msg += f"tokens/s : {tokens_per_s:.1f}  "
        if device_step_time:
            msg += f"device step time : {device_step_time:.4f} s  "
        if grad_norm is not None:
            msg += f"grad norm : {grad_norm:.4f}"
        print(msg, flush=True)
        rec = {"step": step, "step loss": step_loss, "learning rate": learning_rate, "step time": step_time,
               "throughput": throughput, "MFU": MFU, "tokens/s": tokens_per_s,
               "device step time": device_step_time, "grad norm": grad_norm}
        self.jsonl.write(json.dumps(rec) + "\n")
        self.jsonl.flush()
        if self.tb is not None:
            for k, v in rec.items():
                if k != "step" and v is not None:
                    self.tb.add_scalar(k, v, step)

    def close(self):
        self.jsonl.close()
        if self.tb is not None:
            self.tb.close()


class Throughput:
    def __init__(self, batch_size, world_size, grad_accum_usteps, tp_size=1, model=None, seq_length=2048,
                 chip_flops: Optional[float] = None, moving_avg_window_size=10, logging_interval=1,
                 MFU=True, MFU_backpropagation=True):
        """`world_size` is the data-parallel size (train.py:97-105 of the reference passes it so)."""
        self.seqs_per_iteration = batch_size * world_size * grad_accum_usteps * logging_interval
        self.window = collections.deque(maxlen=max(1, math.ceil(moving_avg_window_size / logging_interval)))
        self.start_time = time.time()
        self.batch_size = batch_size * grad_accum_usteps
        self.seq_length = seq_length
        self.tp_size = tp_size or 1
        self.chip_flops = chip_flops if chip_flops is not None else measured_peak_tflops()
        self.MFU = MFU and model in CONFIGS_KWARGS
        self.MFU_backpropagation = MFU_backpropagation
        self.MFU_factor = self.set_mamba_MFU_factor(model) if self.MFU else None

    def set_mamba_MFU_factor(self, model):
        D, layers, N = astuple(CONFIGS_KWARGS[model])
        L = self.seq_length
        per_layer = 12 * L * D ** 2 + 8 * L * D + 2 * L * N * D
        factor = per_layer * layers * self.batch_size / 1e12 / (self.chip_flops * self.tp_size)
        return factor * 3 if self.MFU_backpropagation else factor

    def get_throughput(self):
        now = time.time()
        self.window.append(now - self.start_time)
        self.start_time = now
        avg = sum(self.window) / len(self.window)
        return avg, self.seqs_per_iteration / avg, (self.MFU_factor / avg if self.MFU else None)


class TrainingMetrics:
    """Small JSON store of run metrics keyed by name (nxd_training_utils.py:254-326 of the reference
    carries an equivalent, unused there): `update`, `store_parameters`, read back with `load`."""

    def __init__(self, json_file: str):
        self.json_file = json_file
        self.data = {"metrics": {}, "parameters": {}}
        if os.path.exists(json_file):
            with open(json_file) as f:
                self.data = json.load(f)

    def update(self, **metrics):
        self.data["metrics"].update(metrics)
        self._write()

    def store_parameters(self, **params):
        self.data["parameters"].update({k: str(v) for k, v in params.items()})
        self._write()

    def _write(self):
        tmp = self.json_file + ".tmp"
        with open(tmp, "w") as f:
            json.dump(self.data, f, indent=1)
        os.replace(tmp, self.json_file)
