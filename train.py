"""Pre-training entry point for Mamba-2 and Mamba-2-hybrid models on B200 GPUs.

Same flags and loop as the reference's train.py (flags :245-284, loop :178-232): gradient accumulation,
loss averaged over the data-parallel group, ZeRO-1 AdamW with fp32 master weights, cosine schedule with
warm-up, `LOG` lines from rank 0, periodic sharded checkpoints.  Launch one process per GPU:

    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 train.py --model Mamba7B --tp 8 --use_zero_1 \
        --sequence_parallel_enabled --dtype bfloat16 --data_dir DATA ...

Additions: --synthetic_data, --n_groups, --head_dim, --fused_comm, --resume (optimizer + scheduler +
step, where the reference restores the model only), --profile, --cuda_graph, --heartbeat_timeout.
Between steps the loop reads the kernels' status word (a bounded wait that ran out raises here and no checkpoint
is written from such a state), polls a heartbeat of the other ranks, and reports optimizer steps that were skipped
on the device because the gradient norm was not finite.
"""
from __future__ import annotations

import argparse
import os
import time

import numpy as np
import torch
import torch.distributed as dist
from transformers import get_cosine_schedule_with_warmup

from state_space_models_neuron_b200 import parallel as nxd
from state_space_models_neuron_b200.models import (Mamba2ForCausalLM, Mamba2HybridForCausalLM, get_config)
from state_space_models_neuron_b200.parallel import state as ps
from state_space_models_neuron_b200.utils.data import (DeviceLoader, SyntheticDataset, create_pretraining_dataset,
                                                       get_param_groups_by_weight_decay)
from state_space_models_neuron_b200.utils.logging import Logger, Throughput, get_mixed_precision_config


def build_model_and_optimizer(args):
    config = get_config(
        args.model, args.vocab_size, rmsnorm_within_groups=(not args.rmsnorm_across_groups),
        n_groups=args.n_groups if args.n_groups else args.tp,
        sequence_parallel_enabled=args.sequence_parallel_enabled, dtype=args.dtype, head_dim=args.head_dim,
        b200_recompute_mixer=args.recompute_mixer)
    cfg = nxd.parallel_config(
        tensor_parallel_size=args.tp,
        optimizer_config={"zero_one_enabled": args.use_zero_1, "grad_clipping": True, "max_grad_norm": 1.0},
        sequence_parallel=args.sequence_parallel_enabled,
        mixed_precision_config=get_mixed_precision_config(not args.no_optimizer_fp32),
        backend=args.backend, fused_comm=(args.fused_comm == "on"), init_seed=args.seed,
        device=args.device)

    def get_model():
        cls = Mamba2HybridForCausalLM if "Hybrid" in args.model else Mamba2ForCausalLM
        dev = args.device or ("cuda" if torch.cuda.is_available() else "cpu")
        model = cls(config, device=dev).to(dtype=args.dtype)
        model.train()
        return model

    model = nxd.initialize_parallel_model(cfg, get_model)
    if model.config.tie_word_embeddings:
        assert model.backbone.embeddings.weight is model.lm_head.weight
    groups = get_param_groups_by_weight_decay(model, args.weight_decay)
    opt_cls = nxd.AdamW_LowPrecision if args.no_optimizer_fp32 else nxd.AdamW_FP32OptimParams
    optimizer = nxd.initialize_parallel_optimizer(cfg, opt_cls, groups, lr=args.lr, betas=(args.beta1, args.beta2))
    optimizer.zero_grad()
    return config, cfg, model, optimizer


def run(args):
    torch.manual_seed(args.seed)
    np.random.seed(args.seed)
    config, cfg, model, optimizer = build_model_and_optimizer(args)
    device = next(model.parameters()).device
    dp_size, dp_rank = ps.get_data_parallel_size(), ps.get_data_parallel_rank()
    is_root = ps.is_master()
    scheduler = get_cosine_schedule_with_warmup(optimizer, num_warmup_steps=args.warmup_steps,
                                                num_training_steps=args.max_steps, last_epoch=-1)
    global_step = 0
    if args.checkpoint_load or args.resume:
        content = nxd.load_checkpoint(args.checkpoint_load_dir, tag=args.checkpoint_load_tag, model=model,
                                      optimizer=optimizer if args.resume else None,
                                      scheduler=scheduler if args.resume else None, strict=False)
        if args.resume and content:
            global_step = int(content.get("global_step", 0))
        else:
            optimizer.sync_master_from_params()
        if is_root:
            print(f"loaded checkpoint from {args.checkpoint_load_dir} (step {global_step})", flush=True)

    if is_root:
        print("TP groups:", ps.get_tensor_model_parallel_group(as_list=True))
        print("DP groups:", ps.get_data_parallel_group(as_list=True))
        print("Arguments: ", args)
        n_params = sum(p.numel() for p in set(model.parameters()))
        print(f"Model size: {n_params / 10**6:.1f}M parameters/GPU")
        print(f"Param dtype: {args.dtype}")
        if hasattr(model.backbone, "layer_types"):
            print("Layer allocation:", "".join(model.backbone.layer_types))
        logger = Logger(args, args.dtype, world_size=ps.get_world_size())
        throughput = Throughput(args.batch, dp_size, args.grad_accum_usteps, tp_size=args.tp, model=args.model,
                                seq_length=args.seq_len, logging_interval=args.logging_interval)

    synthetic = SyntheticDataset(args.vocab_size, args.seq_len, seed=args.seed) if args.synthetic_data else None
    loader, _ = create_pretraining_dataset(args.data_dir, args.batch, dp_size, dp_rank, args.seed, synthetic=synthetic)
    device_loader = DeviceLoader(loader, device)

    running_loss = torch.zeros(1, device=device)
    training_step = 0
    use_cuda = device.type == "cuda"
    ev_start = torch.cuda.Event(enable_timing=True) if use_cuda else None
    ev_end = torch.cuda.Event(enable_timing=True) if use_cuda else None
    if use_cuda:
        ev_start.record()

    def save(step):
        nxd.save_checkpoint(args.checkpoint_dir, f"{args.tag}_step_{step}", model, optimizer, scheduler,
                            {"global_step": step, "cli_args": {k: str(v) for k, v in vars(args).items()},
                             "config": model.config.to_dict()},
                            8, False, args.num_kept_checkpoint if args.num_kept_checkpoint > 0 else None)

    prof = None
    if args.profile:
        from state_space_models_neuron_b200.utils.profiling import StepProfiler
        prof = StepProfiler(args.output_dir)

    # ---- failure detection: host-side, between steps (no kernel or collective of this rank is in flight then)
    from state_space_models_neuron_b200.utils.failure import Heartbeat, RankFailure
    heartbeat = None
    if dist.is_initialized() and ps.get_world_size() > 1 and args.heartbeat_timeout > 0:
        store = getattr(dist.distributed_c10d, "_get_default_store", lambda: None)()
        if store is not None:
            heartbeat = Heartbeat(store, ps.get_rank(), ps.get_world_size(), period_s=min(1.0, args.heartbeat_timeout / 4),
                                  timeout_s=args.heartbeat_timeout).start()

    def health_check():
        """Raise if a bounded device-side wait ran out (a fused collective never completed) or a peer stopped
        answering; called at every logging interval and before every checkpoint, never with work in flight that
        this call would not wait for."""
        if use_cuda:
            from state_space_models_neuron_b200.ops import cuda_ops
            torch.cuda.synchronize()
            cuda_ops.check_status()
        if heartbeat is not None:
            heartbeat.check()

    if args.cuda_graph and not use_cuda:
        raise SystemExit("--cuda_graph needs a CUDA device")
    # With --cuda_graph the first optimizer steps run eagerly on their own batches (they are ordinary training
    # steps: allocator, workspaces and kernel attributes settle, data order and step count stay those of an eager
    # run), then the step is captured once and replayed.
    graph_after = global_step + 2 if args.cuda_graph else None
    graphed = None
    skipped_reported = 0

    def finish_optimizer_step(reduced, dev_timer=True):
        """Bookkeeping after an optimizer step: schedule, logging, health check, checkpoint."""
        nonlocal global_step, skipped_reported
        scheduler.step()
        global_step += 1
        if prof is not None:
            prof.step()
        logging_now = global_step % args.logging_interval == 0
        saving_now = args.checkpoint_freq > 0 and global_step % args.checkpoint_freq == 0
        if logging_now or saving_now:
            health_check()
        if is_root and logging_now:
            dev_time = None
            if use_cuda:
                ev_end.record()
                ev_end.synchronize()
                dev_time = ev_start.elapsed_time(ev_end) / 1e3 / args.logging_interval
                ev_start.record()
            step_time, tput, mfu = throughput.get_throughput()
            gn = optimizer.last_grad_norm
            logger.log(global_step, reduced.item(), optimizer.param_groups[0]["lr"], step_time, tput, mfu,
                       tokens_per_s=tput * args.seq_len, device_step_time=dev_time,
                       grad_norm=None if gn is None else float(gn))
            skipped = optimizer.skipped_steps() if hasattr(optimizer, "skipped_steps") else 0
            if skipped > skipped_reported:
                print(f"LOG WARNING {skipped - skipped_reported} optimizer step(s) skipped: non-finite gradient norm "
                      f"(total {skipped})", flush=True)
                skipped_reported = skipped
        if saving_now:
            save(global_step)

    done = global_step >= args.max_steps
    # a resumed run continues with the batch that the interrupted run would have seen next
    skip_batches = global_step * args.grad_accum_usteps if args.resume else 0
    def training_loop():
        nonlocal done, skip_batches, training_step, graphed
        while not done:
            for data in device_loader:
                if skip_batches > 0:
                    skip_batches -= 1
                    continue
                training_step += 1
                boundary = training_step % args.grad_accum_usteps == 0
                if graph_after is not None and global_step >= graph_after:
                    if graphed is None:
                        from state_space_models_neuron_b200.parallel.graph import GraphedAccumulationStep, GraphedTrainStep
                        if args.grad_accum_usteps == 1:
                            graphed = GraphedTrainStep(model, optimizer, data, warmup=0)
                        else:       # one graph per kind of micro-step plus one for the update
                            graphed = GraphedAccumulationStep(model, optimizer, data, args.grad_accum_usteps, warmup=0)
                    if args.grad_accum_usteps == 1:
                        running_loss.add_(graphed(data))
                    else:
                        running_loss.add_(graphed.micro_step(data))
                else:
                    out = model(input_ids=data["input_ids"], labels=data["labels"], return_logits=False)
                    loss = out.loss / args.grad_accum_usteps
                    loss.backward()
                    running_loss.add_(loss.detach())
                    if boundary:
                        optimizer.step()
                        optimizer.zero_grad()
                if boundary:
                    reduced = running_loss / dp_size
                    if dp_size > 1:
                        dist.all_reduce(reduced, group=ps.get_data_parallel_group())
                    reduced = reduced.clone()
                    running_loss.zero_()
                    finish_optimizer_step(reduced)
                if global_step >= args.max_steps:
                    done = True
                    break
        if args.save_last_step and (args.checkpoint_freq <= 0 or global_step % args.checkpoint_freq):
            health_check()
            save(global_step)
        health_check()

    try:
        if args.cuda_graph:
            # graph capture cannot involve the legacy default stream, and autograd remembers the stream on which a
            # parameter's gradient was first accumulated: with --cuda_graph the whole loop runs on a side stream
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                training_loop()
            torch.cuda.current_stream().wait_stream(side)
        else:
            training_loop()
    finally:
        if heartbeat is not None:
            heartbeat.stop()
    if is_root:
        logger.close()
    ps.barrier()
    return global_step


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser()
    p.add_argument("--seed", type=int, default=100)
    p.add_argument("--dtype", default="bfloat16", choices=["float32", "bfloat16"])
    p.add_argument("--batch", type=int, default=1)
    p.add_argument("--vocab_size", type=int, default=50272)
    p.add_argument("--model", default="Mamba130M")
    p.add_argument("--backend", default=None, choices=["nccl", "gloo", "xla", None],
                   help="process-group backend; default nccl on GPUs, gloo on CPU ('xla' is accepted and mapped to the default)")
    p.add_argument("--tp", type=int, default=1)
    p.add_argument("--no_optimizer_fp32", action="store_true")
    p.add_argument("--use_zero_1", action="store_true")
    p.add_argument("--sequence_parallel_enabled", action="store_true")
    p.add_argument("--lr", type=float, default=4e-4)
    p.add_argument("--weight_decay", type=float, default=0.01)
    p.add_argument("--beta1", type=float, default=0.9)
    p.add_argument("--beta2", type=float, default=0.999)
    p.add_argument("--data_dir", type=str, default=None)
    p.add_argument("--warmup_steps", type=int, default=2000)
    p.add_argument("--seq_len", type=int, default=2048)
    p.add_argument("--max_steps", type=int, default=10)
    p.add_argument("--grad_accum_usteps", type=int, default=1)
    p.add_argument("--rmsnorm_across_groups", action="store_true")
    p.add_argument("--debug", "-d", action="store_true")
    p.add_argument("--logging_interval", type=int, default=1)
    p.add_argument("--checkpoint_load", action="store_true")
    p.add_argument("--checkpoint_load_dir", type=str, default=None)
    p.add_argument("--checkpoint_load_tag", type=str, default=None)
    p.add_argument("--checkpoint_freq", type=int, default=-1)
    p.add_argument("--checkpoint_dir", type=str, default="checkpoints")
    p.add_argument("--num_kept_checkpoint", type=int, default=-1)
    p.add_argument("--save_last_step", action="store_true")
    p.add_argument("--output_dir", type=str, default="tensorboard_logs")
    p.add_argument("--tag", type=str, default="exp")
    # additions
    p.add_argument("--synthetic_data", action="store_true", help="uniform random token ids instead of --data_dir")
    p.add_argument("--n_groups", type=int, default=0, help="SSM groups; 0 = TP degree like the reference")
    p.add_argument("--head_dim", type=int, default=None, help="override the preset's Mamba head dim")
    p.add_argument("--fused_comm", default="on", choices=["on", "off"],
                   help="off = library collectives + separate GEMMs (the measured baseline)")
    p.add_argument("--recompute_mixer", action="store_true", help="rebuild conv/scan intermediates in backward")
    p.add_argument("--resume", action="store_true", help="also restore optimizer, scheduler and step")
    p.add_argument("--profile", action="store_true")
    p.add_argument("--cuda_graph", action="store_true",
                   help="capture the whole optimizer step (fwd+bwd+collectives+AdamW) in one CUDA graph and replay it; "
                        "with --grad_accum_usteps > 1: one graph per kind of micro-step plus one for the update; the "
                        "first two optimizer steps run eagerly")
    p.add_argument("--device", default=None)
    p.add_argument("--heartbeat_timeout", type=float, default=60.0,
                   help="seconds without a heartbeat after which a peer rank counts as dead (checked between steps at "
                        "every logging interval and before checkpoints); 0 turns the heartbeat off")
    return p


def main(argv=None):
    args = build_parser().parse_args(argv)
    args.dtype = torch.float32 if args.dtype == "float32" else torch.bfloat16
    if args.backend == "xla":
        args.backend = None
    if args.debug:
        os.environ["SSM_B200_DEBUG"] = "1"
        os.environ.setdefault("NCCL_DEBUG", "INFO")
    if args.data_dir is None and not args.synthetic_data:
        raise SystemExit("pass --data_dir or --synthetic_data")
    ps.initialize_model_parallel(args.tp, backend=args.backend)
    try:
        run(args)
    finally:
        if dist.is_initialized():
            dist.barrier()
            if not args.cuda_graph:      # communicators referenced by a live graph are left to process exit
                dist.destroy_process_group()


if __name__ == "__main__":
    main()
