"""Headline benchmark: training tokens/s of Mamba2-7B (d_model 4096, 64 layers, head_dim 64, d_state 128,
n_groups 8, vocab 50288) in bf16 with TP = N + sequence parallel + ZeRO-1, seq 2048, batch 1 per DP rank,
synthetic uniform-random tokens, random-init weights.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        bench.py --gpus 8 --steps 5 --warmup 3

Rank 0 prints one JSON line.  `value` is device-timed (CUDA events around exactly `steps` optimizer steps,
barrier + synchronize on both sides, max over ranks) with inputs already on the device; `e2e` times the same
steps through the public API with the per-step host->device copy of the batch from pinned memory and the
device->host read of the loss inside the timed region.  `--impl reference` reports why the reference cannot
run on this hardware.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

MODEL = dict(name="Mamba2-7B", hidden_size=4096, num_hidden_layers=64, head_dim=64, num_heads=128, state_size=128,
             n_groups=8, vocab_size=50288, conv_kernel=4)
SEQ_LEN = 2048
BATCH_PER_DP = 1
SMALL = dict(name="Mamba2-tiny", hidden_size=512, num_hidden_layers=4, head_dim=64, num_heads=16, state_size=128,
             n_groups=8, vocab_size=50288, conv_kernel=4)


def measured_baselines(n_gpus: int):
    """(tokens/s of the PyTorch + cuBLAS + NCCL arm, tokens/s of this repo's kernels with NCCL collectives) at this
    GPU count as recorded in baseline/measured.json by earlier runs of `--impl baseline` and `--fused_comm off` on
    the same pool; None where no measurement exists."""
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "measured.json")
    try:
        with open(path) as f:
            rec = json.load(f)
    except (OSError, ValueError):
        return None, None
    key = str(n_gpus)
    return rec.get("pytorch_cublas_nccl", {}).get(key), rec.get("own_kernels_nccl", {}).get(key)


def reference_arm():
    print(json.dumps({"impl": "reference", "unavailable":
                      "reference is Trainium-only (imports neuronx_distributed/torch_xla/neuronxcc NKI, asserts an XLA "
                      "device) and has no setup.py/pyproject.toml: pip install of the reference tree fails, nothing to run on B200"}))


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index: int, period: float = 0.2):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop_evt = threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        nv = self.nv
        names = {nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
                 nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
                 nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
                 nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap"}
        while not self._stop_evt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop_evt.wait(self.period)

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=2)
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "baseline"])
    ap.add_argument("--small", action="store_true", help="tiny model for profiling captures (not a benchmark value)")
    ap.add_argument("--layers", type=int, default=None, help="override layer count (profiling only)")
    ap.add_argument("--fused_comm", default="auto", choices=["auto", "on", "off"],
                    help="auto: time the whole step with each of the two GEMM + collective kernels fused or as NCCL + "
                         "GEMM (four combinations, before the warm-up) and run the fastest; on: both fused; off: NCCL")
    ap.add_argument("--no_e2e", action="store_true")
    ap.add_argument("--graph", default="on", choices=["on", "off"],
                    help="replay the whole training step as one CUDA graph (off = eager launches)")
    ap.add_argument("--shard_of", type=int, default=1,
                    help="analysis only: run ONE rank's share of a TP=k model on one GPU without communication "
                         "(heads, groups and vocabulary divided by k) to see the per-rank compute of TP=k; not a "
                         "benchmark value")
    ap.add_argument("--profile_mode", action="store_true",
                    help="allow fewer than 3 warm-up steps (for profiler captures; not a benchmark value)")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm()
        return
    if args.warmup < 3 and not (args.small or args.profile_mode):
        args.warmup = 3

    import torch
    import torch.distributed as dist
    from state_space_models_neuron_b200 import parallel as nxd
    from state_space_models_neuron_b200.models import Mamba2Config, Mamba2ForCausalLM
    from state_space_models_neuron_b200.ops import cuda_ops
    from state_space_models_neuron_b200.parallel import state as ps
    from state_space_models_neuron_b200.utils.data import get_param_groups_by_weight_decay

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    tp = args.gpus
    ps.initialize_model_parallel(tp, backend="nccl")
    rank = ps.get_rank()
    m = dict(SMALL if args.small else MODEL)
    if args.layers:
        m["num_hidden_layers"] = args.layers
    if args.shard_of > 1:
        k = args.shard_of
        m.update(num_heads=m["num_heads"] // k, n_groups=max(1, m["n_groups"] // k), vocab_size=m["vocab_size"] // k,
                 expand=2.0 / k, name=m["name"] + f" (1/{k} shard, analysis)")
    fused = args.fused_comm in ("on", "auto") and args.impl == "ours"
    if args.impl == "baseline":
        from baseline import nccl_cublas
        # one GPU holds all 126 GB of weights, gradients and optimizer state of the 7B model: the saved scan
        # intermediates of 64 layers do not fit next to them, so only that case recomputes the mixer in backward
        nccl_cublas.enable(checkpoint_mixer=(args.gpus == 1 and not args.small))
    cfg = nxd.parallel_config(
        tensor_parallel_size=tp, optimizer_config={"zero_one_enabled": True, "grad_clipping": True, "max_grad_norm": 1.0},
        sequence_parallel=tp > 1, fused_comm=fused, init_seed=0)
    mc = Mamba2Config(num_heads=m["num_heads"], head_dim=m["head_dim"], vocab_size=m["vocab_size"],
                      hidden_size=m["hidden_size"], state_size=m["state_size"], num_hidden_layers=m["num_hidden_layers"],
                      n_groups=m["n_groups"], expand=m.get("expand", 2), conv_kernel=4, tie_word_embeddings=True, rmsnorm_within_groups=False,
                      sequence_parallel_enabled=tp > 1, dtype=torch.bfloat16, initializer_range=0.02, use_cache=False)
    model = nxd.initialize_parallel_model(cfg, lambda: Mamba2ForCausalLM(mc, device="cuda").to(torch.bfloat16))
    model.train()
    groups = get_param_groups_by_weight_decay(model, 0.1)
    opt = nxd.initialize_parallel_optimizer(cfg, nxd.AdamW_FP32OptimParams, groups, lr=3e-4, betas=(0.9, 0.95))
    opt.zero_grad()

    dp = ps.get_data_parallel_size()
    B, L, V = BATCH_PER_DP, SEQ_LEN, m["vocab_size"]
    g = torch.Generator().manual_seed(1234 + ps.get_data_parallel_rank())
    n_batches = args.warmup + args.steps
    host = [torch.randint(0, V, (B, L), generator=g).pin_memory() for _ in range(n_batches)]
    dev = [h.cuda(non_blocking=True) for h in host]

    def eager_step(ids):
        loss = model(input_ids=ids, labels=ids, return_logits=False).loss
        loss.backward()
        opt.step()
        opt.zero_grad()
        return loss

    fused_fallback = None
    if fused and tp > 1:
        # pre-flight of the fused collective kernels: one eager step; if any rank reports a failed wait, every rank
        # switches to the NCCL collectives (same kernels otherwise) and the JSON line says so
        bad = 0
        try:
            eager_step(dev[0])
            torch.cuda.synchronize()
            cuda_ops.check_status()
        except Exception as e:
            print(f"[rank {rank}] fused collectives failed in the pre-flight step: {e!r}", file=sys.stderr, flush=True)
            bad = 1
        flag = torch.tensor([bad], device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MAX)
        if int(flag.item()):
            from state_space_models_neuron_b200.parallel import fused as fused_switch
            fused_switch.set_enabled(False)
            fused = False
            fused_fallback = "pre-flight step of the fused collective kernels failed on at least one rank; NCCL collectives used"
            torch.cuda.synchronize()
            try:
                cuda_ops.check_status()
            except Exception:
                pass
            opt.zero_grad()
    step, gstep, graph_note = eager_step, None, "off"
    fused_choice = None

    def build_graphed():
        from state_space_models_neuron_b200.parallel.graph import GraphedTrainStep
        try:
            gs = GraphedTrainStep(model, opt, {"input_ids": dev[0], "labels": dev[0]})
        except Exception as e:                       # fall back to eager launches, on every rank or on none
            print(f"[rank {rank}] CUDA graph capture failed, running eager: {e!r}", file=sys.stderr, flush=True)
            gs = None
        ok = torch.tensor([1 if gs is not None else 0], device="cuda")
        if world > 1:
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        return gs if int(ok.item()) else None

    if args.graph == "on" and args.impl == "ours":
        if fused and tp > 1 and args.fused_comm == "auto":
            # the whole graphed step is timed under each on/off combination of the two GEMM + collective kernels
            # (max over ranks, so every rank decides alike); the fastest runs the warm-up and the timed steps
            from state_space_models_neuron_b200.parallel import fused_tune
            graphs = {}

            def build_combo():
                gs = build_graphed()
                if gs is None:
                    return None
                run = lambda: gs({"input_ids": dev[0], "labels": dev[0]})
                graphs[id(run)] = gs
                return run

            def healthy():
                bad = 0
                try:
                    torch.cuda.synchronize()
                    cuda_ops.check_status()
                except RuntimeError as e:
                    print(f"[rank {rank}] fused collectives failed while the step was being tuned: {e!r}", file=sys.stderr, flush=True)
                    bad = 1
                flag = torch.tensor([bad], device="cuda")
                dist.all_reduce(flag, op=dist.ReduceOp.MAX)
                return int(flag.item()) == 0

            try:
                rep = fused_tune.pick_fastest(build_combo, torch.device("cuda", local), reps=3,
                                              release=lambda run: graphs.pop(id(run), None), healthy=healthy)
                gstep = graphs.pop(id(rep["step"])) if rep["step"] is not None else None
                graphs.clear()
                torch.cuda.empty_cache()
                fused_choice = {"chosen": rep["chosen"], "ms_per_step": rep["ms"]}
            except fused_tune.CandidateFailed as e:
                # same decision on every rank (the health check is reduced over the ranks): all collectives through NCCL
                from state_space_models_neuron_b200.parallel import fused as fused_switch
                graphs.clear()
                torch.cuda.empty_cache()
                fused_switch.set_enabled(False)
                fused = False
                fused_fallback = f"{e}; NCCL collectives used"
                opt.zero_grad()
                gstep = build_graphed()
        else:
            gstep = build_graphed()
        if gstep is not None:
            graph_note = "whole step (fwd+bwd+optimizer+collectives) captured once, replayed per step"

            def step(ids):
                return gstep({"input_ids": ids, "labels": ids})

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        loss = step(dev[i])
    barrier()
    cuda_ops.check_status()
    sampler = ClockSampler(local)
    sampler.start()
    launches0 = cuda_ops.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    h0 = time.perf_counter()
    for i in range(args.steps):
        loss = step(dev[args.warmup + i])
    host_issue_ms = (time.perf_counter() - h0) * 1e3 / args.steps     # host time to enqueue one step (no sync)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    launches = cuda_ops.launch_count() - launches0
    if gstep is not None:
        launches = gstep.native_launches_per_step * args.steps
    clocks = sampler.stop()
    last_loss = float(loss.detach())
    cuda_ops.check_status()
    t = torch.tensor([ms], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = t.item()
    tokens = B * dp * L * args.steps
    value = tokens / (ms / 1e3)

    e2e = None
    if not args.no_e2e:
        barrier()
        t0 = time.perf_counter()
        h2d = d2h = 0
        for i in range(args.steps):
            ids = host[args.warmup + i].to("cuda", non_blocking=True)    # pinned host -> device, every step
            h2d = ids.numel() * ids.element_size()
            lval = step(ids).item()                                      # device -> host read of the loss
            d2h = 4
        torch.cuda.synchronize()
        dt_e2e = time.perf_counter() - t0
        t2 = torch.tensor([dt_e2e], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t2, op=dist.ReduceOp.MAX)
        e2e = {"value": tokens / t2.item(), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "ms_per_step": t2.item() * 1e3 / args.steps, "last_loss": lval}

    if rank == 0:
        base_pt, base_nccl = measured_baselines(args.gpus)
        is_headline = args.impl == "ours" and not args.small and not args.layers and args.shard_of == 1
        out = {
            "metric": "train tokens/s (device-timed, max over ranks) Mamba2-7B TP=N seq2048",
            "value": value, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": (value / base_pt) if (base_pt and is_headline) else None,
            "dtype": "bf16", "data": "synthetic uniform-random token ids, random-init weights",
            "impl": args.impl if args.impl != "ours" else "ours",
            "config": {"model": m["name"], "layers": m["num_hidden_layers"], "global_batch": B * dp, "seq_len": L,
                       "parallelism": f"tp{tp}" + ("+sp" if tp > 1 else "") + "+zero1(dp%d)" % dp,
                       "fused_comm": fused, "cuda_graph": graph_note,
                       "l2": "no explicit flush: each step streams >100 GB of weights, gradients and optimizer state, "
                             "far above the 126 MB L2"},
            "clocks": clocks, "gpu_launches": launches, "loss": last_loss, "host_issue_ms_per_step": host_issue_ms,
        }
        if tp > 1:
            from state_space_models_neuron_b200.parallel import fused_ops
            out["fused_kernel_launches"] = dict(fused_ops.CALLS)
            if fused_fallback:
                out["fused_comm_fallback"] = fused_fallback
            if fused_choice:
                out["fused_comm_choice"] = fused_choice
        if e2e is not None:
            out["e2e"] = e2e
        if is_headline:
            out["baselines"] = {"pytorch_cublas_nccl_tokens_per_s": base_pt, "own_kernels_nccl_tokens_per_s": base_nccl,
                                "vs_own_kernels_nccl": (value / base_nccl) if base_nccl else None,
                                "source": "baseline/measured.json"}
            nccl_ms = (fused_choice or {}).get("ms_per_step", {}).get("ag_gemm=nccl,gemm_rs=nccl")
            if nccl_ms:
                # the same step with both collectives as NCCL + plain GEMM, timed in this run by the tuner (3 replays)
                out["baselines"]["own_kernels_nccl_same_run_ms_per_step"] = nccl_ms
                out["baselines"]["vs_own_kernels_nccl_same_run"] = nccl_ms / (ms / args.steps)
        print(json.dumps(out), flush=True)
    # Tear down without destroying NCCL communicators that a live CUDA graph still references (that can block
    # forever): drop the graph, drain the device, meet the other ranks, run the interpreter's registered exit
    # handlers (anything that records which libraries this process loaded runs there) and only then leave the
    # process directly.  A single process holds no communicator and simply returns.
    if gstep is not None:
        gstep.graph.reset()
        gstep = None
    torch.cuda.synchronize()
    if world == 1:
        return
    dist.barrier()
    sys.stdout.flush()
    sys.stderr.flush()
    import atexit
    try:
        atexit._run_exitfuncs()
    finally:
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
