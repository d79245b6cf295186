"""Run under torchrun on 2 GPUs: training with gradient accumulation through CUDA graphs (one graph for the first
micro-step of an optimizer step, one for the following ones, one for the update) must reproduce the losses and the
parameters of the same run with eager launches, with the fused tensor-parallel collectives on.  Exit code 0 on
success.  (The reference accumulates gradients over micro-steps in its training loop, train.py:178-232.)"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from state_space_models_neuron_b200 import parallel as nxd  # noqa: E402
from state_space_models_neuron_b200.models import Mamba2Config, Mamba2ForCausalLM  # noqa: E402
from state_space_models_neuron_b200.ops import cuda_ops  # noqa: E402
from state_space_models_neuron_b200.parallel import state as ps  # noqa: E402
from state_space_models_neuron_b200.parallel.graph import GraphedAccumulationStep  # noqa: E402

ACCUM, STEPS = 4, 5


def build(tp):
    ps.destroy_model_parallel()
    ps.initialize_model_parallel(tp, backend="nccl")
    mc = Mamba2Config(num_heads=16, head_dim=64, vocab_size=2048, hidden_size=512, state_size=128, num_hidden_layers=2,
                      n_groups=8, tie_word_embeddings=True, initializer_range=0.02, sequence_parallel_enabled=tp > 1,
                      dtype=torch.bfloat16)
    cfg = nxd.parallel_config(tp, {"zero_one_enabled": True}, sequence_parallel=tp > 1, init_seed=3, fused_comm=True)
    model = nxd.initialize_parallel_model(cfg, lambda: Mamba2ForCausalLM(mc, device="cuda").to(torch.bfloat16))
    opt = nxd.initialize_parallel_optimizer(cfg, nxd.AdamW_FP32OptimParams,
                                            [{"params": list(model.parameters()), "weight_decay": 0.1}], lr=1e-3)
    opt.zero_grad()
    return model, opt


def main():
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    world = dist.get_world_size()
    g = torch.Generator().manual_seed(0)
    batches = [torch.randint(0, 2048, (1, 1024), generator=g).cuda() for _ in range(ACCUM * STEPS)]

    def eager():
        model, opt = build(world)
        losses = []
        for s in range(STEPS):
            tot = 0.0
            for m in range(ACCUM):
                ids = batches[s * ACCUM + m]
                loss = model(input_ids=ids, labels=ids, return_logits=False).loss / ACCUM
                loss.backward()
                tot += loss.item()
            opt.step()
            opt.zero_grad()
            losses.append(tot)
        return losses, opt.flat_params.float().clone()

    def graphed():
        # graph capture cannot involve the default stream: like train.py --cuda_graph, run everything on a side stream
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            out = graphed_on_side_stream()
        torch.cuda.current_stream().wait_stream(side)
        return out

    def graphed_on_side_stream():
        model, opt = build(world)
        losses, step = [], None
        for s in range(STEPS):
            tot = torch.zeros((), device="cuda")
            for m in range(ACCUM):
                ids = batches[s * ACCUM + m]
                if s < 2:            # the first optimizer steps run eagerly on their own batches, as train.py does
                    loss = model(input_ids=ids, labels=ids, return_logits=False).loss / ACCUM
                    loss.backward()
                    tot += loss.detach()
                    if m == ACCUM - 1:
                        opt.step()
                        opt.zero_grad()
                else:
                    if step is None:
                        step = GraphedAccumulationStep(model, opt, {"input_ids": ids, "labels": ids}, ACCUM, warmup=0)
                    tot += step.micro_step({"input_ids": ids, "labels": ids})
            losses.append(tot.item())
        params = opt.flat_params.float().clone()
        del step
        return losses, params

    a, pa = eager()
    b, pb = graphed()
    torch.cuda.synchronize()
    cuda_ops.check_status()
    ok = all(abs(x - y) < 2e-3 for x, y in zip(a, b))
    diff = (pa - pb).abs().max().item()
    ok = ok and diff < 2e-2
    if dist.get_rank() == 0:
        print("eager  ", a)
        print("graphed", b)
        print("max parameter difference", diff)
        print("OK" if ok else "MISMATCH")
    dist.barrier()
    os._exit(0 if ok else 1)


if __name__ == "__main__":
    main()
