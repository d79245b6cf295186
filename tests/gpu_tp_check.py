"""Run under torchrun on N GPUs: a small bf16 model at TP=N (+SP, +ZeRO-1) must reproduce the loss curve of the
same model at TP=1 (built on every rank from the same seeds).  Exit code 0 on success."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from state_space_models_neuron_b200 import parallel as nxd  # noqa: E402
from state_space_models_neuron_b200.models import (Mamba2Config, Mamba2ForCausalLM, Mamba2HybridConfig,  # noqa: E402
                                                   Mamba2HybridForCausalLM)
from state_space_models_neuron_b200.ops import cuda_ops  # noqa: E402
from state_space_models_neuron_b200.parallel import state as ps  # noqa: E402


def build(tp, sp, hybrid, fused):
    ps.destroy_model_parallel()
    ps.initialize_model_parallel(tp, backend="nccl")
    kw = dict(num_heads=16, head_dim=64, vocab_size=2048, hidden_size=512, state_size=128, num_hidden_layers=2,
              n_groups=8, tie_word_embeddings=True, initializer_range=0.02, sequence_parallel_enabled=sp,
              dtype=torch.bfloat16)
    if hybrid:
        mc = Mamba2HybridConfig(**{**kw, "num_hidden_layers": 4}, attn_num_heads=8, attn_head_dim=128,
                                attn_key_value_heads=8, mlp_hidden_size=1024, hybrid_attention_ratio=0.25,
                                hybrid_mlp_ratio=0.25, residual_in_fp32=False)
        cls = Mamba2HybridForCausalLM
    else:
        mc, cls = Mamba2Config(**kw), Mamba2ForCausalLM
    cfg = nxd.parallel_config(tp, {"zero_one_enabled": True}, sequence_parallel=sp, init_seed=3, fused_comm=fused)
    model = nxd.initialize_parallel_model(cfg, lambda: cls(mc, device="cuda").to(torch.bfloat16))
    opt = nxd.initialize_parallel_optimizer(cfg, nxd.AdamW_FP32OptimParams,
                                            [{"params": list(model.parameters()), "weight_decay": 0.1}], lr=1e-3)
    return model, opt


def build_solo(hybrid):
    """TP=1, DP=1 on this rank alone (no collectives): the reference for the data-parallel check."""
    from state_space_models_neuron_b200.parallel import state as st
    st.destroy_model_parallel()
    st._S = st._State(initialized=True)        # one-rank groups regardless of the launcher's world size
    kw = dict(num_heads=16, head_dim=64, vocab_size=2048, hidden_size=512, state_size=128, num_hidden_layers=2,
              n_groups=8, tie_word_embeddings=True, initializer_range=0.02, dtype=torch.bfloat16)
    cfg = nxd.parallel_config(1, {"zero_one_enabled": False}, init_seed=3, fused_comm=False)
    from state_space_models_neuron_b200.parallel.layers import set_init_seed
    from state_space_models_neuron_b200.parallel import fused as fz
    set_init_seed(3)
    fz.set_enabled(False)
    model = Mamba2ForCausalLM(Mamba2Config(**kw), device="cuda").to(torch.bfloat16)
    model.lm_head.weight = model.backbone.embeddings.weight
    opt = nxd.initialize_parallel_optimizer(cfg, nxd.AdamW_FP32OptimParams,
                                            [{"params": list(model.parameters()), "weight_decay": 0.1}], lr=1e-3)
    return model, opt


def run(model, opt, ids, steps, grads_of=None):
    """Losses of `steps` optimizer steps; with `grads_of` (list of parameter-name substrings) also the fp32 gradients
    of the first step, as the optimizer sees them, for the parameters whose name contains one of them."""
    losses, grads = [], {}

    def snapshot(_):
        if not grads and grads_of:
            for n, p in model.named_parameters():
                if any(k in n for k in grads_of):
                    grads[n] = p.main_grad.detach().float().clone()
    opt.post_reduce_hook = snapshot
    for i in range(steps):
        opt.zero_grad()
        loss = model(input_ids=ids, labels=ids, return_logits=False).loss
        loss.backward()
        opt.step()
        losses.append(loss.item())
    opt.post_reduce_hook = None
    return losses, grads


def main():
    hybrid = "--hybrid" in sys.argv
    fused = "--fused" in sys.argv
    dp_mode = "--dp" in sys.argv            # TP=1, DP=world: exercises the fused ZeRO-1 reduce/AdamW/push kernels
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    world = dist.get_world_size()
    g = torch.Generator().manual_seed(0)
    shape = (1, 1024) if (fused and not dp_mode) else (world if dp_mode else 2, 512)
    ids = torch.randint(0, 2048, shape, generator=g).cuda()
    if dp_mode:
        # single-rank reference: every rank runs the full batch in its own one-rank group
        ps.destroy_model_parallel()
    # replicated parameters (norm weights) have the same full gradient on every rank at any TP degree
    watch = ["norm.weight", "norm_f.weight"] if not dp_mode else None
    m1, o1 = build(1, False, hybrid, False) if not dp_mode else build_solo(hybrid)
    ref, ref_grads = run(m1, o1, ids, 3, watch)
    del m1, o1
    if dp_mode:
        mt, ot = build(1, False, hybrid, fused)
        mine = ids[ps.get_data_parallel_rank():ps.get_data_parallel_rank() + 1]
        got, _ = run(mt, ot, mine, 3)
        t = torch.tensor(got, device="cuda")
        dist.all_reduce(t)
        got = (t / world).tolist()
        assert getattr(ot, "_fused_dp", False) == fused, "fused ZeRO-1 path was not selected"
    else:
        mt, ot = build(world, True, hybrid, fused)
        got, got_grads = run(mt, ot, ids, 3, watch)
    torch.cuda.synchronize()
    cuda_ops.check_status()
    ok = all(abs(a - b) < 0.05 for a, b in zip(ref, got))
    if not dp_mode:
        # gradients of the replicated norm weights after the first backward pass: summed over the sequence shards they
        # must equal the single-GPU gradient (bf16 activations: 3 % of the gradient's largest entry)
        for n, g1 in ref_grads.items():
            gt = got_grads.get(n)
            if gt is None or gt.shape != g1.shape:
                continue
            err = (gt - g1).abs().max().item()
            if err > 0.03 * g1.abs().max().item() + 1e-4:
                ok = False
                if dist.get_rank() == 0:
                    print(f"gradient mismatch {n}: max err {err:.4e} vs max |g| {g1.abs().max().item():.4e}")
    if fused and not dp_mode:
        from state_space_models_neuron_b200.parallel import fused_ops
        ok = ok and fused_ops.CALLS["ag_gemm"] > 0 and fused_ops.CALLS["gemm_rs"] > 0
        if dist.get_rank() == 0:
            print("fused kernel launches", fused_ops.CALLS)
    if dist.get_rank() == 0:
        print("TP=1 losses", ref)
        print(f"TP={world} losses", got, "fused" if fused else "nccl")
        print("OK" if ok else "MISMATCH")
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
