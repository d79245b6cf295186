"""TP / SP / ZeRO-1 equivalence on gloo CPU ranks: T-rank results equal single-rank results."""
import os
import tempfile

import pytest
import torch

from tests.dist_utils import run_ranks


def _cfg(sp=False, hybrid=False):
    from state_space_models_neuron_b200.models import Mamba2Config, Mamba2HybridConfig
    kw = dict(num_heads=4, head_dim=32, vocab_size=256, hidden_size=64, state_size=32, num_hidden_layers=2,
              n_groups=2, tie_word_embeddings=True, initializer_range=0.05, sequence_parallel_enabled=sp,
              dtype=torch.float32)
    if hybrid:
        return Mamba2HybridConfig(**{**kw, "num_hidden_layers": 4}, attn_num_heads=4, attn_head_dim=16,
                                  attn_key_value_heads=2, mlp_hidden_size=128, hybrid_attention_ratio=0.25,
                                  hybrid_mlp_ratio=0.25, residual_in_fp32=False)
    return Mamba2Config(**kw)


def _reference_run(hybrid, steps, path):
    """single process, TP=1: losses, merged params after `steps` optimizer steps."""
    from state_space_models_neuron_b200 import parallel as nxd
    from state_space_models_neuron_b200.models import Mamba2ForCausalLM, Mamba2HybridForCausalLM
    from state_space_models_neuron_b200.parallel import state as ps
    ps.initialize_model_parallel(1)
    cfg = nxd.parallel_config(1, {"zero_one_enabled": False}, device="cpu", init_seed=7)
    cls = Mamba2HybridForCausalLM if hybrid else Mamba2ForCausalLM
    model = nxd.initialize_parallel_model(cfg, lambda: cls(_cfg(False, hybrid)))
    opt = nxd.initialize_parallel_optimizer(cfg, nxd.AdamW_FP32OptimParams,
                                            [{"params": list(model.parameters()), "weight_decay": 0.1}], lr=1e-2)
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, 256, (4, 128), generator=g)
    losses = []
    for _ in range(steps):
        opt.zero_grad()
        loss = model(input_ids=ids, labels=ids).loss
        loss.backward()
        opt.step()
        losses.append(loss.item())
    torch.save({"losses": losses, "sd": {k: v.clone() for k, v in model.state_dict().items()}, "ids": ids}, path)


def _tp_worker(rank, world, tp, sp, zero1, hybrid, steps, ref_path, out_dir):
    from state_space_models_neuron_b200 import parallel as nxd
    from state_space_models_neuron_b200.models import Mamba2ForCausalLM, Mamba2HybridForCausalLM
    from state_space_models_neuron_b200.parallel import state as ps
    from state_space_models_neuron_b200.parallel.layout import merge_state_dicts
    ps.initialize_model_parallel(tp)
    cfg = nxd.parallel_config(tp, {"zero_one_enabled": zero1}, sequence_parallel=sp, device="cpu", init_seed=7)
    cls = Mamba2HybridForCausalLM if hybrid else Mamba2ForCausalLM
    mcfg = _cfg(sp, hybrid)
    model = nxd.initialize_parallel_model(cfg, lambda: cls(mcfg))
    opt = nxd.initialize_parallel_optimizer(cfg, nxd.AdamW_FP32OptimParams,
                                            [{"params": list(model.parameters()), "weight_decay": 0.1}], lr=1e-2)
    ref = torch.load(ref_path, weights_only=False)
    ids = ref["ids"]
    dp, dpr = ps.get_data_parallel_size(), ps.get_data_parallel_rank()
    mine = ids.chunk(dp)[dpr]
    losses = []
    for _ in range(steps):
        opt.zero_grad()
        loss = model(input_ids=mine, labels=mine).loss
        loss.backward()
        opt.step()
        l = loss.detach().clone() / dp
        if dp > 1:
            torch.distributed.all_reduce(l, group=ps.get_data_parallel_group())
        losses.append(l.item())
    for a, b in zip(losses, ref["losses"]):
        assert abs(a - b) < 2e-4, (losses, ref["losses"])
    nxd.save_checkpoint(out_dir, "t", model, opt, None, {"config": mcfg.to_dict()})
    if rank == 0:
        shards = [torch.load(os.path.join(out_dir, "t", "model", f"dp_rank_00_tp_rank_{r:02d}_pp_rank_00.pt"),
                             weights_only=False) for r in range(tp)]
        merged = merge_state_dicts(shards, mcfg)
        for k, v in ref["sd"].items():
            assert torch.allclose(merged[k], v, atol=2e-4, rtol=1e-3), (k, (merged[k] - v).abs().max())


@pytest.mark.parametrize("world,tp,sp,zero1,hybrid", [
    (2, 2, True, False, False),
    (2, 2, False, False, False),
    (2, 1, False, True, False),
    (4, 2, True, True, False),
    (2, 2, True, False, True),
])
def test_parallel_training_matches_single_rank(world, tp, sp, zero1, hybrid):
    with tempfile.TemporaryDirectory() as d:
        ref = os.path.join(d, "ref.pt")
        _run_reference(hybrid, 3, ref)
        run_ranks(_tp_worker, world, tp, sp, zero1, hybrid, 3, ref, os.path.join(d, "ck"))


def _ref_entry(rank, world, hybrid, steps, path):
    _reference_run(hybrid, steps, path)


def _run_reference(hybrid, steps, path):
    run_ranks(_ref_entry, 1, hybrid, steps, path)


def _tp_decode_worker(rank, world, hybrid):
    """TP=2 prefill + token-by-token decode gives the vocabulary shards of the single-rank full forward."""
    from state_space_models_neuron_b200 import parallel as nxd
    from state_space_models_neuron_b200.models import Mamba2Cache, Mamba2ForCausalLM, Mamba2HybridForCausalLM
    from state_space_models_neuron_b200.parallel import state as ps
    from state_space_models_neuron_b200.parallel.layout import shard_state_dict
    cls = Mamba2HybridForCausalLM if hybrid else Mamba2ForCausalLM
    mcfg = _cfg(False, hybrid)
    # full model on every rank (TP=1 state) as the oracle
    ps.initialize_model_parallel(1)
    torch.manual_seed(11)
    full = cls(mcfg).eval()
    ids = torch.randint(0, 256, (2, 256), generator=torch.Generator().manual_seed(5))
    with torch.no_grad():
        ref = full(input_ids=ids).logits
    sd = {k: v.clone() for k, v in full.state_dict().items()}
    ps.destroy_model_parallel()
    ps.initialize_model_parallel(world)
    cfg = nxd.parallel_config(world, {"zero_one_enabled": False}, device="cpu", init_seed=7)
    model = nxd.initialize_parallel_model(cfg, lambda: cls(mcfg)).eval()
    model.load_state_dict(shard_state_dict(sd, mcfg, world, rank), strict=False)
    per = 256 // world
    mine = ref[..., rank * per:(rank + 1) * per]
    with torch.no_grad():
        logits, cache = model.prefill(ids[:, :128])
        assert torch.allclose(logits[:, -1], mine[:, 127], atol=2e-4, rtol=1e-3)
        for t in range(128, 152):
            out = model.step(ids[:, t:t + 1], cache)
            assert torch.allclose(out[:, 0], mine[:, t], atol=3e-4, rtol=1e-3), (t, (out[:, 0] - mine[:, t]).abs().max())
        # greedy generation picks the same tokens as the single-rank model (parallel argmax over vocab shards)
        ps.destroy_model_parallel()
        ps.initialize_model_parallel(1)
        want = full.generate_tokens(ids[:, :130], 6)
        ps.destroy_model_parallel()
        ps.initialize_model_parallel(world)
        got = model.generate_tokens(ids[:, :130], 6)
        assert torch.equal(got, want), (got[:, -6:], want[:, -6:])


def test_tensor_parallel_decode_matches_full_forward():
    # the hybrid model has no decode cache (the reference asserts use_cache is False, mamba2hybrid_attn.py:379)
    run_ranks(_tp_decode_worker, 2, False)


def _gqa_qkv_worker(rank, world):
    """GQAQKVColumnParallelLinear with one KV head replicated over two TP ranks: outputs equal the single-rank
    projections and both copies of the KV weights receive the same (summed) gradient."""
    import torch.distributed as dist
    from state_space_models_neuron_b200.parallel import state as ps
    from state_space_models_neuron_b200.parallel.layers import GQAQKVColumnParallelLinear, set_init_seed
    hd, Hq, Hkv, D = 8, 4, 1, 32
    x = torch.randn(2, 16, D, generator=torch.Generator().manual_seed(1))
    ps.initialize_model_parallel(1)
    set_init_seed(3)
    ref = GQAQKVColumnParallelLinear(D, [Hq * hd, Hkv * hd], kv_size_multiplier=1, head_dim=hd)
    q0, k0, v0 = ref(x)
    (q0.square().sum() + (k0 * 2).sum() + v0.square().sum()).backward()
    ps.destroy_model_parallel()
    ps.initialize_model_parallel(world)
    set_init_seed(3)
    lay = GQAQKVColumnParallelLinear(D, [Hq * hd, Hkv * hd], kv_size_multiplier=2, head_dim=hd)
    assert lay.weight_k.shape == (hd, D) and torch.equal(lay.weight_k, ref.weight_k)      # a full copy per rank
    xr = x.clone().requires_grad_(True)
    q, k, v = lay(xr)
    per = Hq * hd // world
    assert torch.allclose(q, q0[..., rank * per:(rank + 1) * per], atol=1e-6)
    assert torch.allclose(k, k0, atol=1e-6) and torch.allclose(v, v0, atol=1e-6)
    # each rank uses its copy for half of the query heads: loss split accordingly, gradients summed over the copies
    (q.square().sum() + (k * 2).sum() / world + v.square().sum() / world).backward()
    assert torch.allclose(lay.weight_k.grad, ref.weight_k.grad, atol=1e-5), (lay.weight_k.grad - ref.weight_k.grad).abs().max()
    assert torch.allclose(lay.weight_v.grad, ref.weight_v.grad, atol=1e-5)
    assert torch.allclose(lay.weight_q.grad, ref.weight_q.grad[rank * per:(rank + 1) * per], atol=1e-5)


def test_gqa_qkv_linear_kv_replication():
    run_ranks(_gqa_qkv_worker, 2)


def _tuner_agreement_worker(rank, world):
    """Two ranks whose local timings prefer different combinations must end up with the same choice: the times are
    reduced with MAX over the ranks before they are compared."""
    import time
    from state_space_models_neuron_b200.parallel import fused, fused_tune
    # milliseconds per step on (rank 0, rank 1): rank 0 alone would pick the first combination, rank 1 the last one;
    # the slowest rank decides: max = 40, 25, 30, 45 -> the second combination
    cost = {(True, True): (5, 40), (False, True): (25, 20), (True, False): (30, 30), (False, False): (45, 3)}

    def build():
        key = (fused.kernel_enabled("ag_gemm"), fused.kernel_enabled("gemm_rs"))
        step = lambda: time.sleep(cost[key][rank] / 1e3)
        step.key = key
        return step

    rep = fused_tune.pick_fastest(build, "cpu", reps=3)
    assert rep["chosen"] == "ag_gemm=nccl,gemm_rs=fused", rep
    assert fused.kernels() == {"ag_gemm": False, "gemm_rs": True}
    ms = rep["ms"]
    assert ms["ag_gemm=fused,gemm_rs=fused"] >= 39 and ms["ag_gemm=nccl,gemm_rs=nccl"] >= 44 and ms["ag_gemm=nccl,gemm_rs=fused"] < 39


def test_fused_tuner_ranks_agree_on_the_slowest_ranks_time():
    run_ranks(_tuner_agreement_worker, 2)
