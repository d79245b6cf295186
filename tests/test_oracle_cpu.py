"""Config-1 checks on CPU in fp32: chunked SSD scan vs the naive recurrence (outputs, gradients, last
state), conv, gated norm, and decode vs forward token by token."""
import math

import pytest
import torch

from state_space_models_neuron_b200 import ops
from state_space_models_neuron_b200.models import Mamba2Cache, Mamba2Config, Mamba2ForCausalLM
from state_space_models_neuron_b200.ops import oracle
from state_space_models_neuron_b200.parallel.layers import set_init_seed


def _scan_inputs(B=2, L=256, H=8, P=64, G=1, N=64, seed=0, dtype=torch.float64):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, L, H, P, generator=g, dtype=dtype)
    dt = torch.exp(torch.rand(B, L, H, generator=g, dtype=dtype) * (math.log(0.1) - math.log(1e-3)) + math.log(1e-3))
    A = -torch.empty(H, dtype=dtype).uniform_(1, 16, generator=g)
    Bm = torch.randn(B, L, G, N, generator=g, dtype=dtype)
    Cm = torch.randn(B, L, G, N, generator=g, dtype=dtype)
    D = torch.ones(H, dtype=dtype)
    return x, dt, A, Bm, Cm, D


@pytest.mark.parametrize("G,H,P,N", [(1, 8, 64, 64), (2, 4, 32, 16)])
def test_chunked_scan_matches_recurrence(G, H, P, N):
    x, dt, A, Bm, Cm, D = [t.float() for t in _scan_inputs(H=H, P=P, G=G, N=N)]
    y_ref, s_ref = oracle.ssd_recurrence(x, dt, A, Bm, Cm, D)
    y, s = oracle.ssd_chunked(x, dt, A, Bm, Cm, D, 128)
    assert torch.allclose(y, y_ref, atol=1e-4, rtol=1e-4)
    assert torch.allclose(s, s_ref, atol=1e-4, rtol=1e-4)


def test_chunked_scan_gradients_match_recurrence():
    ins = [t.float().requires_grad_(True) for t in _scan_inputs(B=1, L=256, H=2, P=16, G=1, N=16)]
    y_ref, _ = oracle.ssd_recurrence(*ins)
    w = torch.randn_like(y_ref)
    g_ref = torch.autograd.grad((y_ref * w).sum(), ins)
    y, _ = oracle.ssd_chunked(*ins, 128)
    g = torch.autograd.grad((y * w).sum(), ins)
    for a, b in zip(g, g_ref):
        assert torch.allclose(a, b, atol=2e-4, rtol=2e-3), (a - b).abs().max()


def test_scan_initial_state_chaining():
    x, dt, A, Bm, Cm, D = [t.float() for t in _scan_inputs(B=1, L=256, H=2, P=16, G=1, N=16)]
    y_full, s_full = oracle.ssd_chunked(x, dt, A, Bm, Cm, D, 128)
    y1, s1 = oracle.ssd_chunked(x[:, :128], dt[:, :128], A, Bm[:, :128], Cm[:, :128], D, 128)
    y2, s2 = oracle.ssd_chunked(x[:, 128:], dt[:, 128:], A, Bm[:, 128:], Cm[:, 128:], D, 128, initial_state=s1)
    assert torch.allclose(torch.cat([y1, y2], 1), y_full, atol=1e-5)
    assert torch.allclose(s2, s_full, atol=1e-5)


def test_conv_matches_torch_conv1d():
    g = torch.Generator().manual_seed(1)
    x = torch.randn(2, 40, 24, generator=g)
    w = torch.randn(24, 4, generator=g)
    b = torch.randn(24, generator=g)
    ref = torch.nn.functional.conv1d(x.transpose(1, 2), w[:, None, :], b, padding=3, groups=24)[..., :40]
    ref = torch.nn.functional.silu(ref).transpose(1, 2)
    assert torch.allclose(oracle.causal_conv1d_silu(x, w, b), ref, atol=1e-5)


def test_gated_norm_groups():
    g = torch.Generator().manual_seed(2)
    y, z, w = torch.randn(3, 5, 64, generator=g), torch.randn(3, 5, 64, generator=g), torch.rand(64, generator=g)
    out = oracle.gated_rmsnorm(y, z, w, 1e-5, group_size=16)
    h = (y * torch.nn.functional.silu(z)).reshape(3, 5, 4, 16)
    ref = (h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + 1e-5)).reshape(3, 5, 64) * w
    assert torch.allclose(out, ref, atol=1e-5)


def _tiny_model():
    set_init_seed(0)
    cfg = Mamba2Config(num_heads=8, head_dim=64, vocab_size=1024, hidden_size=256, state_size=64,
                       num_hidden_layers=2, n_groups=1, tie_word_embeddings=True, initializer_range=0.02,
                       a_log_init="uniform", layer_norm_epsilon=1e-5)
    return Mamba2ForCausalLM(cfg), cfg


def test_tiny_model_forward_backward_and_decode():
    torch.manual_seed(0)
    model, cfg = _tiny_model()
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 1024, (2, 256), generator=g)
    out = model(input_ids=ids, labels=ids)
    assert out.logits.shape == (2, 256, 1024)
    assert abs(out.loss.item() - math.log(1024)) < 0.5
    out.loss.backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in model.parameters())
    model.eval()
    with torch.no_grad():
        full = model(input_ids=ids).logits
        cache = Mamba2Cache(cfg, 2, dtype=torch.float32)
        steps = torch.cat([model.step(ids[:, i:i + 1], cache) for i in range(256)], dim=1)
        assert torch.allclose(steps, full, atol=1e-3, rtol=3e-2)
        _, cache2 = model.prefill(ids[:, :128])
        tail = torch.cat([model.step(ids[:, i:i + 1], cache2) for i in range(128, 256)], dim=1)
        assert torch.allclose(tail, full[:, 128:], atol=1e-3, rtol=3e-2)


def test_loss_from_hidden_equals_shifted_logits_loss():
    model, _ = _tiny_model()
    ids = torch.randint(0, 1024, (2, 128))
    a = model(input_ids=ids, labels=ids).loss
    b = model(input_ids=ids, labels=ids, return_logits=False).loss
    assert torch.allclose(a, b, atol=1e-5)


def test_matches_huggingface_mamba2_mixer():
    """Independent implementation: transformers' torch Mamba2 forward with the same weights."""
    from transformers import Mamba2Config as HFConfig, Mamba2ForCausalLM as HFModel
    model, cfg = _tiny_model()
    hf_cfg = HFConfig(num_heads=8, head_dim=64, vocab_size=1024, hidden_size=256, state_size=64, num_hidden_layers=2,
                      n_groups=1, tie_word_embeddings=True, chunk_size=128, layer_norm_epsilon=1e-5, expand=2)
    hf = HFModel(hf_cfg).eval()
    missing, unexpected = hf.load_state_dict(model.state_dict(), strict=False)
    assert not unexpected and all("lm_head" in m for m in missing)
    ids = torch.randint(0, 1024, (2, 128))
    with torch.no_grad():
        ours = model(input_ids=ids).logits
        theirs = hf(input_ids=ids).logits
    assert torch.allclose(ours, theirs, atol=2e-4, rtol=1e-3), (ours - theirs).abs().max()


def test_generate_tokens_matches_full_forward_greedy():
    model, _ = _tiny_model()
    model.eval()
    ids = torch.randint(0, 1024, (2, 150))          # 128 tokens prefilled, 22 stepped
    out = model.generate_tokens(ids, max_new_tokens=3)
    assert out.shape == (2, 153) and torch.equal(out[:, :150], ids)
    with torch.no_grad():
        cache = Mamba2Cache(model.config, 2, dtype=torch.float32)
        ref = None
        for t in range(150):
            ref = model.step(ids[:, t:t + 1], cache)
    assert torch.equal(out[:, 150], ref[:, -1].argmax(-1))


def test_hf_style_generate_uses_the_cached_decode_path():
    """`model.generate(...)` (HuggingFace calling convention) gives the same tokens as `generate_tokens`."""
    from state_space_models_neuron_b200.models import Mamba2Config, Mamba2ForCausalLM
    from state_space_models_neuron_b200.parallel import state as ps
    ps.initialize_model_parallel(1)
    torch.manual_seed(0)
    m = Mamba2ForCausalLM(Mamba2Config(num_heads=4, head_dim=32, vocab_size=64, hidden_size=64, state_size=32,
                                       num_hidden_layers=2, n_groups=1)).eval()
    ids = torch.randint(1, 64, (2, 130))
    want = m.generate_tokens(ids, 5)
    assert torch.equal(m.generate(ids, max_new_tokens=5, do_sample=False, eos_token_id=-1), want)
    assert torch.equal(m.generate(input_ids=ids, max_length=135, eos_token_id=-1), want)
    sampled = m.generate(ids, max_new_tokens=3, do_sample=True, temperature=0.7, top_k=4, eos_token_id=-1,
                         generator=torch.Generator().manual_seed(1))
    assert sampled.shape == (2, 133) and torch.equal(sampled[:, :130], ids)
