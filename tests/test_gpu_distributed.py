"""Multi-GPU equivalence (needs >= 2 GPUs): TP=N+SP+ZeRO-1 in bf16 follows the TP=1 loss curve."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _torchrun(n, *extra, port=29611):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "gpu_tp_check.py"), *extra]
    return subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)


@pytest.mark.parametrize("extra", [(), ("--fused",), ("--fused", "--dp"), ("--fused", "--hybrid")])
def test_tp_matches_single_gpu(extra):
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    r = _torchrun(min(n, 8) if n in (2, 4, 8) else 2, *extra, port=29611 + len(extra))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]


def test_fused_collectives_against_torch_distributed():
    """Every fused compute+collective kernel against fp32 matmul + torch.distributed on the same ranks."""
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    world = n if n in (2, 4, 8) else 2
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", "29641", os.path.join(ROOT, "tests", "gpu_collectives_check.py")]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-4000:] + r.stderr[-3000:]


def test_graphed_accumulation_matches_eager():
    """train.py with --cuda_graph and gradient accumulation (three graphs) reproduces the eager run's losses."""
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29651", os.path.join(ROOT, "tests", "gpu_graph_accum_check.py")]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-4000:] + r.stderr[-3000:]


def test_tp_decode_matches_forward():
    """Token-by-token decode under TP=2 (one-kernel all-reduce after out_proj, graph-free) reproduces the logits of
    the full forward pass on every rank's vocabulary shard."""
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29631", os.path.join(ROOT, "mamba2_inference.py"), "--mode", "check", "--model", "Mamba130M",
           "--tp", "2", "--n_groups", "2", "--head_dim", "64", "--batch", "2", "--seq_len", "256"]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
