"""Run under torchrun on T >= 2 GPUs: every fused compute+collective kernel against fp32 `torch.matmul` plus
`torch.distributed` collectives on the same ranks (outputs and gradients), each at least twice in a row so that both
double buffers and their flags are reused, with shapes that exercise edge tiles.  Exit code 0 on success.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 tests/gpu_collectives_check.py
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from state_space_models_neuron_b200.ops import cuda_ops  # noqa: E402
from state_space_models_neuron_b200.parallel import fused, fused_ops, mappings as mp, state as ps, symm  # noqa: E402
from state_space_models_neuron_b200.parallel.cross_entropy import parallel_cross_entropy  # noqa: E402
from state_space_models_neuron_b200.utils.debug import assert_deterministic  # noqa: E402

FAILS = []


def close(name, a, b, atol, rtol=2e-2):
    a, b = a.float(), b.float()
    bad = ((a - b).abs() > atol + rtol * b.abs()).float().mean().item()
    if bad > 0:
        FAILS.append(f"[rank {dist.get_rank()}] {name}: {bad:.5f} of elements off, max err {(a - b).abs().max().item():.4e}")


def rnd(shape, seed, scale=0.5):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, device="cuda", generator=g) * scale).bfloat16()


def gather_rows(x_shard):
    T = dist.get_world_size()
    out = torch.empty(T * x_shard.shape[0], x_shard.shape[1], dtype=x_shard.dtype, device="cuda")
    dist.all_gather_into_tensor(out, x_shard.contiguous())
    return out


def check_ag_gemm(T, r, ws):
    for rep, (Ls, K, N, b_mn) in enumerate([(128, 512, 264, False), (256, 4096, 6286, False), (2048 // T, 1024, 2320, False),
                                            (256, 520, 1024, True), (128, 512, 264, False)]):
        x = rnd((Ls, K), 10 * rep + r)
        w = rnd((K, N) if b_mn else (N, K), 77 + rep)          # same weight on every rank
        if w.shape[1] % 8:
            w = torch.nn.functional.pad(w, (0, (-w.shape[1]) % 8))[:, :w.shape[1]]
        gathered, y = fused_ops._ag_gemm(x, w, b_mn, None, ws)
        full = gather_rows(x)
        if not torch.equal(gathered, full):
            FAILS.append(f"[rank {r}] ag_gemm {Ls}x{K}: gathered rows differ from all_gather")
        ref = full.float() @ (w.float() if b_mn else w.float().t())
        close(f"ag_gemm {Ls}x{K}x{N}", y, ref, atol=0.02 * K ** 0.5 * 0.25 + 0.02)


def check_gemm_rs(T, r, ws, library=False):
    """`library`: the op runs as plain GEMM (bf16 out) + NCCL reduce-scatter.  Every partial block is then rounded to
    bf16 before the sum (relative error 2^-9 each, and again per addition), which the fused kernel avoids for its own
    partial: the bound for that form is elementwise, 2^-8 of the sum of the partials' magnitudes."""
    for rep, (Ls, K, N, b_mn) in enumerate([(128, 256, 384, False), (256, 1024, 4096, False), (2048 // T, 520, 1024, True),
                                            (128, 6286, 512, True)]):
        M = T * Ls
        a = rnd((M, K), 500 + 10 * rep + r)
        if K % 8:
            a = torch.nn.functional.pad(a, (0, (-K) % 8))[:, :K]
        w = rnd((K, N) if b_mn else (N, K), 600 + rep)
        out = fused_ops._gemm_rs(a, w, b_mn, ws)
        part = (a.float() @ (w.float() if b_mn else w.float().t()))
        ref = torch.empty(Ls, N, device="cuda")
        dist.reduce_scatter_tensor(ref, part.contiguous())
        atol = 0.012 * (K * T) ** 0.5 * 0.25 + 0.05
        if library:
            mag = torch.empty(Ls, N, device="cuda")
            dist.reduce_scatter_tensor(mag, part.abs().contiguous())
            atol = atol + mag * 2.0 ** -8
        close(f"gemm_rs{' (library form)' if library else ''} {M}x{K}x{N}", out, ref, atol=atol)


def check_layers_autograd(T, r):
    """Column-parallel (all-gather) and row-parallel (reduce-scatter) linear layers: outputs, input gradients and
    weight gradients of the fused path against the library-collective path on the same data."""
    Ls, D, F = 256, 512, 1024
    x0 = rnd((1, Ls, D), 900 + r)
    w1, w2 = rnd((F, D), 901 + r, 0.05), rnd((D, F), 902 + r, 0.05)
    gy = rnd((1, Ls, D), 903 + r)
    res = []
    for use_fused in (True, False):
        x = x0.clone().requires_grad_(True)
        a, b = w1.clone().requires_grad_(True), w2.clone().requires_grad_(True)
        if use_fused:
            h = fused.all_gather_linear(x, a)
            y = fused.linear_reduce_scatter(h, b)
        else:
            h = cuda_ops.linear(mp.gather_from_sequence_parallel_region(x, True), a)
            y = mp.reduce_scatter_to_sequence_parallel_region(cuda_ops.linear(h, b))
        y.backward(gy)
        res.append((y.detach(), x.grad, a.grad, b.grad))
    for name, u, v, tol in zip(("y", "dx", "dw1", "dw2"), res[0], res[1], (0.05, 0.05, 0.3, 0.3)):
        close(f"layers autograd {name}", u, v, atol=tol)
    # q, k, v behind one all-gather
    ws3 = [rnd((n, D), 910 + i, 0.05) for i, n in enumerate((512, 128, 128))]
    x = x0.clone().requires_grad_(True)
    outs = fused.all_gather_multi_linear(x, ws3)
    full = gather_rows(x0[0])
    for i, (o, w) in enumerate(zip(outs, ws3)):
        close(f"multi-linear output {i}", o[0], full.float() @ w.float().t(), atol=0.1)


def check_lm_head_ce(T, r):
    """LM head with the cross-entropy statistics from the GEMM epilogue (vocabulary shard not a multiple of 8)
    against the unfused path: loss, dX and dW."""
    Ls, D, Vs = 128, 512, 6286 // 2 if T == 2 else 786
    L = Ls * T
    x0 = rnd((1, Ls, D), 1000 + r)
    w0 = rnd((Vs, D), 1001 + r, 0.1)
    g = torch.Generator(device="cuda").manual_seed(5)
    labels = torch.randint(0, Vs * T, (1, L), device="cuda", generator=g)
    labels[0, -1] = -100
    res = []
    for use_fused in (True, False):
        x, w = x0.clone().requires_grad_(True), w0.clone().requires_grad_(True)
        if use_fused:
            y, stats = fused.all_gather_linear(x, w, None, ce=(labels.reshape(-1), r * Vs))
            loss = parallel_cross_entropy(y, labels, stats=stats).sum() / (L - 1)
        else:
            y = cuda_ops.linear(mp.gather_from_sequence_parallel_region(x, True), w)
            fused.set_enabled(False)
            loss = parallel_cross_entropy(y, labels).sum() / (L - 1)
            fused.set_enabled(True)
        loss.backward()
        res.append((loss.detach(), x.grad, w.grad))
    if abs(res[0][0].item() - res[1][0].item()) > 2e-3:
        FAILS.append(f"[rank {r}] LM head + CE loss {res[0][0].item()} vs {res[1][0].item()}")
    close("LM head + CE dx", res[0][1], res[1][1], atol=2e-4, rtol=3e-2)
    close("LM head + CE dw", res[0][2], res[1][2], atol=2e-4, rtol=3e-2)


def check_small_collectives(T, r):
    for n in (1, 7, 4096, 16384):
        for op in ("sum", "max"):
            v = torch.randn(n, device="cuda") + r
            ref = v.clone()
            dist.all_reduce(ref, op=dist.ReduceOp.SUM if op == "sum" else dist.ReduceOp.MAX)
            if not fused.small_allreduce(v, op):
                FAILS.append(f"[rank {r}] small_allreduce not available for n={n}")
            close(f"small_allreduce {op} n={n}", v, ref, atol=1e-5, rtol=1e-6)
    for shape in ((64, 2560), (1, 4096), (8, 512)):
        x = rnd(shape, 1200 + r)
        ref = x.float().clone()
        dist.all_reduce(ref)
        out = fused.allreduce_bf16(x)
        if out is None:
            FAILS.append(f"[rank {r}] allreduce_bf16 not available for {shape}")
        else:
            close(f"allreduce_bf16 {shape}", out, ref, atol=3e-2, rtol=1e-2)


def check_embedding(T, r):
    V, D, B, L = 1024, 512, 1, 256 * T
    Vs = V // T
    g = torch.Generator(device="cuda").manual_seed(3)
    ids = torch.randint(0, V, (B, L), device="cuda", generator=g)
    table = rnd((V, D), 1300)                                # full table, same on every rank
    w = table[r * Vs:(r + 1) * Vs].clone().requires_grad_(True)
    go = rnd((B, L // T, D), 1301 + r)
    for rep in range(2):
        w.grad = None
        out = fused.vocab_embed_scatter(ids, w, r * Vs)
        if out is None:
            FAILS.append(f"[rank {r}] vocab_embed_scatter not available")
            return
        ref = table[ids][:, r * (L // T):(r + 1) * (L // T)]
        if not torch.equal(out, ref):
            FAILS.append(f"[rank {r}] vocab_embed_scatter forward differs")
        out.backward(go)
        gfull = gather_rows(go[0]).float()                  # [L, D] in sequence order (B = 1)
        gref = torch.zeros(Vs, D, device="cuda")
        local = ids[0] - r * Vs
        inside = (local >= 0) & (local < Vs)
        gref.index_add_(0, local.clamp(0, Vs - 1), gfull * inside[:, None])
        close("vocab_embed_scatter dW", w.grad, gref, atol=3e-2, rtol=1e-2)


def check_wraparound(T, r, ws):
    """Sequence numbers that cross 2^31 in the middle of a run: collectives keep synchronising."""
    ws.seq_base.fill_(2 ** 31 - 3 * 65536 + 17)
    torch.cuda.synchronize()
    dist.barrier()
    for step in range(6):
        ws.advance_step()
        x = rnd((128, 512), 1400 + 10 * step + r)
        w = rnd((256, 512), 1450 + step)
        gathered, y = fused_ops._ag_gemm(x, w, False, None, ws)
        close(f"wrap step {step} ag_gemm", y, gather_rows(x).float() @ w.float().t(), atol=0.3)
        v = torch.full((5,), float(r + step), device="cuda")
        fused.small_allreduce(v, "sum")
        want = sum(range(T)) + T * step
        if not torch.equal(v, torch.full_like(v, float(want))):
            FAILS.append(f"[rank {r}] wrap step {step}: small_allreduce gave {v.tolist()} instead of {want}")
    torch.cuda.synchronize()
    if r == 0:
        print("sequence base after the wrap test:", int(ws.seq_base.item()))


def main():
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    T = int(os.environ["WORLD_SIZE"])
    ps.initialize_model_parallel(T, backend="nccl")
    r = ps.get_rank()
    fused.set_enabled(True)
    fused_ops.install()
    ws = symm.get_workspace(2048, 6400, torch.device("cuda"))
    check_ag_gemm(T, r, ws)
    check_gemm_rs(T, r, ws)
    check_layers_autograd(T, r)
    check_lm_head_ce(T, r)
    check_small_collectives(T, r)
    check_embedding(T, r)
    # same inputs, same rank, twice: the fused kernels must be bit-reproducible (fixed reduction orders)
    xs, wd = rnd((128, 512), 40 + r), rnd((264, 512), 41)
    assert_deterministic(lambda a, b: fused_ops._ag_gemm(a, b, False, None, ws)[1], [xs, wd])
    ad, w2 = rnd((128 * T, 256), 42 + r), rnd((384, 256), 43)
    assert_deterministic(lambda a, b: fused_ops._gemm_rs(a, b, False, ws), [ad, w2])
    check_wraparound(T, r, ws)
    # the same checks with each kernel switched to its library form (NCCL collective + plain GEMM): what the
    # step-level tuner falls back to op by op
    for name in ("ag_gemm", "gemm_rs"):
        fused.set_kernel(name, False)
    check_ag_gemm(T, r, ws)
    check_gemm_rs(T, r, ws, library=True)
    check_layers_autograd(T, r)
    check_lm_head_ce(T, r)
    for name in ("ag_gemm", "gemm_rs"):
        fused.set_kernel(name, True)
    if fused_ops.CALLS.get("ag_gemm_library", 0) == 0 or fused_ops.CALLS.get("gemm_rs_library", 0) == 0:
        FAILS.append(f"[rank {r}] the library forms of the fused ops did not run: {dict(fused_ops.CALLS)}")
    torch.cuda.synchronize()
    try:
        cuda_ops.check_status()
    except RuntimeError as e:
        FAILS.append(f"[rank {r}] {e}")
    bad = torch.tensor([len(FAILS)], device="cuda")
    dist.all_reduce(bad)
    for f in FAILS:
        print(f, flush=True)
    if r == 0:
        print("fused kernel launches", dict(fused_ops.CALLS))
        print("OK" if int(bad.item()) == 0 else f"MISMATCH ({int(bad.item())} failures over all ranks)")
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if int(bad.item()) == 0 else 1)


if __name__ == "__main__":
    main()
