"""GEMM scheduling variants (CTA pairs, K-split tail tiles, cross-entropy epilogue) and the fused
compute+collective GEMMs, each against fp32 `torch.matmul`.

The collective variants are exercised on ONE GPU by playing one rank of a T-rank group: all T "ranks'" buffers
live on this device, the contributions of the other ranks are written (and their flags set) before the launch, so
the kernel under test pushes, waits, computes and reduces exactly as it does with real peers, without a second
process.  The multi-process versions of these checks are in `gpu_collectives_check.py`.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

AG_GROUPS = 4
FLAG_SLOTS = 32


def _close(a, b, atol, rtol=2e-2, frac=1.0):
    a, b = a.float(), b.float()
    ok = (a - b).abs() <= atol + rtol * b.abs()
    assert ok.float().mean().item() >= frac, f"only {ok.float().mean().item():.6f} close; max err {(a - b).abs().max().item():.4e}"


@pytest.fixture(autouse=True)
def _status():
    yield
    from state_space_models_neuron_b200.ops import cuda_ops
    torch.cuda.synchronize()
    cuda_ops.check_status()


def _rand(shape, seed, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, device="cuda", generator=g) * scale).bfloat16()


# shapes chosen to hit: pair tiles with an odd number of 128-row blocks, tails of a few tiles that get cut along K,
# fewer tiles than SMs (everything is tail), N edges that are not a multiple of 8 or 64, K edges
SHAPES = [(2048, 2320, 4096), (2048, 4096, 1024), (384, 6286, 520), (2176, 2560, 2048), (64, 2560, 5120),
          (18560, 4096, 256), (640, 1000, 4096)]


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("layout", ["tn", "nn", "tt"])
def test_gemm_schedules(M, N, K, layout):
    from state_space_models_neuron_b200.ops import cuda_ops
    a, b = _rand((M, K), M + K, 0.5), _rand((N, K), N + K, 0.5)
    ref = a.float() @ b.float().t()
    a_mn, b_mn = layout == "tt", layout in ("nn", "tt")
    A = a.t().contiguous() if a_mn else a
    Bm = b.t().contiguous() if b_mn else b
    if A.shape[1] % 8 or Bm.shape[1] % 8:
        pad = lambda t: torch.nn.functional.pad(t, (0, (-t.shape[1]) % 8))[:, :t.shape[1]]
        A, Bm = pad(A), pad(Bm)
    tol = 0.02 * (K ** 0.5) * 0.25 + 0.02
    out = cuda_ops.gemm(A, Bm, a_mn=a_mn, b_mn=b_mn)
    _close(out, ref, atol=tol)
    f32 = cuda_ops.gemm(A, Bm, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    _close(f32, ref, atol=1e-2 + 1e-4 * K ** 0.5, rtol=1e-3)
    acc = torch.full((M, (N + 3) // 4 * 4), 2.0, device="cuda")[:, :N]
    cuda_ops.gemm(A, Bm, a_mn=a_mn, b_mn=b_mn, out=acc, accumulate=True)
    _close(acc, ref + 2.0, atol=1e-2 + 1e-4 * K ** 0.5, rtol=1e-3)
    ss = torch.zeros(1, device="cuda")
    f32b = cuda_ops.gemm(A, Bm, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32, sumsq=ss)
    _close(f32b, ref, atol=1e-2 + 1e-4 * K ** 0.5, rtol=1e-3)
    want = (ref.double() ** 2).sum().item()
    assert abs(ss.item() - want) <= 2e-3 * want


@pytest.mark.parametrize("pair,split,bn", [(0, 1, 0), (0, 2, 128), (0, 2, 192), (0, 0, 256), (2, 2, 256), (2, 2, 128), (2, 0, 0), (1, 1, 0)])
def test_gemm_forced_tilings(pair, split, bn):
    """Every tile family without the K-split tail, with it wherever possible (2) and where the cost rule takes it (1),
    on shapes whose last wave is partial."""
    from state_space_models_neuron_b200.ops import cuda_ops, native
    lib = native.lib()
    lib.ssm_gemm_set_options(pair, split, bn)
    try:
        for M, N, K in [(2048, 2320, 4096), (2176, 4096, 1024), (64, 2560, 5120), (1152, 1000, 520)]:
            a, b = _rand((M, K), M, 0.5), _rand((N, K), N, 0.5)
            ref = a.float() @ b.float().t()
            _close(cuda_ops.gemm(a, b), ref, atol=0.02 * K ** 0.5 * 0.25 + 0.02)
            bt = b.t().contiguous()
            if bt.shape[1] % 8:
                bt = torch.nn.functional.pad(bt, (0, (-bt.shape[1]) % 8))[:, :N]
            f32 = cuda_ops.gemm(a, bt, b_mn=True, out_dtype=torch.float32)
            _close(f32, ref, atol=1e-2 + 1e-4 * K ** 0.5, rtol=1e-3)
    finally:
        lib.ssm_gemm_set_options(1, 1, 0)


def test_gemm_repeated_launches_reuse_split_scratch():
    """Tail tiles exchange partial sums through a scratch buffer and arrival counters that must be clean again after
    every launch: run a tail-heavy shape many times back to back."""
    from state_space_models_neuron_b200.ops import cuda_ops
    a, b = _rand((2048, 4096), 1, 0.5), _rand((2320, 4096), 2, 0.5)
    ref = a.float() @ b.float().t()
    outs = [cuda_ops.gemm(a, b) for _ in range(12)]
    for o in outs:
        _close(o, ref, atol=0.35)
    assert all(torch.equal(outs[0], o) for o in outs[1:])


@pytest.mark.parametrize("M,N,K,vs", [(2048, 6286, 512, 6286 * 3), (256, 1000, 256, 0), (1024, 12572, 256, 12572)])
def test_gemm_cross_entropy_epilogue(M, N, K, vs):
    """Statistics from the GEMM epilogue equal those of a separate pass over the stored bf16 logits."""
    from state_space_models_neuron_b200.ops import cuda_ops, oracle
    a, b = _rand((M, K), 3, 1.0), _rand((N, K), 4, 0.3)
    g = torch.Generator(device="cuda").manual_seed(9)
    labels = torch.randint(0, 8 * N, (M,), device="cuda", generator=g)
    labels[::7] = -100
    labels[1::5] = vs + torch.randint(0, N, (len(labels[1::5]),), device="cuda", generator=g)
    y, (m, s, t) = cuda_ops.gemm_ce(a, b, labels, vs)
    _close(y, a.float() @ b.float().t(), atol=0.15)
    rm, rs, rt = oracle.ce_partials(y.float(), labels, vs)
    assert torch.equal(m, rm)
    _close(s, rs, atol=1e-5, rtol=2e-3)
    assert torch.equal(t, rt)


def test_linear_ce_loss_and_grads_match_separate_pass():
    from state_space_models_neuron_b200 import ops
    from state_space_models_neuron_b200.parallel.cross_entropy import parallel_cross_entropy
    x0, w0 = _rand((1, 512, 256), 5), _rand((1000, 256), 6, 0.1)
    labels = torch.randint(0, 1000, (1, 512), device="cuda")
    labels[0, -1] = -100
    res = []
    for fused in (True, False):
        x, w = x0.clone().requires_grad_(True), w0.clone().requires_grad_(True)
        if fused:
            y, stats = ops.linear_ce(x, w, labels.reshape(-1), 0)
            assert stats is not None
            loss = parallel_cross_entropy(y, labels, stats=stats).sum() / 511
        else:
            loss = parallel_cross_entropy(ops.linear(x, w), labels).sum() / 511
        loss.backward()
        res.append((loss.item(), x.grad.float(), w.grad.float()))
    assert abs(res[0][0] - res[1][0]) < 1e-4
    _close(res[0][1], res[1][1], atol=1e-6, rtol=1e-2)
    _close(res[0][2], res[1][2], atol=1e-6, rtol=1e-2)
    xr, wr = x0.float().requires_grad_(True), w0.float().requires_grad_(True)
    lr = torch.nn.functional.cross_entropy((xr @ wr.t()).reshape(-1, 1000), labels.reshape(-1), ignore_index=-100)
    assert abs(lr.item() - res[0][0]) < 2e-2


# ------------------------------------------------------------------------------------------------------
# one rank of a T-rank fused collective, all buffers on this GPU
# ------------------------------------------------------------------------------------------------------
def _ptrs(tensors):
    arr = (ctypes.c_void_p * 8)()
    for i, t in enumerate(tensors):
        arr[i] = t if isinstance(t, int) else t.data_ptr()
    return arr


def _fused(A, B, C, M, N, K, lda, ldb, ldc, b_mn, mode, T, me, seq, seq_base, flags, ag=None, rs=None, ce=None):
    from state_space_models_neuron_b200.ops import cuda_ops
    P, ll = cuda_ops._P, cuda_ops._ll
    null = _ptrs([])
    ag = ag or dict(on=0, rows=0, base=0, src=None, src_ld=0, dst=null, dst_ld=0, counter=None)
    rs = rs or dict(on=0, rows=0, base=0, land=null, ld=0, counters=None, local=None, slot_stride=0, out=None, out_ld=0)
    ce = ce or dict(labels=None, vocab_start=0, tmax=None, tsum=None, tgt=None)
    cuda_ops._run("ssm_gemm_bf16_fused", P(A), P(B), P(C), M, N, K, ll(lda), ll(ldb), ll(ldc), 0, int(b_mn), mode,
                  P(None), 0, P(cuda_ops.status_tensor(A.device)), cuda_ops._st(), T, me, seq, P(seq_base), _ptrs(flags),
                  ag["on"], ag["rows"], ag["base"], P(ag["src"]), ll(ag["src_ld"]), ag["dst"], ll(ag["dst_ld"]),
                  P(ag["counter"]),
                  rs["on"], rs["rows"], rs["base"], rs["land"], ll(rs["ld"]), P(rs["counters"]), P(rs["local"]),
                  ll(rs["slot_stride"]), P(rs["out"]), ll(rs["out_ld"]),
                  P(ce["labels"]), ll(ce["vocab_start"]), P(ce["tmax"]), P(ce["tsum"]), P(ce["tgt"]))


@pytest.mark.parametrize("T,me,Ls,K,N,b_mn", [(2, 0, 1024, 512, 2320, False), (8, 5, 256, 1024, 6286, False),
                                               (4, 3, 512, 256, 1024, True), (8, 0, 128, 512, 264, False)])
def test_all_gather_gemm_one_rank_of_T(T, me, Ls, K, N, b_mn):
    M = T * Ls
    shards = [_rand((Ls, K), 100 + s, 0.5) for s in range(T)]
    w = _rand((K, N) if b_mn else (N, K), 7, 0.5)
    if w.shape[1] % 8:
        w = torch.nn.functional.pad(w, (0, (-w.shape[1]) % 8))[:, :w.shape[1]]
    gathers = [torch.zeros(M, K, device="cuda", dtype=torch.bfloat16) for _ in range(T)]
    flags = [torch.zeros(256, device="cuda", dtype=torch.int32) for _ in range(T)]
    seq_base = torch.tensor([70000], device="cuda", dtype=torch.int32)
    counter = torch.zeros(8, device="cuda", dtype=torch.int32)
    base = FLAG_SLOTS * 1              # all-gather kind, parity 1
    for rep, seq in enumerate((5, 9)):         # twice in a row: counters and flags of the first call must not leak
        want_seq = 70000 + seq
        for s in range(T):
            if s != me:                          # what the peers' pushes would have left on this rank
                gathers[me][s * Ls:(s + 1) * Ls] = shards[s]
                flags[me][base + s * AG_GROUPS: base + (s + 1) * AG_GROUPS] = want_seq
        ld = (N + 7) // 8 * 8
        y = torch.zeros(M, ld, device="cuda", dtype=torch.bfloat16)[:, :N]
        _fused(gathers[me], w, y, M, N, K, K, w.stride(0), y.stride(0), b_mn, 0, T, me, seq, seq_base, flags,
               ag=dict(on=1, rows=Ls, base=base, src=shards[me], src_ld=K, dst=_ptrs(gathers), dst_ld=K, counter=counter))
        torch.cuda.synchronize()
        full = torch.cat(shards).float()
        ref = full @ (w.float() if b_mn else w.float().t())
        _close(y, ref, atol=0.02 * K ** 0.5 * 0.25 + 0.02)
        kb = (K + 63) // 64
        per = (kb + AG_GROUPS - 1) // AG_GROUPS
        groups = (kb + per - 1) // per                     # column groups of the shard, each with its own flag
        for t in range(T):
            assert torch.equal(gathers[t][me * Ls:(me + 1) * Ls], shards[me]), f"push to rank {t} incomplete"
            got = flags[t][base + me * AG_GROUPS: base + me * AG_GROUPS + groups]
            assert (got == want_seq).all(), (t, got.tolist())
        assert int(counter.abs().sum()) == 0


@pytest.mark.parametrize("T,me,Ls,K,N,b_mn", [(2, 1, 1024, 512, 512, False), (8, 2, 256, 1024, 4096, False),
                                               (4, 0, 512, 6286, 1024, True), (8, 7, 128, 256, 384, False)])
def test_gemm_reduce_scatter_one_rank_of_T(T, me, Ls, K, N, b_mn):
    M = T * Ls
    Kp = (K + 7) // 8 * 8
    a = torch.nn.functional.pad(_rand((M, K), 11, 0.5), (0, Kp - K))[:, :K]
    w = _rand((K, N) if b_mn else (N, K), 12, 0.5)
    if w.shape[1] % 8:
        w = torch.nn.functional.pad(w, (0, (-w.shape[1]) % 8))[:, :w.shape[1]]
    lands = [torch.zeros(T, Ls, N, device="cuda", dtype=torch.bfloat16) for _ in range(T)]
    flags = [torch.zeros(256, device="cuda", dtype=torch.int32) for _ in range(T)]
    seq_base = torch.tensor([2 ** 31 - 3], device="cuda", dtype=torch.int32)     # sequence numbers wrap in this test
    counters = torch.zeros(8, device="cuda", dtype=torch.int32)
    base = FLAG_SLOTS * 2              # reduce-scatter kind, parity 0
    full = a.float() @ (w.float() if b_mn else w.float().t())
    for seq in (2, 6):
        want_seq = (2 ** 31 - 3 + seq + 2 ** 31) % 2 ** 32 - 2 ** 31       # int32 wrap-around
        others = [_rand((Ls, N), 300 + s + seq, 0.5) for s in range(T)]
        for s in range(T):
            if s != me:
                lands[me][s] = others[s]
                flags[me][base + s] = want_seq
        out = torch.zeros(Ls, N, device="cuda", dtype=torch.bfloat16)
        land_ptrs = _ptrs([lands[o][me] for o in range(T)])
        _fused(a, w, None, M, N, K, a.stride(0), w.stride(0), 0, b_mn, 3, T, me, seq, seq_base, flags,
               rs=dict(on=1, rows=Ls, base=base, land=land_ptrs, ld=N, counters=counters, local=lands[me],
                       slot_stride=Ls * N, out=out, out_ld=N))
        torch.cuda.synchronize()
        tol = 0.02 * K ** 0.5 * 0.25 + 0.02
        for o in range(T):
            if o == me:          # this rank's own rows never take the detour through the landing zone
                continue
            _close(lands[o][me], full[o * Ls:(o + 1) * Ls], atol=tol)
            assert int(flags[o][base + me]) == want_seq
        ref = full[me * Ls:(me + 1) * Ls] + sum(others[s].float() for s in range(T) if s != me)
        _close(out, ref, atol=2e-2 + 0.004 * K ** 0.5, rtol=1e-2)
        assert int(counters.abs().sum()) == 0
