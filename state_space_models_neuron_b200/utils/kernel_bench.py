"""Run one kernel of the framework on one shape: the small case used for `ncu` captures and the CUDA-event
timing behind the roofline numbers in `profiles/`.

    python -m state_space_models_neuron_b200.utils.kernel_bench gemm --m 2048 --n 18560 --k 4096 --iters 20
    python -m state_space_models_neuron_b200.utils.kernel_bench gemm --m 2048 --n 4096 --k 1024 --trace
    python -m state_space_models_neuron_b200.utils.kernel_bench ssd --seq 2048 --heads 128 --groups 8 --iters 10
    python -m state_space_models_neuron_b200.utils.kernel_bench norm|conv|attn|adamw ...
    python -m torch.distributed.run --nproc-per-node T --master-addr 127.0.0.1 -m \
        state_space_models_neuron_b200.utils.kernel_bench ag_gemm|gemm_rs --seq 2048 --gemm_k 4096 --gemm_n 18560
        (fused collective + GEMM over T ranks; --gemm_n / --gemm_k are the GLOBAL sizes, each rank takes 1/T; the time is the
        max over ranks and the roofline is the slower of FLOPs at the measured GEMM peak and NVLink bytes at the
        measured 770 GB/s per direction)

Prints one JSON line: time per launch (CUDA events, after warm-up, L2 flushed between launches by writing a
256 MiB buffer), achieved TFLOP/s or GB/s and the fraction of the measured peak from MEASURED_PEAKS.json.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from ..ops import cuda_ops


TRACE_SLOTS = 24          # int64 time stamps per CTA written by the GEMM kernel (GEMM_TRACE_SLOTS in ops/csrc/gemm.cu)


def _peaks():
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    for base in (os.getcwd(), here):
        p = os.path.join(base, "MEASURED_PEAKS.json")
        if os.path.exists(p):
            with open(p) as f:
                d = json.load(f)
            return d.get("bf16_tflops", 1590.0), d.get("hbm_gbs", 6650.0), "measured"
    return 1590.0, 6650.0, "fallback"


def time_kernel(fn, iters: int, warmup: int = 3, flush: bool = True) -> float:
    scratch = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if scratch is not None:
            scratch.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    cuda_ops.check_status()
    return total / iters


def plan_gemm(a):
    """`gemm --plan`: the tiling and work distribution the library picks for this shape (no launch, works without a GPU)."""
    from . import debug
    for accumulate in (False, True):
        print(json.dumps({"kernel": "gemm-plan", "m": a.m, "n": a.n, "k": a.k, "accumulate": accumulate,
                          **debug.gemm_plan(a.m, a.n, a.k, accumulate=accumulate)}))


def bench_gemm(a):
    A = torch.randn(a.m, a.k, device="cuda").bfloat16()
    B = torch.randn(a.n, a.k, device="cuda").bfloat16()
    if a.layout == "tn":
        fn = lambda: cuda_ops.gemm(A, B)
    elif a.layout == "nn":
        Bt = B.t().contiguous()
        fn = lambda: cuda_ops.gemm(A, Bt, b_mn=True)
    else:
        At, Bt = A.t().contiguous(), B.t().contiguous()
        out = torch.zeros(a.m, a.n, device="cuda")
        fn = lambda: cuda_ops.gemm(At, Bt, a_mn=True, b_mn=True, out=out, accumulate=False)
    ms = time_kernel(fn, a.iters)
    return ms, 2.0 * a.m * a.n * a.k, None


def trace_gemm(a):
    """Timeline of one GEMM launch from the kernel's own timestamps (global timer, one record per CTA): when the
    first operands land, when each accumulator is complete, how long the epilogue takes."""
    import ctypes
    from ..ops import native
    lib = native.lib()
    A = torch.randn(a.m, a.k, device="cuda").bfloat16()
    B = torch.randn(a.n, a.k, device="cuda").bfloat16()
    odt = torch.float32 if a.fp32_out else torch.bfloat16
    for _ in range(3):
        cuda_ops.gemm(A, B, out_dtype=odt)
    torch.cuda.synchronize()
    tr = torch.zeros(148 * TRACE_SLOTS, dtype=torch.int64, device="cuda")
    lib.ssm_gemm_set_trace(ctypes.c_void_p(tr.data_ptr()))
    cuda_ops.gemm(A, B, out_dtype=odt)
    torch.cuda.synchronize()
    lib.ssm_gemm_set_trace(ctypes.c_void_p(0))
    t = tr.view(148, TRACE_SLOTS).cpu().double()
    t0 = t[:, 0][t[:, 0] > 0].min()
    names = [(0, "CTA set-up done"), (8, "first TMA load issued"), (1, "first stage landed"),
             (2, "first tile: MMAs issued"), (4, "first tile: accumulator complete"), (5, "first tile: epilogue done"),
             (3, "last tile: MMAs issued"), (6, "last tile: accumulator complete"), (7, "last tile: epilogue done"),
             (9, "producer finished"), (10, "CTA done")]
    out = {"kernel": "gemm-trace", "m": a.m, "n": a.n, "k": a.k, "out": str(odt), "events_us": {}}
    for slot, name in names:
        col = t[:, slot]
        col = col[col > 0]
        if len(col):
            out["events_us"][name] = {"ctas": int(len(col)), "min": round(float((col.min() - t0) / 1e3), 2),
                                      "median": round(float((col.median() - t0) / 1e3), 2),
                                      "max": round(float((col.max() - t0) / 1e3), 2)}
    print(json.dumps(out))


def bench_ssd(a):
    from .. import ops
    H, P, G, N, L, Bz = a.heads, 64, a.groups, 128, a.seq, a.batch
    x = torch.randn(Bz, L, H, P, device="cuda").bfloat16().requires_grad_(True)
    dt = (torch.rand(Bz, L, H, device="cuda") * 4 - 4).bfloat16().requires_grad_(True)
    A = -(torch.rand(H, device="cuda") * 15 + 1)
    Bm = (torch.randn(Bz, L, G, N, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    Cm = (torch.randn(Bz, L, G, N, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    D, bias = torch.ones(H, device="cuda"), torch.zeros(H, device="cuda")
    if a.backward:
        y = ops.ssd_chunk_scan(x, dt, A, Bm, Cm, D, bias)
        gy = torch.randn_like(y)
        fn = lambda: torch.autograd.grad(y, [x, dt, Bm, Cm], gy, retain_graph=True)
    else:
        fn = lambda: ops.ssd_chunk_scan(x.detach(), dt.detach(), A, Bm.detach(), Cm.detach(), D, bias)
    ms = time_kernel(fn, a.iters)
    byts = 2.0 * Bz * L * (2 * H * P + 2 * G * N + H) * (3 if a.backward else 1)
    return ms, None, byts


def bench_norm(a):
    from .. import ops
    rows, d = a.rows, a.cols
    y = torch.randn(1, rows, d, device="cuda").bfloat16().requires_grad_(True)
    z = torch.randn(1, rows, d, device="cuda").bfloat16().requires_grad_(True)
    w = torch.ones(d, device="cuda").bfloat16().requires_grad_(True)
    if a.backward:
        out = ops.gated_rmsnorm(y, z, w, 1e-5, a.group)
        go = torch.randn_like(out)
        fn = lambda: torch.autograd.grad(out, [y, z, w], go, retain_graph=True)
        byts = 2.0 * rows * d * 5
    else:
        fn = lambda: ops.gated_rmsnorm(y.detach(), z.detach(), w.detach(), 1e-5, a.group)
        byts = 2.0 * rows * d * 3
    return time_kernel(fn, a.iters), None, byts


def bench_conv(a):
    from .. import ops
    x = torch.randn(a.batch, a.seq, a.cols, device="cuda").bfloat16().requires_grad_(True)
    w = (torch.randn(a.cols, 1, 4, device="cuda") * 0.3).bfloat16().requires_grad_(True)
    b = torch.zeros(a.cols, device="cuda").bfloat16().requires_grad_(True)
    if a.backward:
        out = ops.causal_conv1d_silu(x, w, b)
        go = torch.randn_like(out)
        fn = lambda: torch.autograd.grad(out, [x, w, b], go, retain_graph=True)
        byts = 2.0 * a.batch * a.seq * a.cols * 3
    else:
        fn = lambda: ops.causal_conv1d_silu(x.detach(), w.detach(), b.detach())
        byts = 2.0 * a.batch * a.seq * a.cols * 2
    return time_kernel(fn, a.iters), None, byts


def bench_attn(a):
    from .. import ops
    q = torch.randn(a.batch, a.seq, a.heads, 128, device="cuda").bfloat16().requires_grad_(True)
    k = torch.randn(a.batch, a.seq, a.groups, 128, device="cuda").bfloat16().requires_grad_(True)
    v = torch.randn(a.batch, a.seq, a.groups, 128, device="cuda").bfloat16().requires_grad_(True)
    fl = 4.0 * a.batch * a.heads * a.seq * a.seq * 128 / 2
    if a.backward:
        o = ops.attention(q, k, v)
        go = torch.randn_like(o)
        fn = lambda: torch.autograd.grad(o, [q, k, v], go, retain_graph=True)
        fl *= 2.5
    else:
        fn = lambda: ops.attention(q.detach(), k.detach(), v.detach())
    return time_kernel(fn, a.iters), fl, None


def bench_adamw(a):
    n = a.n
    master, m, v = [torch.zeros(n, device="cuda") for _ in range(3)]
    g = torch.randn(n, device="cuda")
    out = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    clip = torch.ones(1, device="cuda")
    fn = lambda: cuda_ops.adamw_step(master, m, v, g, out, clip, 1e-3, 0.9, 0.95, 1e-8, 0.1, 1)
    return time_kernel(fn, a.iters, flush=False), None, 30.0 * n


NVLINK_GBS = 770.0      # measured peer-copy bandwidth per direction per GPU on this pool


def _dist_setup():
    from ..parallel import state as ps
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    ps.initialize_model_parallel(world, backend="nccl")
    return ps, world


def _time_collective(fn, iters, warmup=5, graph=True):
    """Device time per call, max over ranks.  The `iters` calls are captured into one CUDA graph and replayed so
    that the host (tensor-map encoding, Python) is off the clock, as it is in the graphed training step."""
    import torch.distributed as dist
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(warmup):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = None
    if graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(iters):
                fn()
        g.replay()                      # one untimed replay
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    if g is not None:
        g.replay()
    else:
        for _ in range(iters):
            fn()
    b.record()
    torch.cuda.synchronize()
    cuda_ops.check_status()
    t = torch.tensor([a.elapsed_time(b) / iters], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    del g
    return t.item()


def bench_fused(a):
    """all-gather + GEMM (`ag_gemm`) or GEMM + reduce-scatter (`gemm_rs`) as the training step runs them, and the
    same operation through NCCL + the plain GEMM kernel for comparison."""
    import torch.distributed as dist
    from ..parallel import fused_ops, mappings as mp, symm
    ps, T = _dist_setup()
    L, Ls = a.seq, a.seq // T
    ws = symm.get_workspace(L, max(a.k, a.n) if a.kernel == "ag_gemm" else a.n, torch.device("cuda"))
    g = torch.Generator(device="cuda").manual_seed(ps.get_rank())
    if a.kernel == "ag_gemm":
        K, N = a.k, a.n // T
        x = torch.randn(1, Ls, K, device="cuda", generator=g).bfloat16()
        w = torch.randn(N, K, device="cuda", generator=g).bfloat16()
        fused_fn = lambda: fused_ops._ag_gemm(x.reshape(Ls, K), w, False, None, ws)
        lib_fn = lambda: cuda_ops.gemm(mp.all_gather_seq(x).reshape(L, K), w)
        xfull = torch.randn(L, K, device="cuda", generator=g).bfloat16()
        plain_fn = lambda: cuda_ops.gemm(xfull, w)
        flops, link = 2.0 * L * N * K, (T - 1) * Ls * K * 2.0
    else:
        K, N = a.k // T, a.n
        x = torch.randn(L, K, device="cuda", generator=g).bfloat16()
        w = torch.randn(N, K, device="cuda", generator=g).bfloat16()
        fused_fn = lambda: fused_ops._gemm_rs(x, w, False, ws)
        lib_fn = lambda: mp.reduce_scatter_seq(cuda_ops.gemm(x, w).reshape(1, L, N))
        plain_fn = lambda: cuda_ops.gemm(x, w)
        flops, link = 2.0 * L * N * K, (T - 1) * Ls * N * 2.0

    def stepped(fn):
        def run():
            symm.advance_step()
            fn()
        return run
    if a.trace:
        # in-kernel timeline of one fused call (timestamps from the global timer, one record per CTA)
        import ctypes
        from ..ops import native
        lib = native.lib()
        for _ in range(3):
            stepped(fused_fn)()
        torch.cuda.synchronize()
        dist.barrier()
        tr = torch.zeros(148 * TRACE_SLOTS, dtype=torch.int64, device="cuda")
        lib.ssm_gemm_set_trace(ctypes.c_void_p(tr.data_ptr()))
        stepped(fused_fn)()
        torch.cuda.synchronize()
        lib.ssm_gemm_set_trace(ctypes.c_void_p(0))
        t = tr.view(148, TRACE_SLOTS).cpu().double()
        t0 = t[:, 0][t[:, 0] > 0].min()
        names = [(0, "set-up done"), (16, "push: first box in shared memory"), (17, "push: all boxes issued"),
                 (18, "push: own boxes of group 0 complete"), (20, "push: flag of group 0 published"), (11, "push finished"), (12, "first remote group arrived"), (1, "first stage landed"),
                 (4, "first accumulator complete"), (5, "first epilogue done"), (6, "last accumulator complete"),
                 (7, "last epilogue done"), (9, "producer finished"), (14, "tiles stored, flags published"),
                 (13, "tail: all sources seen"), (10, "CTA done")]
        out = {"kernel": a.kernel + "-trace", "rank": dist.get_rank(), "ranks": T, "events_us": {}}
        for slot, name in names:
            col = t[:, slot]
            col = col[col > 0]
            if len(col):
                out["events_us"][name] = [round(float((col.min() - t0) / 1e3), 1), round(float((col.median() - t0) / 1e3), 1),
                                          round(float((col.max() - t0) / 1e3), 1)]
        if a.trace_dump and dist.get_rank() == 0:
            # raw per-CTA records of rank 0, microseconds from the first CTA's start (0 = event not reached)
            rel = torch.where(t > 0, (t - t0) / 1e3, torch.zeros_like(t))
            with open(a.trace_dump, "w") as f:
                json.dump({"slots": {str(k): v for k, v in names}, "cta_us": [[round(float(x), 1) for x in row] for row in rel]}, f)
        for r in range(T):
            if r == dist.get_rank():
                print(json.dumps(out), flush=True)
            dist.barrier()
        torch.cuda.synchronize()
        os._exit(0)
    ms = _time_collective(stepped(fused_fn), a.iters)
    ms_lib = _time_collective(lib_fn, a.iters)
    ms_plain = _time_collective(plain_fn, a.iters)
    tf_peak, _, src = _peaks()
    roof_ms = max(flops / (tf_peak * 1e9), link / (NVLINK_GBS * 1e6))
    if dist.get_rank() == 0:
        print(json.dumps({"kernel": a.kernel, "ranks": T, "M": L, "N": N, "K": K, "ms_fused": ms, "ms_nccl_plus_gemm": ms_lib,
                          "ms_gemm_alone": ms_plain,
                          "roofline_ms": roof_ms, "compute_ms_at_%s_peak" % src: flops / (tf_peak * 1e9),
                          "nvlink_ms_at_770GBs": link / (NVLINK_GBS * 1e6), "frac_of_roofline": roof_ms / ms,
                          "timing": "calls captured in one CUDA graph, CUDA events around the replay, max over ranks"}))
    torch.cuda.synchronize()
    dist.barrier()
    os._exit(0)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["gemm", "ssd", "norm", "conv", "attn", "adamw", "ag_gemm", "gemm_rs"])
    ap.add_argument("--m", "--gemm_m", type=int, default=2048)
    ap.add_argument("--n", "--gemm_n", type=int, default=4096)   # --gemm_* spellings: torchrun rejects "--n"
    ap.add_argument("--k", "--gemm_k", type=int, default=4096)
    ap.add_argument("--layout", default="tn", choices=["tn", "nn", "tt"])
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--heads", type=int, default=128)
    ap.add_argument("--groups", type=int, default=8)
    ap.add_argument("--rows", type=int, default=2048)
    ap.add_argument("--cols", type=int, default=8192)
    ap.add_argument("--group", type=int, default=8192)
    ap.add_argument("--backward", action="store_true")
    ap.add_argument("--trace", action="store_true", help="gemm: print the in-kernel pipeline timeline instead of timing")
    ap.add_argument("--plan", action="store_true", help="gemm: print the tiling / K-split plan for the shape and exit (no GPU needed)")
    ap.add_argument("--fp32_out", action="store_true", help="gemm --trace: fp32 output (gradient epilogue)")
    ap.add_argument("--trace_dump", default="", help="ag_gemm / gemm_rs --trace: also write rank 0's per-CTA records to this JSON file")
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args(argv)
    if a.kernel in ("ag_gemm", "gemm_rs"):
        return bench_fused(a)
    if a.kernel == "gemm" and a.plan:
        return plan_gemm(a)
    if a.kernel == "gemm" and a.trace:
        return trace_gemm(a)
    ms, flops, byts = {"gemm": bench_gemm, "ssd": bench_ssd, "norm": bench_norm, "conv": bench_conv,
                       "attn": bench_attn, "adamw": bench_adamw}[a.kernel](a)
    tf_peak, bw_peak, src = _peaks()
    out = {"kernel": a.kernel, "args": {k: v for k, v in vars(a).items() if k != "kernel"}, "ms": ms}
    if flops:
        out["tflops"] = flops / ms / 1e9
        out["frac_of_%s_bf16_peak" % src] = out["tflops"] / tf_peak
    if byts:
        out["gbs"] = byts / ms / 1e6
        out["frac_of_%s_hbm_peak" % src] = out["gbs"] / bw_peak
    print(json.dumps(out))


if __name__ == "__main__":
    main()
