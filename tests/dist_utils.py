"""Spawn gloo CPU ranks for distributed tests (rendezvous through a temp file, no network)."""
import os
import tempfile
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _entry(rank, world, path, fn, args, errq):
    try:
        torch.set_num_threads(1)
        dist.init_process_group("gloo", init_method=f"file://{path}", rank=rank, world_size=world)
        fn(rank, world, *args)
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        errq.put((rank, traceback.format_exc()))
        raise


def run_ranks(fn, world: int, *args, timeout: float = 300.0):
    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "rdzv")
        procs = [ctx.Process(target=_entry, args=(r, world, path, fn, args, errq)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout)
        alive = [p for p in procs if p.is_alive()]
        for p in alive:
            p.kill()
        msgs = []
        while not errq.empty():
            msgs.append(errq.get())
        assert not alive, "ranks timed out"
        assert not msgs and all(p.exitcode == 0 for p in procs), "\n".join(f"rank {r}:\n{m}" for r, m in msgs)
