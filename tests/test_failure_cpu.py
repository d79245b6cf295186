"""Failure detection without touching a GPU: failures are made on the host (a rank that exits, a heartbeat that
stops, a truncated checkpoint shard, NaN gradients)."""
import os
import tempfile
import time

import pytest
import torch
import torch.distributed as dist

from state_space_models_neuron_b200.utils.failure import Heartbeat, RankFailure, skip_step_on_nonfinite
from tests.dist_utils import run_ranks


def test_heartbeat_detects_silent_rank():
    store = dist.HashStore()
    a = Heartbeat(store, 0, 2, period_s=0.05, timeout_s=0.4).start()
    b = Heartbeat(store, 1, 2, period_s=0.05, timeout_s=0.4).start()
    time.sleep(0.3)
    assert a.dead_ranks() == []
    b.stop()                      # rank 1 goes silent between steps
    deadline = time.time() + 5
    while time.time() < deadline and not a.dead_ranks():
        time.sleep(0.1)
    with pytest.raises(RankFailure):
        a.check()
    a.stop()


def _rank_that_leaves(rank, world):
    """rank 1 raises between steps; rank 0 learns of it through the store before its next collective."""
    store = dist.distributed_c10d._get_default_store()
    hb = Heartbeat(store, rank, world, period_s=0.05, timeout_s=0.5, prefix="t").start()
    t = torch.ones(4)
    dist.all_reduce(t)            # step 1: everyone present
    if rank == 1:
        hb.stop()
        store.set("left/1", "1")
        time.sleep(1.5)           # stays alive only so the spawner's final barrier can complete
        return
    deadline = time.time() + 10
    detected = False
    while time.time() < deadline:
        if hb.dead_ranks():
            detected = True
            break
        time.sleep(0.1)
    assert detected, "rank 0 did not notice that rank 1 stopped"
    hb.stop()


def test_rank_leaving_between_steps_is_noticed_on_the_host():
    run_ranks(_rank_that_leaves, 2)


def test_truncated_checkpoint_shard_is_rejected_and_newest_points_to_complete_one():
    from state_space_models_neuron_b200.parallel import checkpoint as ck
    from state_space_models_neuron_b200.parallel import state as ps
    ps.initialize_model_parallel(1)
    with tempfile.TemporaryDirectory() as d:
        ck.save_checkpoint(d, "a", {"w": torch.arange(10.)}, None, None, {"global_step": 1})
        assert ck.newest_tag(d) == "a"
        # a crash while writing tag "b": shard half-written, never published
        os.makedirs(os.path.join(d, "b", "model"))
        with open(os.path.join(d, "b", "model", ck.shard_file_name(0, 0) + ".tmp"), "wb") as f:
            f.write(b"\x00" * 10)
        assert ck.newest_tag(d) == "a" and ck.list_tags(d) == ["a"]
        # corrupt the published shard: loading must fail loudly, not return garbage
        p = os.path.join(d, "a", "model", ck.shard_file_name(0, 0))
        data = open(p, "rb").read()
        open(p, "wb").write(data[: len(data) // 2])

        class M(torch.nn.Module):
            def __init__(self):
                super().__init__()
                self.w = torch.nn.Parameter(torch.zeros(10))
        with pytest.raises(Exception):
            ck.load_checkpoint(d, None, model=M())


def test_nan_gradients_skip_the_step():
    from state_space_models_neuron_b200.parallel import state as ps
    from state_space_models_neuron_b200.parallel.zero1 import Zero1Optimizer
    ps.initialize_model_parallel(1)
    p = torch.nn.Parameter(torch.ones(256))
    opt = Zero1Optimizer([{"params": [p]}], lr=0.1)
    opt.zero_grad()
    (p * float("nan")).sum().backward()
    assert skip_step_on_nonfinite(opt)
    assert torch.equal(p.detach(), torch.ones(256))
    opt.zero_grad()
    (p * 2).sum().backward()
    assert not skip_step_on_nonfinite(opt)
    opt.step()
    assert (p.detach() < 1).all()
